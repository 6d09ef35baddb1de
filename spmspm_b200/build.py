"""In-tree build of libSpMM_API.so (nvcc, sm_100a only)."""
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))


def build(verbose=False):
    r = subprocess.run(["make", "-C", os.path.join(_HERE, "csrc"), "-j", "4"], capture_output=True, text=True)
    if verbose or r.returncode != 0:
        print(r.stdout[-4000:])
        print(r.stderr[-4000:])
    if r.returncode != 0:
        raise RuntimeError("building libSpMM_API.so failed")
    return os.path.join(_HERE, "libSpMM_API.so")
