"""The C-ABI library loads and exports every symbol include/spmm_b200.h and include/SpMM_API.cuh declare.

No compute entry point is called here (no GPU in this tier of the suite).
"""
import ctypes
import os
import re
import subprocess

from conftest import ROOT


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "spmm_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(spb_\w+|Our_GenSparseMatrixBinFile)\s*\(", text)))


def test_header_declares_expected_entry_points():
    names = _declared_functions()
    for n in ("spb_encode_host", "spb_encode_device", "spb_spmm_bitmap_v3", "spb_splitk_reduce",
              "Our_GenSparseMatrixBinFile"):
        assert n in names


def test_library_exports_every_declared_symbol(lib_built):
    from spmspm_b200 import _lib
    for name in _declared_functions():
        assert hasattr(lib_built, name), name
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    for name in _lib.SIGNATURES:
        assert name in _declared_functions(), f"{name} bound but not declared in the header"


def test_library_exports_reference_mangled_symbols(lib_built):
    from spmspm_b200 import _lib
    for sym in _lib.MANGLED:
        ctypes.cast(getattr(lib_built, sym), ctypes.c_void_p)


def test_version_and_error_string(lib_built):
    assert lib_built.spb_version() >= 100
    assert isinstance(lib_built.spb_last_error(), bytes)


def test_reference_header_compiles_against_the_library(tmp_path, lib_built):
    """A translation unit written like the reference's callers compiles and links unchanged."""
    src = tmp_path / "caller.cu"
    src.write_text(r'''
#include "SpMM_API.cuh"
int main(int argc, char**) {
    if (argc > 100) {  // never executed: link check only
        half* v; int *a, *b, *c; uint64_t* bm; int mx;
        InitSparseMatrixA_bitmap(nullptr, 64, 64, 8, 16, 64, 8, 64, 64, &v, &a, &b, &c, &bm, mx);
        SpMM_SplitK_API_bitmap_v3(0, nullptr, v, c, b, bm, a, v, v, 64, 16, 64, v, 1);
        Our_GenSparseMatrixBinFile(nullptr, 64, 64, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr);
    }
    return 0;
}
''')
    exe = tmp_path / "caller"
    libdir = os.path.join(ROOT, "spmspm_b200")
    r = subprocess.run(["/usr/local/cuda/bin/nvcc", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a",
                        "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe), "-L", libdir,
                        "-l:libSpMM_API.so", "-Xlinker", f"-rpath={libdir}"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    assert subprocess.run([str(exe)]).returncode == 0


def test_split_k_suggestion_and_schedule_switch_without_gpu(lib_built):
    """The suggestion is pure host arithmetic (148 SMs assumed when no device answers): it never leaves an empty
    last range, and it follows the schedule switch."""
    from spmspm_b200 import _lib
    lib = _lib.load()
    assert lib.spb_set_schedule(0) in (0, 1, 2)
    for M, N, K in [(28672, 16, 7168), (4096, 16, 4096), (5120, 16, 5120), (5120, 32, 20480), (64, 16, 64), (128, 8, 192),
                    (15360, 8, 5120), (1152, 16, 36864)]:
        for mode in (0, 1):
            lib.spb_set_schedule(mode)
            sk = lib.spb_suggest_split_k(M, N, K)
            kt = K // 64
            assert 1 <= sk <= min(32, kt)
            avg = (kt - 1) // sk + 1
            assert (sk - 1) * avg < kt                      # no empty last range
    lib.spb_set_schedule(1)
    assert lib.spb_suggest_split_k(28672, 16, 7168) > 1     # static: 224 items on 148 SMs want a split
    lib.spb_set_schedule(0)
    assert lib.spb_suggest_split_k(28672, 16, 7168) == 1    # balanced shares fill the SMs without one
    assert lib.spb_set_schedule(7) == -1 and lib.spb_set_schedule(0) == 0


def test_spmm_entry_points_reject_bad_arguments_without_launching(lib_built):
    """Shapes, null pointers and misaligned pointers are turned into error codes before any CUDA call is made, by the
    plain entry point and by the fused all-gather one alike (bulk copies and tensor maps fault on the device on a
    pointer that is not 16-byte aligned)."""
    from spmspm_b200 import _lib
    lib = _lib.load()
    INVALID, MISALIGNED = 1, 716          # cudaErrorInvalidValue, cudaErrorMisalignedAddress
    ok = 0x10000                          # never dereferenced: every call below fails its checks first
    args = dict(vals=ok, gt=ok, mt=ok, bm=ok, mx=ok, B=ok, C=ok, ws=ok)

    def spmm(M=128, N=16, K=128, sk=1, **over):
        a = dict(args, **over)
        return lib.spb_spmm_bitmap_v3(None, None, a["vals"], a["gt"], a["mt"], a["bm"], a["mx"], a["B"], a["C"], M, N, K,
                                      a["ws"], sk)

    assert spmm(M=100) == INVALID and spmm(K=0) == INVALID and spmm(N=0) == INVALID
    assert spmm(sk=3) == INVALID                      # more ranges than k-tiles
    assert spmm(vals=None) == INVALID and spmm(C=None) == INVALID and spmm(sk=2, ws=None) == INVALID
    for name in ("vals", "mt", "bm", "B", "C"):
        assert spmm(**{name: ok + 2}) == MISALIGNED, name
    assert spmm(sk=2, ws=ok + 8) == MISALIGNED
    assert b"16-byte" in lib.spb_last_error()

    peers = (ctypes.c_void_p * 2)(ok, ok)

    def gather(M=128, N=16, K=128, sk=1, n_peers=2, rank=0, M_full=256, row0=0, **over):
        a = dict(args, **over)
        return lib.spb_spmm_bitmap_v3_allgather(None, a["vals"], a["gt"], a["mt"], a["bm"], a["mx"], a["B"], peers, peers,
                                                n_peers, rank, M, N, K, M_full, row0, None, a["ws"], sk)

    assert gather(n_peers=9) == INVALID and gather(rank=2) == INVALID and gather(row0=192) == INVALID
    assert gather(M=96) == INVALID and gather(vals=None) == INVALID and gather(sk=2, ws=None) == INVALID
    for name in ("vals", "mt", "bm", "B"):
        assert gather(**{name: ok + 4}) == MISALIGNED, name
    assert gather(sk=2, ws=ok + 2) == MISALIGNED

    def linear(act=0, bias=ok, res=ok, **over):
        a = dict(args, **over)
        return lib.spb_linear_bitmap_v3(None, a["vals"], a["gt"], a["mt"], a["bm"], a["mx"], a["B"], a["C"], 128, 16, 128,
                                        bias, res, act, a["ws"], 1)

    assert linear(act=2) == INVALID and linear(act=-1) == INVALID and linear(vals=None) == INVALID
    assert linear(bias=ok + 2) == MISALIGNED and linear(res=ok + 8) == MISALIGNED
    assert lib.spb_linear_allreduce_finish(None, ok, ok, ok, 1, 128, 16, ok + 2, None, 0) == INVALID
    assert lib.spb_linear_allreduce_finish(None, ok, ok, ok, 1, 128, 16, None, None, 3) == INVALID
    assert lib.spb_linear_allreduce_finish(None, ok, ok, None, 1, 128, 16, None, None, 0) == INVALID


def test_launch_counter_is_callable_without_a_gpu(lib_built):
    from spmspm_b200 import _lib
    lib = _lib.load()
    n = lib.spb_launch_count()
    assert isinstance(n, int) and n >= 0
    # rejected calls launch nothing
    assert lib.spb_spmm_bitmap_v3(None, None, None, None, None, None, None, None, None, 128, 16, 128, None, 1) != 0
    assert lib.spb_launch_count() == n
