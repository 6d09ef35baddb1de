"""Regenerates the encoder fixtures in this directory from the reference's own encoder.

Run in a container that has the reference sources (oracle/Makefile builds them into
oracle/_ref):   python tests/golden/make_golden.py
Each .npz holds the dense input (fp16 bit patterns) and the five arrays plus max_nnz that the
reference's InitSparseMatrixA_bitmap (csrc/SpMM_API.cuh:112-241) returned for it; operand_b/*.npz hold the same for
the fork's encoder of a compressed second operand, InitSparseMatrixA_bitmap_v6_B (csrc/spmm_test_utils.h:523-652).
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
import oracle  # noqa: E402


def cases():
    rng = np.random.default_rng(20250101)

    def rnd(M, K, s):
        A = (rng.standard_normal((M, K)) * 0.02).astype(np.float16)
        A[rng.random((M, K)) < s] = 0
        return A.view(np.uint16)

    out = {"rand_64x64_s50": rnd(64, 64, 0.5), "rand_128x192_s60": rnd(128, 192, 0.6),
           "rand_192x64_s90": rnd(192, 64, 0.9), "dense_64x64": rnd(64, 64, 0.0),
           "empty_64x128": np.zeros((64, 128), np.uint16)}
    # special values: -0.0 and +0.0 are dropped, NaN / inf / subnormals are kept
    sp = rnd(64, 64, 0.7)
    specials = np.array([0x8000, 0x0000, 0x7E00, 0xFE00, 0x7C00, 0xFC00, 0x0001, 0x8001, 0x03FF, 0x7BFF], np.uint16)
    idx = rng.choice(64 * 64, size=400, replace=False)
    sp.reshape(-1)[idx] = specials[rng.integers(0, len(specials), 400)]
    out["specials_64x64"] = sp
    # exactly one non-zero per 8x8 tile, at every bit position in turn
    one = np.zeros((64, 64), np.uint16)
    for t in range(64):
        r0, c0 = 8 * (t // 8), 8 * (t % 8)
        one[r0 + t // 8, c0 + t % 8] = 0x3C00 + t
    out["one_per_tile_64x64"] = one
    return out


def main():
    assert oracle.have_ref(), "oracle/_ref is not built (needs the reference sources)"
    for name, A in cases().items():
        e = oracle.ref_encode(A)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), A=A, vals=e.vals, tile_nnz=e.tile_nnz, mtile=e.mtile,
                            gtile=e.gtile, bitmap=e.bitmap, max_nnz=np.int32(e.max_nnz))
        print(name, A.shape, "val_count", e.vals.size, "max_nnz", e.max_nnz)
    assert oracle.have_ref_b(), "oracle/_ref/libref_encoder_b.so is not built"
    os.makedirs(os.path.join(HERE, "operand_b"), exist_ok=True)
    for name, A in cases().items():
        e = oracle.ref_encode_b(A)
        np.savez_compressed(os.path.join(HERE, "operand_b", name + ".npz"), A=A, vals=e.vals, tile_nnz=e.tile_nnz,
                            mtile=e.mtile, gtile=e.gtile, bitmap=e.bitmap, max_nnz=np.int32(e.max_nnz))
        print("operand_b", name, A.shape, "val_count", e.vals.size, "max_nnz", e.max_nnz)


if __name__ == "__main__":
    main()
