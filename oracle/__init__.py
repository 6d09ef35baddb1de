"""ctypes front-end of the CPU oracle (oracle.c) and of the compiled reference encoder.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke test and by the
benchmark's CPU-baseline leg.  The shipped package never imports this module.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "liboracle.so")
_REF = os.path.join(_HERE, "_ref", "libref_encoder.so")
_REF_SPMM = os.path.join(_HERE, "_ref", "libref_style_spmm.so")

_u16p = ctypes.POINTER(ctypes.c_uint16)
_i32p = ctypes.POINTER(ctypes.c_int)
_u64p = ctypes.POINTER(ctypes.c_uint64)
_f32p = ctypes.POINTER(ctypes.c_float)


def build(force=False):
    """Compile liboracle.so (and _ref/ when the reference sources are present)."""
    if force or not os.path.exists(_LIB) or os.path.getmtime(_LIB) < os.path.getmtime(os.path.join(_HERE, "oracle.c")):
        subprocess.run(["make", "-C", _HERE, "liboracle.so"], check=True, capture_output=True)
    # REF_DIR (the csrc directory of a checkout of the reference) overrides the Makefile's default
    ref_dir = os.environ.get("REF_DIR") or _makefile_ref_dir()
    if ref_dir and os.path.isdir(ref_dir) and (force or not os.path.exists(_REF) or not os.path.exists(_REF_SPMM)
                                                     or not os.path.exists(os.path.join(_HERE, "_ref", "libref_encoder_b.so"))):
        subprocess.run(["make", "-C", _HERE, "ref", f"REF_DIR={ref_dir}"], check=True, capture_output=True)


def _makefile_ref_dir():
    """Default of REF_DIR in the Makefile beside this file."""
    try:
        for line in open(os.path.join(_HERE, "Makefile")):
            if line.startswith("REF_DIR ?="):
                return line.split("=", 1)[1].strip()
    except OSError:
        pass
    return None


def _p(a, t):
    return a.ctypes.data_as(t)


_lib = None
_ref = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB)
        _lib.oracle_encode_bitmap_v3.restype = ctypes.c_int
        _lib.oracle_total_error.restype = ctypes.c_double
        _lib.oracle_total_error.argtypes = [_u16p, _u16p, ctypes.c_size_t]
        _lib.oracle_h2f.restype = ctypes.c_float
        _lib.oracle_h2f.argtypes = [ctypes.c_uint16]
        _lib.oracle_f2h.restype = ctypes.c_uint16
        _lib.oracle_f2h.argtypes = [ctypes.c_float]
    return _lib


def have_ref():
    return os.path.exists(_REF)


def ref():
    global _ref
    if _ref is None:
        _ref = ctypes.CDLL(_REF)
        _ref.ref_encode_bitmap_v3.restype = ctypes.c_int
        _ref.ref_free.argtypes = [ctypes.c_void_p]
    return _ref


def have_ref_style():
    return os.path.exists(_REF_SPMM)


_ref_spmm = None


def ref_style_spmm(stream, vals, gtile, mtile, bitmap, B, C, M, N, K, workspace, split_k, max_nnz):
    """The reference-style mma.sync / cp.async SpMM (oracle/ref_style_spmm.cu, built from the reference's device
    functions) on device pointers given as integers.  A GPU comparator and numerics pin for tests and bench.py.
    N in {8, 16, 32, 64, k*128}; for N = 8 the buffer behind B must be readable for 16 rows."""
    global _ref_spmm
    if _ref_spmm is None:
        _ref_spmm = ctypes.CDLL(_REF_SPMM)
        _ref_spmm.ref_style_spmm.restype = ctypes.c_int
        _ref_spmm.ref_style_spmm.argtypes = [ctypes.c_void_p] * 7 + [ctypes.c_int] * 3 + [ctypes.c_void_p, ctypes.c_int,
                                                                                      ctypes.c_int]
    rc = _ref_spmm.ref_style_spmm(stream, vals, gtile, mtile, bitmap, B, C, M, N, K, workspace, split_k, max_nnz)
    if rc != 0:
        raise RuntimeError(f"ref_style_spmm failed: cudaError {rc}")


def _as_u16(a):
    a = np.ascontiguousarray(a)
    if a.dtype == np.float16:
        a = a.view(np.uint16)
    assert a.dtype == np.uint16
    return a


class Encoded:
    """The five arrays of the bitmap-v3 format plus max_nnz, as numpy arrays."""

    def __init__(self, M, K, vals, tile_nnz, mtile, gtile, bitmap, max_nnz):
        self.M, self.K = M, K
        self.vals, self.tile_nnz, self.mtile, self.gtile, self.bitmap = vals, tile_nnz, mtile, gtile, bitmap
        self.max_nnz = int(max_nnz)
        self.G = (M // 64) * (K // 64)

    def same_as(self, o):
        return (self.max_nnz == o.max_nnz and np.array_equal(self.vals, o.vals)
                and np.array_equal(self.tile_nnz, o.tile_nnz) and np.array_equal(self.mtile, o.mtile)
                and np.array_equal(self.gtile, o.gtile) and np.array_equal(self.bitmap, o.bitmap))


def encode(A):
    """oracle.c restatement of the encoder.  A: [M,K] float16/uint16."""
    A = _as_u16(A)
    M, K = A.shape
    assert M % 64 == 0 and K % 64 == 0
    G = (M // 64) * (K // 64)
    vals = np.empty(M * K + 8 * G + 8, np.uint16)
    tile_nnz = np.empty(max(M * K // 64, 1), np.int32)
    mtile = np.empty(max(4 * G, 1), np.int32)
    gtile = np.empty(G + 1, np.int32)
    bitmap = np.empty(max(M * K // 64, 1), np.uint64)
    mx = ctypes.c_int(0)
    g = lib().oracle_encode_bitmap_v3(_p(A, _u16p), M, K, _p(vals, _u16p), _p(tile_nnz, _i32p), _p(mtile, _i32p),
                                      _p(gtile, _i32p), _p(bitmap, _u64p), ctypes.byref(mx))
    assert g == G
    n = int(gtile[G])
    return Encoded(M, K, vals[:n].copy(), tile_nnz[:M * K // 64], mtile[:4 * G], gtile, bitmap[:M * K // 64], mx.value)


_REF_B = os.path.join(_HERE, "_ref", "libref_encoder_b.so")
_ref_b = None


def have_ref_b():
    return os.path.exists(_REF_B)


def encode_b(A):
    """oracle.c restatement of the fork's encoder for a compressed second operand (InitSparseMatrixA_bitmap_v6_B)."""
    A = _as_u16(A)
    M, K = A.shape
    assert M % 64 == 0 and K % 64 == 0
    G = (M // 64) * (K // 64)
    vals = np.empty(M * K + 8 * G + 8, np.uint16)
    tile_nnz = np.empty(max(M * K // 64, 1), np.int32)
    mtile = np.empty(max(16 * G, 1), np.int32)
    gtile = np.empty(G + 1, np.int32)
    bitmap = np.empty(max(M * K // 64, 1), np.uint64)
    mx = ctypes.c_int(0)
    fn = lib().oracle_encode_bitmap_v6_b
    fn.restype = ctypes.c_int
    g = fn(_p(A, _u16p), M, K, _p(vals, _u16p), _p(tile_nnz, _i32p), _p(mtile, _i32p), _p(gtile, _i32p), _p(bitmap, _u64p),
           ctypes.byref(mx))
    assert g == G
    n = int(gtile[G])
    return Encoded(M, K, vals[:n].copy(), tile_nnz[:M * K // 64], mtile[:16 * G], gtile, bitmap[:M * K // 64], mx.value)


def decode_b(enc):
    """Dense [M,K] uint16 image of a matrix in the second-operand layout."""
    out = np.empty((enc.M, enc.K), np.uint16)
    fn = lib().oracle_decode_bitmap_v6_b
    fn.restype = None
    fn(_p(np.ascontiguousarray(enc.vals if enc.vals.size else np.zeros(1, np.uint16)), _u16p), _p(enc.gtile, _i32p),
       _p(enc.bitmap, _u64p), enc.M, enc.K, _p(out, _u16p))
    return out


def ref_encode_b(A):
    """The reference's own InitSparseMatrixA_bitmap_v6_B (compiled into oracle/_ref)."""
    global _ref_b
    A = _as_u16(A)
    M, K = A.shape
    G = (M // 64) * (K // 64)
    if _ref_b is None:
        _ref_b = ctypes.CDLL(_REF_B)
        _ref_b.ref_encode_bitmap_v6_b.restype = ctypes.c_int
        _ref_b.ref_b_free.argtypes = [ctypes.c_void_p]
    vals, tn, mt, gt, bm = _u16p(), _i32p(), _i32p(), _i32p(), _u64p()
    mx = ctypes.c_int(0)
    g = _ref_b.ref_encode_bitmap_v6_b(_p(A, _u16p), M, K, ctypes.byref(vals), ctypes.byref(tn), ctypes.byref(mt),
                                      ctypes.byref(gt), ctypes.byref(bm), ctypes.byref(mx))
    assert g == G
    gtile = np.ctypeslib.as_array(gt, (G + 1,)).copy()
    n = int(gtile[G])
    nt = M * K // 64
    out = Encoded(M, K, (np.ctypeslib.as_array(vals, (n,)).copy() if n else np.zeros(0, np.uint16)),
                  np.ctypeslib.as_array(tn, (max(nt, 1),))[:nt].copy(),
                  np.ctypeslib.as_array(mt, (max(16 * G, 1),))[:16 * G].copy(), gtile,
                  np.ctypeslib.as_array(bm, (max(nt, 1),))[:nt].copy(), mx.value)
    for p in (vals, tn, mt, gt, bm):
        _ref_b.ref_b_free(ctypes.cast(p, ctypes.c_void_p))
    return out


def ref_encode(A):
    """The reference's own InitSparseMatrixA_bitmap (compiled into oracle/_ref)."""
    A = _as_u16(A)
    M, K = A.shape
    G = (M // 64) * (K // 64)
    r = ref()
    vals, tn, mt, gt, bm = _u16p(), _i32p(), _i32p(), _i32p(), _u64p()
    mx = ctypes.c_int(0)
    g = r.ref_encode_bitmap_v3(_p(A, _u16p), M, K, ctypes.byref(vals), ctypes.byref(tn), ctypes.byref(mt),
                               ctypes.byref(gt), ctypes.byref(bm), ctypes.byref(mx))
    assert g == G
    gtile = np.ctypeslib.as_array(gt, (G + 1,)).copy()
    n = int(gtile[G])
    nt = M * K // 64
    out = Encoded(M, K,
                  (np.ctypeslib.as_array(vals, (n,)).copy() if n else np.zeros(0, np.uint16)),
                  np.ctypeslib.as_array(tn, (max(nt, 1),))[:nt].copy(),
                  np.ctypeslib.as_array(mt, (max(4 * G, 1),))[:4 * G].copy(),
                  gtile,
                  np.ctypeslib.as_array(bm, (max(nt, 1),))[:nt].copy(), mx.value)
    for p in (vals, tn, mt, gt, bm):
        r.ref_free(ctypes.cast(p, ctypes.c_void_p))
    return out


def ref_gen_bin_files(dense_path, M, K, prefix):
    """The reference's own Our_GenSparseMatrixBinFile (compiled into oracle/_ref) on `dense_path`; writes the six
    files `prefix`.{NZWeights,gtile,mtile,ltile,intile,OutputSizes}.bin.  The reference prints a summary line and
    calls exit(-1) on I/O errors, so only call it with files that exist."""
    r = ref()
    names = [prefix + sfx for sfx in (".NZWeights.bin", ".gtile.bin", ".mtile.bin", ".ltile.bin", ".intile.bin",
                                      ".OutputSizes.bin")]
    r.ref_gen_bin_files.restype = None
    r.ref_gen_bin_files.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.c_int] + [ctypes.c_char_p] * 6
    r.ref_gen_bin_files(dense_path.encode(), M, K, *[n.encode() for n in names])
    return names


def decode(enc):
    A = np.empty((enc.M, enc.K), np.uint16)
    vals = enc.vals if enc.vals.size else np.zeros(1, np.uint16)
    lib().oracle_decode_bitmap_v3(_p(vals, _u16p), _p(enc.mtile, _i32p), _p(enc.gtile, _i32p),
                                  _p(enc.bitmap, _u64p), enc.M, enc.K, _p(A, _u16p))
    return A


def gemm_f32(A, B):
    """A [M,K] fp16 row-major, B [N,K] fp16 (column-major KxN) -> C [N,M] float32."""
    A, B = _as_u16(A), _as_u16(B)
    M, K = A.shape
    N = B.shape[0]
    assert B.shape[1] == K
    C = np.empty((N, M), np.float32)
    lib().oracle_gemm_f32(_p(A, _u16p), _p(B, _u16p), _p(C, _f32p), M, N, K)
    return C


def spmm_f32(enc, B):
    """fp32 product straight from the compressed form (decode + GEMM) -> C [N,M] float32."""
    B = _as_u16(B)
    N = B.shape[0]
    C = np.empty((N, enc.M), np.float32)
    vals = enc.vals if enc.vals.size else np.zeros(1, np.uint16)
    lib().oracle_spmm_f32(_p(vals, _u16p), _p(enc.mtile, _i32p), _p(enc.gtile, _i32p), _p(enc.bitmap, _u64p),
                          _p(B, _u16p), _p(C, _f32p), enc.M, N, enc.K)
    return C


def spmm_splitk_f16(A, B, split_k):
    """The reference's split-K rounding chain on a dense copy of A -> C [N,M] uint16 (fp16 bits)."""
    A, B = _as_u16(A), _as_u16(B)
    M, K = A.shape
    N = B.shape[0]
    C = np.empty((N, M), np.uint16)
    lib().oracle_spmm_splitk_f16(_p(A, _u16p), _p(B, _u16p), _p(C, _u16p), M, N, K, int(split_k))
    return C


def splitk_reduce(partials, M, N, split_k):
    partials = _as_u16(partials)
    C = np.empty((N, M), np.uint16)
    lib().oracle_splitk_reduce(_p(partials, _u16p), _p(C, _u16p), M, N, int(split_k))
    return C


def total_error(a, b):
    a, b = _as_u16(a).ravel(), _as_u16(b).ravel()
    return lib().oracle_total_error(_p(a, _u16p), _p(b, _u16p), a.size)


def num_threads():
    return lib().oracle_num_threads()


def set_num_threads(n):
    """Threads for the OpenMP loops of the oracle from now on (see oracle_set_num_threads)."""
    lib().oracle_set_num_threads(int(n))
    return num_threads()
