"""Loader for libSpMM_API.so (the C ABI declared in include/spmm_b200.h).

The library is built in-tree by spmspm_b200.build.build(); there is no Python or
CPU fallback: if the shared object is missing, loading raises.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# SPMSPM_B200_LIB names another build of the same library (e.g. one compiled with other tuning constants).
LIB_PATH = os.environ.get("SPMSPM_B200_LIB") or os.path.join(_HERE, "libSpMM_API.so")

_u16p = ctypes.POINTER(ctypes.c_uint16)
_i32p = ctypes.POINTER(ctypes.c_int)
_u64p = ctypes.POINTER(ctypes.c_uint64)
_vp = ctypes.c_void_p

# name -> (restype, argtypes); every symbol include/spmm_b200.h declares
SIGNATURES = {
    "spb_version": (ctypes.c_int, []),
    "spb_last_error": (ctypes.c_char_p, []),
    "spb_encode_host": (ctypes.c_int, [_vp, ctypes.c_int, ctypes.c_int, ctypes.POINTER(_u16p), ctypes.POINTER(_i32p),
                                       ctypes.POINTER(_i32p), ctypes.POINTER(_i32p), ctypes.POINTER(_u64p), _i32p]),
    "spb_encode_b_host": (ctypes.c_int, [_vp, ctypes.c_int, ctypes.c_int, ctypes.POINTER(_u16p), ctypes.POINTER(_i32p),
                                         ctypes.POINTER(_i32p), ctypes.POINTER(_i32p), ctypes.POINTER(_u64p), _i32p]),
    "spb_decode_operand_b": (ctypes.c_int, [_vp, _vp, _vp, _vp, ctypes.c_int, ctypes.c_int, _vp]),
    "spb_spmspm_bitmap_v3": (ctypes.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, ctypes.c_int, ctypes.c_int,
                                            ctypes.c_int, _vp, ctypes.c_int]),
    "spb_free_host": (None, [_vp]),
    "spb_encode_scratch_bytes": (ctypes.c_size_t, [ctypes.c_int, ctypes.c_int]),
    "spb_encode_device": (ctypes.c_int, [_vp, _vp, ctypes.c_int, ctypes.c_int, _vp, ctypes.c_size_t, _vp, _vp, _vp,
                                         _vp, _vp, _vp, _vp]),
    "Our_GenSparseMatrixBinFile": (None, [ctypes.c_char_p, ctypes.c_int, ctypes.c_int] + [ctypes.c_char_p] * 6),
    "spb_gen_bin_files": (ctypes.c_int, [ctypes.c_char_p, ctypes.c_int, ctypes.c_int] + [ctypes.c_char_p] * 6),
    "spb_load_bin_files": (ctypes.c_int, [ctypes.c_char_p] * 6 + [ctypes.c_int, ctypes.c_int, ctypes.POINTER(_u16p),
                                          ctypes.POINTER(_i32p), ctypes.POINTER(_i32p), ctypes.POINTER(_u64p), _i32p, _i32p]),
    "spb_spmm_bitmap_v3": (ctypes.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, ctypes.c_int, ctypes.c_int,
                                          ctypes.c_int, _vp, ctypes.c_int]),
    "spb_spmm_bitmap_v3_noalloc": (ctypes.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, ctypes.c_int, ctypes.c_int,
                                                  ctypes.c_int, ctypes.c_int]),
    "spb_splitk_reduce": (ctypes.c_int, [_vp, _vp, _vp, ctypes.c_int, ctypes.c_int, ctypes.c_int]),
    "spb_suggest_split_k": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, ctypes.c_int]),
    "spb_set_schedule": (ctypes.c_int, [ctypes.c_int]),
    "spb_init": (ctypes.c_int, [_vp]),
    "spb_release": (ctypes.c_int, [_vp]),
    "spb_set_weight_prefetch": (ctypes.c_int, [ctypes.c_int]),
    "spb_spmm_bitmap_v3_allgather": (ctypes.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, ctypes.c_int, ctypes.c_int,
                                                    ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, _vp, _vp, ctypes.c_int]),
    "spb_wait_flags": (ctypes.c_int, [_vp, _vp, ctypes.c_int]),
    "spb_spmm_bitmap_v3_allreduce": (ctypes.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, ctypes.c_int, ctypes.c_int,
                                                    ctypes.c_int, ctypes.c_int, ctypes.c_int, _vp, _vp, ctypes.c_int]),
    "spb_allreduce_finish": (ctypes.c_int, [_vp, _vp, _vp, _vp, ctypes.c_int, ctypes.c_int, ctypes.c_int]),
    "spb_linear_bitmap_v3": (ctypes.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                            _vp, _vp, ctypes.c_int, _vp, ctypes.c_int]),
    "spb_linear_allreduce_finish": (ctypes.c_int, [_vp, _vp, _vp, _vp, ctypes.c_int, ctypes.c_int, ctypes.c_int, _vp, _vp,
                                                   ctypes.c_int]),
    "spb_launch_count": (ctypes.c_ulonglong, []),
    "spb_device_status": (ctypes.c_int, [_i32p]),
    "spb_reset_device_status": (ctypes.c_int, []),
}

# C++-mangled symbols of the reference header (include/SpMM_API.cuh)
MANGLED = [
    "_Z25SpMM_SplitK_API_bitmap_v3P11CUstream_stPK6__halfS3_PKiS5_PKmS5_S3_PS1_iiiS8_i",
    "_Z24InitSparseMatrixA_bitmapP6__halfiiiiiiiiPS0_PPiS3_S3_PPmRi",
    # the fork's forms with a compressed second operand (csrc/SpMM_API.cuh:47-53, csrc/spmm_test_utils.h:523)
    "_Z25SpMM_SplitK_API_bitmap_v3P11CUstream_stPK6__halfS3_PKiS5_PKmS5_S3_S3_S5_S5_S7_S5_PS1_iiiS8_i",
    "_Z29InitSparseMatrixA_bitmap_v6_BP6__halfiiiiiiiiPS0_PPiS3_S3_PPmRi",
]

NOALLOC_MAX_SCRATCH_BYTES = 16 << 20  # SPB_NOALLOC_MAX_SCRATCH_BYTES in include/spmm_b200.h

_lib = None


def load():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
                "(nvcc, sm_100a). There is no fallback path.")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def last_error():
    return load().spb_last_error().decode()
