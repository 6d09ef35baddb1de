"""Host-side mirror of the reference's SpMM library interface, over the C ABI.

Names and argument meaning follow the reference (csrc/SpMM_API.cuh):
  InitSparseMatrixA_bitmap      -> init_sparse_matrix_a_bitmap   (:112)
  SpMM_SplitK_API_bitmap_v3     -> spmm_splitk_api_bitmap_v3     (:47)
  Our_GenSparseMatrixBinFile    -> our_gen_sparse_matrix_bin_file (:243)
PyTorch is used only to hold device memory and streams.
"""
import ctypes
from dataclasses import dataclass

import numpy as np
import torch

from . import _lib


class SpmmError(RuntimeError):
    pass


def _check(code, what):
    if code != 0:
        raise SpmmError(f"{what} failed: cudaError {code}: {_lib.last_error()}")


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


def _stream_ptr(stream=None):
    s = stream if stream is not None else torch.cuda.current_stream()
    return ctypes.c_void_p(s.cuda_stream)


# --------------------------------------------------------------------------- encoder (host)

@dataclass
class HostEncoded:
    """Host arrays in the reference's bitmap-v3 format (what InitSparseMatrixA_bitmap returns)."""
    M: int
    K: int
    vals: np.ndarray       # uint16 [val_count]        Compressed_Val
    tile_nnz: np.ndarray   # int32  [M*K/64]           TileOffsets (per-8x8 counts)
    mtile: np.ndarray      # int32  [4*G]              TileOffsets_median
    gtile: np.ndarray      # int32  [G+1]              TileOffsets_global
    bitmap: np.ndarray     # uint64 [M*K/64]
    max_nnz: int

    @property
    def G(self):
        return (self.M // 64) * (self.K // 64)


def init_sparse_matrix_a_bitmap_v6_b(B_h):
    """Encode a host fp16 matrix [rows, cols] in the fork's second-operand layout (InitSparseMatrixA_bitmap_v6_B,
    csrc/spmm_test_utils.h:523-652) on the GPU; HostEncoded.mtile then holds 16 offsets per global tile."""
    return init_sparse_matrix_a_bitmap(B_h, _second_operand=True)


def init_sparse_matrix_a_bitmap(A_h, _second_operand=False):
    """Encode a host fp16 matrix [M,K] on the GPU; returns HostEncoded (bit-identical to the reference)."""
    A_h = np.ascontiguousarray(A_h)
    if A_h.dtype == np.float16:
        A_h = A_h.view(np.uint16)
    if A_h.dtype != np.uint16 or A_h.ndim != 2:
        raise SpmmError("A must be a 2-D float16/uint16 array")
    M, K = A_h.shape
    lib = _lib.load()
    u16p, i32p, u64p = ctypes.POINTER(ctypes.c_uint16), ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_uint64)
    vals, tn, mt, gt, bm = u16p(), i32p(), i32p(), i32p(), u64p()
    mx = ctypes.c_int(0)
    fn = lib.spb_encode_b_host if _second_operand else lib.spb_encode_host
    g = fn(ctypes.c_void_p(A_h.ctypes.data), M, K, ctypes.byref(vals), ctypes.byref(tn),
           ctypes.byref(mt), ctypes.byref(gt), ctypes.byref(bm), ctypes.byref(mx))
    try:
        if g < 0:
            raise SpmmError(f"InitSparseMatrixA_bitmap failed ({g}): {_lib.last_error()}")
        nt = M * K // 64
        gtile = np.ctypeslib.as_array(gt, (g + 1,)).copy()
        n = int(gtile[g])
        out = HostEncoded(
            M, K,
            np.ctypeslib.as_array(vals, (n,)).copy() if n else np.zeros(0, np.uint16),
            np.ctypeslib.as_array(tn, (nt,)).copy(),
            np.ctypeslib.as_array(mt, ((16 if _second_operand else 4) * g,)).copy(),
            gtile,
            np.ctypeslib.as_array(bm, (nt,)).copy(),
            mx.value)
    finally:
        for p in (vals, tn, mt, gt, bm):
            lib.spb_free_host(ctypes.cast(p, ctypes.c_void_p))
    return out


def our_gen_sparse_matrix_bin_file(dense, M, K, val, gtile, mtile, bitmap, max_nnz, sizes):
    """Non-exiting form of Our_GenSparseMatrixBinFile: raises on failure."""
    enc = [s.encode() for s in (dense, val, gtile, mtile, bitmap, max_nnz, sizes)]
    rc = _lib.load().spb_gen_bin_files(enc[0], M, K, *enc[1:])
    if rc != 0:
        raise SpmmError(_lib.last_error())


# --------------------------------------------------------------------------- on-disk format

BIN_SUFFIXES = (".NZWeights.bin", ".gtile.bin", ".mtile.bin", ".ltile.bin", ".intile.bin", ".OutputSizes.bin")


def bin_file_names(prefix):
    """The six file names the reference's converter derives from a dense weight file `prefix`.bin
    (end2end_inference/ft_tools/huggingface_opt_convert_Phase2.py:70-76), in the argument order of
    Our_GenSparseMatrixBinFile: values, global offsets, median offsets, bitmaps, max_nnz, sizes."""
    return tuple(prefix + sfx for sfx in BIN_SUFFIXES)


def load_bin_files(prefix, M, K):
    """Read the six files of one weight matrix (spb_load_bin_files) into a HostEncoded.

    The per-8x8-tile counts are not part of the on-disk format (csrc/SpMM_API.cuh:288-319 writes five arrays
    and the sizes); tile_nnz is rebuilt from the bitmaps."""
    names = [n.encode() for n in bin_file_names(prefix)]
    lib = _lib.load()
    u16p, i32p, u64p = ctypes.POINTER(ctypes.c_uint16), ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_uint64)
    vals, mt, gt, bm = u16p(), i32p(), i32p(), u64p()
    mx, n = ctypes.c_int(0), ctypes.c_int(0)
    rc = lib.spb_load_bin_files(*names, M, K, ctypes.byref(vals), ctypes.byref(mt), ctypes.byref(gt), ctypes.byref(bm),
                                ctypes.byref(mx), ctypes.byref(n))
    if rc != 0:
        raise SpmmError(f"load_bin_files({prefix}) failed: {_lib.last_error()}")
    try:
        G = (M // 64) * (K // 64)
        bitmap = np.ctypeslib.as_array(bm, (64 * G,)).copy()
        bits = np.unpackbits(bitmap.view(np.uint8)).reshape(-1, 64).sum(axis=1).astype(np.int32)
        out = HostEncoded(M, K,
                          np.ctypeslib.as_array(vals, (n.value,)).copy() if n.value else np.zeros(0, np.uint16),
                          bits, np.ctypeslib.as_array(mt, (4 * G,)).copy(),
                          np.ctypeslib.as_array(gt, (G + 1,)).copy(), bitmap, mx.value)
    finally:
        for p in (vals, mt, gt, bm):
            lib.spb_free_host(ctypes.cast(p, ctypes.c_void_p))
    return out


RANK_LISTS = ("val_count_List", "num_gtiles_List", "num_mtiles_List", "num_ltiles_List", "SplitK_List")


def write_rank_lists(directory, rank, prefixes, split_ks):
    """The five per-rank list files FasterTransformer's loader reads before it allocates the weight buffers
    (third_party/ft_spinfer.patch:3133-3147): one int32 per weight matrix, in `prefixes` order, taken from each
    matrix's .OutputSizes file as the reference's converter does (huggingface_opt_convert_Phase2.py:329-360);
    a matrix that was left dense (no .OutputSizes file) gets zeros and Split_K 0."""
    import os
    rows = []
    for prefix, sk in zip(prefixes, split_ks):
        f = prefix + ".OutputSizes.bin"
        if os.path.exists(f):
            sz = np.fromfile(f, dtype=np.int32)
            if sz.shape[0] != 4:
                raise SpmmError(f"{f} must hold four int32")
            rows.append([int(sz[0]), int(sz[1]), int(sz[2]), int(sz[3]), int(sk)])
        else:
            rows.append([0, 0, 0, 0, 0])
    arr = np.asarray(rows, dtype=np.int32).reshape(-1, 5)
    for col, name in enumerate(RANK_LISTS):
        arr[:, col].copy().tofile(os.path.join(directory, f"{name}.{rank}.bin"))


def read_rank_lists(directory, rank):
    """Inverse of write_rank_lists: dict name -> int32 array (one entry per weight matrix)."""
    import os
    return {name: np.fromfile(os.path.join(directory, f"{name}.{rank}.bin"), dtype=np.int32) for name in RANK_LISTS}


# --------------------------------------------------------------------------- encoder (device)

@dataclass
class BitmapMatrix:
    """A weight matrix resident on the GPU in bitmap-v3 form."""
    M: int
    K: int
    vals: torch.Tensor      # float16 [>= val_count]
    gtile: torch.Tensor     # int32 [G+1]
    mtile: torch.Tensor     # int32 [4G]
    bitmap: torch.Tensor    # int64 view of uint64 [M*K/64]
    max_nnz: torch.Tensor   # int32 [1] (device; the kernel dereferences it)
    tile_nnz: torch.Tensor = None
    val_count: int = -1

    @property
    def G(self):
        return (self.M // 64) * (self.K // 64)

    def algorithmic_bytes(self, N):
        """Bytes one SpMM must move: packed values, bitmaps, offsets, activations, output."""
        G = self.G
        return 2 * self.val_count + 8 * (self.M * self.K // 64) + 4 * (G + 1) + 16 * G + 2 * self.K * N + 2 * self.M * N

    def shard_rows(self, rank, world):
        """Rows [rank*M/world, (rank+1)*M/world) as a BitmapMatrix that shares storage where it can.

        Global tiles are ordered row-block-major, so a row shard is a contiguous slice of
        every array; only the global offsets need re-basing.
        """
        if self.M % (64 * world):
            raise SpmmError("M/world must be a multiple of 64")
        Ms = self.M // world
        gk = self.K // 64
        g0, g1 = rank * (Ms // 64) * gk, (rank + 1) * (Ms // 64) * gk
        gt_h = self.gtile[[g0, g1]].cpu()
        o0, o1 = int(gt_h[0]), int(gt_h[1])
        gtile = (self.gtile[g0:g1 + 1] - o0).contiguous()
        sizes = gtile[1:] - gtile[:-1]
        mx = sizes.max().to(torch.int32).reshape(1) if sizes.numel() else torch.zeros(1, dtype=torch.int32, device=self.vals.device)
        return BitmapMatrix(Ms, self.K, self.vals[o0:o1], gtile, self.mtile[4 * g0:4 * g1],
                            self.bitmap[64 * g0:64 * g1], mx,
                            self.tile_nnz[64 * g0:64 * g1] if self.tile_nnz is not None else None, o1 - o0)


def encode_device(A, stream=None):
    """Encode a CUDA fp16 tensor [M,K] on the GPU (spb_encode_device)."""
    if not (A.is_cuda and A.dtype == torch.float16 and A.dim() == 2 and A.is_contiguous()):
        raise SpmmError("A must be a contiguous CUDA float16 matrix")
    M, K = A.shape
    if M % 64 or K % 64:
        raise SpmmError("M and K must be multiples of 64")
    lib = _lib.load()
    dev = A.device
    G = (M // 64) * (K // 64)
    nt = M * K // 64
    tile_nnz = torch.empty(nt, dtype=torch.int32, device=dev)
    mtile = torch.empty(4 * G, dtype=torch.int32, device=dev)
    gtile = torch.empty(G + 1, dtype=torch.int32, device=dev)
    bitmap = torch.empty(nt, dtype=torch.int64, device=dev)
    max_nnz = torch.zeros(1, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    scratch = torch.empty(lib.spb_encode_scratch_bytes(M, K), dtype=torch.uint8, device=dev)
    cap = M * K + 8 * G
    vals = torch.empty(cap, dtype=torch.float16, device=dev)
    with torch.cuda.device(dev):
        _check(lib.spb_encode_device(_stream_ptr(stream), _ptr(A), M, K, _ptr(vals), cap, _ptr(tile_nnz), _ptr(mtile),
                                     _ptr(gtile), _ptr(bitmap), _ptr(max_nnz), _ptr(scratch), _ptr(status)),
               "spb_encode_device")
    n = int(gtile[G].item())
    if int(status.item()) != 0:
        raise SpmmError("encoder overflowed its value buffer")
    # release the worst-case buffer (an all-zero matrix keeps 16 bytes so the pointer is never null)
    vals = vals[:n].clone() if n else torch.zeros(8, dtype=torch.float16, device=dev)
    return BitmapMatrix(M, K, vals, gtile, mtile, bitmap, max_nnz, tile_nnz, n)


def to_device(enc: HostEncoded, device="cuda"):
    """Upload reference-format host arrays (what the FT loader does with the .bin files)."""
    dev = torch.device(device)
    mx = enc.max_nnz
    return BitmapMatrix(
        enc.M, enc.K,
        torch.from_numpy(enc.vals.view(np.float16).copy()).to(dev) if enc.vals.size else torch.zeros(8, dtype=torch.float16, device=dev),
        torch.from_numpy(enc.gtile.copy()).to(dev),
        torch.from_numpy(enc.mtile.copy()).to(dev),
        torch.from_numpy(enc.bitmap.view(np.int64).copy()).to(dev),
        torch.tensor([mx], dtype=torch.int32, device=dev),
        torch.from_numpy(enc.tile_nnz.copy()).to(dev),
        int(enc.vals.size))


# --------------------------------------------------------------------------- SpMM

def spmm_splitk_api_bitmap_v3(stream, A, Compressed_A, TileOffsets, TileOffsets_Median, bitmap, max_nnz_intile, B, C,
                              M_Global, N_Global, K_Global, Reduction_Workspace, Split_K):
    """Same argument list as the reference's SpMM_SplitK_API_bitmap_v3 (csrc/SpMM_API.cuh:47); tensors for pointers.

    A is ignored (FasterTransformer passes nullptr).  Raises SpmmError with the CUDA error code on failure.
    """
    lib = _lib.load()
    code = lib.spb_spmm_bitmap_v3(_stream_ptr(stream), _ptr(A), _ptr(Compressed_A), _ptr(TileOffsets),
                                  _ptr(TileOffsets_Median), _ptr(bitmap), _ptr(max_nnz_intile), _ptr(B), _ptr(C),
                                  M_Global, N_Global, K_Global, _ptr(Reduction_Workspace), Split_K)
    _check(code, "SpMM_SplitK_API_bitmap_v3")


_initialised = set()


def init(stream=None):
    """spb_init for the current device and `stream` (default: torch's current stream): creates the scratch of the
    balanced schedule and of the fused all-gather.  Allocates and synchronises; not during stream capture."""
    s = stream if stream is not None else torch.cuda.current_stream()
    key = (torch.cuda.current_device(), s.cuda_stream)
    if key not in _initialised:
        _check(_lib.load().spb_init(ctypes.c_void_p(s.cuda_stream)), "spb_init")
        _initialised.add(key)


def release(stream=None):
    """spb_release: give back the scratch `init` created for the current device and `stream` (waits for the stream)."""
    s = stream if stream is not None else torch.cuda.current_stream()
    _check(_lib.load().spb_release(ctypes.c_void_p(s.cuda_stream)), "spb_release")
    _initialised.discard((torch.cuda.current_device(), s.cuda_stream))
    _no_scratch.discard((torch.cuda.current_device(), s.cuda_stream))


_no_scratch = set()


def _init_if_possible(stream):
    """The Python wrappers prepare a stream the first time they see it, unless it is being captured (the C entry
    points never do: they fall back to the static schedule on a stream spb_init was not called for).  When the
    device's scratch sets are all taken the stream simply stays without one: the calls then run the static schedule."""
    s = stream if stream is not None else torch.cuda.current_stream()
    key = (torch.cuda.current_device(), s.cuda_stream)
    if key in _initialised or key in _no_scratch or torch.cuda.is_current_stream_capturing():
        return
    try:
        init(s)
    except SpmmError:
        _no_scratch.add(key)


def suggest_split_k(M, N, K):
    return _lib.load().spb_suggest_split_k(M, N, K)


SCHEDULE_AUTO, SCHEDULE_STATIC, SCHEDULE_BALANCED = 0, 1, 2


def set_schedule(mode):
    """spb_set_schedule: SCHEDULE_AUTO (default), SCHEDULE_STATIC or SCHEDULE_BALANCED; returns the previous mode."""
    prev = _lib.load().spb_set_schedule(int(mode))
    if prev < 0:
        raise SpmmError("set_schedule: mode must be SCHEDULE_AUTO, SCHEDULE_STATIC or SCHEDULE_BALANCED")
    return prev


def spmm(W: BitmapMatrix, B, split_k=None, out=None, workspace=None, stream=None):
    """C[N,M] = (W @ B^T)^T with B given as [N,K] (the reference's column-major K x N)."""
    if not (B.is_cuda and B.dtype == torch.float16 and B.dim() == 2 and B.is_contiguous() and B.shape[1] == W.K):
        raise SpmmError("B must be a contiguous CUDA float16 [N,K] tensor")
    N = B.shape[0]
    if split_k is None:
        split_k = suggest_split_k(W.M, N, W.K)
    if out is None:
        out = torch.empty((N, W.M), dtype=torch.float16, device=B.device)
    if split_k > 1 and workspace is None:
        workspace = torch.empty(split_k * N * W.M, dtype=torch.float16, device=B.device)
    with torch.cuda.device(B.device):
        _init_if_possible(stream)
        spmm_splitk_api_bitmap_v3(stream, None, W.vals, W.gtile, W.mtile, W.bitmap, W.max_nnz, B, out, W.M, N, W.K,
                                  workspace, split_k)
    return out


ACT_NONE, ACT_RELU = 0, 1


def _check_tail(M, N, bias, residual, activation, device):
    if activation not in (ACT_NONE, ACT_RELU):
        raise SpmmError("activation must be ACT_NONE or ACT_RELU")
    if bias is not None and not (bias.is_cuda and bias.device == device and bias.dtype == torch.float16
                                 and bias.is_contiguous() and tuple(bias.shape) == (M,)):
        raise SpmmError("bias must be a contiguous CUDA float16 [M] tensor")
    if residual is not None and not (residual.is_cuda and residual.device == device and residual.dtype == torch.float16
                                     and residual.is_contiguous() and tuple(residual.shape) == (N, M)):
        raise SpmmError("residual must be a contiguous CUDA float16 [N,M] tensor")


def linear(W: BitmapMatrix, B, bias=None, residual=None, activation=ACT_NONE, split_k=None, out=None, workspace=None,
           stream=None):
    """spb_linear_bitmap_v3: out[N,M] = residual + act(spmm(W, B) + bias), every step rounded to fp16 (the bits of
    spmm followed by the separate element-wise fp16 operations), in the launches of the SpMM itself."""
    if not (B.is_cuda and B.dtype == torch.float16 and B.dim() == 2 and B.is_contiguous() and B.shape[1] == W.K):
        raise SpmmError("B must be a contiguous CUDA float16 [N,K] tensor")
    N = B.shape[0]
    _check_tail(W.M, N, bias, residual, activation, B.device)
    if split_k is None:
        split_k = suggest_split_k(W.M, N, W.K)
    if out is None:
        out = torch.empty((N, W.M), dtype=torch.float16, device=B.device)
    elif not (out.is_cuda and out.dtype == torch.float16 and out.is_contiguous() and tuple(out.shape) == (N, W.M)):
        raise SpmmError("out must be a contiguous CUDA float16 [N,M] tensor")
    if split_k > 1 and workspace is None:
        workspace = torch.empty(split_k * N * W.M, dtype=torch.float16, device=B.device)
    if split_k > 1 and workspace.numel() < split_k * N * W.M:
        raise SpmmError("workspace too small for split_k * N * M halves")
    with torch.cuda.device(B.device):
        _init_if_possible(stream)
        code = _lib.load().spb_linear_bitmap_v3(_stream_ptr(stream), _ptr(W.vals), _ptr(W.gtile), _ptr(W.mtile),
                                                _ptr(W.bitmap), _ptr(W.max_nnz), _ptr(B), _ptr(out), W.M, N, W.K,
                                                _ptr(bias) if bias is not None else None,
                                                _ptr(residual) if residual is not None else None, int(activation),
                                                _ptr(workspace) if workspace is not None else None, split_k)
    _check(code, "spb_linear_bitmap_v3")
    return out


def decode_operand_b(Bc: BitmapMatrix, out=None, stream=None):
    """spb_decode_operand_b: a matrix in the second-operand layout (to_device of init_sparse_matrix_a_bitmap_v6_b)
    expanded to dense fp16 [rows, cols]."""
    if out is None:
        out = torch.empty((Bc.M, Bc.K), dtype=torch.float16, device=Bc.vals.device)
    with torch.cuda.device(out.device):
        code = _lib.load().spb_decode_operand_b(_stream_ptr(stream), _ptr(Bc.vals), _ptr(Bc.gtile), _ptr(Bc.bitmap), Bc.M, Bc.K,
                                                _ptr(out))
    _check(code, "spb_decode_operand_b")
    return out


def spmspm(W: BitmapMatrix, Bc: BitmapMatrix, split_k=None, out=None, workspace=None, stream=None):
    """spb_spmspm_bitmap_v3: C[N,M] with both operands bitmap-compressed; Bc encodes the stored [N,K] activations in
    the second-operand layout."""
    if Bc.K != W.K:
        raise SpmmError("the compressed second operand must be [N,K]")
    N = Bc.M
    if split_k is None:
        split_k = suggest_split_k(W.M, N, W.K)
    if out is None:
        out = torch.empty((N, W.M), dtype=torch.float16, device=W.vals.device)
    if split_k > 1 and workspace is None:
        workspace = torch.empty(split_k * N * W.M, dtype=torch.float16, device=W.vals.device)
    with torch.cuda.device(W.vals.device):
        _init_if_possible(stream)
        code = _lib.load().spb_spmspm_bitmap_v3(_stream_ptr(stream), _ptr(W.vals), _ptr(W.gtile), _ptr(W.mtile), _ptr(W.bitmap),
                                                _ptr(W.max_nnz), _ptr(Bc.vals), _ptr(Bc.gtile), _ptr(Bc.bitmap), _ptr(out),
                                                W.M, N, W.K, _ptr(workspace) if workspace is not None else None, split_k)
    _check(code, "spb_spmspm_bitmap_v3")
    return out


def spmm_noalloc(W: BitmapMatrix, B, split_k, out, stream=None):
    """spb_spmm_bitmap_v3_noalloc: split-K SpMM whose partial sums use the library's built-in scratch array.

    For callers that must not allocate device memory: `out` has to be supplied, nothing is allocated here or in
    the library.  Raises SpmmError when split_k * M * N * 2 bytes exceed the built-in array.
    """
    if not (B.is_cuda and B.dtype == torch.float16 and B.dim() == 2 and B.is_contiguous() and B.shape[1] == W.K):
        raise SpmmError("B must be a contiguous CUDA float16 [N,K] tensor")
    N = B.shape[0]
    if not (out.is_cuda and out.dtype == torch.float16 and out.is_contiguous() and tuple(out.shape) == (N, W.M)):
        raise SpmmError("out must be a contiguous CUDA float16 [N,M] tensor")
    with torch.cuda.device(B.device):
        code = _lib.load().spb_spmm_bitmap_v3_noalloc(_stream_ptr(stream), _ptr(W.vals), _ptr(W.gtile), _ptr(W.mtile),
                                                      _ptr(W.bitmap), _ptr(W.max_nnz), _ptr(B), _ptr(out), W.M, N, W.K,
                                                      split_k)
    _check(code, "spb_spmm_bitmap_v3_noalloc")
    return out


def spmm_allgather(W: BitmapMatrix, B, C_peers, flag_peers, n_peers, rank, M_full, row_offset, B_flags=None,
                   split_k=1, workspace=None, stream=None):
    """spb_spmm_bitmap_v3_allgather: SpMM of a row shard whose output rows are stored into every rank's buffer.

    C_peers / flag_peers are ctypes arrays of n_peers device pointers (see spmspm_b200.dist.PeerGather); B_flags is
    the local flag tensor of the exchange that produced B, if B is a gathered buffer not yet waited for."""
    if not (B.is_cuda and B.dtype == torch.float16 and B.dim() == 2 and B.is_contiguous() and B.shape[1] == W.K):
        raise SpmmError("B must be a contiguous CUDA float16 [N,K] tensor")
    if split_k > 1 and workspace is None:
        workspace = torch.empty(split_k * B.shape[0] * W.M, dtype=torch.float16, device=B.device)
    with torch.cuda.device(B.device):
        _init_if_possible(stream)
        code = _lib.load().spb_spmm_bitmap_v3_allgather(_stream_ptr(stream), _ptr(W.vals), _ptr(W.gtile), _ptr(W.mtile),
                                                        _ptr(W.bitmap), _ptr(W.max_nnz), _ptr(B), C_peers, flag_peers,
                                                        n_peers, rank, W.M, B.shape[0], W.K, M_full, row_offset,
                                                        _ptr(B_flags), _ptr(workspace), split_k)
    _check(code, "spb_spmm_bitmap_v3_allgather")


def spmm_allreduce(W: BitmapMatrix, B, part_peers, flag_peers, n_peers, rank, B_flags=None, split_k=1, workspace=None,
                   stream=None):
    """spb_spmm_bitmap_v3_allreduce: SpMM of a column shard whose partial result goes to slot `rank` of every rank's
    buffer (see spmspm_b200.dist.PeerReduce)."""
    if not (B.is_cuda and B.dtype == torch.float16 and B.dim() == 2 and B.is_contiguous() and B.shape[1] == W.K):
        raise SpmmError("B must be a contiguous CUDA float16 [N,K_shard] tensor")
    if split_k > 1 and workspace is None:
        workspace = torch.empty(split_k * B.shape[0] * W.M, dtype=torch.float16, device=B.device)
    with torch.cuda.device(B.device):
        _init_if_possible(stream)
        code = _lib.load().spb_spmm_bitmap_v3_allreduce(_stream_ptr(stream), _ptr(W.vals), _ptr(W.gtile), _ptr(W.mtile),
                                                        _ptr(W.bitmap), _ptr(W.max_nnz), _ptr(B), part_peers, flag_peers,
                                                        n_peers, rank, W.M, B.shape[0], W.K, _ptr(B_flags),
                                                        _ptr(workspace), split_k)
    _check(code, "spb_spmm_bitmap_v3_allreduce")


def allreduce_finish(out, parts_local, flags_local, n_peers, stream=None, bias=None, residual=None, activation=ACT_NONE):
    """spb_linear_allreduce_finish: bounded wait for all ranks' partials, then their fp32 sum in rank order, rounded
    once, then the linear layer's tail (bias, activation, residual; see `linear`).  One launch."""
    N, M = out.shape
    _check_tail(M, N, bias, residual, activation, out.device)
    with torch.cuda.device(out.device):
        code = _lib.load().spb_linear_allreduce_finish(_stream_ptr(stream), _ptr(out), _ptr(parts_local), _ptr(flags_local),
                                                       n_peers, M, N, _ptr(bias) if bias is not None else None,
                                                       _ptr(residual) if residual is not None else None, int(activation))
    _check(code, "spb_linear_allreduce_finish")
    return out


def wait_flags(flags, n_peers, stream=None):
    """spb_wait_flags: bounded device-side wait until every rank's rows of the current exchange have arrived."""
    with torch.cuda.device(flags.device):
        code = _lib.load().spb_wait_flags(_stream_ptr(stream), _ptr(flags), n_peers)
    _check(code, "spb_wait_flags")


def splitk_reduce(C, workspace, M, N, split_k, stream=None):
    _check(_lib.load().spb_splitk_reduce(_stream_ptr(stream), _ptr(C), _ptr(workspace), M, N, split_k),
           "spb_splitk_reduce")


def launch_count():
    """spb_launch_count: kernel launches issued by the library in this process so far."""
    return int(_lib.load().spb_launch_count())


def device_status():
    st = ctypes.c_int(0)
    _check(_lib.load().spb_device_status(ctypes.byref(st)), "spb_device_status")
    return st.value


def reset_device_status():
    _check(_lib.load().spb_reset_device_status(), "spb_reset_device_status")
