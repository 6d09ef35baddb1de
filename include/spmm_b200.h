/*
 * C ABI of the B200 (sm_100a) implementation of the bitmap-v3 sparse SpMM path.
 *
 * Every entry point is extern "C" with plain pointers and sizes.  Each one names
 * the reference interface it replaces (path inside the reference project:line).
 * The same shared library also exports the reference's own C++-mangled symbols
 * (declared in include/SpMM_API.cuh) so that code written against the reference
 * header links unchanged.
 *
 * Conventions
 *   - fp16 values travel as uint16_t bit patterns.
 *   - "stream" is a cudaStream_t passed as void*.
 *   - A is M x K row-major; B is K x N column-major (stored [N][K]); C is M x N
 *     column-major (stored [N][M]).  M and K must be multiples of 64.
 *   - Functions returning int return 0 (cudaSuccess) or a cudaError_t value,
 *     unless stated otherwise; spb_last_error() gives a message for the calling
 *     thread's last failure.
 *   - There is no CPU fallback: without a usable CUDA device every compute
 *     entry point fails.
 */
#ifndef SPMM_B200_H
#define SPMM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Library version (major*10000 + minor*100 + patch). */
int spb_version(void);

/* Message describing the calling thread's most recent failure ("" if none). */
const char* spb_last_error(void);

/* ------------------------------------------------------------------ encoder */

/*
 * Host-buffer encoder.  Replaces InitSparseMatrixA_bitmap
 * (csrc/SpMM_API.cuh:112-241) for the tile shape all of its callers pass
 * (8,16,64,8,64,64; csrc/SpMM_API.cuh:275).  A_h is a host pointer to M*K fp16
 * values; the work is done on the current CUDA device.  On success the five
 * output arrays are malloc()ed and owned by the caller (free() or
 * spb_free_host), exactly like the reference, and bit-identical to it:
 *   vals      gtile[G] halves (packed non-zeros, each 64x64 tile padded with
 *             +0.0 to a multiple of 8)
 *   tile_nnz  M*K/64 ints (non-zeros per 8x8 tile; the reference's "TileOffsets")
 *   mtile     4*G ints written; allocated M*K/64 ints like the reference (csrc/SpMM_API.cuh:137)
 *   gtile     G+1 ints
 *   bitmap    M*K/64 uint64
 *   max_nnz   largest padded 64x64-tile count (not rounded to 64)
 * Returns G = (M/64)*(K/64), or -1 when an allocation fails (reference
 * behaviour), or -(1000+cudaError) when a CUDA call fails.
 */
int spb_encode_host(const uint16_t* A_h, int M, int K, uint16_t** vals, int** tile_nnz, int** mtile, int** gtile,
                    uint64_t** bitmap, int* max_nnz);

void spb_free_host(void* p);

/*
 * Device-buffer encoder (no reference counterpart: the reference encodes on the
 * CPU only; csrc/SpMM_API.cuh:112).  All pointers are device pointers.
 * Asynchronous on `stream`.  vals_capacity is the room at vals_d in halves;
 * M*K + 8*G always suffices.  After completion gtile_d[G] holds the number of
 * halves written and *max_nnz_d the largest padded tile count.  If the values
 * do not fit, nothing is written past the capacity and *status_d (optional,
 * may be NULL) is set to 1.  scratch_d needs spb_encode_scratch_bytes(M,K).
 */
size_t spb_encode_scratch_bytes(int M, int K);
int spb_encode_device(void* stream, const uint16_t* A_d, int M, int K, uint16_t* vals_d, size_t vals_capacity,
                      int* tile_nnz_d, int* mtile_d, int* gtile_d, uint64_t* bitmap_d, int* max_nnz_d,
                      void* scratch_d, int* status_d);

/*
 * File-level encoder, same name, arguments, output files and failure
 * behaviour (message + exit(-1)) as the reference's
 * Our_GenSparseMatrixBinFile (csrc/SpMM_API.cuh:243-320): reads M*K halves,
 * encodes, rounds max_nnz up to a multiple of 64 and writes the six files.
 * spb_gen_bin_files is the same but returns non-zero instead of exiting.
 */
void Our_GenSparseMatrixBinFile(char* DenseMatrixFileName, int M, int K, char* Compressed_ValFileName,
                                char* bitmap_TileOffsets_globalFileName, char* bitmap_TileOffsets_medianFileName,
                                char* bitmapFileName, char* max_nnz_intileFileName, char* OutputSizesFileName);
int spb_gen_bin_files(const char* dense, int M, int K, const char* val, const char* gtile, const char* mtile,
                      const char* bitmap, const char* max_nnz, const char* sizes);

/*
 * Loader of the six files Our_GenSparseMatrixBinFile writes (csrc/SpMM_API.cuh:288-319), the counterpart of
 * what FasterTransformer's patched weight loader does with them (third_party/ft_spinfer.patch:2336-2357:
 * loadDataArrayFromBin of .NZWeights, .gtile, .mtile, .ltile and .intile into device buffers whose sizes come
 * from the per-rank list files).  Pure host code.  `sizes` is the .OutputSizes file; it is checked against M and K
 * ([val_count, G+1, 4G, 64G]).  On success the four arrays are malloc()ed and owned by the caller (free() or
 * spb_free_host): vals val_count halves, gtile G+1 ints, mtile 4G ints, bitmap 64G uint64; *max_nnz_out is the
 * content of the .intile file (the largest padded tile count, rounded up to a multiple of 64 by the writer).
 * Returns 0, or cudaErrorInvalidValue when a file is missing, short or inconsistent (message in spb_last_error).
 */
int spb_load_bin_files(const char* val, const char* gtile, const char* mtile, const char* bitmap, const char* max_nnz,
                       const char* sizes, int M, int K, uint16_t** vals_out, int** mtile_out, int** gtile_out,
                       uint64_t** bitmap_out, int* max_nnz_out, int* val_count_out);

/*
 * The fork's extension: a bitmap-compressed SECOND operand (reference csrc/spmm_test_utils.h:523-652,
 * InitSparseMatrixA_bitmap_v6_B as called at csrc/spmm_test.cu:205, and the 19-argument
 * SpMM_SplitK_API_bitmap_v3 of csrc/SpMM_API.cuh:47-53).  The layout differs from the weight's: 64 x 64 global
 * tiles in row-major order, inside each the 16 x 16 median tiles column by column (16 median offsets per global
 * tile), inside those the four 8 x 8 tiles row-major; bitmaps, zero padding to 8 values per global tile and max_nnz
 * as for the weight.  spb_encode_b_host encodes a row-major [rows][cols] fp16 matrix on the GPU and returns host
 * arrays like spb_encode_host (mtile holds 16 * G ints).  spb_decode_operand_b expands such a matrix into dense fp16
 * [rows][cols] on the device.  spb_spmspm_bitmap_v3 is the SpMM with the activations given in that form: the
 * compressed B describes the stored [N_Global][K_Global] matrix (N_Global, K_Global multiples of 64); it is expanded
 * into memory taken from the stream's pool (cudaMallocAsync / cudaFreeAsync: asynchronous, legal under capture) and
 * the SpMM then runs as spb_spmm_bitmap_v3.  Corrupt offsets set the device status word and expand to zeros.
 */
int spb_encode_b_host(const uint16_t* B_h, int rows, int cols, uint16_t** vals, int** tile_nnz, int** mtile, int** gtile,
                      uint64_t** bitmap, int* max_nnz);
int spb_decode_operand_b(void* stream, const uint16_t* Compressed_B, const int* TileOffsets_B, const uint64_t* bitmap_B,
                         int rows, int cols, uint16_t* dense_out);
int spb_spmspm_bitmap_v3(void* stream, const uint16_t* Compressed_A, const int* TileOffsets, const int* TileOffsets_Median,
                         const uint64_t* bitmap, const int* max_nnz_intile, const uint16_t* Compressed_B,
                         const int* TileOffsets_B, const uint64_t* bitmap_B, uint16_t* C, int M_Global, int N_Global,
                         int K_Global, uint16_t* Reduction_Workspace, int Split_K);

/* --------------------------------------------------------------------- SpMM */

/*
 * C = A_sparse * B.  Replaces SpMM_SplitK_API_bitmap_v3 (csrc/SpMM_API.cuh:47-110;
 * the 14-argument dense-B form that FasterTransformer's patched wrapper calls,
 * third_party/ft_spinfer.patch:3736-3749).  Argument order and meaning are the
 * reference's: A is ignored (may be NULL); Compressed_A, TileOffsets (global
 * tile offsets), TileOffsets_Median, bitmap, max_nnz_intile (device pointer to
 * one int), B, C and Reduction_Workspace are device pointers.  With Split_K > 1
 * the k-tiles are cut into Split_K ranges exactly as the reference does
 * (csrc/SpMM_Kernel.cuh:35-43), fp16 partials go to Reduction_Workspace
 * ([Split_K][N][M], at least Split_K*M*N halves) and are summed in fp32 in range
 * order (csrc/Reduction_Kernel.cuh:24-44).  Asynchronous on `stream`; never
 * allocates, frees or synchronises (like the reference's entry point); the first
 * call on a device raises the kernels' shared-memory limit (cudaFuncSetAttribute),
 * which spb_init also does.
 * N may be any positive value (the reference accepts only 8,16,32,64 and
 * multiples of 128; csrc/SpMM_API.cuh:60-96): activation tiles of 16, 32, 64, 128 or 256
 * columns, wider N is cut into tiles of 256 columns.  Returns a cudaError_t value;
 * invalid shapes give cudaErrorInvalidValue and launch nothing.
 */
int spb_spmm_bitmap_v3(void* stream, const uint16_t* A, const uint16_t* Compressed_A, const int* TileOffsets,
                       const int* TileOffsets_Median, const uint64_t* bitmap, const int* max_nnz_intile,
                       const uint16_t* B, uint16_t* C, int M_Global, int N_Global, int K_Global,
                       uint16_t* Reduction_Workspace, int Split_K);

/*
 * The same SpMM for callers that can neither pass a reduction workspace nor let the library allocate
 * one (no counterpart in the reference, whose callers always bring their own workspace).  Typical
 * callers: a serving process that fixes its device-memory plan at start-up and bans allocation while
 * requests run, a plug-in that is only given the framework's input and output tensors, code executing
 * during stream capture.  The fp16 split-K partials go to an array of
 * SPB_NOALLOC_MAX_SCRATCH_BYTES that is part of the library's device image (each GPU that loads the
 * library holds it until the process ends).  The call performs no cudaMalloc/cudaFree and uses no
 * allocating library routine.
 *   - Split_K*M*N*2 bytes must fit the array; larger requests fail with cudaErrorInvalidValue and
 *     launch nothing.  Split_K == 1 needs no scratch and has no size limit.
 *   - The first call on a device looks up the array's device address (cudaGetSymbolAddress) and
 *     raises the shared-memory limit of the kernels of every activation width at once; make that
 *     first call (or a call of spb_init) outside any stream capture.
 *   - All calls share the one array and it keeps whatever the previous call left; the kernels
 *     overwrite every partial they later read, so no clearing is needed, but two calls whose
 *     kernels overlap on the GPU (different streams) race on it: serialise them.
 * Arguments as spb_spmm_bitmap_v3 without A and Reduction_Workspace.
 */
#define SPB_NOALLOC_MAX_SCRATCH_BYTES (16u << 20)
int spb_spmm_bitmap_v3_noalloc(void* stream, const uint16_t* Compressed_A, const int* TileOffsets,
                               const int* TileOffsets_Median, const uint64_t* bitmap, const int* max_nnz_intile,
                               const uint16_t* B, uint16_t* C, int M_Global, int N_Global, int K_Global, int Split_K);

/*
 * One-time preparation of (current device, stream), no counterpart in the reference: raises the kernels'
 * shared-memory limit and creates the library-owned scratch (39 MB of fp32 partial sums and 4 MB of arrival
 * counters) that the balanced work schedule, the split-K reduction fused into the SpMM kernel and the fused
 * all-gather / all-reduce use on that stream.  Allocates device memory and
 * synchronises the device, so call it once per stream at start-up, outside stream capture (up to 16 streams per
 * device at a time, see spb_release).  Without it every SpMM entry point still works, under the static schedule with a separate reduction
 * launch, and still allocates nothing; spb_spmm_bitmap_v3_allgather and spb_spmm_bitmap_v3_allreduce need it.
 */
int spb_init(void* stream);

/*
 * Gives back what spb_init created for (current device, stream): waits for the stream's work, then frees the scratch.
 * For hosts that create and destroy streams over their lifetime (a device serves up to 16 initialised streams at a
 * time; spb_init fails with cudaErrorMemoryAllocation beyond that, and SpMM calls on a stream without scratch use the
 * static schedule).  Not during stream capture.  Returns 0 also when the stream had no scratch.
 */
int spb_release(void* stream);

/*
 * Launch overlap of consecutive SpMM calls on one stream (no counterpart in the reference).  The SpMM kernel is
 * launched with programmatic stream serialization; with the setting on (default) its weight-streaming warps start
 * fetching Compressed_A, the offsets, the bitmaps and max_nnz_intile as soon as its thread blocks are resident,
 * while the slowest thread blocks of the stream's preceding kernel are still running; activations, outputs,
 * workspaces and all scratch are only touched after that kernel has completed.  This is safe whenever the weight
 * arrays are not written by a kernel that can still be running when the SpMM's thread blocks start, which holds
 * for everything that does not itself release its dependents early (this library's SpMM kernels do, and never
 * write weights).  Turn it off (0) if a kernel that releases its dependents early (griddepcontrol.launch_dependents /
 * cudaTriggerProgrammaticLaunchCompletion) writes weight arrays right before an SpMM on the same stream.
 * Returns the previous setting.  Process-wide.
 */
int spb_set_weight_prefetch(int on);

/*
 * Split-K reduction alone.  Replaces the SplitK_Reduction launch
 * (csrc/SpMM_API.cuh:106-108, csrc/Reduction_Kernel.cuh:24-44).
 */
int spb_splitk_reduce(void* stream, uint16_t* C, const uint16_t* Reduction_Workspace, int M_Global, int N_Global,
                      int Split_K);

/*
 * Split_K this library would pick for a shape on the current device (the
 * reference keeps a per-M table in its converter,
 * end2end_inference/ft_tools/huggingface_opt_convert_Phase2.py:23).
 */
int spb_suggest_split_k(int M, int N, int K);

/* Number of kernel launches this library has issued in this process so far (all entry points, all threads). */
unsigned long long spb_launch_count(void);

/*
 * Work schedule of spb_spmm_bitmap_v3 (no counterpart in the reference, whose grid is one CTA per
 * output tile and split-K range, csrc/SpMM_API.cuh:61-67).
 *   SPB_SCHEDULE_STATIC: one work item per 128-row block and split-K range, no scratch.
 *   SPB_SCHEDULE_BALANCED: the k-tiles of all ranges are laid end to end and every SM takes an equal
 *     share; a range that is cut between SMs is summed in fp32 through scratch memory the library owns
 *     (39 MB per stream, created by spb_init), and rounded to fp16 once, where the reference
 *     rounds it.  The scratch belongs to the stream: a graph captured on a stream must not run at the
 *     same time as other calls made on that stream.  Calls on a stream spb_init was not called for, and
 *     spb_spmm_bitmap_v3_noalloc, use the static schedule.
 *   SPB_SCHEDULE_AUTO (default): per call, whichever of the two a cost model expects to be faster.
 * Both give the same result up to the order of the fp32 additions inside a range.
 * Returns the previous mode, or -1 for an invalid mode.  Process-wide.
 */
#define SPB_SCHEDULE_AUTO 0
#define SPB_SCHEDULE_STATIC 1
#define SPB_SCHEDULE_BALANCED 2
int spb_set_schedule(int mode);

/*
 * SpMM of one row shard fused with the all-gather of the output rows (no counterpart in the reference, which
 * is single-GPU; its caller runs an NCCL all-gather after the GEMM for the M-split of tensor parallelism).
 * C_peers[q] is rank q's output buffer [N_Global][M_full] (fp16, column-major M_full x N like C above) as
 * mapped into this process, q = 0..n_peers-1, this rank's own buffer included; the rows of this shard
 * (M_shard of them, starting at row_offset) are stored into all of them.  flag_peers[q] is rank q's flag
 * array of n_peers + 2 uint32, zero before the first use: when the launch has finished, entry `rank` of
 * every array receives this rank's launch count.  spb_wait_flags enqueues a kernel that waits (bounded; on
 * expiry the device status word is set) until the local array shows the next launch of every rank; work
 * enqueued behind it sees the gathered rows.  Every rank must make the same sequence of calls on a buffer,
 * and a buffer may be written again only after every rank has consumed it (use two buffers in turn).
 * B_flags, when not null, is the local flag array of the exchange that produced B (a buffer gathered by an
 * earlier call): instead of a spb_wait_flags kernel in between, this launch itself waits for that exchange,
 * only in the warp that loads the activation tiles and with the same bound, while the weights already stream
 * in; it counts as the one consumer of that exchange (do not also call spb_wait_flags for it).
 * With Split_K > 1 the fp16 partial sums go to Reduction_Workspace (Split_K*M_shard*N_Global halves) as in
 * spb_spmm_bitmap_v3 and the reduction kernel does the stores to the peers and the flags.
 * Peer memory is only ever written, never loaded from.  Needs spb_init on the calling stream.
 */
int spb_spmm_bitmap_v3_allgather(void* stream, const uint16_t* Compressed_A, const int* TileOffsets,
                                 const int* TileOffsets_Median, const uint64_t* bitmap, const int* max_nnz_intile,
                                 const uint16_t* B, uint16_t* const* C_peers, uint32_t* const* flag_peers, int n_peers,
                                 int rank, int M_shard, int N_Global, int K_Global, int M_full, int row_offset,
                                 uint32_t* B_flags, uint16_t* Reduction_Workspace, int Split_K);
int spb_wait_flags(void* stream, uint32_t* flags, int n_peers);

/*
 * K-split of tensor parallelism with a one-shot all-reduce over peer stores (no counterpart in the reference, whose
 * caller runs an NCCL all-reduce after the out-proj and FC2 GEMMs; per-rank shapes in
 * end2end_inference/ft_tools/huggingface_opt_convert_Phase2.py:284-285).  This rank holds the columns
 * [rank*K/n, (rank+1)*K/n) of the weight (K_shard of them, encoded as a matrix of its own) and the matching slice
 * of the activations B [N][K_shard].  part_peers[q] is rank q's buffer of n_peers partial results
 * [n_peers][N_Global][M_Global] (fp16) as mapped into this process; this rank's product goes to slot `rank` of all of
 * them, and entry `rank` of every flag array (n_peers + 2 uint32, zero before the first use) receives this rank's
 * launch count, exactly as in spb_spmm_bitmap_v3_allgather, whose rules on call sequence, buffer reuse, B_flags and
 * Split_K apply.  spb_allreduce_finish then waits (bounded; on expiry the device status word is set) for all ranks'
 * partials in this rank's own buffer and writes C = fp16(sum over ranks in rank order of float(partial)) with the
 * split-K reduction's arithmetic.  Peer memory is only ever written.  Needs spb_init on the calling stream.
 */
int spb_spmm_bitmap_v3_allreduce(void* stream, const uint16_t* Compressed_A, const int* TileOffsets,
                                 const int* TileOffsets_Median, const uint64_t* bitmap, const int* max_nnz_intile,
                                 const uint16_t* B, uint16_t* const* part_peers, uint32_t* const* flag_peers, int n_peers,
                                 int rank, int M_Global, int N_Global, int K_shard, uint32_t* B_flags,
                                 uint16_t* Reduction_Workspace, int Split_K);
int spb_allreduce_finish(void* stream, uint16_t* C, const uint16_t* parts_local, uint32_t* flags_local, int n_peers,
                         int M_Global, int N_Global);

/*
 * Linear layer: the SpMM with the element-wise kernels that FasterTransformer runs after each GEMM of the OPT
 * decoder folded into the place where the result is rounded to fp16 (the SpMM kernel's epilogue, its fused split-K
 * reduction, or the reduction launch): bias add after QKV and FC1, ReLU after FC1, bias and residual add after the
 * attention output projection and FC2 (third_party/ft_spinfer.patch:623-862 FFN, 1459-1573 and 1704-1811
 * attention).  With y = the SpMM result as spb_spmm_bitmap_v3 rounds it:
 *     y = fp16(y + bias[m])        bias: M_Global fp16 values, or NULL
 *     y = y <= 0 ? 0 : y           activation 1 (ReLU); 0 = none
 *     C = fp16(residual + y)       residual: fp16 [N_Global][M_Global] like C, or NULL (may be C itself)
 * every step rounded to fp16, so the result has the bits of spb_spmm_bitmap_v3 followed by separate element-wise
 * fp16 kernels.  All other arguments, checks and return values as spb_spmm_bitmap_v3; bias and residual must be
 * 16-byte aligned.  spb_linear_allreduce_finish is spb_allreduce_finish with the same tail applied to the sum over
 * the ranks (residual and bias are added once, after the reduction); both run as one kernel launch.
 */
int spb_linear_bitmap_v3(void* stream, const uint16_t* Compressed_A, const int* TileOffsets, const int* TileOffsets_Median,
                         const uint64_t* bitmap, const int* max_nnz_intile, const uint16_t* B, uint16_t* C, int M_Global,
                         int N_Global, int K_Global, const uint16_t* bias, const uint16_t* residual, int activation,
                         uint16_t* Reduction_Workspace, int Split_K);
int spb_linear_allreduce_finish(void* stream, uint16_t* C, const uint16_t* parts_local, uint32_t* flags_local, int n_peers,
                                int M_Global, int N_Global, const uint16_t* bias, const uint16_t* residual,
                                int activation);

/*
 * Status word of the current device: 0 when no kernel of this library has hit a
 * bounded wait that ran out or an inconsistent offset since the last reset.
 * Synchronises the device.  spb_reset_device_status clears it.
 */
int spb_device_status(int* status_out);
int spb_reset_device_status(void);

#ifdef __cplusplus
}
#endif
#endif /* SPMM_B200_H */
