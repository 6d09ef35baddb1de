// Internal declarations shared by the translation units of libSpMM_API.so.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stddef.h>

namespace spb {

// Error codes kept in the per-device status word (see spb_device_status).
enum DeviceStatus : int {
    kStatusOk = 0,
    kStatusWaitTimeout = 1,    // a bounded mbarrier wait ran out
    kStatusBadOffsets = 2,     // a global-tile chunk was larger than max_nnz_intile allows
    kStatusEncodeOverflow = 4, // encoder: packed values did not fit the caller's buffer
};

// Address of the calling device's status word (device memory, one int).
cudaError_t device_status_ptr(int** out);

// ---- encoder (encoder.cu) -------------------------------------------------
size_t encode_scratch_bytes(int M, int K);
// Pass 1+2: bitmaps, per-tile counts, median offsets, global offsets, max.
cudaError_t encode_count_and_scan(cudaStream_t s, const uint16_t* A, int M, int K, int* tile_nnz, int* mtile,
                                  int* gtile, uint64_t* bitmap, int* max_nnz, void* scratch, int fmt = 0);
// Pass 3: packed values.
cudaError_t encode_pack(cudaStream_t s, const uint16_t* A, int M, int K, const int* gtile, const uint64_t* bitmap,
                        uint16_t* vals, size_t vals_capacity, int* status, int fmt = 0);
// fmt: 0 = the weight layout (InitSparseMatrixA_bitmap), 1 = the fork's layout for a compressed second operand
// (InitSparseMatrixA_bitmap_v6_B: 16 median offsets per global tile, mtile holds 16 * G ints).
constexpr int kFmtWeight = 0, kFmtOperandB = 1;
// Expands a matrix [rows][cols] in the second-operand layout into dense fp16 (sparse_b.cu).
cudaError_t decode_operand_b(cudaStream_t s, const uint16_t* vals, const int* gtile, const uint64_t* bitmap, int rows,
                             int cols, uint16_t* dense, int* status);

// ---- split-K reduction (reduction.cu) --------------------------------------
// Element-wise tail of a linear layer (see epilogue.cuh): bias [M] fp16 or null, residual in the layout of the
// destination or null, activation 0 (none) or 1 (ReLU).
struct Epilogue {
    const uint16_t* bias = nullptr;
    const uint16_t* residual = nullptr;
    int activation = 0;
    bool any() const { return bias || residual || activation; }
};
// ep.residual is indexed like C; wait_flags/wait_n: first wait (bounded) until the n sequence numbers of an
// exchange have arrived (see exchange.cu), for partials that other GPUs write
cudaError_t splitk_reduce(cudaStream_t s, uint16_t* C, const uint16_t* ws, int M, int N, int split_k,
                          const Epilogue& ep = Epilogue(), uint32_t* wait_flags = nullptr, int wait_n = 0, int* status = nullptr);

// ---- SpMM (spmm_kernel.cu) --------------------------------------------------
struct SpmmArgs {
    const uint16_t* vals;
    const int* gtile;
    const int* mtile;
    const uint64_t* bitmap;
    const int* max_nnz;
    const uint16_t* B;
    uint16_t* out;  // C when split_k == 1, else the fp16 partial workspace
    // split_k > 1: where the reduced result belongs (C), so that the kernel may do the reduction itself; when it
    // does, *reduce_fused is set and the caller must not launch the reduction
    uint16_t* final_out = nullptr;
    bool* reduce_fused = nullptr;
    int M, N, K, split_k;
    // Fused all-gather (n_out > 0): the result rows go to rows row0.. of n_out buffers [N][ld_out] (this GPU's
    // and its peers'), then entry flag_index of n_flags flag arrays gets the launch's sequence number (the
    // incremented value of *sequence).  With split_k > 1 that happens only if the kernel fuses the reduction
    // (*reduce_fused); otherwise the caller's reduction launch has to store the rows and write the flags.
    uint16_t* outs[8] = {};
    uint32_t* flags[8] = {};
    int n_out = 0, ld_out = 0, row0 = 0, n_flags = 0, flag_index = 0;
    uint32_t* sequence = nullptr;
    // flag array (on this GPU) of the exchange that produced B, or null; wait_n ranks
    uint32_t* wait_flags = nullptr;
    int wait_n = 0;
    // applied by the kernel wherever it writes final rows; with split_k > 1 and no fused reduction the caller's
    // reduction launch has to apply it
    Epilogue ep;
};
cudaError_t wait_flags_launch(cudaStream_t s, uint32_t* flags, int n, int* status);
cudaError_t exchange_counter(cudaStream_t s, int** out);  // a zeroed int of the stream's scratch, for CTA counting
cudaError_t spmm_launch(cudaStream_t s, const SpmmArgs& a);
cudaError_t init_stream(cudaStream_t s);  // scratch of the balanced schedule / fused exchange for this stream
cudaError_t release_stream(cudaStream_t s);  // gives that scratch back (synchronises the stream)
int suggest_split_k(int M, int N, int K);
// Work schedule of the SpMM kernel: 1 = static (one work item per split-K range, no scratch), 2 = balanced
// (equal k-tile shares per SM, fp32 exchange through library-owned scratch) whenever possible, 0 = whichever
// the cost model expects to be faster for the shape.
int set_schedule(int mode);
int set_weight_prefetch(int on);     // returns the previous setting          // returns the previous mode, -1 for an invalid one
void push_static_schedule();         // calling thread only, nestable
void pop_static_schedule();
cudaError_t reset_schedule_scratch();  // clears the arrival counters of the current device

void set_error(const char* fmt, ...);
// Kernel launches this library has issued in this process (every launch site counts itself): lets a caller state
// how many kernels a piece of work takes, e.g. by reading the counter around the capture of a CUDA graph.
void count_launch(int n = 1);
bool aligned16(const void* p);
// Argument checks of the SpMM entry points (api.cu): cudaSuccess, or an error code with the message set.
cudaError_t check_spmm_args(const char* who, const void* vals, const void* gtile, const void* mtile, const void* bitmap,
                            const void* max_nnz, const void* B, int M, int N, int K, const void* ws, int split_k);

}  // namespace spb
