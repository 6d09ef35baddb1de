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
                                  int* gtile, uint64_t* bitmap, int* max_nnz, void* scratch);
// Pass 3: packed values.
cudaError_t encode_pack(cudaStream_t s, const uint16_t* A, int M, int K, const int* gtile, const uint64_t* bitmap,
                        uint16_t* vals, size_t vals_capacity, int* status);

// ---- split-K reduction (reduction.cu) --------------------------------------
cudaError_t splitk_reduce(cudaStream_t s, uint16_t* C, const uint16_t* ws, int M, int N, int split_k);

// ---- SpMM (spmm_kernel.cu) --------------------------------------------------
struct SpmmArgs {
    const uint16_t* vals;
    const int* gtile;
    const int* mtile;
    const uint64_t* bitmap;
    const int* max_nnz;
    const uint16_t* B;
    uint16_t* out;  // C when split_k == 1, else the fp16 partial workspace
    int M, N, K, split_k;
};
cudaError_t spmm_launch(cudaStream_t s, const SpmmArgs& a);
int suggest_split_k(int M, int N, int K);
// Work schedule of the SpMM kernel: 1 = static (one work item per split-K range, no scratch), 2 = balanced
// (equal k-tile shares per SM, fp32 exchange through library-owned scratch) whenever possible, 0 = whichever
// the cost model expects to be faster for the shape.
int set_schedule(int mode);          // returns the previous mode, -1 for an invalid one
void push_static_schedule();         // calling thread only, nestable
void pop_static_schedule();
cudaError_t reset_schedule_scratch();  // clears the arrival counters of the current device

void set_error(const char* fmt, ...);

}  // namespace spb
