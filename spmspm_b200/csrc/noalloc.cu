// Split-K SpMM for callers that may not allocate device memory.
//
// Some hosts of this library cannot hand it a reduction workspace and cannot let it create one: an
// inference server that plans all of its device memory at start-up and forbids allocation on the
// request path, a plug-in that only ever sees the framework's input and output buffers, or any code
// that runs while a stream is being captured, where cudaMalloc is not allowed.  For them the fp16
// split-K partials live in a fixed array inside the library's device image instead of in a
// caller-provided workspace.
#include "../../include/spmm_b200.h"
#include "common.cuh"

namespace {

// Partial sums of one call: [Split_K][N][M] fp16.  Part of the module image: every GPU that loads the
// library keeps these bytes until the process exits.
static __device__ __align__(256) unsigned char g_splitk_scratch[SPB_NOALLOC_MAX_SCRATCH_BYTES];

// In host code the array's name is only a handle; the device address has to be asked for, once per
// device, with that device current.
cudaError_t scratch_address(uint16_t** out)
{
    static uint16_t* cache[64] = {nullptr};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!cache[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_splitk_scratch);
        if (e != cudaSuccess) {
            spb::set_error("spb_spmm_bitmap_v3_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            return e;
        }
        cache[dev] = static_cast<uint16_t*>(p);
    }
    *out = cache[dev];
    return cudaSuccess;
}

}  // namespace

extern "C" int spb_spmm_bitmap_v3_noalloc(void* stream, const uint16_t* Compressed_A, const int* TileOffsets,
                                          const int* TileOffsets_Median, const uint64_t* bitmap,
                                          const int* max_nnz_intile, const uint16_t* B, uint16_t* C, int M_Global,
                                          int N_Global, int K_Global, int Split_K)
{
    if (M_Global <= 0 || N_Global <= 0 || K_Global <= 0 || Split_K < 1) {
        spb::set_error("spb_spmm_bitmap_v3_noalloc: M, N, K and Split_K must be positive");
        return (int)cudaErrorInvalidValue;
    }
    uint16_t* ws = nullptr;
    if (Split_K > 1) {
        const unsigned long long need = 2ull * (unsigned long long)Split_K * (unsigned long long)M_Global *
                                        (unsigned long long)N_Global;
        if (need > (unsigned long long)SPB_NOALLOC_MAX_SCRATCH_BYTES) {
            spb::set_error("spb_spmm_bitmap_v3_noalloc: Split_K*M*N*2 = %llu bytes of partial sums exceed the built-in "
                           "scratch of %llu bytes; lower Split_K or use spb_spmm_bitmap_v3 with your own workspace",
                           need, (unsigned long long)SPB_NOALLOC_MAX_SCRATCH_BYTES);
            return (int)cudaErrorInvalidValue;
        }
        cudaError_t e = scratch_address(&ws);
        if (e != cudaSuccess) return (int)e;
    }
    // The SpMM kernel writes every partial of every range (empty ranges as zeros) before the reduction
    // reads them, so nothing in the scratch has to be cleared between calls.
    // The static work schedule is the one that needs no library-owned buffers.
    spb::push_static_schedule();
    const int rc = spb_spmm_bitmap_v3(stream, nullptr, Compressed_A, TileOffsets, TileOffsets_Median, bitmap,
                                      max_nnz_intile, B, C, M_Global, N_Global, K_Global, ws, Split_K);
    spb::pop_static_schedule();
    return rc;
}
