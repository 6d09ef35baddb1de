// SpMSpM: both operands bitmap-compressed (the fork's extension, reference csrc/SpMM_API.cuh:47-53: the
// 19-argument SpMM_SplitK_API_bitmap_v3, and csrc/spmm_test_utils.h:523-652: InitSparseMatrixA_bitmap_v6_B).
//
// The second operand is small next to the weight at decode sizes and no larger than it in the fork's own tests, and
// the SpMM kernel wants it as a dense, swizzled shared-memory tile fetched by TMA.  So the compressed B is expanded
// once per call into a dense [N][K] array taken from the stream's memory pool (cudaMallocAsync: no synchronisation,
// legal under stream capture) by an HBM-bound kernel, and the SpMM then runs exactly as for a dense B.
// Traffic of the expansion: compressed bytes in, 2 * N * K bytes out.
#include "../../include/spmm_b200.h"
#include "common.cuh"

namespace spb {
namespace {

// One CTA per 64x64 global tile, thread t <-> (tile t / 4 in storage order, rows 2 * (t % 4) and + 1 of that tile).
__global__ void __launch_bounds__(256)
decode_b_kernel(const uint16_t* __restrict__ vals, const int* __restrict__ gtile, const uint64_t* __restrict__ bitmap,
                int GK, int cols, uint16_t* __restrict__ dense, long long val_capacity, int* __restrict__ status)
{
    __shared__ int tstart[64];
    __shared__ int warp_total;
    const int g = blockIdx.x, gm = g / GK, gk = g % GK, t = threadIdx.x;
    const long long base = gtile[g], end = gtile[g + 1];
    const bool bad = base < 0 || end < base || end - base > 4096 || (val_capacity >= 0 && end > val_capacity);
    if (t < 64) {
        const uint64_t bm = bitmap[(size_t)g * 64 + t];
        const int cnt = __popcll(bm);
        // inclusive scan over the 64 tiles (two warps)
        int x = cnt;
        const int lane = t & 31;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int y = __shfl_up_sync(0xffffffffu, x, d);
            if (lane >= d) x += y;
        }
        if (t == 31) warp_total = x;
        asm volatile("bar.sync 1, 64;" ::: "memory");
        if (t >= 32) x += warp_total;
        tstart[t] = x - cnt;
    }
    __syncthreads();
    if (bad) {   // corrupt offsets: report, write zeros
        if (t == 0 && status) atomicOr(status, (int)kStatusBadOffsets);
    }
    const int tile = t >> 2;
    // storage order of the second-operand layout: 16-column step outer, 16-row step, then the 2x2 tiles row-major
    const int mk = tile >> 4, mm = (tile >> 2) & 3, i = (tile >> 1) & 1, j = tile & 1;
    const uint64_t bm = bitmap[(size_t)g * 64 + tile];
    const int avail = (int)(end - base);
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const int r = 2 * (t & 3) + u;
        int off = tstart[tile] + __popcll(bm & ((1ull << (8 * r)) - 1ull));
        const uint32_t mask = (uint32_t)(bm >> (8 * r)) & 0xffu;
        uint16_t o[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const bool set = (mask >> c) & 1u;
            o[c] = (set && !bad && off < avail) ? vals[base + off] : (uint16_t)0;
            off += set ? 1 : 0;
        }
        const int row = gm * 64 + 16 * mm + 8 * i + r, col = gk * 64 + 8 * (2 * mk + j);
        uint4 w;
        w.x = o[0] | ((uint32_t)o[1] << 16);
        w.y = o[2] | ((uint32_t)o[3] << 16);
        w.z = o[4] | ((uint32_t)o[5] << 16);
        w.w = o[6] | ((uint32_t)o[7] << 16);
        *reinterpret_cast<uint4*>(dense + (size_t)row * cols + col) = w;
    }
}

}  // namespace

cudaError_t decode_operand_b(cudaStream_t s, const uint16_t* vals, const int* gtile, const uint64_t* bitmap, int rows,
                             int cols, uint16_t* dense, int* status)
{
    const int GK = cols / 64, G = (rows / 64) * GK;
    if (G <= 0) return cudaSuccess;
    count_launch();
    decode_b_kernel<<<G, 256, 0, s>>>(vals, gtile, bitmap, GK, cols, dense, -1, status);
    return cudaGetLastError();
}

}  // namespace spb

extern "C" int spb_decode_operand_b(void* stream, const uint16_t* Compressed_B, const int* TileOffsets_B,
                                    const uint64_t* bitmap_B, int rows, int cols, uint16_t* dense_out)
{
    if (!Compressed_B || !TileOffsets_B || !bitmap_B || !dense_out || rows <= 0 || cols <= 0 || (rows % 64) || (cols % 64) ||
        !spb::aligned16(dense_out)) {
        spb::set_error("spb_decode_operand_b: non-null pointers, rows and cols positive multiples of 64, 16-byte aligned output");
        return (int)cudaErrorInvalidValue;
    }
    int* status = nullptr;
    cudaError_t e = spb::device_status_ptr(&status);
    if (e != cudaSuccess) return (int)e;
    return (int)spb::decode_operand_b((cudaStream_t)stream, Compressed_B, TileOffsets_B, bitmap_B, rows, cols, dense_out, status);
}
