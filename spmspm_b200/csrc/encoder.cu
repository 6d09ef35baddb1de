// GPU encoder: dense fp16 row-major A[M][K] -> bitmap-v3 format, bit-identical
// to the reference's CPU encoder InitSparseMatrixA_bitmap
// (reference csrc/SpMM_API.cuh:112-241).
//
// Three launches, all HBM-bound byte/integer work:
//   count : one CTA per 64x64 global tile; 16-byte coalesced loads, one mask
//           byte per 8-element row segment, bitmaps + per-tile counts + median
//           offsets + padded global-tile count + running maximum.
//   scan  : exclusive prefix of the padded counts -> global tile offsets.
//   pack  : re-reads the tile, compacts non-zeros in the reference's order into
//           shared memory (zero-padded to a multiple of 8) and streams the
//           chunk out with 16-byte stores.
#include "common.cuh"

namespace spb {
namespace {

constexpr int kEncThreads = 256;

// Tile index, inside its 64x64 global tile, of the 8x8 tile holding element
// (row, 8*cc): median tile row>>4, 16-column group cc>>1, then the 2x2 order of
// reference csrc/SpMM_API.cuh:170-176 (column half outer, row half inner).
// kFmt 1 is the layout of the fork's encoder for the second operand, InitSparseMatrixA_bitmap_v6_B
// (reference csrc/spmm_test_utils.h:523-652, called with median tiles of 16 x 16): median tiles column-major inside
// the global tile (16-column step outer, 16-row step inner, :566-567), the 2x2 tiles of a median tile row-major
// (:575-578), and one median offset per 16x16 median tile (16 per global tile, :564, :617-621).
template <int kFmt>
__device__ __forceinline__ int tile_of(int row, int cc)
{
    if (kFmt == 0) return 16 * (row >> 4) + 4 * (cc >> 1) + 2 * (cc & 1) + ((row >> 3) & 1);
    return 16 * (cc >> 1) + 4 * (row >> 4) + 2 * ((row >> 3) & 1) + (cc & 1);
}

// Bit c set when the c-th fp16 of the 16-byte segment is kept.  The reference
// keeps a value iff __half2float(v) != 0.0f (csrc/SpMM_API.cuh:189): +-0 are
// dropped, NaN and subnormals stay.
__device__ __forceinline__ uint32_t nonzero_mask(const uint4& v)
{
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t m = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        m |= ((w[i] & 0x00007fffu) ? 1u : 0u) << (2 * i);
        m |= ((w[i] & 0x7fff0000u) ? 1u : 0u) << (2 * i + 1);
    }
    return m;
}

__device__ __forceinline__ uint4 load_segment(const uint16_t* A, int K, int gm, int gk, int row, int cc)
{
    const uint16_t* p = A + (size_t)(gm * 64 + row) * K + (size_t)gk * 64 + cc * 8;
    return __ldg(reinterpret_cast<const uint4*>(p));
}

// Inclusive scan of one int per thread over the first 64 threads of the CTA.
// Every thread of warps 0 and 1 must call it.
__device__ __forceinline__ int scan64(int v, int* warp_total)
{
    const int lane = threadIdx.x & 31;
    int x = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        int y = __shfl_up_sync(0xffffffffu, x, d);
        if (lane >= d) x += y;
    }
    if (threadIdx.x == 31) *warp_total = x;
    // named barrier over the two participating warps
    asm volatile("bar.sync 1, 64;" ::: "memory");
    if (threadIdx.x >= 32) x += *warp_total;
    return x;
}

template <int kFmt>
__global__ void __launch_bounds__(kEncThreads)
encode_count_kernel(const uint16_t* __restrict__ A, int K, int GK, int* __restrict__ tile_nnz,
                    int* __restrict__ mtile, int* __restrict__ gcount, uint64_t* __restrict__ bitmap,
                    int* __restrict__ max_nnz)
{
    __shared__ __align__(8) uint8_t rowmask[64 * 8];
    __shared__ int warp_total;
    const int g = blockIdx.x, gm = g / GK, gk = g % GK;
    const int t = threadIdx.x;
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const int row = u * 32 + (t >> 3), cc = t & 7;
        const uint4 v = load_segment(A, K, gm, gk, row, cc);
        rowmask[tile_of<kFmt>(row, cc) * 8 + (row & 7)] = (uint8_t)nonzero_mask(v);
    }
    __syncthreads();
    if (t < 64) {
        const uint64_t bm = *reinterpret_cast<const uint64_t*>(&rowmask[t * 8]);
        const int cnt = __popcll(bm);
        bitmap[(size_t)g * 64 + t] = bm;
        tile_nnz[(size_t)g * 64 + t] = cnt;
        const int incl = scan64(cnt, &warp_total);
        if (kFmt == 0) {
            if ((t & 15) == 0) mtile[(size_t)g * 4 + (t >> 4)] = incl - cnt;
        } else {
            if ((t & 3) == 0) mtile[(size_t)g * 16 + (t >> 2)] = incl - cnt;
        }
        if (t == 63) {
            const int padded = (incl + 7) & ~7;  // reference csrc/SpMM_API.cuh:216-220
            gcount[g] = padded;
            atomicMax(max_nnz, padded);
        }
    }
}

// gtile[0] = 0, gtile[g+1] = sum of counts[0..g].  Single CTA.
__global__ void __launch_bounds__(1024) encode_scan_kernel(const int* __restrict__ counts, int* __restrict__ gtile, int G)
{
    __shared__ int warp_sums[32];
    __shared__ int carry_s;
    const int t = threadIdx.x, lane = t & 31, w = t >> 5;
    if (t == 0) {
        carry_s = 0;
        gtile[0] = 0;
    }
    __syncthreads();
    for (int base = 0; base < G; base += 1024) {
        const int i = base + t;
        int x = (i < G) ? counts[i] : 0;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            int y = __shfl_up_sync(0xffffffffu, x, d);
            if (lane >= d) x += y;
        }
        if (lane == 31) warp_sums[w] = x;
        __syncthreads();
        if (w == 0) {
            int s = warp_sums[lane];
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                int y = __shfl_up_sync(0xffffffffu, s, d);
                if (lane >= d) s += y;
            }
            warp_sums[lane] = s;
        }
        __syncthreads();
        const int carry = carry_s;
        const int incl = carry + x + (w ? warp_sums[w - 1] : 0);
        if (i < G) gtile[i + 1] = incl;
        __syncthreads();
        if (t == 1023) carry_s = incl;
        __syncthreads();
    }
}

template <int kFmt>
__global__ void __launch_bounds__(kEncThreads)
encode_pack_kernel(const uint16_t* __restrict__ A, int K, int GK, const int* __restrict__ gtile,
                   uint16_t* __restrict__ vals, size_t capacity, int* __restrict__ status)
{
    __shared__ __align__(8) uint8_t rowmask[64 * 8];
    __shared__ int tstart[64];
    __shared__ int warp_total;
    __shared__ __align__(16) uint16_t stage[4096 + 8];
    const int g = blockIdx.x, gm = g / GK, gk = g % GK;
    const int t = threadIdx.x;
    uint4 v[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const int row = u * 32 + (t >> 3), cc = t & 7;
        v[u] = load_segment(A, K, gm, gk, row, cc);
        rowmask[tile_of<kFmt>(row, cc) * 8 + (row & 7)] = (uint8_t)nonzero_mask(v[u]);
    }
    __syncthreads();
    if (t < 64) {
        const uint64_t bm = *reinterpret_cast<const uint64_t*>(&rowmask[t * 8]);
        const int cnt = __popcll(bm);
        const int incl = scan64(cnt, &warp_total);
        tstart[t] = incl - cnt;
    }
    __syncthreads();
    const size_t base = (size_t)gtile[g];
    const int padded = gtile[g + 1] - gtile[g];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const int row = u * 32 + (t >> 3), cc = t & 7, r = row & 7;
        const int tile = tile_of<kFmt>(row, cc);
        const uint64_t bm = *reinterpret_cast<const uint64_t*>(&rowmask[tile * 8]);
        int off = tstart[tile] + __popcll(bm & ((1ull << (8 * r)) - 1ull));
        const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint16_t lo = (uint16_t)(w[i] & 0xffffu), hi = (uint16_t)(w[i] >> 16);
            if (lo & 0x7fffu) stage[off++] = lo;
            if (hi & 0x7fffu) stage[off++] = hi;
        }
    }
    // zero padding up to the multiple of 8 (at most 7 halves)
    {
        const int total = tstart[63] + __popcll(*reinterpret_cast<const uint64_t*>(&rowmask[63 * 8]));
        if (t < padded - total) stage[total + t] = 0;
    }
    __syncthreads();
    if (base + (size_t)padded > capacity) {
        if (t == 0 && status) atomicOr(status, (int)kStatusEncodeOverflow);
        return;
    }
    uint4* dst = reinterpret_cast<uint4*>(vals + base);
    const uint4* src = reinterpret_cast<const uint4*>(stage);
    for (int i = t; i < padded / 8; i += kEncThreads) dst[i] = src[i];
}

__global__ void encode_init_kernel(int* max_nnz)
{
    *max_nnz = 0;
}

}  // namespace

size_t encode_scratch_bytes(int M, int K)
{
    const size_t G = (size_t)(M / 64) * (size_t)(K / 64);
    return (G + 1) * sizeof(int);
}

cudaError_t encode_count_and_scan(cudaStream_t s, const uint16_t* A, int M, int K, int* tile_nnz, int* mtile,
                                  int* gtile, uint64_t* bitmap, int* max_nnz, void* scratch, int fmt)
{
    const int GK = K / 64, G = (M / 64) * GK;
    count_launch(G > 0 ? 3 : 2);
    encode_init_kernel<<<1, 1, 0, s>>>(max_nnz);
    if (G > 0) {
        if (fmt == 0)
            encode_count_kernel<0><<<G, kEncThreads, 0, s>>>(A, K, GK, tile_nnz, mtile, (int*)scratch, bitmap, max_nnz);
        else
            encode_count_kernel<1><<<G, kEncThreads, 0, s>>>(A, K, GK, tile_nnz, mtile, (int*)scratch, bitmap, max_nnz);
    }
    encode_scan_kernel<<<1, 1024, 0, s>>>((const int*)scratch, gtile, G);
    return cudaGetLastError();
}

cudaError_t encode_pack(cudaStream_t s, const uint16_t* A, int M, int K, const int* gtile, const uint64_t* bitmap,
                        uint16_t* vals, size_t vals_capacity, int* status, int fmt)
{
    (void)bitmap;
    const int GK = K / 64, G = (M / 64) * GK;
    if (G > 0) count_launch();
    if (G > 0 && fmt == 0) encode_pack_kernel<0><<<G, kEncThreads, 0, s>>>(A, K, GK, gtile, vals, vals_capacity, status);
    if (G > 0 && fmt != 0) encode_pack_kernel<1><<<G, kEncThreads, 0, s>>>(A, K, GK, gtile, vals, vals_capacity, status);
    return cudaGetLastError();
}

}  // namespace spb
