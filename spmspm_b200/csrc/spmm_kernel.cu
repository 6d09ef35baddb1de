// SpMM over the bitmap-v3 format for sm_100a:  C[M x N] = A_sparse[M x K] * B[K x N].
//
// Replaces the reference's SpMM_Kernel_bitmap_v3 (reference csrc/SpMM_Kernel.cuh:18-199,
// an mma.sync + cp.async kernel) with a persistent, warp-specialised kernel:
//
//   producer warp   streams the compressed weight (packed values, bitmaps, median
//                   offsets of two vertically adjacent 64x64 global tiles) with
//                   1-D bulk copies and the activation tile with a 2-D TMA load into a
//                   ring of shared-memory stages, completion on mbarriers;
//   decode warps    (groups of 4 warps, one thread per weight row) expand the bitmaps:
//                   a first pass turns the 128 tile bitmaps of the stage into per-row
//                   value offsets with byte-wise popcounts + a 16-lane prefix sum, a second
//                   pass
//                   gathers each row's values and writes the dense 128 x 64 fp16 tile
//                   straight into tensor memory (tcgen05.st) as the MMA's A operand;
//   MMA warp        one thread issues tcgen05.mma (M=128, N=16..128, K=16, fp16 in,
//                   fp32 accumulate in TMEM), A from TMEM, B from the swizzled smem tile;
//   epilogue warps  read the accumulator (tcgen05.ld), round to fp16 and store C or the
//                   split-K partial, column-major as the reference does
//                   (reference csrc/SpMM_Kernel.cuh:192-198).
//
// Work item = (row block of 128 rows, split-K range); the split-K ranges are cut exactly
// like the reference's (reference csrc/SpMM_Kernel.cuh:35-43).  Every wait is bounded: when
// one runs out the CTA records it in the device status word and leaves without touching
// tensor memory again.
#include "common.cuh"
#include <cuda.h>
#include <cuda_fp16.h>
#include <mutex>

namespace spb {
namespace {

#ifndef SPB_DECODE_GROUPS
#define SPB_DECODE_GROUPS 3
#endif
constexpr int kDecodeGroups = SPB_DECODE_GROUPS;  // each group: 4 warps, one thread per weight row
constexpr int kProducerWarp = 0;
constexpr int kMmaWarp = 1;
constexpr int kEpilogueWarp0 = 2;     // warps 2..5
constexpr int kDecodeWarp0 = 6;       // warps 6..
constexpr int kThreads = 32 * (kDecodeWarp0 + 4 * kDecodeGroups);
constexpr int kABufs = 2 * kDecodeGroups;  // A-operand buffers in TMEM (32 columns each)
constexpr int kMaxStages = 24;
// Per-row metadata of one stage: word = value offset (16 bit) | row mask << 16 | row count << 24.
// Rows 0-3 and rows 4-7 of a tile live in two regions whose distance is 16 mod 32 words and every
// 16-tile median group is shifted by 8 words, so that the 32 rows a warp reads at once fall into
// 32 different banks.
constexpr int kMetaRegionWords = 592;
constexpr int kMetaBufBytes = 2 * kMetaRegionWords * 4;
constexpr int kMetaBytes = ((kDecodeGroups * 2 * kMetaBufBytes + 1023) / 1024) * 1024;
constexpr int kHeaderBytes = 1024;
constexpr int kLutOffset = 640;       // two 16-entry selector tables inside the header
constexpr uint32_t kSpinLimit = 1u << 22;

struct KernelParams {
    const uint16_t* vals;
    const int* gtile;
    const int* mtile;
    const uint64_t* bitmap;
    const int* max_nnz;
    uint16_t* out;
    int* status;
    int M, N, K, split_k;
    int kt_total, avg_kt, row_blocks, gm_total, n_tiles, num_items;
    uint32_t smem_bytes;
};

// ------------------------------------------------------------------ PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("{ .reg .b64 st; mbarrier.arrive.shared::cta.b64 st, [%0]; }" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("{ .reg .b64 st; mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1; }" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false (and raises *abort_flag) when the limit is reached or when
// another thread of the CTA has already given up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag)
{
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if (mbar_try(bar, parity)) return true;
        if (i > 64) {
            if (*abort_flag) return false;
            __nanosleep(40);
        }
    }
    *abort_flag = 1;
    return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            dst),
        "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void tc_fence_before()
{
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after()
{
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem desc], kind::f16.
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tc_st_32x32b_x32(uint32_t taddr, const uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
        "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tc_wait_st()
{
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_wait_ld()
{
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// AND-reduction of a predicate over the `n` threads of named barrier `id`.
__device__ __forceinline__ bool bar_and(int id, int n, bool pred)
{
    uint32_t out;
    asm volatile(
        "{ .reg .pred p, q; setp.ne.u32 p, %3, 0; barrier.cta.red.and.pred q, %1, %2, p; selp.u32 %0, 1, 0, q; }"
        : "=r"(out)
        : "r"(id), "r"(n), "r"((uint32_t)pred)
        : "memory");
    return out != 0;
}

// Shared-memory descriptor of a K-major, 128-byte-swizzled tile (rows of 64 fp16 = 128 B,
// 8-row groups 1024 B apart), as written by the 2-D TMA load of the activation tile.
__device__ __forceinline__ uint64_t make_b_desc(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);
    d |= (uint64_t)1 << 16;            // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;  // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;            // descriptor version for sm_100
    d |= (uint64_t)2 << 61;            // SWIZZLE_128B
    return d;
}

struct Item {
    int nt, y, batch, k0, nk;
};
__device__ __forceinline__ Item decode_item(const KernelParams& p, int item)
{
    Item it;
    const int per_nt = p.row_blocks * p.split_k;
    it.nt = item / per_nt;
    const int rem = item - it.nt * per_nt;
    it.y = rem / p.split_k;
    it.batch = rem - it.y * p.split_k;
    it.k0 = it.batch * p.avg_kt;
    int k1 = it.k0 + p.avg_kt;
    if (k1 > p.kt_total) k1 = p.kt_total;
    it.nk = k1 > it.k0 ? k1 - it.k0 : 0;
    return it;
}

__device__ __forceinline__ void tc_st_32x32b_x16(uint32_t taddr, const uint32_t* r)
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(
            taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
// prmt.b32 in its default mode: selector nibble bits 2:0 pick one of the 8 source bytes, bit 3
// replaces the byte by 8 copies of its sign bit.
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel)
{
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr)
{
    uint32_t v;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void lds32x3(uint32_t addr, uint32_t& a, uint32_t& b, uint32_t& c)
{
    asm volatile("ld.shared.b32 %0, [%3];\n\tld.shared.b32 %1, [%3+4];\n\tld.shared.b32 %2, [%3+8];"
                 : "=&r"(a), "=&r"(b), "=&r"(c)
                 : "r"(addr));
}

// Selector tables for expanding a row segment with byte permutes.  A row's 8-bit mask is split in
// two nibbles.  The low nibble's (up to 4) values are the first values of the row, the high
// nibble's the last, so the low half is expanded from a window starting at the row's first value
// and the high half from a window ending at its last value.
//   low  entry: sel(pos 0,1 from {v0,v1 | zero})  |  sel(pos 2,3 from {v0..v3}) << 16
//   high entry: sel(pos 4,5 from {v[k-4..k-1]})   |  sel(pos 6,7 from {v[k-2],v[k-1] | zero}) << 16
__device__ __forceinline__ uint32_t lut_low_entry(uint32_t n)
{
    const uint32_t b0 = n & 1, b1 = (n >> 1) & 1, b2 = (n >> 2) & 1;
    const uint32_t p0 = b0 ? 0x10u : 0x54u;
    const uint32_t p1 = b1 ? (b0 ? 0x32u : 0x10u) : 0x54u;
    const uint32_t i2 = b0 + b1, i3 = i2 + b2;
    const uint32_t s1 = (0x10u + 0x22u * i2) | ((0x10u + 0x22u * i3) << 8);
    return (p0 | (p1 << 8)) | (s1 << 16);
}
__device__ __forceinline__ uint32_t lut_high_entry(uint32_t n)
{
    const uint32_t b5 = (n >> 1) & 1, b6 = (n >> 2) & 1, b7 = (n >> 3) & 1;
    const uint32_t h4 = 3 - (b5 + b6 + b7), h5 = 3 - (b6 + b7);
    const uint32_t s2 = (0x10u + 0x22u * h4) | ((0x10u + 0x22u * h5) << 8);
    const uint32_t p6 = b6 ? (b7 ? 0x10u : 0x32u) : 0x54u;
    const uint32_t p7 = b7 ? 0x32u : 0x54u;
    return s2 | ((p6 | (p7 << 8)) << 16);
}

// Expand one 8-element row segment described by `meta` (see kMetaRegionWords) into 4 registers
// of packed fp16.  vbase: shared address of the stage's value region; lut: shared address of the
// selector tables.
__device__ __forceinline__ void decode_unit(uint32_t meta, uint32_t vbase, uint32_t lut, uint32_t* o)
{
    const uint32_t off2 = (meta << 1) & 0x1fffeu;  // byte offset of the row's first value
    const uint32_t k2 = (meta >> 23) & 0x1eu;      // 2 * number of values in the row
    const uint32_t mask = (meta >> 16) & 0xffu;
    uint32_t x0, x1, x2, y0, y1, y2;
    lds32x3(vbase + (off2 & ~3u), x0, x1, x2);
    const uint32_t ot2 = off2 + k2 - 8u;           // byte offset of the value 4 before the row's end
    lds32x3(vbase + (ot2 & ~3u), y0, y1, y2);
    const uint32_t L = lds32(lut + ((mask & 15u) << 2));
    const uint32_t H = lds32(lut + 64u + ((mask >> 4) << 2));
    const uint32_t selb = 0x3210u + ((off2 >> 1) & 1u) * 0x2222u;
    const uint32_t selt = 0x3210u + ((ot2 >> 1) & 1u) * 0x2222u;
    const uint32_t b0 = prmt(x0, x1, selb), b1 = prmt(x1, x2, selb);
    const uint32_t t0 = prmt(y0, y1, selt), t1 = prmt(y1, y2, selt);
    // 0xffff per kept position: mask bit -> sign bit of a byte -> replicated by the permute
    const uint32_t z1 = (mask & 0x0cu) * 0x1020u, z2 = (mask & 0x30u) * 0x0408u;
    const uint32_t k1 = prmt(z1, z1, 0x9988u), k2m = prmt(z2, z2, 0x9988u);
    o[0] = prmt(b0, 0u, L);
    o[1] = prmt(b0, b1, L >> 16) & k1;
    o[2] = prmt(t0, t1, H) & k2m;
    o[3] = prmt(t1, 0u, H >> 16);
}

template <int NPAD>
__global__ void __launch_bounds__(kThreads, 1)
spmm_bitmap_tcgen05_kernel(const KernelParams p, const __grid_constant__ CUtensorMap tmap_b)
{
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment for the swizzled activation tiles
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t pad = (uint32_t)(smem - smem_raw);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // ---- carve-up ------------------------------------------------------------------------
    int max_nnz = *p.max_nnz;
    if (max_nnz < 8) max_nnz = 8;
    if (max_nnz > 4096) max_nnz = 4096;
    const uint32_t vmax = ((uint32_t)max_nnz * 2 + 127) & ~127u;  // bytes per value chunk
    constexpr uint32_t kBTile = NPAD * 128;
    const uint32_t off_v0 = kBTile, off_v1 = kBTile + vmax, off_bm = kBTile + 2 * vmax, off_mt = off_bm + 1024;
    const uint32_t stage_bytes = (off_mt + 32 + 1023) & ~1023u;
    const uint32_t avail = p.smem_bytes - pad - kHeaderBytes - kMetaBytes;
    int S = (int)(avail / stage_bytes);
    if (S > kMaxStages) S = kMaxStages;

    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
    const uint32_t bar_full = smem_u32(bars);                         // [kMaxStages]
    const uint32_t bar_empty = bar_full + 8 * kMaxStages;             // [kMaxStages]
    const uint32_t bar_aready = bar_empty + 8 * kMaxStages;           // [kABufs]
    const uint32_t bar_afree = bar_aready + 8 * kABufs;               // [kABufs]
    const uint32_t bar_accfull = bar_afree + 8 * kABufs;              // [2]
    const uint32_t bar_accempty = bar_accfull + 16;                   // [2]
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + 8 * (2 * kMaxStages + 2 * kABufs + 4));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
    uint8_t* meta_base = smem + kHeaderBytes;
    uint8_t* stage_base = smem + kHeaderBytes + kMetaBytes;

    constexpr uint32_t kTmemCols = (2 * NPAD + 32 * kABufs) <= 256 ? 256 : 512;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kMaxStages; ++i) {
            mbar_init(bar_full + 8 * i, 1);
            mbar_init(bar_empty + 8 * i, 5);  // 4 decode warps + the MMA commit
        }
        for (int i = 0; i < kABufs; ++i) {
            mbar_init(bar_aready + 8 * i, 4);
            mbar_init(bar_afree + 8 * i, 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar_accfull + 8 * i, 1);
            mbar_init(bar_accempty + 8 * i, 4);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (threadIdx.x >= 32 && threadIdx.x < 64) {
        uint32_t* lut = reinterpret_cast<uint32_t*>(smem + kLutOffset);
        const uint32_t n = threadIdx.x - 32;
        lut[n] = n < 16 ? lut_low_entry(n) : lut_high_entry(n - 16);
    }
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_holder;
    const uint32_t tmem_a0 = tmem_base + 2 * NPAD;

    if (S < 2) {
        // Not enough shared memory for a pipeline (cannot happen with the launch configuration
        // used by the host code); leave cleanly.
        if (threadIdx.x == 0) atomicOr(p.status, (int)kStatusBadOffsets);
    } else if (warp == kProducerWarp) {
        // ================================================================= producer
        uint32_t it = 0;
        bool ok = true;
        for (int item = blockIdx.x; item < p.num_items && ok; item += gridDim.x) {
            const Item w = decode_item(p, item);
            const bool chunk1 = (2 * w.y + 1) < p.gm_total;
            const size_t g_row0 = (size_t)(2 * w.y) * p.kt_total + w.k0;
            for (int kk0 = 0; kk0 < w.nk && ok; kk0 += 32) {
                const int kk = kk0 + lane;
                int o0a = 0, o0b = 0, o1a = 0, o1b = 0;
                if (kk < w.nk) {
                    o0a = __ldg(p.gtile + g_row0 + kk);
                    o0b = __ldg(p.gtile + g_row0 + kk + 1);
                    if (chunk1) {
                        o1a = __ldg(p.gtile + g_row0 + p.kt_total + kk);
                        o1b = __ldg(p.gtile + g_row0 + p.kt_total + kk + 1);
                    }
                }
                const int n_here = min(32, w.nk - kk0);
                for (int j = 0; j < n_here && ok; ++j) {
                    const int a0 = __shfl_sync(0xffffffffu, o0a, j), b0 = __shfl_sync(0xffffffffu, o0b, j);
                    const int a1 = __shfl_sync(0xffffffffu, o1a, j), b1 = __shfl_sync(0xffffffffu, o1b, j);
                    if (lane == 0) {
                        const uint32_t slot = it % (uint32_t)S, round = it / (uint32_t)S;
                        if (round > 0) ok = mbar_wait(bar_empty + 8 * slot, (round - 1) & 1, abort_flag);
                        if (ok) {
                            uint32_t n0 = (uint32_t)(b0 - a0) * 2, n1 = (uint32_t)(b1 - a1) * 2;
                            if (b0 < a0 || n0 > vmax || b1 < a1 || n1 > vmax) {
                                atomicOr(p.status, (int)kStatusBadOffsets);
                                n0 = 0;
                                n1 = 0;
                            }
                            const uint32_t full = bar_full + 8 * slot;
                            const uint32_t sbase = smem_u32(stage_base + (size_t)slot * stage_bytes);
                            const uint32_t tx = kBTile + n0 + n1 + (chunk1 ? 2u : 1u) * (512u + 16u);
                            mbar_expect_tx(full, tx);
                            const size_t g0 = g_row0 + kk0 + j;
                            tma_load_2d(sbase, &tmap_b, (w.k0 + kk0 + j) * 64, w.nt * NPAD, full);
                            if (n0) bulk_g2s(sbase + off_v0, p.vals + a0, n0, full);
                            bulk_g2s(sbase + off_bm, p.bitmap + g0 * 64, 512, full);
                            bulk_g2s(sbase + off_mt, p.mtile + g0 * 4, 16, full);
                            if (chunk1) {
                                const size_t g1 = g0 + p.kt_total;
                                if (n1) bulk_g2s(sbase + off_v1, p.vals + a1, n1, full);
                                bulk_g2s(sbase + off_bm + 512, p.bitmap + g1 * 64, 512, full);
                                bulk_g2s(sbase + off_mt + 16, p.mtile + g1 * 4, 16, full);
                            }
                        }
                    }
                    ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
                    ++it;
                }
            }
        }
    } else if (warp == kMmaWarp) {
        // ================================================================= MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(NPAD >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
            uint32_t it = 0, idx = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < p.num_items && ok; item += gridDim.x) {
                const Item w = decode_item(p, item);
                if (w.nk == 0) continue;
                const uint32_t accbuf = idx & 1;
                if (idx >= 2) ok = mbar_wait(bar_accempty + 8 * accbuf, ((idx >> 1) - 1) & 1, abort_flag);
                const uint32_t d_tmem = tmem_base + accbuf * NPAD;
                for (int kk = 0; kk < w.nk && ok; ++kk, ++it) {
                    const uint32_t slot = it % (uint32_t)S, round = it / (uint32_t)S;
                    const uint32_t abuf = it % kABufs, around = it / kABufs;
                    ok = mbar_wait(bar_full + 8 * slot, round & 1, abort_flag) &&
                         mbar_wait(bar_aready + 8 * abuf, around & 1, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t bdesc = make_b_desc(smem_u32(stage_base + (size_t)slot * stage_bytes));
                    const uint32_t a_tmem = tmem_a0 + 32 * abuf;
#pragma unroll
                    for (int s = 0; s < 4; ++s)
                        tc_mma_ts(d_tmem, a_tmem + 8 * s, bdesc + 2 * s, idesc, (kk > 0 || s > 0) ? 1u : 0u);
                    tc_commit(bar_afree + 8 * abuf);
                    tc_commit(bar_empty + 8 * slot);
                }
                if (ok) tc_commit(bar_accfull + 8 * accbuf);
                ++idx;
            }
        }
        __syncwarp();
    } else if (warp < kDecodeWarp0) {
        // ================================================================= epilogue
        const int quad = warp & 3;
        const int row_in_block = quad * 32 + lane;
        uint32_t idx = 0;
        bool ok = true;
        for (int item = blockIdx.x; item < p.num_items && ok; item += gridDim.x) {
            const Item w = decode_item(p, item);
            const int grow = w.y * 128 + row_in_block;
            uint16_t* out = p.out + (p.split_k > 1 ? (size_t)w.batch * p.M * p.N : (size_t)0);
            if (w.nk == 0) {
                for (int n = 0; n < NPAD; ++n) {
                    const int col = w.nt * NPAD + n;
                    if (col < p.N && grow < p.M) out[(size_t)col * p.M + grow] = 0;
                }
                continue;
            }
            const uint32_t accbuf = idx & 1;
            ok = mbar_wait(bar_accfull + 8 * accbuf, (idx >> 1) & 1, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const uint32_t t_acc = tmem_base + ((uint32_t)(quad * 32) << 16) + accbuf * NPAD;
#pragma unroll
            for (int c = 0; c < NPAD / 16; ++c) {
                uint32_t r[16];
                tc_ld_32x32b_x16(t_acc + 16 * c, r);
                tc_wait_ld();
                if (c == NPAD / 16 - 1) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_accempty + 8 * accbuf);
                }
#pragma unroll
                for (int n = 0; n < 16; ++n) {
                    const int col = w.nt * NPAD + c * 16 + n;
                    if (col < p.N && grow < p.M)
                        out[(size_t)col * p.M + grow] = __half_as_ushort(__float2half_rn(__uint_as_float(r[n])));
                }
            }
            ++idx;
        }
    } else {
        // ================================================================= decode
        const int dw = warp - kDecodeWarp0;
        const int group = dw >> 2;
        const int quad = warp & 3;             // TMEM lane quadrant this warp may access
        const int row = quad * 32 + lane;      // weight row inside the 128-row block == tile index in pass 1
        const int bar_id = 1 + group;
        uint8_t* meta_g = meta_base + group * (2 * kMetaBufBytes);
        const uint32_t lut = smem_u32(smem + kLutOffset);
        // pass 1: this thread owns tile `row` of the stage (tile t of chunk t>>6)
        const int chunk = row >> 6, rr = row & 63;
        const uint32_t p1_word = (uint32_t)row * 4 + 8 * (uint32_t)(row >> 4);
        // pass 2: the 8 tiles crossing this weight row are tbase + 2q, q = 0..7
        const int tbase = chunk * 64 + 16 * (rr >> 4) + ((rr >> 3) & 1);
        const int r_in_tile = rr & 7;
        const uint32_t p2_word = (uint32_t)(r_in_tile >> 2) * kMetaRegionWords + (uint32_t)tbase * 4 +
                                 (uint32_t)(r_in_tile & 3) + 8 * (uint32_t)(tbase >> 4);

        uint32_t it = 0, mine = 0;
        bool ok = true;
        for (int item = blockIdx.x; item < p.num_items && ok; item += gridDim.x) {
            const Item w = decode_item(p, item);
            const bool chunk1 = (2 * w.y + 1) < p.gm_total;
            const bool valid = (chunk == 0) || chunk1;
            for (int kk = 0; kk < w.nk; ++kk, ++it) {
                if ((int)(it % kDecodeGroups) != group) continue;
                const uint32_t slot = it % (uint32_t)S, round = it / (uint32_t)S;
                const uint32_t abuf = it % kABufs, around = it / kABufs;
                const bool got = mbar_wait(bar_full + 8 * slot, round & 1, abort_flag);
                const uint8_t* st = stage_base + (size_t)slot * stage_bytes;
                uint32_t* meta = reinterpret_cast<uint32_t*>(meta_g + (mine & 1) * kMetaBufBytes);
                ++mine;
                // ---- pass 1: per-row value offsets, masks and counts of tile `row`
                {
                    uint2 bm = make_uint2(0u, 0u);
                    int mt = 0;
                    if (got && valid) {
                        bm = reinterpret_cast<const uint2*>(st + off_bm)[row];
                        mt = reinterpret_cast<const int*>(st + off_mt)[chunk * 4 + (rr >> 4)];
                    }
                    // per-byte population counts (one byte of the bitmap = one tile row)
                    uint32_t a = bm.x - ((bm.x >> 1) & 0x55555555u);
                    a = (a & 0x33333333u) + ((a >> 2) & 0x33333333u);
                    a = (a + (a >> 4)) & 0x0f0f0f0fu;
                    uint32_t b = bm.y - ((bm.y >> 1) & 0x55555555u);
                    b = (b & 0x33333333u) + ((b >> 2) & 0x33333333u);
                    b = (b + (b >> 4)) & 0x0f0f0f0fu;
                    const uint32_t ia = a * 0x01010101u, ib = b * 0x01010101u;  // inclusive byte prefixes
                    const uint32_t tl = ia >> 24;
                    const int cnt = (int)(tl + (ib >> 24));
                    int x = cnt;                                               // 16-lane scan: tiles of a median tile
#pragma unroll
                    for (int d = 1; d < 16; d <<= 1) {
                        const int y = __shfl_up_sync(0xffffffffu, x, d, 16);
                        if ((lane & 15) >= d) x += y;
                    }
                    const uint32_t base = (uint32_t)chunk * (vmax >> 1) + (uint32_t)mt + (uint32_t)(x - cnt);
                    const uint32_t base_hi = base + tl;
                    const uint32_t ea = ia << 8, eb = ib << 8;                   // exclusive prefixes, byte 0 == 0
                    uint4 lo4, hi4;
                    uint32_t* lo_w = reinterpret_cast<uint32_t*>(&lo4);
                    uint32_t* hi_w = reinterpret_cast<uint32_t*>(&hi4);
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        const uint32_t s1 = (uint32_t)r | ((uint32_t)(4 + r) << 4);
                        const uint32_t s2 = (uint32_t)r | (4u << 8) | (5u << 12);
                        lo_w[r] = prmt(ea, prmt(bm.x, a, s1), s2) + base;
                        hi_w[r] = prmt(eb, prmt(bm.y, b, s1), s2) + base_hi;
                    }
                    *reinterpret_cast<uint4*>(meta + p1_word) = lo4;
                    *reinterpret_cast<uint4*>(meta + kMetaRegionWords + p1_word) = hi4;
                }
                ok = bar_and(bar_id, 128, got && !*abort_flag);
                if (!ok) break;
                // ---- pass 2: thread <-> weight row; gather its 64 values, 8 per tile
                const uint32_t vbase = smem_u32(st + off_v0);
                const uint32_t maddr = smem_u32(meta + p2_word);
                uint32_t a[32];
#pragma unroll
                for (int q = 0; q < 8; ++q) decode_unit(lds32(maddr + 32 * q), vbase, lut, a + 4 * q);
                // ---- hand the dense rows to the tensor core through TMEM
                bool fr = true;
                if (around > 0) fr = mbar_wait(bar_afree + 8 * abuf, (around - 1) & 1, abort_flag);
                fr = __all_sync(0xffffffffu, fr);
                if (fr) {
                    tc_fence_after();
                    const uint32_t ta = tmem_a0 + 32 * abuf + ((uint32_t)(quad * 32) << 16);
                    tc_st_32x32b_x16(ta, a);
                    tc_st_32x32b_x16(ta + 16, a + 16);
                    tc_wait_st();
                    tc_fence_before();
                }
                __syncwarp();
                if (lane == 0) {
                    if (fr) mbar_arrive(bar_aready + 8 * abuf);
                    mbar_arrive(bar_empty + 8 * slot);
                }
            }
        }
    }

    // ---- teardown ----------------------------------------------------------------------------
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (*abort_flag) {
        if (threadIdx.x == 0) {
            atomicOr(p.status, (int)kStatusWaitTimeout);
            // give copies that may still be in flight a bounded chance to land before the CTA's
            // shared memory is released
            for (int i = 0; i < S; ++i)
                for (uint32_t spin = 0; spin < 4096; ++spin)
                    if (mbar_try(bar_full + 8 * i, 0) || mbar_try(bar_full + 8 * i, 1)) break;
        }
        __syncthreads();
    }
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// ------------------------------------------------------------------------------ host side

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn()
{
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    });
    return fn;
}

struct DeviceInfo {
    int sms = 0;
    int max_smem = 0;
    bool ok = false;
};
DeviceInfo device_info()
{
    static DeviceInfo cache[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return DeviceInfo();
    if (!cache[dev].ok) {
        DeviceInfo d;
        cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev);
        cudaDeviceGetAttribute(&d.max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
        d.ok = d.sms > 0;
        cache[dev] = d;
    }
    return cache[dev];
}

template <int NPAD>
cudaError_t launch_t(cudaStream_t s, const SpmmArgs& a, const DeviceInfo& di, int* status)
{
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) {
        set_error("cuTensorMapEncodeTiled is not available from the driver");
        return cudaErrorNotSupported;
    }
    CUtensorMap tmap;
    const cuuint64_t dims[2] = {(cuuint64_t)a.K, (cuuint64_t)a.N};
    const cuuint64_t strides[1] = {(cuuint64_t)a.K * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)NPAD};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(&tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<uint16_t*>(a.B), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed (%d) for B=%p K=%d N=%d", (int)r, (const void*)a.B, a.K, a.N);
        return cudaErrorInvalidValue;
    }
    KernelParams p;
    p.vals = a.vals;
    p.gtile = a.gtile;
    p.mtile = a.mtile;
    p.bitmap = a.bitmap;
    p.max_nnz = a.max_nnz;
    p.out = a.out;
    p.status = status;
    p.M = a.M;
    p.N = a.N;
    p.K = a.K;
    p.split_k = a.split_k;
    p.kt_total = a.K / 64;
    p.avg_kt = (p.kt_total - 1) / a.split_k + 1;  // reference csrc/SpMM_Kernel.cuh:36
    p.gm_total = a.M / 64;
    p.row_blocks = (p.gm_total + 1) / 2;
    p.n_tiles = (a.N + NPAD - 1) / NPAD;
    p.num_items = p.n_tiles * p.row_blocks * a.split_k;
    p.smem_bytes = (uint32_t)di.max_smem;

    static bool attr_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(spmm_bitmap_tcgen05_kernel<NPAD>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, di.max_smem);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    const int grid = p.num_items < di.sms ? p.num_items : di.sms;
    spmm_bitmap_tcgen05_kernel<NPAD><<<grid, kThreads, di.max_smem, s>>>(p, tmap);
    return cudaGetLastError();
}

}  // namespace

int suggest_split_k(int M, int N, int K)
{
    (void)N;
    DeviceInfo di = device_info();
    const int sms = di.ok ? di.sms : 148;
    const int row_blocks = (M / 64 + 1) / 2;
    const int kt = K / 64;
    if (row_blocks <= 0 || kt <= 0) return 1;
    // Smallest split whose item count fills the SMs at least ~twice, while keeping each
    // range at least 8 k-tiles long.
    int best = 1;
    double best_cost = 1e30;
    for (int sk = 1; sk <= 32 && sk <= kt; ++sk) {
        const int avg = (kt - 1) / sk + 1;
        if ((sk - 1) * avg >= kt) continue;  // would leave an empty last range
        if (avg < 4 && sk > 1) break;
        const long items = (long)row_blocks * sk;
        const long waves = (items + sms - 1) / sms;
        // time ~ waves * (avg + fixed per-item overhead) ; + a small cost per extra partial
        const double cost = (double)waves * (avg + 3.0) + 0.15 * sk;
        if (cost < best_cost - 1e-9) {
            best_cost = cost;
            best = sk;
        }
    }
    return best;
}

cudaError_t spmm_launch(cudaStream_t s, const SpmmArgs& a)
{
    DeviceInfo di = device_info();
    if (!di.ok) {
        set_error("no usable CUDA device");
        return cudaErrorNoDevice;
    }
    int* status = nullptr;
    cudaError_t e = device_status_ptr(&status);
    if (e != cudaSuccess) return e;
    if (a.N <= 16) return launch_t<16>(s, a, di, status);
    if (a.N <= 32) return launch_t<32>(s, a, di, status);
    if (a.N <= 64) return launch_t<64>(s, a, di, status);
    return launch_t<128>(s, a, di, status);
}

}  // namespace spb
