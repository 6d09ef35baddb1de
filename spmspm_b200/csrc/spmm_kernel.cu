// SpMM over the bitmap-v3 format for sm_100a:  C[M x N] = A_sparse[M x K] * B[K x N].
//
// Replaces the reference's SpMM_Kernel_bitmap_v3 (reference csrc/SpMM_Kernel.cuh:18-199,
// an mma.sync + cp.async kernel) with a persistent, warp-specialised kernel:
//
//   producer warps  three warps stream the compressed weight (packed values; bitmaps and median
//                   offsets; activation tiles) of two vertically adjacent 64x64 global tiles with
//                   1-D bulk copies and the activation tile with a 2-D TMA load into a ring of
//                   shared-memory stages of four k-tiles each, completion on mbarriers;
//   decode warps    (4 groups of 4 warps, one group per k-tile of a stage, one thread per weight
//                   row) expand the bitmaps in a single pass: each thread reads the bitmaps of
//                   the 8 tiles its row crosses, keeps a running sum of the tile sizes of its
//                   median tile, finds its row's values with popcounts, expands them with byte
//                   permutes driven by two nibble tables and writes the dense 128 x 64 fp16 tile
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
#include <cstdio>
#include <mutex>

namespace spb {
namespace {

// Warp roles, by warpgroup (4 warps) so that each role can resize its register file share:
//   warpgroup 0: warp 1 MMA issuer, warps 0, 2, 3 producers (each issues a share of the copies)
//   warpgroup 1: epilogue (one warp per TMEM lane quadrant)
//   warpgroup 2..: decode groups (one warp per quadrant each)
#ifndef SPB_KT
#define SPB_KT 4
#endif
// A pipeline stage holds kKT consecutive k-tiles of one 128-row block.  The four decode groups are
// split into kSets sets of kKT groups; set s expands the stages s, s + kSets, ..., one group per k-tile.
// Smaller stages mean more stages in the shared-memory ring (the loop producer -> HBM -> decode ->
// MMA -> release is latency-bound), larger ones mean fewer copies per byte.
constexpr int kKT = SPB_KT;
constexpr int kDecodeGroups = 4;
constexpr int kSets = kDecodeGroups / kKT;
static_assert(kKT * kSets == kDecodeGroups, "kKT must be 1, 2 or 4");
constexpr int kMmaWarp = 1;
constexpr int kEpilogueWarp0 = 4;
constexpr int kDecodeWarp0 = 8;
constexpr int kThreads = 32 * (kDecodeWarp0 + 4 * kDecodeGroups);
// Registers per thread after the roles have resized (the launch gives every thread
// 65536 / kThreads rounded down to a multiple of 8).
constexpr int kRegsControl = 40, kRegsEpilogue = 56, kRegsDecode = 96;
// The register file is handed out per warp in blocks of 512 registers (16 per thread), so the budget
// is checked on rounded-up sizes; a resize that cannot be satisfied blocks the warp for ever.
constexpr int regs_rounded(int r) { return (r + 15) / 16 * 16; }
static_assert(128 * regs_rounded(kRegsControl) + 128 * regs_rounded(kRegsEpilogue) +
                      128 * kDecodeGroups * regs_rounded(kRegsDecode) <= 65536 - 2048,
              "register budget (keep slack: a resize that can never be satisfied would block for ever)");
constexpr int kMaxStages = 24;
constexpr int kHeaderBytes = 1024;
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
// Same, for the control warps, which spend most of their time waiting for the decode warps: after a
// few quick tries they sleep between polls so that their polling does not take issue slots and
// integer-pipe cycles from the decode warps of the same scheduler.
__device__ __forceinline__ bool mbar_wait_patient(uint32_t bar, uint32_t parity, volatile int* abort_flag)
{
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if (mbar_try(bar, parity)) return true;
        if (i >= 4) {
            if (*abort_flag) return false;
            __nanosleep(150);
        }
    }
    *abort_flag = 1;
    return false;
}
// Same, for waits that last a whole work item: polls rarely so that the waiting warp leaves the
// issue slots to the others.
__device__ __forceinline__ bool mbar_wait_relaxed(uint32_t bar, uint32_t parity, volatile int* abort_flag)
{
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if (mbar_try(bar, parity)) return true;
        if (*abort_flag) return false;
        __nanosleep(400);
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
// Register-file resizing of the calling warpgroup (all of its warps must execute it).
template <int N>
__device__ __forceinline__ void reg_alloc()
{
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void reg_dealloc()
{
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
// True in exactly one lane of a converged warp.
__device__ __forceinline__ bool elect_one()
{
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.b32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
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
__device__ __forceinline__ void tc_st_32x32b_x8(uint32_t taddr, const uint32_t* r)
{
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(r[0]),
                 "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
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

__device__ __forceinline__ void lds64(uint32_t addr, uint32_t& a, uint32_t& b)
{
    asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(a), "=r"(b) : "r"(addr));
}

// Selector tables for expanding a row segment with byte permutes.  A row's 8-bit mask is split in
// two nibbles.  The low nibble's (up to 4) values are the first values of the row, the high
// nibble's the last, so positions 0-3 are filled from a 4-value window starting at the row's first
// value and positions 4-7 from a 4-value window ending at its last value.  Every output register
// (two positions) is one permute of a 2-value window and a zero register:
//   pair_sel(lo, hi, first): selector placing the window's values at the kept positions.
// Low-nibble entry  {sel(pos 0,1) | window(pos 2,3) << 16, sel(pos 2,3)}
// High-nibble entry {sel(pos 6,7) | window(pos 4,5) << 16, sel(pos 4,5)}
// where window(...) is the permute selector that cuts the 2-value window out of the 4-value one.
__device__ __forceinline__ uint32_t pair_sel_bottom(uint32_t lo, uint32_t hi)
{
    // window = {next value, the one after}; zero register in bytes 4..7
    const uint32_t p_lo = lo ? 0x10u : 0x54u;
    const uint32_t p_hi = hi ? (lo ? 0x32u : 0x10u) : 0x54u;
    return p_lo | (p_hi << 8);
}
__device__ __forceinline__ uint32_t pair_sel_top(uint32_t lo, uint32_t hi)
{
    // window = {second to last value, last value}
    const uint32_t p_hi = hi ? 0x32u : 0x54u;
    const uint32_t p_lo = lo ? (hi ? 0x10u : 0x32u) : 0x54u;
    return p_lo | (p_hi << 8);
}
__device__ __forceinline__ uint2 lut_low_entry(uint32_t n)
{
    const uint32_t b0 = n & 1, b1 = (n >> 1) & 1, b2 = (n >> 2) & 1, b3 = (n >> 3) & 1;
    const uint32_t win = 0x3210u + 0x2222u * (b0 + b1);  // values b0+b1, b0+b1+1 of the 4-value window
    return make_uint2(pair_sel_bottom(b0, b1) | (win << 16), pair_sel_bottom(b2, b3));
}
__device__ __forceinline__ uint2 lut_high_entry(uint32_t n)
{
    const uint32_t b4 = n & 1, b5 = (n >> 1) & 1, b6 = (n >> 2) & 1, b7 = (n >> 3) & 1;
    const uint32_t win = 0x3210u + 0x2222u * (2 - (b6 + b7));  // the two values before those of pos 6,7
    return make_uint2(pair_sel_top(b6, b7) | (win << 16), pair_sel_top(b4, b5));
}

// Expansion of one 8-element row segment (one row of one 8x8 tile) into 4 registers of packed fp16,
// split into a load half and a compute half so that the loads of several segments can be in flight
// together.  lut: shared address of the selector tables.
#ifndef SPB_UNIT_BATCH
#define SPB_UNIT_BATCH 2
#endif
constexpr int kUnitBatch = SPB_UNIT_BATCH;  // row segments whose loads are issued together (1, 2 or 4)
struct UnitLoads {
    uint32_t x0, x1, x2, y0, y1, y2, l0, l1, h0, h1, sb, st;
};
__device__ __forceinline__ void lds32x3_before(uint32_t addr, uint32_t& a, uint32_t& b, uint32_t& c)
{
    asm volatile("ld.shared.b32 %0, [%3+-8];\n\tld.shared.b32 %1, [%3+-4];\n\tld.shared.b32 %2, [%3];"
                 : "=&r"(a), "=&r"(b), "=&r"(c)
                 : "r"(addr));
}
// Load half: everything a row segment needs is derived from the tile's 64-bit bitmap (lo, hi)
// in the thread that expands it.  `run` is the shared address where the values of this tile *pair*
// (the tile of rows 0-7 and the one of rows 8-15 of the same 16-row median tile and 8-column slice)
// start; it is advanced past the pair.  The other tile's count comes from the lane 8 away.
//   below_lo/below_hi  thread constants: bitmap bits of the tile rows above this thread's row
//   rsel               permute selector moving this row's mask byte to byte 0
//   second             all ones in the threads of the second tile of the pair, else zero
__device__ __forceinline__ void unit_load_sp(uint32_t lo, uint32_t hi, uint32_t& run, uint32_t below_lo,
                                             uint32_t below_hi, uint32_t rsel, uint32_t second, uint32_t lut,
                                             UnitLoads& u)
{
    const uint32_t cnt = __popc(lo) + __popc(hi);
    const uint32_t other = __shfl_xor_sync(0xffffffffu, cnt, 8);
    const uint32_t tile = run + 2u * (other & second);
    run += 2u * (cnt + other);
    const uint32_t w0 = tile + 2u * (__popc(lo & below_lo) + __popc(hi & below_hi));
    const uint32_t g = prmt(lo, hi, rsel);                 // row mask in byte 0 (bytes 1-3 are not clean)
    const uint32_t wt = w0 + 2u * __popc(g & 0xffu);       // address just past the row's last value
    lds32x3(w0 & ~3u, u.x0, u.x1, u.x2);
    lds32x3_before(wt & ~3u, u.y0, u.y1, u.y2);            // window of the 4 values before wt
    lds64(lut + (g & 15u) * 8u, u.l0, u.l1);
    lds64(lut + 128u + (g & 0xf0u), u.h0, u.h1);           // high-nibble entries are 16 bytes apart
    u.sb = w0 << 3;
    u.st = wt << 3;
}
__device__ __forceinline__ void unit_expand(const UnitLoads& u, uint32_t* o)
{
    const uint32_t b0 = __funnelshift_r(u.x0, u.x1, u.sb), b1 = __funnelshift_r(u.x1, u.x2, u.sb);
    const uint32_t t0 = __funnelshift_r(u.y0, u.y1, u.st), t1 = __funnelshift_r(u.y1, u.y2, u.st);
    o[0] = prmt(b0, 0u, u.l0);
    o[1] = prmt(prmt(b0, b1, u.l0 >> 16), 0u, u.l1);
    o[2] = prmt(prmt(t0, t1, u.h0 >> 16), 0u, u.h1);
    o[3] = prmt(t1, 0u, u.h0);
}

template <int NPAD>
__global__ void __launch_bounds__(kThreads, 1)
spmm_bitmap_tcgen05_kernel(const KernelParams p, const __grid_constant__ CUtensorMap tmap_b)
{
    // selector tables: low nibble entries [0,16); high nibble entry n at index 16 + 2n (16 bytes apart,
    // so that the nibble's bit position can be used as the offset)
    __shared__ __align__(16) uint2 lut_tab[48];
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment for the swizzled activation tiles
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t pad = (uint32_t)(smem - smem_raw);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // ---- carve-up ------------------------------------------------------------------------
    // A stage holds kKT consecutive k-tiles of one 128-row block: the activation tiles, then for each
    // of the two 64-row global-tile rows one contiguous run of packed values, the bitmaps and the
    // median offsets, then the start of every global tile's values inside its run.
    int max_nnz = *p.max_nnz;
    if (max_nnz < 8) max_nnz = 8;
    if (max_nnz > 4096) max_nnz = 4096;
    const uint32_t vmax = ((uint32_t)max_nnz * 2 + 127) & ~127u;  // bytes per global tile, upper bound
    constexpr uint32_t kBTile = NPAD * 128;
    const uint32_t off_v0 = kKT * kBTile, off_v1 = off_v0 + kKT * vmax;
    const uint32_t off_bm0 = off_v1 + kKT * vmax, off_bm1 = off_bm0 + kKT * 512;
    const uint32_t off_mt0 = off_bm1 + kKT * 512, off_mt1 = off_mt0 + kKT * 16;
    const uint32_t off_rel = off_mt1 + kKT * 16;  // [2][kKT] uint32: byte offset of a tile's values in its run
    const uint32_t stage_bytes = (off_rel + 8 * kKT + 1023) & ~1023u;
    const uint32_t avail = p.smem_bytes - pad - kHeaderBytes;
    int S = (int)(avail / stage_bytes);
    if (S > kMaxStages) S = kMaxStages;

    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
    const uint32_t bar_full = smem_u32(bars);                         // [kMaxStages]
    const uint32_t bar_empty = bar_full + 8 * kMaxStages;             // [kMaxStages]
    const uint32_t bar_aready = bar_empty + 8 * kMaxStages;           // [2 * kSets]
    const uint32_t bar_accfull = bar_aready + 8 * 2 * kSets;          // [2]
    const uint32_t bar_accempty = bar_accfull + 16;                   // [2]
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + 8 * (2 * kMaxStages + 2 * kSets + 4));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
    const uint32_t stage0 = smem_u32(smem + kHeaderBytes);

    // Back-to-back tcgen05.mma into one accumulator are serialised by the tensor core, and at these
    // tiny N every instruction is pure latency, so the four k-steps of a k-tile go to different
    // accumulators (summed in the epilogue).
    constexpr int kNAcc = 4;
    constexpr int kAccBufs = NPAD <= 32 ? 2 : 1;
    constexpr uint32_t kAccCols = kAccBufs * kNAcc * NPAD;
    constexpr uint32_t kACols = 2 * kSets * kKT * 32;  // A operands of two stages per set
    static_assert(kAccCols + kACols <= 512, "TMEM budget");
    constexpr uint32_t kTmemCols = 512;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kMaxStages; ++i) {
            mbar_init(bar_full + 8 * i, 1);
            mbar_init(bar_empty + 8 * i, 4 * kKT + 1);  // every decode warp + the MMA commit
        }
        for (int i = 0; i < 2 * kSets; ++i) mbar_init(bar_aready + 8 * i, 4 * kKT);
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar_accfull + 8 * i, 1);
            mbar_init(bar_accempty + 8 * i, 4);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (threadIdx.x >= 32 && threadIdx.x < 64) {
        const uint32_t n = threadIdx.x - 32;
        if (n < 16) {
            lut_tab[n] = lut_low_entry(n);
        } else {
            lut_tab[16 + 2 * (n - 16)] = lut_high_entry(n - 16);
            lut_tab[17 + 2 * (n - 16)] = make_uint2(0u, 0u);
        }
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
    const uint32_t tmem_a0 = tmem_base + kAccCols;

    // The A operands of n_abuf stages live in TMEM: two per set when the ring is deep enough, else one.
    // A decode warp may overwrite a buffer once the MMAs of the stage n_abuf back have completed, which
    // it learns from that stage's empty barrier; with a ring no deeper than n_abuf the full barrier of
    // its own stage already implies it.
    const uint32_t n_abuf = S > 2 * kSets ? 2u * kSets : (uint32_t)kSets;
    const bool reuse_wait = (uint32_t)S > n_abuf;
    const bool two_deep = n_abuf == 2u * kSets;
    if (S < 1) {
        // A single stage does not fit (cannot happen with the launch configuration used by the host
        // code); leave cleanly.
        if (threadIdx.x == 0) atomicOr(p.status, (int)kStatusBadOffsets);
    } else if (warp < kEpilogueWarp0) {
        reg_dealloc<kRegsControl>();
        if (warp != kMmaWarp) {
            // ================================================================= producers
            // Issuing a bulk copy costs the issuing thread on the order of a hundred cycles, so the
            // copies of a stage are shared by three warps that walk the same stage sequence:
            //   warp 0  arms the full barrier, writes the run offsets, copies the packed values
            //   warp 2  copies bitmaps and median offsets
            //   warp 3  loads the activation tiles
            const int prole = warp == 0 ? 0 : warp - 1;
            // Global-tile offsets are read in batches of 32 consecutive k-tiles (lane l holds the offset of
            // k-tile base + l of both 64-row global-tile rows) and one batch ahead, so that the latency of
            // these loads never sits between two stages.
            constexpr int kOffBatch = 28;  // k-tiles a batch advances by; a stage needs up to base + 27 + kKT
            struct Batch {
                int item, base, v0, v1;
                Item w;
            };
            auto load_batch = [&](Batch& b) {
                b.v0 = 0;
                b.v1 = 0;
                if (prole != 0 || b.item >= p.num_items) return;
                const size_t g = (size_t)(2 * b.w.y) * p.kt_total + b.w.k0 + b.base;
                if (lane <= b.w.nk - b.base) {
                    b.v0 = __ldg(p.gtile + g + lane);
                    if ((2 * b.w.y + 1) < p.gm_total) b.v1 = __ldg(p.gtile + g + p.kt_total + lane);
                }
            };
            auto next_nonempty = [&](int it, Item& w) -> int {
                do {
                    it += gridDim.x;
                    if (it < p.num_items) w = decode_item(p, it);
                } while (it < p.num_items && w.nk == 0);
                return it;
            };
            auto batch_after = [&](const Batch& b) -> Batch {
                Batch n = b;
                if (b.base + kOffBatch < b.w.nk) {
                    n.base = b.base + kOffBatch;
                } else {
                    n.base = 0;
                    n.item = next_nonempty(b.item, n.w);
                }
                return n;
            };
            uint32_t slot = 0, round = 0;
            bool ok = true;
            int item = blockIdx.x, kk0 = 0;
            Item w = decode_item(p, item < p.num_items ? item : 0);
            if (item < p.num_items && w.nk == 0) item = next_nonempty(item, w);
            Batch cur;
            cur.item = item;
            cur.base = 0;
            cur.w = w;
            load_batch(cur);
            Batch nxt = batch_after(cur);
            load_batch(nxt);
            while (item < p.num_items && ok) {
                const Item cw = w;
                const int ckk0 = kk0;
                if (cur.item != item || ckk0 - cur.base >= kOffBatch) {  // this stage starts the next batch
                    cur = nxt;
                    nxt = batch_after(cur);
                    load_batch(nxt);
                }
                const int bidx = ckk0 - cur.base;
                // advance to the next stage
                kk0 += kKT;
                if (kk0 >= w.nk) {
                    kk0 = 0;
                    item = next_nonempty(item, w);
                }

                const bool chunk1 = (2 * cw.y + 1) < p.gm_total;
                const int nv = min(kKT, cw.nk - ckk0);
                const size_t g0 = (size_t)(2 * cw.y) * p.kt_total + cw.k0 + ckk0;
                const int a0 = __shfl_sync(0xffffffffu, cur.v0, bidx), e0 = __shfl_sync(0xffffffffu, cur.v0, bidx + nv);
                const int a1 = __shfl_sync(0xffffffffu, cur.v1, bidx), e1 = __shfl_sync(0xffffffffu, cur.v1, bidx + nv);
                const int r0 = __shfl_sync(0xffffffffu, cur.v0, bidx + (lane & 7));
                const int r1 = __shfl_sync(0xffffffffu, cur.v1, bidx + (lane & 7));
                if (round > 0) ok = mbar_wait_patient(bar_empty + 8 * slot, (round - 1) & 1, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                uint32_t n0 = (uint32_t)(e0 - a0) * 2, n1 = chunk1 ? (uint32_t)(e1 - a1) * 2 : 0u;
                if (e0 < a0 || n0 > (uint32_t)nv * vmax || (chunk1 && (e1 < a1 || n1 > (uint32_t)nv * vmax))) {
                    if (lane == 0 && prole == 0) atomicOr(p.status, (int)kStatusBadOffsets);
                    n0 = 0;
                    n1 = 0;
                }
                const uint32_t sbase = stage0 + slot * stage_bytes;
                const uint32_t full = bar_full + 8 * slot;
                // where each global tile's values start inside the run (clamped: corrupt offsets must
                // not lead the decode warps outside the stage)
                if (prole == 0 && (lane < kKT || (lane >= 8 && lane < 8 + kKT))) {
                    const uint32_t rel = (uint32_t)(lane < 8 ? r0 - a0 : r1 - a1) * 2;
                    const uint32_t idx = lane < 8 ? (uint32_t)lane : (uint32_t)(kKT + lane - 8);
                    asm volatile("st.shared.b32 [%0], %1;" ::"r"(sbase + off_rel + 4 * idx),
                                 "r"(min(rel, (uint32_t)kKT * vmax))
                                 : "memory");
                }
                __syncwarp();
                // one elected lane issues this warp's copies with warp-uniform operands
                if (elect_one()) {
                    if (prole == 0) {
                        const uint32_t tx =
                            (uint32_t)nv * kBTile + n0 + n1 + (chunk1 ? 2u : 1u) * (uint32_t)nv * (512u + 16u);
                        mbar_expect_tx(full, tx);
                        if (n0) bulk_g2s(sbase + off_v0, p.vals + a0, n0, full);
                        if (n1) bulk_g2s(sbase + off_v1, p.vals + a1, n1, full);
                    } else if (prole == 1) {
                        bulk_g2s(sbase + off_bm0, p.bitmap + g0 * 64, (uint32_t)nv * 512u, full);
                        bulk_g2s(sbase + off_mt0, p.mtile + g0 * 4, (uint32_t)nv * 16u, full);
                        if (chunk1) {
                            bulk_g2s(sbase + off_bm1, p.bitmap + (g0 + p.kt_total) * 64, (uint32_t)nv * 512u, full);
                            bulk_g2s(sbase + off_mt1, p.mtile + (g0 + p.kt_total) * 4, (uint32_t)nv * 16u, full);
                        }
                    } else {
                        for (int j = 0; j < nv; ++j)  // activation tile of k-tile j
                            tma_load_2d(sbase + (uint32_t)j * kBTile, &tmap_b, (cw.k0 + ckk0 + j) * 64, cw.nt * NPAD,
                                        full);
                    }
                }
                __syncwarp();
                if (++slot == (uint32_t)S) {
                    slot = 0;
                    ++round;
                }
            }
        } else if (warp == kMmaWarp) {
            // ================================================================= MMA issuer
            // The whole warp runs the loop with warp-uniform state (so addresses and descriptors stay
            // in uniform registers); one elected lane issues.  A stage's A operands are ready when all
            // decode warps have arrived on aready; they only arrive after the stage's full barrier
            // completed, so the activation tiles have landed too.  One commit per stage arrives on
            // its empty barrier: the producer may refill the stage and the decode warps may
            // overwrite the TMEM A buffers.
            constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(NPAD >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
            uint32_t idx = 0, slot = 0, abuf = 0, apar = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < p.num_items && ok; item += gridDim.x) {
                const Item w = decode_item(p, item);
                if (w.nk == 0) continue;
                const uint32_t accbuf = idx % kAccBufs;
                if (idx >= (uint32_t)kAccBufs)
                    ok = __all_sync(0xffffffffu,
                                    mbar_wait_patient(bar_accempty + 8 * accbuf, ((idx / kAccBufs) - 1) & 1, abort_flag));
                const uint32_t d_tmem = tmem_base + accbuf * (kNAcc * NPAD);
                for (int kk0 = 0; kk0 < w.nk && ok; kk0 += kKT) {
                    const int nv = min(kKT, w.nk - kk0);
                    ok = __all_sync(0xffffffffu, mbar_wait_patient(bar_aready + 8 * abuf, apar, abort_flag));
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sbase = stage0 + slot * stage_bytes;
                    if (elect_one()) {
                        for (int sub = 0; sub < nv; ++sub) {
                            const uint64_t bdesc = make_b_desc(sbase + (uint32_t)sub * kBTile);
                            const uint32_t a_tmem = tmem_a0 + (abuf * kKT + (uint32_t)sub) * 32;
#pragma unroll
                            for (int s = 0; s < 4; ++s)
                                tc_mma_ts(d_tmem + (s % kNAcc) * NPAD, a_tmem + 8 * s, bdesc + 2 * s, idesc,
                                          (kk0 > 0 || sub > 0 || s >= kNAcc) ? 1u : 0u);
                        }
                        tc_commit(bar_empty + 8 * slot);
                    }
                    __syncwarp();
                    if (++slot == (uint32_t)S) slot = 0;
                    if (++abuf == n_abuf) {
                        abuf = 0;
                        apar ^= 1u;
                    }
                }
                if (ok && elect_one()) tc_commit(bar_accfull + 8 * accbuf);
                __syncwarp();
                ++idx;
            }
        }
    } else if (warp < kDecodeWarp0) {
        reg_dealloc<kRegsEpilogue>();
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
            const uint32_t accbuf = idx % kAccBufs;
            ok = mbar_wait_relaxed(bar_accfull + 8 * accbuf, (idx / kAccBufs) & 1, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const uint32_t t_acc = tmem_base + ((uint32_t)(quad * 32) << 16) + accbuf * (kNAcc * NPAD);
#pragma unroll
            for (int c = 0; c < NPAD / 16; ++c) {
                uint32_t r[16];
                tc_ld_32x32b_x16(t_acc + 16 * c, r);
#pragma unroll
                for (int j = 1; j < kNAcc; ++j) {
                    uint32_t r2[16];
                    tc_ld_32x32b_x16(t_acc + j * NPAD + 16 * c, r2);
                    tc_wait_ld();
#pragma unroll
                    for (int n = 0; n < 16; ++n) r[n] = __float_as_uint(__uint_as_float(r[n]) + __uint_as_float(r2[n]));
                }
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
        // Decode group g (4 warps, one per TMEM lane quadrant) belongs to set g / kKT and expands k-tile
        // g % kKT of every stage of its set.  Every warp works alone, one thread per weight row: a row
        // crosses 8 bitmap tiles per k-tile; the thread reads their bitmaps, keeps a running sum of the
        // tile sizes inside its 16-row median tile (the other tile of each pair is counted by the lane
        // 8 away), finds its row's values with popcounts and expands them.
        reg_alloc<kRegsDecode>();
        const int dw = warp - kDecodeWarp0;
        const int group = dw >> 2;
        const int set = group / kKT, sub = group % kKT;
        const int quad = warp & 3;             // TMEM lane quadrant this warp may access
        const int row = quad * 32 + lane;      // weight row inside the 128-row block
        const uint32_t lut = smem_u32(lut_tab);
        const int chunk = row >> 6, rr = row & 63;   // 64-row global-tile row of the block, row inside it
        const int r_in_tile = rr & 7;
        const uint32_t my_v = chunk ? off_v1 : off_v0;
        const uint32_t my_mt = (chunk ? off_mt1 : off_mt0) + (uint32_t)sub * 16 + 4 * (uint32_t)(rr >> 4);
        const uint32_t my_rel = off_rel + 4 * (uint32_t)(chunk * kKT + sub);
        // bitmap of the first of the row's 8 tiles (they are 16 bytes apart): median tile rr >> 4, row half
        // (rr >> 3) & 1 of the 2 x 2 tile order
        const uint32_t sp_bm = (chunk ? off_bm1 : off_bm0) + (uint32_t)sub * 512 +
                               8 * (uint32_t)(16 * (rr >> 4) + ((rr >> 3) & 1));
        const uint32_t below_lo = r_in_tile < 4 ? (1u << (8 * r_in_tile)) - 1u : 0xffffffffu;
        const uint32_t below_hi = r_in_tile <= 4 ? 0u : (1u << (8 * (r_in_tile - 4))) - 1u;
        const uint32_t rsel = 0x4440u | (uint32_t)r_in_tile;
        const uint32_t second = ((rr >> 3) & 1) ? 0xffffffffu : 0u;

        uint32_t slot = 0, round = 0, mine = 0;
        int turn = 0;      // stage counter modulo kSets: this warp's set works when turn == set
        uint32_t abuf = (uint32_t)set;  // TMEM A buffer (in stages) of this set's next stage
        uint32_t bar_old = 0, par_old = 0, bar_new = 0, par_new = 0;  // empty barriers of this set's last two stages
        bool ok = true;
        for (int item = blockIdx.x; item < p.num_items && ok; item += gridDim.x) {
            const Item w = decode_item(p, item);
            const bool chunk1 = (2 * w.y + 1) < p.gm_total;
            const bool valid = (chunk == 0) || chunk1;
            for (int kk0 = 0; kk0 < w.nk; kk0 += kKT) {
                if (turn != set) {  // another set's stage: only follow the ring
                    if (++turn == kSets) turn = 0;
                    if (++slot == (uint32_t)S) {
                        slot = 0;
                        ++round;
                    }
                    continue;
                }
                const bool active = sub < w.nk - kk0;  // this group's k-tile exists in the stage
                ok = mbar_wait(bar_full + 8 * slot, round & 1, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                const uint32_t st = stage0 + slot * stage_bytes;
                uint32_t a[32];
                if (active) {
                    // ---- thread <-> weight row.  Per batch of row segments: the bitmaps of their tiles, each
                    // tile's start (running sum over the median tile), the row's start, the expansion, and
                    // the store of the finished registers to tensor memory.
                    bool fr = true;  // the TMEM A buffer may be rewritten once the MMAs that read it have completed
                    if (reuse_wait) {
                        if (two_deep) {
                            if (mine >= 2) fr = mbar_wait(bar_old, par_old, abort_flag);
                        } else if (mine >= 1) {
                            fr = mbar_wait(bar_new, par_new, abort_flag);
                        }
                    }
                    fr = __all_sync(0xffffffffu, fr);
                    const uint32_t ta = tmem_a0 + (abuf * kKT + (uint32_t)sub) * 32 + ((uint32_t)(quad * 32) << 16);
                    if (fr) tc_fence_after();
                    uint32_t run = st + my_v;
                    if (valid) {
                        const uint32_t mt = lds32(st + my_mt), rel = lds32(st + my_rel);
                        // clamped so that corrupt offsets can never point outside the stage
                        run += min(rel + 2 * mt, (uint32_t)kKT * vmax);
                    }
#pragma unroll
                    for (int q0 = 0; q0 < 8; q0 += kUnitBatch) {
                        uint32_t blo[kUnitBatch], bhi[kUnitBatch];
                        UnitLoads u[kUnitBatch];
#pragma unroll
                        for (int q = 0; q < kUnitBatch; ++q) {
                            blo[q] = bhi[q] = 0u;
                            if (valid) lds64(st + sp_bm + 16 * (q0 + q), blo[q], bhi[q]);
                        }
#pragma unroll
                        for (int q = 0; q < kUnitBatch; ++q)
                            unit_load_sp(blo[q], bhi[q], run, below_lo, below_hi, rsel, second, lut, u[q]);
#pragma unroll
                        for (int q = 0; q < kUnitBatch; ++q) unit_expand(u[q], a + 4 * (q0 + q));
                        if (fr) {
                            if (kUnitBatch == 4) {
                                tc_st_32x32b_x16(ta + 4 * q0, a + 4 * q0);
                            } else if (kUnitBatch == 2) {
                                tc_st_32x32b_x8(ta + 4 * q0, a + 4 * q0);
                            } else if (q0 & 1) {
                                tc_st_32x32b_x8(ta + 4 * (q0 - 1), a + 4 * (q0 - 1));
                            }
                        }
                    }
                    if (fr) {
                        tc_wait_st();
                        tc_fence_before();
                    }
                    ok = fr;
                } else {
                    // A group without a k-tile in this stage still arrives on aready.  Arrivals are
                    // not tagged with a phase, so it must not run ahead of the stage two back either:
                    // an early arrival would complete that stage's aready phase in place of a warp
                    // that is still decoding.
                    if (reuse_wait) {
                        if (two_deep) {
                            if (mine >= 2) ok = mbar_wait(bar_old, par_old, abort_flag);
                        } else if (mine >= 1) {
                            ok = mbar_wait(bar_new, par_new, abort_flag);
                        }
                    }
                    ok = __all_sync(0xffffffffu, ok);
                }
                __syncwarp();
                if (lane == 0 && ok) {
                    mbar_arrive(bar_aready + 8 * abuf);
                    mbar_arrive(bar_empty + 8 * slot);
                }
                bar_old = bar_new;
                par_old = par_new;
                bar_new = bar_empty + 8 * slot;
                par_new = round & 1;
                ++mine;
                abuf += kSets;
                if (abuf >= n_abuf) abuf -= n_abuf;
                if (++turn == kSets) turn = 0;
                if (++slot == (uint32_t)S) {
                    slot = 0;
                    ++round;
                }
                if (!ok) break;
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
    const int dyn_smem = di.max_smem - 1024;  // the kernel also has a small static table
    p.smem_bytes = (uint32_t)dyn_smem;

    static bool attr_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(spmm_bitmap_tcgen05_kernel<NPAD>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, dyn_smem);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    const int grid = p.num_items < di.sms ? p.num_items : di.sms;
    spmm_bitmap_tcgen05_kernel<NPAD><<<grid, kThreads, dyn_smem, s>>>(p, tmap);
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
    // Activation tile width: the smallest of 16/32/64 that holds N; wider N is cut into tiles of 64
    // columns (each re-reads and re-expands the weight).
    if (a.N <= 16) return launch_t<16>(s, a, di, status);
    if (a.N <= 32) return launch_t<32>(s, a, di, status);
    return launch_t<64>(s, a, di, status);
}

}  // namespace spb
