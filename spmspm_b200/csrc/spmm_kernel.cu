// SpMM over the bitmap-v3 format for sm_100a:  C[M x N] = A_sparse[M x K] * B[K x N].
//
// Replaces the reference's SpMM_Kernel_bitmap_v3 (reference csrc/SpMM_Kernel.cuh:18-199,
// an mma.sync + cp.async kernel) with a persistent, warp-specialised kernel:
//
//   producer warps  three warps stream the compressed weight (packed values; bitmaps and median
//                   offsets; activation tiles) of two vertically adjacent 64x64 global tiles with
//                   1-D bulk copies and the activation tile with a 2-D TMA load into a ring of
//                   shared-memory stages of four k-tiles each (two for activation tiles of 128 and
//                   256 columns), completion on mbarriers;
//   decode warps    (6 groups of 4 warps for activation tiles up to 64 columns, 4 groups for the
//                   wide tiles; the k-tiles are dealt to the groups in turn, one thread per weight
//                   row) expand the bitmaps: per k-tile a warp first works out where the values of
//                   its 32 tiles start (one tile per lane: population count of the bitmap, prefix
//                   sum over the 16 tiles of a median tile by shuffles), then every thread, for
//                   each of the 8 tiles its row crosses, finds its row's values with population
//                   counts, expands them with byte permutes driven by a selector table and writes
//                   the dense 128 x 64 fp16 tile straight into tensor memory (tcgen05.st) as the
//                   MMA's A operand.  Every k-tile's A operand block has its own ready/free
//                   barriers, so a group only ever waits for the tensor core's work on its own
//                   k-tiles;
//   MMA warp        one thread issues tcgen05.mma (M=128, N=16..256, K=16, fp16 in,
//                   fp32 accumulate in TMEM), A from TMEM, B from the swizzled smem tile;
//   epilogue warps  read the accumulator (tcgen05.ld), round to fp16 and store C or the
//                   split-K partial, column-major as the reference does
//                   (reference csrc/SpMM_Kernel.cuh:192-198); under the static schedule the last
//                   CTA of a row block also sums the split-K partials (the reference's
//                   SplitK_Reduction, csrc/Reduction_Kernel.cuh:24-44); the exchange variants add
//                   the element-wise tail of a linear layer and the stores to other GPUs' buffers.
//
// Work is scheduled in one of two ways (see Walk).  Static: a work item is (row block of 128 rows,
// split-K range), the ranges cut exactly like the reference's (reference csrc/SpMM_Kernel.cuh:35-43),
// items dealt to the CTAs round-robin.  Balanced: all k-tiles of all items are laid end to end and
// every CTA takes an equal share; a range that is cut between CTAs is summed in fp32 through scratch
// memory, by whichever of its CTAs finishes last, without anybody waiting.  Every wait in the kernel is
// bounded: when one runs out the CTA records it in the device status word and leaves without
// touching tensor memory again.
#include "common.cuh"
#include "epilogue.cuh"
#include <cuda.h>
#include <cuda_fp16.h>
#include <cstdio>
#include <atomic>
#include <mutex>

#ifndef SPB_PROF
#define SPB_PROF 0  // development only: per-phase clock sums of one decode warp, the MMA warp and a producer warp
#endif
#ifndef SPB_UNIT
#define SPB_UNIT 1  // k-tiles a decode group expands per turn (2 measured 3 % slower: the decode warps are bound by
                    // instruction issue, so paying the chain of waits once per two k-tiles buys nothing)
#endif
namespace spb {
#if SPB_PROF
__device__ unsigned long long g_prof[32];
#define PROF_T(i) do { const uint32_t t_ = clock(); pacc[i] += t_ - plast; plast = t_; } while (0)
// time line of a launch: earliest and latest %globaltimer (ns) over all CTAs at event i, in g_prof[32 + 2 * i], [33 + 2 * i]
__device__ unsigned long long g_tl[32];
#define PROF_EV(i) do { unsigned long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); \
                        atomicMin(&g_tl[2 * (i)], t_); atomicMax(&g_tl[2 * (i) + 1], t_); } while (0)
#else
#define PROF_T(i) do {} while (0)
#define PROF_EV(i) do {} while (0)
#endif
namespace {

// Warp roles, by warpgroup (4 warps) so that each role can resize its register file share:
//   warpgroup 0: warp 1 MMA issuer, warps 0, 2, 3 producers (each issues a share of the copies)
//   warpgroup 1: epilogue (one warp per TMEM lane quadrant)
//   warpgroup 2..: decode groups (one warp per quadrant each)
// A pipeline stage holds kKT consecutive k-tiles of one 128-row block, one for each of the four decode
// groups.  (Stages of one or two k-tiles mean more stages in the shared-memory ring and more copies per
// byte; they measured 1.7x and 1.15x slower: a producer warp spends about 2300 cycles per stage whatever the stage
// holds, so two-k-tile stages cap the kernel near 0.6 us per k-tile; the 32-column tile ran 108 instead of 83 us with
// them.)  Activation tiles wider than 64 columns leave room for two k-tiles per stage only (stage_kt).
constexpr int kKT = 4;
__host__ __device__ constexpr int stage_kt(int npad) { return npad > 64 ? 2 : 4; }
// Decode groups.  The k-tiles of the CTA's whole sequence are dealt to the groups in turn (k-tile t goes to
// group t % groups), so a stage gives a group at most one k-tile as long as there are at least kKT groups.
// Six groups at 64 registers per thread (nobody resizes) for activation tiles up to 64 columns, four at 96 registers
// for the wide tiles (measured: six groups are 2-6 % faster up to 64 columns, 19 % slower at 128).
#ifdef SPB_GROUPS
__host__ __device__ constexpr int decode_groups(int) { return SPB_GROUPS; }
#else
__host__ __device__ constexpr int decode_groups(int npad) { return npad <= 64 ? 6 : 4; }
#endif
// A operand blocks in tensor memory (32 columns = one k-tile each), used in turn: k-tile t uses block t % kABlocks.
// Eight blocks, two per decode group: a group can start its next k-tile while the tensor core still reads its last
// one.  A power of two, so that block and barrier phase of the t-th k-tile of the CTA's sequence are t % 8 and
// (t / 8) % 2 with no bookkeeping (twelve blocks with per-block phase bits measured 2 % slower).
constexpr int kABlocks = 8;
constexpr int kMmaWarp = 1;
constexpr int kEpilogueWarp0 = 4;
constexpr int kDecodeWarp0 = 8;
__host__ __device__ constexpr int threads_for(int npad) { return 32 * (kDecodeWarp0 + 4 * decode_groups(npad)); }
// Registers per thread after the roles have resized.  A CTA owns the registers it was launched with
// (65536 / threads rounded down to a multiple of 8 per thread, what ptxas reports for the kernel), and a warp
// that grows can only take what other warps of the CTA have given back: if the sizes below added up to more
// than the launch allocation, the last warps to grow would block for ever (checked at compile time in the kernel).
// With six groups the launch allocation (64 registers) is what the decode loop needs: nobody resizes.
constexpr int kRegsControl = 40, kRegsEpilogue = 56;
__host__ __device__ constexpr int regs_launch(int groups) { return 65536 / (32 * (kDecodeWarp0 + 4 * groups)) / 8 * 8; }
__host__ __device__ constexpr int regs_decode(int groups) { return groups == 4 ? 96 : groups == 5 ? 80 : 64; }
constexpr int kMaxPeers = 8;
constexpr int kMaxStages = 24;
// Shared-memory header: barriers and flags (1 KB), one tile table per decode warp, then the selector table.
//   tile table   32 entries (the warp's tiles of the k-tile it is expanding) of 16 bytes:
//                {bitmap rows 0-3, address of the first value of rows 0-3, bitmap rows 4-7, address of the first value of rows 4-7}
//   selector table  indexed by a row's 8-bit mask: {low-nibble entry, high-nibble entry} (see lut_low_entry), 16 copies
//                interleaved so that the 16 lanes of a half warp always read 16 different 8-byte slots
constexpr int kUnit = SPB_UNIT;
constexpr int kTileTabBytes = 512 * kUnit;
constexpr int kLutBytes = 256 * 16 * 8;
__host__ __device__ constexpr int header_bytes(int groups) { return 1024 + kTileTabBytes * 4 * groups + kLutBytes; }
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
    // balanced schedule: fp32 sums of partial runs, 2 slots of 128 x NPAD per CTA, and one arrival counter per item
    float* partials;
    int* counters;
    int balanced, units;
    int weights_ahead;  // 1: the weight-streaming warps do not wait for the stream's preceding kernel
    // element-wise tail of a linear layer (exchange variants only), applied where final rows are written:
    // bias by weight row, residual at the position of the row in the first destination buffer
    const uint16_t* ep_bias;
    const uint16_t* ep_res;
    int ep_act;
    int ep_on;
    // Output: normally one buffer [N][M] (or the split-K partials).  For the fused all-gather the rows of this
    // launch go to rows row0.. of n_out buffers [N][ld_out], this GPU's and its peers' (peer memory mapped
    // into this process), and when the last CTA has finished, the launch's sequence number is written to
    // entry flag_index of every peer's flag array.
    uint16_t* outs[kMaxPeers];
    uint32_t* flags[kMaxPeers];
    int n_out, ld_out, row0, n_flags, flag_index;
    // Split-K under the static schedule with the reduction fused in: the fp16 partials go to outs[0] as usual; the
    // CTAs of a row block count themselves on red_counters[activation tile * row_blocks + row block], and the
    // one that completes the count sums the partials (fp32, in range order: the arithmetic of the separate
    // reduction kernel) into rows red_row0.. of n_red buffers [N][red_ld].  red_counters == null: no fused reduction.
    uint16_t* red_outs[kMaxPeers];
    int* red_counters;
    int n_red, red_ld, red_row0;
    uint32_t* sequence;  // this GPU's count of fused launches on these buffers
    int* done;           // CTAs of the launch that have finished
    // The activations of this launch are the result of an earlier exchange: its flag array on this GPU
    // ([wait_n] ranks' sequence numbers, then this GPU's own launch count, then the number of exchanges
    // consumed so far).  The warp that loads the activation tiles polls it, everything else starts at once.
    uint32_t* wait_flags;
    int wait_n;
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

// Named barrier 1: the 128 threads of the epilogue warps.
__device__ __forceinline__ void bar_sync_epilogue()
{
    asm volatile("bar.sync 1, 128;" ::: "memory");
}
__device__ __forceinline__ bool bar_and_epilogue(bool pred)
{
    uint32_t r;
    asm volatile(
        "{ .reg .pred p, q; setp.ne.u32 p, %1, 0; bar.red.and.pred q, 1, 128, p; selp.u32 %0, 1, 0, q; }"
        : "=r"(r)
        : "r"((uint32_t)pred)
        : "memory");
    return r != 0;
}
static_assert((kABlocks & (kABlocks - 1)) == 0, "block and phase of a k-tile come from its sequence number by mask and shift");
// A work item is a run of k-tiles of one 128-row block (and one activation tile column): a whole split-K
// range, or, with the balanced schedule, a piece of one.
__device__ __forceinline__ int ld_acquire_gpu(const int* p)
{
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
struct Item {
    int nt, y, batch, k0, nk;
    int id;        // index of the (activation tile, row block, split-K range) this run belongs to
    bool partial;  // the run does not cover its whole range: its sum goes through the fp32 scratch
};
// Start of CTA c's share of the units (k-tiles of all row blocks, in item order) under the balanced schedule.
// The host only chooses this schedule when (units + 1) * gridDim.x fits into 31 bits.
__device__ __forceinline__ int share_begin(const KernelParams& p, int c)
{
    return (int)(((uint32_t)c * (uint32_t)p.units) / gridDim.x);
}
// The CTA whose share holds unit u: the largest c with share_begin(c) <= u.
__device__ __forceinline__ int share_owner(const KernelParams& p, int u)
{
    return (int)((((uint32_t)u + 1u) * gridDim.x - 1u) / (uint32_t)p.units);
}
// Walks the work items of this CTA.  Static schedule: items blockIdx.x, + gridDim.x, ... with the
// split-K ranges cut exactly like the reference's (reference csrc/SpMM_Kernel.cuh:35-43).  Balanced
// schedule: all k-tiles of all ranges are laid end to end and every CTA takes an equal share of them; a
// share is cut into runs at the range boundaries.  The runs that cover only part of their range (at most
// the first and the last of the share) come first, the shorter one before the longer one, then the
// whole ranges: the exchange of partial sums then happens while the CTA still has work, and the last
// run of a CTA is long enough to hide it.
struct Walk {
    int begin, end;      // this CTA's share (balanced) / next item and item count (static)
    int lo_end, hi_beg;  // end of the partial run at the low end, start of the one at the high end
    int pos, phase;      // position inside the current phase (-1: not entered), phase 0..2
    int order;           // which part each phase walks: 2 bits per phase, 0 low run, 1 high run, 2 middle, 3 nothing
    __device__ __forceinline__ void range_of(const KernelParams& p, int u, int& r0, int& r1) const
    {
        const int row = u / p.kt_total, k = u - row * p.kt_total;
        const int ks = (k / p.avg_kt) * p.avg_kt;
        int ke = ks + p.avg_kt;
        if (ke > p.kt_total) ke = p.kt_total;
        r0 = row * p.kt_total + ks;
        r1 = row * p.kt_total + ke;
    }
    template <bool kBalanced>
    __device__ __forceinline__ void init(const KernelParams& p)
    {
        pos = -1;
        phase = 0;
        if (!kBalanced) {
            begin = blockIdx.x;
            end = p.num_items;
            lo_end = hi_beg = order = 0;
            return;
        }
        begin = share_begin(p, blockIdx.x);
        end = share_begin(p, blockIdx.x + 1);
        lo_end = begin;
        hi_beg = end;
        order = 0x3e;  // middle, nothing, nothing
        if (begin >= end) return;
        int r0, r1;
        range_of(p, begin, r0, r1);
        const bool lo = r0 != begin || r1 > end;  // the first range of the share is not whole
        if (lo) lo_end = r1 < end ? r1 : end;
        bool hi = false;
        if (lo_end < end) {
            range_of(p, end - 1, r0, r1);
            hi = r1 > end;
            if (hi) hi_beg = r0;  // >= lo_end: both are range boundaries
        }
        if (lo && hi)
            order = (lo_end - begin <= end - hi_beg) ? (0 | 1 << 2 | 2 << 4) : (1 | 0 << 2 | 2 << 4);
        else if (lo)
            order = 0 | 2 << 2 | 3 << 4;
        else if (hi)
            order = 1 | 2 << 2 | 3 << 4;
    }
    template <bool kBalanced>
    __device__ __forceinline__ bool next(const KernelParams& p, Item& it)
    {
        if (!kBalanced) {
            if (begin >= end) return false;
            const int per_nt = p.row_blocks * p.split_k;
            it.nt = begin / per_nt;
            const int rem = begin - it.nt * per_nt;
            it.y = rem / p.split_k;
            it.batch = rem - it.y * p.split_k;
            it.k0 = it.batch * p.avg_kt;  // reference csrc/SpMM_Kernel.cuh:36-43
            int k1 = it.k0 + p.avg_kt;
            if (k1 > p.kt_total) k1 = p.kt_total;
            it.nk = k1 > it.k0 ? k1 - it.k0 : 0;
            it.id = begin;
            it.partial = false;
            begin += gridDim.x;
            return true;
        }
        for (;;) {
            if (phase > 2) return false;
            const int part = (order >> (2 * phase)) & 3;
            const int a = part == 0 ? begin : part == 1 ? hi_beg : lo_end;
            const int b = part == 0 ? lo_end : part == 1 ? end : part == 2 ? hi_beg : a;
            if (pos < 0) pos = a;
            if (pos >= b) {
                ++phase;
                pos = -1;
                continue;
            }
            const int row = pos / p.kt_total, k = pos - row * p.kt_total;
            it.nt = row / p.row_blocks;
            it.y = row - it.nt * p.row_blocks;
            it.batch = k / p.avg_kt;
            const int ks = it.batch * p.avg_kt;
            int ke = ks + p.avg_kt;
            if (ke > p.kt_total) ke = p.kt_total;
            int e = k + (b - pos);
            if (e > ke) e = ke;
            it.k0 = k;
            it.nk = e - k;
            it.id = row * p.split_k + it.batch;
            it.partial = k != ks || e != ke;
            pos += it.nk;
            return true;
        }
    }
};

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
// Low-nibble entry  sel(pos 0,1) | sel(pos 2,3) << 16
// High-nibble entry sel(pos 6,7) | sel(pos 4,5) << 16
// The 2-value window of positions 2,3 starts (number of values at positions 0,1) values into the 4-value
// window, the one of positions 4,5 ends (number of values at positions 6,7) values before its end; the
// permute selectors that cut them out are computed from those counts.  The tables are kept to 32-bit
// entries because the decode warps are bound by shared-memory wavefronts, not by arithmetic: a 4-byte load
// from a 64-byte table is one conflict-free wavefront, an 8-byte one at least two.
__host__ __device__ constexpr uint32_t pair_sel_bottom(uint32_t lo, uint32_t hi)
{
    // window = {next value, the one after}; zero register in bytes 4..7
    const uint32_t p_lo = lo ? 0x10u : 0x54u;
    const uint32_t p_hi = hi ? (lo ? 0x32u : 0x10u) : 0x54u;
    return p_lo | (p_hi << 8);
}
__host__ __device__ constexpr uint32_t pair_sel_top(uint32_t lo, uint32_t hi)
{
    // window = {second to last value, last value}
    const uint32_t p_hi = hi ? 0x32u : 0x54u;
    const uint32_t p_lo = lo ? (hi ? 0x10u : 0x32u) : 0x54u;
    return p_lo | (p_hi << 8);
}
__host__ __device__ constexpr uint32_t lut_low_entry(uint32_t n)
{
    const uint32_t b0 = n & 1, b1 = (n >> 1) & 1, b2 = (n >> 2) & 1, b3 = (n >> 3) & 1;
    return pair_sel_bottom(b0, b1) | (pair_sel_bottom(b2, b3) << 16);
}
__host__ __device__ constexpr uint32_t lut_high_entry(uint32_t n)
{
    const uint32_t b4 = n & 1, b5 = (n >> 1) & 1, b6 = (n >> 2) & 1, b7 = (n >> 3) & 1;
    return pair_sel_top(b6, b7) | (pair_sel_top(b4, b5) << 16);
}

// The selector table as it lies in shared memory: entry (mask g, copy c) at 8 * (16 * g + c) bytes, c = 0..15, so
// that the 16 lanes of a half warp, each reading its own copy, always touch 16 different 8-byte bank pairs.
// Built at compile time; every CTA fetches it with one bulk copy.
struct SelectorTable {
    uint32_t v[2 * 16 * 256];
    constexpr SelectorTable() : v{}
    {
        for (uint32_t g = 0; g < 256; ++g)
            for (uint32_t c = 0; c < 16; ++c) {
                v[2 * (16 * g + c)] = lut_low_entry(g & 15u);
                v[2 * (16 * g + c) + 1] = lut_high_entry(g >> 4);
            }
    }
};
static_assert(sizeof(SelectorTable) == kLutBytes, "selector table size");
__device__ __align__(128) const SelectorTable g_selector_table = SelectorTable();

// Expansion of one 8-element row segment (one row of one 8x8 tile) into 4 registers of packed fp16,
// split into a load half and a compute half so that the loads of several segments can be in flight
// together.  lut: shared address of the selector tables.
struct UnitLoads {
    uint32_t x0, x1, x2, y0, y1, y2, l, h, c01, c67, sb, st;
};
__device__ __forceinline__ void lds32x3_before(uint32_t addr, uint32_t& a, uint32_t& b, uint32_t& c)
{
    asm volatile("ld.shared.b32 %0, [%3+-8];\n\tld.shared.b32 %1, [%3+-4];\n\tld.shared.b32 %2, [%3];"
                 : "=&r"(a), "=&r"(b), "=&r"(c)
                 : "r"(addr));
}
// Load half for one row segment, from a tile table entry: w = bitmap of the tile's rows 0-3 or 4-7 (the half this
// thread's row is in), half = shared address of the first value of that half.
//   below   thread constant: bitmap bits of the rows of the half above this thread's row
//   rsel    permute selector moving this row's mask byte to byte 0 of a zero word
//   lutlane shared address of this lane's copy of the selector table
__device__ __forceinline__ void unit_load3(uint32_t w, uint32_t half, uint32_t below, uint32_t rsel, uint32_t lutlane,
                                           UnitLoads& u)
{
    const uint32_t w0 = half + 2u * __popc(w & below);
    const uint32_t g = prmt(w, 0u, rsel);                  // row mask, zero-extended
    const uint32_t wt = w0 + 2u * __popc(g);               // address just past the row's last value
    lds32x3(w0 & ~3u, u.x0, u.x1, u.x2);
    lds32x3_before(wt & ~3u, u.y0, u.y1, u.y2);            // window of the 4 values before wt
    lds64(lutlane + g * 128u, u.l, u.h);
    u.c01 = __popc(g & 3u);                                // values at positions 0,1
    u.c67 = __popc(g & 0xc0u);                             // values at positions 6,7
    u.sb = w0 << 3;
    u.st = wt << 3;
}
__device__ __forceinline__ void unit_expand(const UnitLoads& u, uint32_t* o)
{
    const uint32_t b0 = __funnelshift_r(u.x0, u.x1, u.sb), b1 = __funnelshift_r(u.x1, u.x2, u.sb);
    const uint32_t t0 = __funnelshift_r(u.y0, u.y1, u.st), t1 = __funnelshift_r(u.y1, u.y2, u.st);
    const uint32_t win_lo = 0x3210u + 0x2222u * u.c01, win_hi = 0x7654u - 0x2222u * u.c67;
    o[0] = prmt(b0, 0u, u.l);
    o[1] = prmt(prmt(b0, b1, win_lo), 0u, u.l >> 16);
    o[2] = prmt(prmt(t0, t1, win_hi), 0u, u.h >> 16);
    o[3] = prmt(t1, 0u, u.h);
}

// kExchange: the variant used by the fused all-gather (several output buffers, completion flags, activations
// that come out of an earlier exchange).  The plain variant carries none of that code: the decode loop is
// sensitive to the size of the kernel around it (the same source with the exchange code compiled in ran 5 %
// slower on calls that never used it).  kBalanced: the work schedule (see Walk); the static variant carries
// no code for the exchange of partial sums.
template <int NPAD, bool kExchange, bool kBalanced>
__global__ void __launch_bounds__(threads_for(NPAD), 1)
spmm_bitmap_tcgen05_kernel(const KernelParams p, const __grid_constant__ CUtensorMap tmap_b)
{
    // this width's k-tiles per stage and A operand blocks (they hide the file-scope defaults of the same names)
    constexpr int kKT = stage_kt(NPAD);
    constexpr int kDecodeGroups = decode_groups(NPAD);
    constexpr int kThreads = threads_for(NPAD);
    constexpr int kRegsLaunch = regs_launch(kDecodeGroups), kRegsDecode = regs_decode(kDecodeGroups);
    constexpr bool kResize = kRegsDecode > kRegsLaunch;
    constexpr int kHeaderBytes = header_bytes(kDecodeGroups);
    static_assert(kDecodeGroups >= kKT && kDecodeGroups <= 6, "a stage must not give a group two k-tiles; 32 warps at most");
    static_assert(kRegsControl % 8 == 0 && kRegsEpilogue % 8 == 0 && kRegsDecode % 8 == 0, "register counts come in eights");
    static_assert(!kResize || 128 * kRegsControl + 128 * kRegsEpilogue + 128 * kDecodeGroups * kRegsDecode <= kRegsLaunch * kThreads,
                  "register budget: the resized roles must fit into the CTA's launch allocation");
    static_assert(!kResize || (kRegsControl <= kRegsLaunch && kRegsEpilogue <= kRegsLaunch && kRegsDecode >= kRegsLaunch),
                  "roles that shrink must not exceed, roles that grow must not undercut the launch allocation");
    static_assert(kHeaderBytes % 1024 == 0, "the stages behind the header must stay 1024-byte aligned");
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment for the swizzled activation tiles
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t pad = (uint32_t)(smem - smem_raw);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) PROF_EV(0);

    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
    const uint32_t bar_full = smem_u32(bars);                         // [kMaxStages]
    const uint32_t bar_empty = bar_full + 8 * kMaxStages;             // [kMaxStages]
    const uint32_t bar_aready = bar_empty + 8 * kMaxStages;           // [kABlocks]: A operand block written
    const uint32_t bar_afree = bar_aready + 8 * kABlocks;             // [kABlocks]: ... read by its MMAs
    const uint32_t bar_accfull = bar_afree + 8 * kABlocks;            // [2]
    const uint32_t bar_accempty = bar_accfull + 16;                   // [2]
    const uint32_t bar_lut = bar_accempty + 16;                       // the selector table has landed
    const uint32_t bar_b = bar_lut + 8;                               // [kMaxStages]: a stage's activation tiles have landed
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + 8 * (3 * kMaxStages + 2 * kABlocks + 5));
    static_assert(8 * (3 * kMaxStages + 2 * kABlocks + 5) + 16 <= 1024, "barriers and flags fit the first KB of the header");
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
    volatile int* finisher = reinterpret_cast<volatile int*>(tmem_holder + 2);
    const uint32_t stage0 = smem_u32(smem + kHeaderBytes);

    // Back-to-back tcgen05.mma into one accumulator are serialised by the tensor core, and at these
    // tiny N every instruction is pure latency, so the four k-steps of a k-tile go to different
    // accumulators (summed in the epilogue).
    constexpr int kNAcc = NPAD <= 16 ? 4 : NPAD <= 64 ? 2 : 1;
    constexpr int kAccBufs = NPAD <= 128 ? 2 : 1;
    constexpr uint32_t kAccCols = kAccBufs * kNAcc * NPAD;
    constexpr uint32_t kACols = kABlocks * 32;
    static_assert(kAccCols + kACols <= 512, "TMEM budget");
    constexpr uint32_t kTmemCols = 512;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kMaxStages; ++i) {
            mbar_init(bar_full + 8 * i, 1);
            // The activation tiles complete on a barrier of their own, which only the MMA warp waits on: the
            // decode warps can then expand the weights of a stage (all the full barrier covers) before the
            // activations exist, i.e. while the stream's preceding kernel is still running.
            mbar_init(bar_b + 8 * i, 1);
            mbar_init(bar_empty + 8 * i, 4 * kDecodeGroups + 1);  // every decode warp + the MMA commit
        }
        for (int i = 0; i < kABlocks; ++i) {
            mbar_init(bar_aready + 8 * i, 4);  // the four warps of the group that expanded the k-tile
            mbar_init(bar_afree + 8 * i, 1);   // the commit after the k-tile's MMAs
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar_accfull + 8 * i, 1);
            mbar_init(bar_accempty + 8 * i, 4);
        }
        mbar_init(bar_lut, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // the selector table is the library's own constant data: it can be fetched before the preceding kernel of
        // the stream has finished
        mbar_expect_tx(bar_lut, (uint32_t)kLutBytes);
        bulk_g2s(smem_u32(smem + 1024 + kTileTabBytes * 4 * kDecodeGroups), &g_selector_table, (uint32_t)kLutBytes, bar_lut);
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

    // Programmatic dependent launch.  Everything above touches only this CTA's shared and tensor memory, so it
    // overlaps the tail of the preceding kernel of the stream.  From here on the roles differ in what they may
    // do before that kernel has completed (griddepcontrol.wait):
    //   - the warps that stream the weight (packed values, bitmaps, offsets, max_nnz_intile) do not wait at all.
    //     The weight arrays are never written by this library's SpMM kernels, the only kernels that let a
    //     dependent start before they have finished; any other kernel ahead in the stream has completed all
    //     its thread blocks before this one starts.  So the ring of stages fills with weights while the
    //     slowest CTAs of the preceding SpMM are still in their epilogue;
    //   - the warp that loads the activation tiles, the epilogue warps (stores to C, to the partial sums, to
    //     the peers; the scratch of the schedules) and everything that reads the exchange flags wait first.
    // Kernels queued behind this one may be set up as soon as every CTA has passed this point.
    if (threadIdx.x == 0) PROF_EV(1);
    if (!p.weights_ahead) asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (threadIdx.x == 0) PROF_EV(2);

    // ---- carve-up ------------------------------------------------------------------------
    // A stage holds kKT consecutive k-tiles of one 128-row block: the activation tiles, then for each
    // of the two 64-row global-tile rows one contiguous run of packed values, the bitmaps and the
    // median offsets, then the start of every global tile's values inside its run.
    // The stage size depends on max_nnz_intile, a load from global memory that takes most of a microsecond.  The
    // load is issued here; what is derived from it (SPB_CARVE) is computed by each role only after the part of
    // its start-up that does not need it (walking to its first work item, fetching the first tile offsets), so
    // that nobody sits on the load.  (Issuing it, and an L2 prefetch of the first tile offsets, before the set-up
    // instead was measured: no difference.)
    int max_nnz_ld;
    asm volatile("ld.global.cg.s32 %0, [%1];" : "=r"(max_nnz_ld) : "l"(p.max_nnz));
    constexpr uint32_t kBTile = NPAD * 128;
#define SPB_CARVE()                                                                                                   \
    const int max_nnz = max_nnz_ld < 8 ? 8 : max_nnz_ld > 4096 ? 4096 : max_nnz_ld;                                   \
    const uint32_t vmax = ((uint32_t)max_nnz * 2 + 127) & ~127u; /* bytes per global tile, upper bound */             \
    const uint32_t off_v0 = kKT * kBTile, off_v1 = off_v0 + kKT * vmax;                                               \
    const uint32_t off_bm0 = off_v1 + kKT * vmax, off_bm1 = off_bm0 + kKT * 512;                                      \
    const uint32_t off_mt0 = off_bm1 + kKT * 512, off_mt1 = off_mt0 + kKT * 16;                                       \
    const uint32_t off_rel = off_mt1 + kKT * 16; /* [2][kKT] uint32: byte offset of a tile's values in its run */     \
    const uint32_t stage_bytes = (off_rel + 8 * kKT + 1023) & ~1023u;                                                 \
    const int S = min((int)((p.smem_bytes - pad - kHeaderBytes) / stage_bytes), kMaxStages);                          \
    (void)off_v0; (void)off_bm0; (void)off_bm1; (void)off_mt0; (void)off_mt1; (void)off_rel; (void)S; (void)vmax; (void)off_v1


    // The A operands of two stages live in TMEM (buffer = stage parity), one 32-column block per k-tile.
    // Every block has its own pair of barriers: aready (the group that expanded the k-tile has written it)
    // and afree (the MMAs that read it have completed), so that a decode group only ever waits for the
    // tensor core's work on its own k-tiles, never for another group.  Which phase of a block's barriers
    // comes next is kept as one bit per block (ph) by everybody who walks the stage sequence.
    if (warp < kEpilogueWarp0) {
        if constexpr (kResize) reg_dealloc<kRegsControl>();
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
            // position in the CTA's sequence of non-empty work items
            struct Cursor {
                Walk wk;
                Item w;
                int seq;
                bool valid;
            };
            auto advance = [&](Cursor& c) {
                do {
                    c.valid = c.wk.template next<kBalanced>(p, c.w);
                } while (c.valid && c.w.nk == 0);
                ++c.seq;
            };
            struct Batch {
                Cursor c;
                int base, v0, v1;
            };
            auto load_batch = [&](Batch& b) {
                b.v0 = 0;
                b.v1 = 0;
                if (prole != 0 || !b.c.valid) return;
                const size_t g = (size_t)(2 * b.c.w.y) * p.kt_total + b.c.w.k0 + b.base;
                if (lane <= b.c.w.nk - b.base) {
                    // (through L2 only: with the launch overlap above, a line of this SM's L1 could predate the
                    // kernel that wrote the array)
                    b.v0 = __ldcg(p.gtile + g + lane);
                    if ((2 * b.c.w.y + 1) < p.gm_total) b.v1 = __ldcg(p.gtile + g + p.kt_total + lane);
                }
            };
            auto batch_after = [&](const Batch& b) -> Batch {
                Batch n = b;
                if (b.base + kOffBatch < b.c.w.nk) {
                    n.base = b.base + kOffBatch;
                } else {
                    n.base = 0;
                    if (n.c.valid) advance(n.c);
                }
                return n;
            };
            uint32_t slot = 0, round = 0;
            bool ok = true;
            int kk0 = 0;
            Cursor st;
            st.wk.template init<kBalanced>(p);
            st.seq = -1;
            advance(st);
            Batch cur;
            cur.c = st;
            cur.base = 0;
            load_batch(cur);
            Batch nxt = batch_after(cur);
            load_batch(nxt);
            SPB_CARVE();
#if SPB_PROF
            uint32_t pacc[8] = {0, 0, 0, 0, 0, 0, 0, 0}, plast = clock();
#endif
            if (S < 1) {
                // A single stage does not fit (cannot happen with the launch configuration used by the host
                // code): nothing is copied, the other warps give up on their bounded waits.
                if (lane == 0 && prole == 0) atomicOr(p.status, (int)kStatusBadOffsets);
                *abort_flag = 1;
                ok = false;
            }
            if (prole == 2) asm volatile("griddepcontrol.wait;" ::: "memory");  // the activations come from the preceding kernel
            if (kExchange && ok && prole == 2 && p.wait_flags && st.valid) {
                // the activations come out of an exchange between the GPUs: bounded wait for every rank's rows
                bool here = lane >= p.wait_n;
                // the count of consumed exchanges and the first look at the flags travel together (the plain
                // load first: nothing may pass an acquire load that is still under way)
                const uint32_t want = *reinterpret_cast<volatile uint32_t*>(p.wait_flags + p.wait_n + 1) + 1u;
                uint32_t v = 0;
                if (!here) asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p.wait_flags + lane) : "memory");
                here = here || (int32_t)(v - want) >= 0;
                for (uint32_t i = 0; i < kSpinLimit && !here; ++i) {
                    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p.wait_flags + lane) : "memory");
                    here = (int32_t)(v - want) >= 0;
                    if (!here) {
                        if (*abort_flag) break;
                        __nanosleep(100);
                    }
                }
                if (!here) *abort_flag = 1;
                ok = __all_sync(0xffffffffu, here);
                // the rows were written through the generic proxy by other GPUs, the tile loads below read them
                // through the async proxy
                asm volatile("fence.proxy.async.global;" ::: "memory");
            }
            while (st.valid && ok) {
                const Item cw = st.w;
                const int ckk0 = kk0;
                if (cur.c.seq != st.seq || ckk0 - cur.base >= kOffBatch) {  // this stage starts the next batch
                    cur = nxt;
                    nxt = batch_after(cur);
                    load_batch(nxt);
                }
                const int bidx = ckk0 - cur.base;
                // advance to the next stage
                kk0 += kKT;
                if (kk0 >= cw.nk) {
                    kk0 = 0;
                    advance(st);
                }

                const bool chunk1 = (2 * cw.y + 1) < p.gm_total;
                const int nv = min(kKT, cw.nk - ckk0);
                const size_t g0 = (size_t)(2 * cw.y) * p.kt_total + cw.k0 + ckk0;
                const int a0 = __shfl_sync(0xffffffffu, cur.v0, bidx), e0 = __shfl_sync(0xffffffffu, cur.v0, bidx + nv);
                const int a1 = __shfl_sync(0xffffffffu, cur.v1, bidx), e1 = __shfl_sync(0xffffffffu, cur.v1, bidx + nv);
                const int r0 = __shfl_sync(0xffffffffu, cur.v0, bidx + (lane & 7));
                const int r1 = __shfl_sync(0xffffffffu, cur.v1, bidx + (lane & 7));
                PROF_T(0);
                if (round > 0) ok = mbar_wait_patient(bar_empty + 8 * slot, (round - 1) & 1, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                PROF_T(1);
                uint32_t n0 = (uint32_t)(e0 - a0) * 2, n1 = chunk1 ? (uint32_t)(e1 - a1) * 2 : 0u;
                // Offsets of a well-formed matrix are non-negative multiples of 8 values (every global tile is
                // padded to 16 bytes); anything else would make a bulk copy read from a wrong or misaligned address.
                const bool bad0 = a0 < 0 || e0 < a0 || ((a0 | e0) & 7) || n0 > (uint32_t)nv * vmax;
                const bool bad1 = chunk1 && (a1 < 0 || e1 < a1 || ((a1 | e1) & 7) || n1 > (uint32_t)nv * vmax);
                if (bad0 || bad1) {
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
                        const uint32_t tx = n0 + n1 + (chunk1 ? 2u : 1u) * (uint32_t)nv * (512u + 16u);
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
                        mbar_expect_tx(bar_b + 8 * slot, (uint32_t)nv * kBTile);
                        for (int j = 0; j < nv; ++j)  // activation tile of k-tile j
                            tma_load_2d(sbase + (uint32_t)j * kBTile, &tmap_b, (cw.k0 + ckk0 + j) * 64, cw.nt * NPAD,
                                        bar_b + 8 * slot);
                    }
                }
                __syncwarp();
                if (++slot == (uint32_t)S) {
                    slot = 0;
                    ++round;
                }
                PROF_T(2);
#if SPB_PROF
                if (pacc[7] == 0 && prole == 0 && lane == 0) PROF_EV(3);
                ++pacc[7];
#endif
            }
#if SPB_PROF
            if (lane == 0) {
                for (int i = 0; i < 3; ++i) atomicAdd(&g_prof[12 + 4 * prole + i], (unsigned long long)pacc[i]);
                atomicAdd(&g_prof[12 + 4 * prole + 3], (unsigned long long)pacc[7]);
            }
#endif
        } else if (warp == kMmaWarp) {
            // ================================================================= MMA issuer
            // The whole warp runs the loop with warp-uniform state (so addresses and descriptors stay
            // in uniform registers); one elected lane issues.  A k-tile's A operand is ready when the four
            // warps of its group have arrived on its aready barrier; they only arrive after the stage's
            // full barrier completed, so the activation tile has landed too.  A commit per k-tile tells
            // the decode groups that the block may be rewritten; the last one of a stage also arrives on
            // the stage's empty barrier, for the producers.
            constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(NPAD >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
            uint32_t idx = 0, slot = 0, sround = 0, tseq = 0;  // tseq: sequence number of the stage's first k-tile
            bool ok = true;
            Walk wk;
            wk.template init<kBalanced>(p);
            Item w;
            SPB_CARVE();
#if SPB_PROF
            uint32_t pacc[8] = {0, 0, 0, 0, 0, 0, 0, 0}, plast = clock();
#endif
            while (ok && wk.template next<kBalanced>(p, w)) {
                if (w.nk == 0) continue;
                const uint32_t accbuf = idx % kAccBufs;
                if (idx >= (uint32_t)kAccBufs)
                    ok = __all_sync(0xffffffffu,
                                    mbar_wait_patient(bar_accempty + 8 * accbuf, ((idx / kAccBufs) - 1) & 1, abort_flag));
                const uint32_t d_tmem = tmem_base + accbuf * (kNAcc * NPAD);
                for (int kk0 = 0; kk0 < w.nk && ok; kk0 += kKT) {
                    const int nv = min(kKT, w.nk - kk0);
                    const uint32_t sbase = stage0 + slot * stage_bytes;
                    ok = __all_sync(0xffffffffu, mbar_wait_patient(bar_b + 8 * slot, sround & 1u, abort_flag));  // activation tiles
                    for (int sub = 0; sub < nv && ok; ++sub) {
                        const uint32_t t = tseq + (uint32_t)sub, blk = t % kABlocks;
                        PROF_T(0);
                        ok = __all_sync(0xffffffffu, mbar_wait_patient(bar_aready + 8 * blk, (t / kABlocks) & 1u, abort_flag));
                        if (!ok) break;
                        PROF_T(1);
                        tc_fence_after();
                        if (elect_one()) {
                            const uint64_t bdesc = make_b_desc(sbase + (uint32_t)sub * kBTile);
                            const uint32_t a_tmem = tmem_a0 + blk * 32;
#pragma unroll
                            for (int s = 0; s < 4; ++s)
                                tc_mma_ts(d_tmem + (s % kNAcc) * NPAD, a_tmem + 8 * s, bdesc + 2 * s, idesc,
                                          (kk0 > 0 || sub > 0 || s >= kNAcc) ? 1u : 0u);
                            tc_commit(bar_afree + 8 * blk);
                            if (sub == nv - 1) tc_commit(bar_empty + 8 * slot);
                        }
                        __syncwarp();
                        PROF_T(2);
#if SPB_PROF
                        if (pacc[6] == 0 && lane == 0) { PROF_EV(5); pacc[6] = 1; }
#endif
                    }
                    tseq += (uint32_t)nv;
                    if (++slot == (uint32_t)S) {
                        slot = 0;
                        ++sround;
                    }
                }
                if (ok && elect_one()) tc_commit(bar_accfull + 8 * accbuf);
                __syncwarp();
                ++idx;
            }
            if (lane == 0) PROF_EV(6);
#if SPB_PROF
            if (lane == 0)
                for (int i = 0; i < 3; ++i) atomicAdd(&g_prof[8 + i], (unsigned long long)pacc[i]);
#endif
        }
    } else if (warp < kDecodeWarp0) {
        if constexpr (kResize) reg_dealloc<kRegsEpilogue>();
        // ================================================================= epilogue
        asm volatile("griddepcontrol.wait;" ::: "memory");  // before the first access to C, the scratch or the flags
        const int quad = warp & 3;
        const int row_in_block = quad * 32 + lane;
        uint32_t idx = 0;
        bool ok = true;
        Walk wk;
        wk.template init<kBalanced>(p);
        Item w;
        const bool leader = warp == kEpilogueWarp0 && lane == 0;
        // Fused exchange: this launch's number and the count of consumed exchanges are read now, long before
        // they are needed (launches on one set of buffers are ordered by the stream, so nobody changes them
        // in between), so that the end of the kernel is a chain of stores without loads.
        uint32_t my_seq = 0, consumed = 0;
        if (kExchange && leader && p.done) {
            if (p.n_flags > 0) my_seq = *reinterpret_cast<volatile uint32_t*>(p.sequence) + 1u;
            if (p.wait_flags) consumed = *reinterpret_cast<volatile uint32_t*>(p.wait_flags + p.wait_n + 1) + 1u;
        }
        // Fused split-K reduction (static schedule): called by the four epilogue warps after they have stored their
        // item's fp16 partial.  One thread publishes the CTA's stores and counts the CTA on the row block's counter;
        // the CTA that completes the count re-reads all Split_K partials of its 128 x NPAD block (they sit in L2) and
        // writes the sums: 8 consecutive rows per thread with 16-byte accesses, fp32 sums in range order, one
        // rounding, exactly what splitk_reduce_kernel computes.
        auto reduce_if_last = [&](const Item& it) {
            bar_sync_epilogue();
            if (leader) {
                // one acquire-release atomic: it publishes the CTA's partial (the barrier ordered the other
                // threads' stores before it) and, for the CTA that completes the count, makes the others' visible
                int* cnt = p.red_counters + it.nt * p.row_blocks + it.y;
                int before;
                asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(before) : "l"(cnt) : "memory");
                const bool last = before == p.split_k - 1;
                if (last) *cnt = 0;  // ready for the next launch
                *finisher = last;
            }
            bar_sync_epilogue();
            if (!*finisher) return;
            const int t = (warp - kEpilogueWarp0) * 32 + lane;
            const int rowg = it.y * 128 + (t & 15) * 8;
            if (rowg >= p.M) return;
            const size_t mn = (size_t)p.M * p.N;
            const int col_end = min(p.N, (it.nt + 1) * NPAD);
            for (int col = it.nt * NPAD + (t >> 4); col < col_end; col += 8) {
                const uint16_t* src = p.outs[0] + (size_t)col * p.M + rowg;
                float acc[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] = 0.f;
                for (int s2 = 0; s2 < p.split_k; ++s2) {
                    const uint4 v = __ldcg(reinterpret_cast<const uint4*>(src + (size_t)s2 * mn));
                    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 f = __half22float2(h[j]);
                        acc[2 * j] += f.x;
                        acc[2 * j + 1] += f.y;
                    }
                }
                uint4 o;
                __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
                for (int j = 0; j < 4; ++j) oh[j] = __floats2half2_rn(acc[2 * j], acc[2 * j + 1]);
                const size_t at = (size_t)col * p.red_ld + (size_t)p.red_row0 + rowg;
                if (kExchange && p.ep_on)
                    o = ep_apply8(o, p.ep_bias ? p.ep_bias + rowg : nullptr, p.ep_res ? p.ep_res + at : nullptr, p.ep_act);
                for (int q = 0; q < p.n_red; ++q) *reinterpret_cast<uint4*>(p.red_outs[q] + at) = o;
            }
        };
        while (ok && wk.template next<kBalanced>(p, w)) {
            const int grow = w.y * 128 + row_in_block;
            // element (col, grow) of this launch's result, in every output buffer
            const size_t out0 = (p.split_k > 1 ? (size_t)w.batch * p.M * p.N : (size_t)0) + (size_t)p.row0 + (size_t)grow;
            const int n_out = kExchange ? p.n_out : 1;
            auto store = [&](int col, uint16_t v) {
                const size_t at = out0 + (size_t)col * p.ld_out;
                for (int q = 0; q < n_out; ++q) p.outs[q][at] = v;
            };
            if (w.nk == 0) {
                for (int n = 0; n < NPAD; ++n) {
                    const int col = w.nt * NPAD + n;
                    if (col < p.N && grow < p.M) store(col, (uint16_t)0);
                }
                if (!kBalanced && p.red_counters) reduce_if_last(w);
                continue;
            }
            // A run that is only part of its range: the CTAs that share the range (c_first..c_last, in k
            // order) leave their fp32 sums in their scratch slots and count themselves on the range's
            // counter; whoever completes the count adds the sums up in k order, so the result does not
            // depend on who that is, and writes the fp16 result.  Nobody waits for anybody.
            int c_first = 0, c_last = 0, u0 = 0, arrived = 0;
            if ((kBalanced && w.partial)) {
                const int row = w.nt * p.row_blocks + w.y;
                u0 = row * p.kt_total + w.batch * p.avg_kt;
                int u1 = u0 + p.avg_kt;
                if (u1 > (row + 1) * p.kt_total) u1 = (row + 1) * p.kt_total;
                c_first = share_owner(p, u0);
                c_last = share_owner(p, u1 - 1);
                // Look at the counter while the MMAs of the run are still in flight: if all the others
                // have arrived already (the usual case for a CTA's last run) this CTA completes the range
                // straight from its registers, without publishing its own sums first.
                if (leader) arrived = ld_acquire_gpu(p.counters + w.id);
            }
            // Tail of a linear layer (exchange variants): the row's bias is fetched now, the residual values of a
            // 16-column chunk before the chunk's accumulators are read, so that no global-memory latency sits
            // between the reads of tensor memory (the accumulators are released after the last of them).
            const bool tail = kExchange && p.ep_on && p.split_k == 1 && grow < p.M;
            const bool tail_bias = tail && p.ep_bias != nullptr, tail_res = tail && p.ep_res != nullptr;
            const uint16_t ep_b = tail_bias ? p.ep_bias[grow] : (uint16_t)0;
            const int tail_act = p.ep_act;
            uint16_t ep_r[16];
#pragma unroll
            for (int n = 0; n < 16; ++n) ep_r[n] = 0;
            const uint32_t accbuf = idx % kAccBufs;
            ok = mbar_wait_relaxed(bar_accfull + 8 * accbuf, (idx / kAccBufs) & 1, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            bool direct = false;
            if ((kBalanced && w.partial)) {
                if (leader) {
                    // the run may have been long: look again before taking the slower way
                    if (arrived != c_last - c_first) arrived = ld_acquire_gpu(p.counters + w.id);
                    *finisher = arrived == c_last - c_first;
                }
                // the four warps meet on a named barrier below, so they must agree to go on
                ok = bar_and_epilogue(ok);
                direct = *finisher != 0;
            }
            if (!ok) break;
            tc_fence_after();
            const uint32_t t_acc = tmem_base + ((uint32_t)(quad * 32) << 16) + accbuf * (kNAcc * NPAD);
            // the first contributor used its second slot unless its share starts with this range
            const int slot_first = (kBalanced && w.partial) && share_begin(p, c_first) != u0 ? 1 : 0;
            auto slot_of = [&](int cc) -> float* {
                return p.partials + (size_t)(2 * cc + (cc == c_first ? slot_first : 0)) * (128 * NPAD) + row_in_block;
            };
            float* mine = slot_of((int)blockIdx.x);
            // adds the sums of all contributors to acc in k order (own: the registers r when have_own)
            auto add_all = [&](float* acc, const uint32_t* r, int c, bool have_own) {
#pragma unroll 1
                for (int cc = c_first; cc <= c_last; ++cc) {
                    if (have_own && cc == (int)blockIdx.x) {
#pragma unroll
                        for (int n = 0; n < 16; ++n) acc[n] += __uint_as_float(r[n]);
                    } else {
                        const float* src = slot_of(cc) + c * 16 * 128;
                        float v[16];
#pragma unroll
                        for (int n = 0; n < 16; ++n) v[n] = __ldcg(src + n * 128);
#pragma unroll
                        for (int n = 0; n < 16; ++n) acc[n] += v[n];
                    }
                }
            };
            // the same without own registers: two contributors' sums are fetched together
            auto add_all_pairs = [&](float* acc, int c) {
#pragma unroll 1
                for (int cc = c_first; cc <= c_last; cc += 2) {
                    const bool two = cc + 1 <= c_last;
                    const float* s0 = slot_of(cc) + c * 16 * 128;
                    const float* s1 = slot_of(two ? cc + 1 : cc) + c * 16 * 128;
                    float v0[16], v1[16];
#pragma unroll
                    for (int n = 0; n < 16; ++n) v0[n] = __ldcg(s0 + n * 128);
#pragma unroll
                    for (int n = 0; n < 16; ++n) v1[n] = __ldcg(s1 + n * 128);
#pragma unroll
                    for (int n = 0; n < 16; ++n) {
                        acc[n] += v0[n];
                        if (two) acc[n] += v1[n];
                    }
                }
            };
            // 16 columns of the result to every output buffer: the loop over the buffers is the outer one so
            // that the 16 stores to a buffer are issued back to back (the end of the kernel waits for them)
            auto write_out = [&](const float* acc, int c) {
                uint16_t h[16];
#pragma unroll
                for (int n = 0; n < 16; ++n) h[n] = __half_as_ushort(__float2half_rn(acc[n]));
                const int col0 = w.nt * NPAD + c * 16;
                if (kExchange && tail) {   // these are final rows: two columns per step
                    const __half2 b2 = __half2half2(__ushort_as_half(ep_b));
#pragma unroll
                    for (int n = 0; n < 16; n += 2) {
                        const __half2 y = ep_pair(__halves2half2(__ushort_as_half(h[n]), __ushort_as_half(h[n + 1])), tail_bias, b2, tail_act,
                                                  tail_res, __halves2half2(__ushort_as_half(ep_r[n]), __ushort_as_half(ep_r[n + 1])));
                        h[n] = __half_as_ushort(__low2half(y));
                        h[n + 1] = __half_as_ushort(__high2half(y));
                    }
                }
                if (grow < p.M) {
#pragma unroll 1
                    for (int q = 0; q < n_out; ++q) {
                        uint16_t* o = p.outs[q] + out0 + (size_t)col0 * p.ld_out;
#pragma unroll
                        for (int n = 0; n < 16; ++n)
                            if (col0 + n < p.N) o[(size_t)n * p.ld_out] = h[n];
                    }
                }
            };
#pragma unroll(kExchange && NPAD >= 128 ? 1 : 16)
            for (int c = 0; c < NPAD / 16; ++c) {
                if (kExchange && tail_res) {
                    const int col0 = w.nt * NPAD + c * 16;
#pragma unroll
                    for (int n = 0; n < 16; ++n)
                        ep_r[n] = col0 + n < p.N ? p.ep_res[out0 + (size_t)(col0 + n) * p.ld_out] : (uint16_t)0;
                }
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
                if (!(kBalanced && w.partial)) {
                    float acc[16];
#pragma unroll
                    for (int n = 0; n < 16; ++n) acc[n] = __uint_as_float(r[n]);
                    write_out(acc, c);
                } else if (direct) {
                    float acc[16];
#pragma unroll
                    for (int n = 0; n < 16; ++n) acc[n] = 0.f;
                    add_all(acc, r, c, true);
                    write_out(acc, c);
                } else {
#pragma unroll
                    for (int n = 0; n < 16; ++n) __stcg(mine + (c * 16 + n) * 128, __uint_as_float(r[n]));
                }
            }
            if ((kBalanced && w.partial) && direct) {
                if (leader) p.counters[w.id] = 0;  // ready for the next launch
            } else if ((kBalanced && w.partial)) {
                // One thread publishes the CTA's partial sums (its fence covers the stores the barrier
                // ordered before it) and counts the arrival; its second fence makes the other CTAs' sums
                // visible to the threads that pass the second barrier.
                bar_sync_epilogue();
                if (leader) {
                    __threadfence();
                    const int before = atomicAdd(p.counters + w.id, 1);
                    if (before == c_last - c_first) __threadfence();
                    *finisher = before == c_last - c_first;
                }
                bar_sync_epilogue();
                if (*finisher) {
#pragma unroll 1
                    for (int c = 0; c < NPAD / 16; ++c) {
                        float acc[16];
#pragma unroll
                        for (int n = 0; n < 16; ++n) acc[n] = 0.f;
                        if (kExchange && tail_res) {
                            const int col0 = w.nt * NPAD + c * 16;
#pragma unroll
                            for (int n = 0; n < 16; ++n)
                                ep_r[n] = col0 + n < p.N ? p.ep_res[out0 + (size_t)(col0 + n) * p.ld_out] : (uint16_t)0;
                        }
                        add_all_pairs(acc, c);
                        write_out(acc, c);
                    }
                    if (leader) p.counters[w.id] = 0;
                }
            }
            if (!kBalanced && p.red_counters) reduce_if_last(w);
            ++idx;
        }
        if (leader) PROF_EV(7);
        if (kExchange && p.done) {
            // Fused all-gather: every thread's stores to the peers are made visible system-wide before the CTA
            // counts itself as finished; the CTA that completes the count numbers the launch and tells the peers.
            // (the barrier orders the other threads' stores before the leader's system-scope fence, which is
            // cumulative: one fence per CTA instead of one per thread)
            bar_sync_epilogue();
            if (leader && p.n_flags > 0) __threadfence_system();
            if (leader && atomicAdd(p.done, 1) == (int)gridDim.x - 1) {
                *p.done = 0;
                if (p.n_flags > 0) {
                    __threadfence();  // the other CTAs' counts (each behind its own system-scope fence) were seen
                    *p.sequence = my_seq;
                    for (int q = 0; q < p.n_flags; ++q)
                        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.flags[q] + p.flag_index), "r"(my_seq)
                                     : "memory");
                }
                if (p.wait_flags) p.wait_flags[p.wait_n + 1] = consumed;  // every CTA of this launch has read it
            }
        }
    } else {
        // ================================================================= decode
        // Decode group g is four warps, one per TMEM lane quadrant, one thread per weight row.  The k-tiles of the
        // CTA's stage sequence are cut into units of kUnit k-tiles of one stage and dealt to the groups in turn.
        // Per unit a warp first works out, one tile per lane, where the values of its 32 tiles of each k-tile start
        // (population count of the bitmap, prefix sum over the 16 tiles of a median tile by shuffles) and leaves
        // {bitmap half, start of the half's values} pairs in its tile table; then every thread expands, for each of
        // the 8 tiles its row crosses, its row segment and writes it to tensor memory.  The barrier checks and the
        // prefix sums are a chain of dependent instructions: it is paid once per unit.
        if constexpr (kResize) reg_alloc<kRegsDecode>();
        const int dw = warp - kDecodeWarp0;
        const int group = dw >> 2;
        const int quad = warp & 3;             // TMEM lane quadrant this warp may access
        const int row = quad * 32 + lane;      // weight row inside the 128-row block
        const int chunk = row >> 6, rr = row & 63;   // 64-row global-tile row of the block, row inside it
        const int r_in_tile = rr & 7;
        SPB_CARVE();
        const uint32_t my_v = chunk ? off_v1 : off_v0;
        const uint32_t rel0 = off_rel + 4 * (uint32_t)(chunk * kKT);
        // Lane l looks after tile l & 15 of median tile 2 * (quad & 1) + (l >> 4) of each k-tile of the unit.
        const uint32_t tile_tab = smem_u32(smem + 1024) + (uint32_t)dw * kTileTabBytes;
        const uint32_t tile_bm0 = (chunk ? off_bm1 : off_bm0) + 8 * (uint32_t)(32 * (quad & 1) + lane);
        const uint32_t tile_mt0 = (chunk ? off_mt1 : off_mt0) + 4 * (uint32_t)(2 * (quad & 1) + (lane >> 4));
        // This row's entry of the table for the first tile it crosses (the others are 32 bytes apart: the tiles of a
        // median tile are stored in pairs, rows 0-7 then rows 8-15 of each 8-column step), the half its row is in.
        const uint32_t ent = tile_tab + 16 * (uint32_t)(16 * (lane >> 4) + ((lane >> 3) & 1)) + 8 * (uint32_t)(r_in_tile >> 2);
        const uint32_t below = (r_in_tile & 3) ? (1u << (8 * (r_in_tile & 3))) - 1u : 0u;
        const uint32_t rsel4 = 0x4440u | (uint32_t)(r_in_tile & 3);
        const uint32_t lutlane = smem_u32(smem + 1024 + kTileTabBytes * 4 * kDecodeGroups) + 8 * (uint32_t)(lane & 15);

        uint32_t slot = 0, round = 0, rot = 0, tseq = 0;  // tseq: sequence number of the stage's first k-tile
        bool ok = true;
        Walk wk;
        wk.template init<kBalanced>(p);
        Item w;
        ok = __all_sync(0xffffffffu, mbar_wait(bar_lut, 0, abort_flag));  // the selector table
#if SPB_PROF
        uint32_t pacc[8] = {0, 0, 0, 0, 0, 0, 0, 0}, plast = clock();
#endif
        while (ok && wk.template next<kBalanced>(p, w)) {
            const bool valid = chunk == 0 || (2 * w.y + 1) < p.gm_total;
            for (int kk0 = 0; kk0 < w.nk && ok; kk0 += kKT) {
                const int nv = min(kKT, w.nk - kk0);
                const int nun = (nv + kUnit - 1) / kUnit;  // units in this stage
                const int usub = (int)(((uint32_t)group + (uint32_t)kDecodeGroups - rot) % (uint32_t)kDecodeGroups);  // this group's unit
                rot = (rot + (uint32_t)nun) % (uint32_t)kDecodeGroups;
                // Every group, with or without a unit, waits for the stage: it arrives on the stage's empty
                // barrier below and must not get a ring round ahead of it.
                PROF_T(0);
                ok = mbar_wait(bar_full + 8 * slot, round & 1, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                PROF_T(1);
#if SPB_PROF
                if (dw == 0 && lane == 0 && pacc[7] == 0 && plast != 0xffffffffu) { PROF_EV(4); }
#endif
                if (usub < nun) {
                    const int sub0 = usub * kUnit, nk = min(kUnit, nv - sub0);  // the unit's k-tiles of the stage
                    const uint32_t st = stage0 + slot * stage_bytes;
                    {   // starts of the warp's 32 tiles of each k-tile: running sum of the tile sizes inside each median tile
                        uint32_t lo[kUnit], hi[kUnit], base[kUnit], cnt[kUnit], x[kUnit];
#pragma unroll
                        for (int j = 0; j < kUnit; ++j) {
                            lo[j] = hi[j] = 0u;
                            base[j] = st + my_v;
                            if (valid && j < nk) {
                                lds64(st + tile_bm0 + (uint32_t)(sub0 + j) * 512, lo[j], hi[j]);
                                const uint32_t mt = lds32(st + tile_mt0 + (uint32_t)(sub0 + j) * 16);
                                const uint32_t rel = lds32(st + rel0 + 4 * (uint32_t)(sub0 + j));
                                // clamped so that corrupt offsets can never point outside the stage
                                base[j] += min(rel + 2 * mt, (uint32_t)kKT * vmax);
                            }
                        }
#pragma unroll
                        for (int j = 0; j < kUnit; ++j) x[j] = cnt[j] = __popc(lo[j]) + __popc(hi[j]);
#pragma unroll
                        for (int d = 1; d < 16; d <<= 1) {
#pragma unroll
                            for (int j = 0; j < kUnit; ++j) {
                                const uint32_t y = __shfl_up_sync(0xffffffffu, x[j], d, 16);
                                if ((lane & 15) >= d) x[j] += y;
                            }
                        }
                        __syncwarp();  // every lane has read the previous unit's tables
#pragma unroll
                        for (int j = 0; j < kUnit; ++j) {
                            const uint32_t ts_lo = base[j] + 2 * (x[j] - cnt[j]), ts_hi = ts_lo + 2 * __popc(lo[j]);
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(tile_tab + 512 * j + 16 * (uint32_t)lane),
                                         "r"(lo[j]), "r"(ts_lo), "r"(hi[j]), "r"(ts_hi)
                                         : "memory");
                        }
                        __syncwarp();
                    }
                    PROF_T(2);
#pragma unroll
                    for (int j = 0; j < kUnit; ++j) {
                        if (j >= nk || !ok) continue;
                        const uint32_t t = tseq + (uint32_t)(sub0 + j), blk = t % kABlocks;
                        // the MMAs of the block's previous k-tile (a barrier nobody has arrived on yet passes a wait
                        // for the phase before its first, so the block's first use needs no special case)
                        ok = mbar_wait(bar_afree + 8 * blk, ((t / kABlocks) & 1u) ^ 1u, abort_flag);
                        ok = __all_sync(0xffffffffu, ok);
                        if (!ok) continue;
                        tc_fence_after();
                        PROF_T(3);
                        const uint32_t ta = tmem_a0 + blk * 32 + ((uint32_t)(quad * 32) << 16);
                        uint32_t a[32];
#pragma unroll
                        for (int q0 = 0; q0 < 8; q0 += 2) {
                            uint32_t wq[2], hq[2];
                            UnitLoads u[2];
#pragma unroll
                            for (int q = 0; q < 2; ++q) lds64(ent + 512 * j + 32 * (q0 + q), wq[q], hq[q]);
#pragma unroll
                            for (int q = 0; q < 2; ++q) unit_load3(wq[q], hq[q], below, rsel4, lutlane, u[q]);
#pragma unroll
                            for (int q = 0; q < 2; ++q) unit_expand(u[q], a + 4 * (q0 + q));
                            tc_st_32x32b_x8(ta + 4 * q0, a + 4 * q0);
                        }
                        PROF_T(4);
                        tc_wait_st();
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar_aready + 8 * blk);
                        PROF_T(5);
#if SPB_PROF
                        ++pacc[7];
#endif
                    }
                    if (!ok) break;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_empty + 8 * slot);
                tseq += (uint32_t)nv;
                if (++slot == (uint32_t)S) {
                    slot = 0;
                    ++round;
                }
                PROF_T(6);
            }
        }
#if SPB_PROF
        if (dw == 0 && lane == 0)
            for (int i = 0; i < 8; ++i) atomicAdd(&g_prof[i], (unsigned long long)pacc[i]);
#endif
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
            SPB_CARVE();
            for (uint32_t spin = 0; spin < 4096; ++spin)
                if (mbar_try(bar_lut, 0)) break;
            for (int i = 0; i < S; ++i)
                for (uint32_t spin = 0; spin < 4096; ++spin)
                    if ((mbar_try(bar_full + 8 * i, 0) || mbar_try(bar_full + 8 * i, 1)) &&
                        (mbar_try(bar_b + 8 * i, 0) || mbar_try(bar_b + 8 * i, 1)))
                        break;
        }
        __syncthreads();
    }
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
    if (threadIdx.x == 0) PROF_EV(8);
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

// ---------------------------------------------------------------- scratch of the balanced schedule
// Owned by the library, one set per (device, stream) so that calls on different streams never share
// counters; calls on one stream are ordered by the stream.  Created by spb_init(stream) only: the SpMM
// entry points themselves never allocate or synchronise (the reference's entry point is asynchronous and
// allocation-free, reference csrc/SpMM_API.cuh:47-110); on a stream that was never initialised they use
// the static schedule, which needs no scratch.
constexpr int kScratchSets = 16;
constexpr int kCounterCap = 1 << 20;
struct ScratchSet {
    float* partials = nullptr;
    int* counters = nullptr;
    cudaStream_t stream = nullptr;
    bool taken = false;
};
std::mutex g_scratch_mu;
ScratchSet g_scratch[64][kScratchSets];
std::atomic<int> g_weights_ahead{1};  // see spb_set_weight_prefetch
std::atomic<int> g_schedule{0};       // 0: by the cost model, 1: always static, 2: balanced whenever possible
thread_local int t_static_depth = 0;  // > 0: this thread's calls use the static schedule

const ScratchSet* scratch_for(cudaStream_t st, int dev, int sms, bool may_create)
{
    std::lock_guard<std::mutex> lock(g_scratch_mu);
    ScratchSet* sets = g_scratch[dev];
    for (int i = 0; i < kScratchSets; ++i)
        if (sets[i].taken && sets[i].stream == st) return &sets[i];
    if (!may_create) return nullptr;
    for (int i = 0; i < kScratchSets; ++i) {
        if (sets[i].taken) continue;
        ScratchSet n;
        const size_t pbytes = (size_t)2 * sms * 128 * 256 * sizeof(float);  // two slots of 128 x (widest tile) per CTA
        if (cudaMalloc(&n.partials, pbytes) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        if (cudaMalloc(&n.counters, (size_t)(kCounterCap + 16) * sizeof(int)) != cudaSuccess ||
            cudaMemset(n.counters, 0, (size_t)(kCounterCap + 16) * sizeof(int)) != cudaSuccess ||
            cudaDeviceSynchronize() != cudaSuccess) {
            cudaGetLastError();
            cudaFree(n.partials);
            if (n.counters) cudaFree(n.counters);
            return nullptr;
        }
        n.stream = st;
        n.taken = true;
        sets[i] = n;
        return &sets[i];
    }
    return nullptr;  // more streams than sets: the static schedule needs none
}

bool stream_is_capturing(cudaStream_t st)
{
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cs) != cudaSuccess) {
        cudaGetLastError();
        return true;  // e.g. the legacy stream while another stream captures: stay on the safe side
    }
    return cs != cudaStreamCaptureStatusNone;
}

// Cost model of the two schedules, in units of one k-tile of one 128-row block on one SM (about 0.45 us),
// fitted to timings of OPT-shaped matrices at N = 16 and 32.  Every work item after an SM's first costs
// about 4 k-tiles (pipeline hand-over), a split-K reduction launch about 3.  The exchange of partial sums at
// the end of a balanced kernel costs about 6 plus 2.2 per round of loads: one round per 16 columns and per
// other SM that shares a range.  With activation tiles of 128 and 256 columns a k-tile takes 1.15 and 1.85 units
// (the tensor core's and the decode warps' shared-memory traffic add up), and the fp16 partials of a split-K run
// (written once, read once, at about 4 TB/s out of L2 and HBM) stop being negligible.
double tile_units(int npad) { return npad <= 64 ? 1.0 : npad <= 128 ? 1.15 : 1.85; }
double item_units(int npad) { return npad <= 64 ? 4.0 : 4.0 + npad / 16; }   // hand-over between work items: the epilogue grows with the tile
double reduction_cost(int row_blocks, int n_tiles, int sk, int npad)
{
    if (sk <= 1) return 0.0;
    const double bytes = 2.0 * (sk + 1) * (128.0 * row_blocks) * ((double)n_tiles * npad);
    return 3.0 + 0.15 * sk + bytes / 4.0e6 / 0.45;
}
double static_cost(int row_blocks, int n_tiles, int kt, int sk, int sms, int npad)
{
    const int avg = (kt - 1) / sk + 1;
    const long items = (long)row_blocks * n_tiles * sk;
    const long waves = (items + sms - 1) / sms;
    return (double)waves * (tile_units(npad) * avg + item_units(npad)) - item_units(npad) + reduction_cost(row_blocks, n_tiles, sk, npad);
}
double balanced_cost(int row_blocks, int n_tiles, int kt, int sk, int sms, int npad)
{
    const double units = (double)row_blocks * n_tiles * kt;
    const long items = (long)row_blocks * n_tiles * sk;
    const int avg = (kt - 1) / sk + 1;
    const double share = units / (units < sms ? units : sms);
    const bool cuts = items % sms != 0 || avg * sk != kt;  // some range is shared between SMs
    double exchange = 0.0;
    if (cuts) {
        double others = avg / share;
        others = others <= 1.0 ? 1.0 : (double)(long)(others + 0.999);
        exchange = 6.0 + 2.2 * (npad / 16) * others;
    }
    // the balanced variant of the kernel needs about 4 % longer per k-tile than the static one
    return 1.04 * tile_units(npad) * share + exchange + reduction_cost(row_blocks, n_tiles, sk, npad);
}
bool prefer_balanced(int row_blocks, int n_tiles, int kt, int sk, int sms, int npad)
{
    return balanced_cost(row_blocks, n_tiles, kt, sk, sms, npad) < static_cost(row_blocks, n_tiles, kt, sk, sms, npad);
}

template <int NPAD>
cudaError_t prepare_width(int dyn_smem)
{
    cudaError_t e = cudaFuncSetAttribute(spmm_bitmap_tcgen05_kernel<NPAD, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, dyn_smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(spmm_bitmap_tcgen05_kernel<NPAD, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, dyn_smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(spmm_bitmap_tcgen05_kernel<NPAD, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, dyn_smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(spmm_bitmap_tcgen05_kernel<NPAD, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, dyn_smem);
    return e;
}
// Raises the dynamic shared-memory limit of all kernel variants on the current device, the first time it is
// called for that device.
cudaError_t prepare_kernels(int dev, int dyn_smem)
{
    static std::mutex mu;
    static bool done[64] = {};
    std::lock_guard<std::mutex> lock(mu);
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (done[dev]) return cudaSuccess;
    cudaError_t e = prepare_width<16>(dyn_smem);
    if (e == cudaSuccess) e = prepare_width<32>(dyn_smem);
    if (e == cudaSuccess) e = prepare_width<64>(dyn_smem);
    if (e == cudaSuccess) e = prepare_width<128>(dyn_smem);
    if (e == cudaSuccess) e = prepare_width<256>(dyn_smem);
    if (e == cudaSuccess) done[dev] = true;
    return e;
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
    int dev = 0;
    cudaGetDevice(&dev);
    // Balanced schedule: every CTA gets the same number of k-tiles; needs the library's scratch.
    const long long units = (long long)p.n_tiles * p.row_blocks * p.kt_total;
    const bool no_empty_range = (long long)(a.split_k - 1) * p.avg_kt < p.kt_total;
    p.partials = nullptr;
    p.counters = nullptr;
    p.balanced = 0;
    p.units = 0;
    // Where the result goes.  Split_K == 1: straight to the final destination, C or (fused all-gather) the peers'
    // buffers.  Split_K > 1: fp16 partials to the workspace (a.out); the final destination is written by the
    // fused reduction when that is possible (decided below), else by the caller's reduction launch.
    const bool split = a.split_k > 1;
    const bool gather = a.n_out > 0;
    const bool direct_gather = gather && !split;
    for (int q = 0; q < kMaxPeers; ++q) {
        p.outs[q] = direct_gather && q < a.n_out ? a.outs[q] : nullptr;
        p.flags[q] = nullptr;
        p.red_outs[q] = nullptr;
    }
    if (!direct_gather) p.outs[0] = a.out;
    p.n_out = direct_gather ? a.n_out : 1;
    p.ld_out = direct_gather ? a.ld_out : a.M;
    p.row0 = direct_gather ? a.row0 : 0;
    p.n_flags = 0;
    p.red_counters = nullptr;
    p.n_red = 0;
    p.red_ld = 0;
    p.red_row0 = 0;
    if (a.reduce_fused) *a.reduce_fused = false;
    p.flag_index = a.flag_index;
    p.sequence = a.sequence;
    p.done = nullptr;
    p.wait_flags = a.wait_flags;
    p.wait_n = a.wait_n;
    p.weights_ahead = g_weights_ahead.load();
    p.ep_bias = a.ep.bias;
    p.ep_res = a.ep.residual;
    p.ep_act = a.ep.activation;
    p.ep_on = a.ep.any() ? 1 : 0;
    const int mode = g_schedule.load();
    if (mode != 1 && t_static_depth == 0 && (units + 1) * di.sms < (1LL << 31) && p.num_items <= kCounterCap &&
        no_empty_range && (mode == 2 || prefer_balanced(p.row_blocks, p.n_tiles, p.kt_total, a.split_k, di.sms, NPAD))) {
        // the scratch spb_init created for this stream, if it was called
        if (const ScratchSet* sc = scratch_for(s, dev, di.sms, false)) {
            p.partials = sc->partials;
            p.counters = sc->counters;
            p.balanced = 1;
            p.units = (int)units;
        }
    }
    // Fused split-K reduction: static schedule, a final destination, the stream's counters (spb_init)
    bool red_fused = false;
    if (split && !p.balanced && t_static_depth == 0 && (gather || a.final_out) && p.n_tiles * p.row_blocks <= kCounterCap &&
        ((size_t)a.M * a.N) % 8 == 0) {
        if (const ScratchSet* sc = scratch_for(s, dev, di.sms, false)) {
            p.red_counters = sc->counters;
            p.n_red = gather ? a.n_out : 1;
            for (int q = 0; q < p.n_red; ++q) p.red_outs[q] = gather ? a.outs[q] : a.final_out;
            p.red_ld = gather ? a.ld_out : a.M;
            p.red_row0 = gather ? a.row0 : 0;
            red_fused = true;
            if (a.reduce_fused) *a.reduce_fused = true;
        }
    }
    // the kernel tells the peers itself when it also writes the final rows
    if (gather && (!split || red_fused)) {
        p.n_flags = a.n_flags;
        for (int q = 0; q < kMaxPeers; ++q) p.flags[q] = q < a.n_flags ? a.flags[q] : nullptr;
    }
    if (p.n_flags > 0 || p.wait_flags) {
        // the count of finished CTAs lives behind the arrival counters of the stream's scratch
        const ScratchSet* sc = scratch_for(s, dev, di.sms, false);
        if (!sc) {
            set_error("fused all-gather: spb_init has not been called for this stream");
            return cudaErrorNotReady;
        }
        p.done = sc->counters + kCounterCap;
    }

    const bool exchange = gather || p.wait_flags != nullptr || p.ep_on;
    const int variant = (exchange ? 2 : 0) + (p.balanced ? 1 : 0);
    auto kernel = variant == 3   ? spmm_bitmap_tcgen05_kernel<NPAD, true, true>
                  : variant == 2 ? spmm_bitmap_tcgen05_kernel<NPAD, true, false>
                  : variant == 1 ? spmm_bitmap_tcgen05_kernel<NPAD, false, true>
                                 : spmm_bitmap_tcgen05_kernel<NPAD, false, false>;
    {   // every variant of every activation-tile width, once per device: a later call never changes a kernel attribute
        cudaError_t e = prepare_kernels(dev, dyn_smem);
        if (e != cudaSuccess) return e;
    }
    const long long work = p.balanced ? units : (long long)p.num_items;
    const int grid = work < di.sms ? (int)work : di.sms;
    // Programmatic dependent launch: this kernel's set-up may overlap the end of the stream's previous
    // kernel; the kernel itself waits for that kernel before it touches global memory.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(threads_for(NPAD));
    cfg.dynamicSmemBytes = (size_t)dyn_smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    count_launch();
    return cudaLaunchKernelEx(&cfg, kernel, p, tmap);
}

}  // namespace

cudaError_t exchange_counter(cudaStream_t s, int** out)
{
    DeviceInfo di = device_info();
    int dev = 0;
    if (!di.ok || cudaGetDevice(&dev) != cudaSuccess) return cudaErrorNoDevice;
    const ScratchSet* sc = scratch_for(s, dev, di.sms, false);
    if (!sc) {
        set_error("fused all-gather: spb_init has not been called for this stream");
        return cudaErrorNotReady;
    }
    *out = sc->counters + kCounterCap + 1;
    return cudaSuccess;
}

#if SPB_PROF
}  // namespace spb
extern "C" int spb_debug_prof(unsigned long long* out, int clear)
{
    cudaError_t e = cudaMemcpyFromSymbol(out, spb::g_prof, sizeof(unsigned long long) * 32);
    if (e == cudaSuccess) e = cudaMemcpyFromSymbol(out + 32, spb::g_tl, sizeof(unsigned long long) * 32);
    if (e == cudaSuccess && clear) {
        unsigned long long z[32] = {}, t[32];
        for (int i = 0; i < 32; ++i) t[i] = (i & 1) ? 0ull : ~0ull;
        e = cudaMemcpyToSymbol(spb::g_prof, z, sizeof(z));
        if (e == cudaSuccess) e = cudaMemcpyToSymbol(spb::g_tl, t, sizeof(t));
    }
    return (int)e;
}
namespace spb {
#endif
// Creates the scratch of the balanced schedule and of the fused exchange for (current device, stream) and raises
// the kernels' shared-memory limit; allocates and synchronises, so it must run outside stream capture.
cudaError_t init_stream(cudaStream_t s)
{
    DeviceInfo di = device_info();
    int dev = 0;
    if (!di.ok || cudaGetDevice(&dev) != cudaSuccess) {
        set_error("spb_init: no usable CUDA device");
        return cudaErrorNoDevice;
    }
    if (stream_is_capturing(s)) {
        set_error("spb_init: the stream is being captured");
        return cudaErrorStreamCaptureUnsupported;
    }
    cudaError_t e = prepare_kernels(dev, di.max_smem - 1024);
    if (e != cudaSuccess) return e;
    int* status = nullptr;
    e = device_status_ptr(&status);
    if (e != cudaSuccess) return e;
    if (!scratch_for(s, dev, di.sms, true)) {
        set_error("spb_init: no scratch set left (%d streams per device) or out of device memory", kScratchSets);
        return cudaErrorMemoryAllocation;
    }
    return cudaSuccess;
}

// Gives back the scratch spb_init created for (current device, stream), after the stream's work has completed.
cudaError_t release_stream(cudaStream_t s)
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (stream_is_capturing(s)) {
        set_error("spb_release: the stream is being captured");
        return cudaErrorStreamCaptureUnsupported;
    }
    e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return e;
    std::lock_guard<std::mutex> lock(g_scratch_mu);
    for (int i = 0; i < kScratchSets; ++i) {
        ScratchSet& set = g_scratch[dev][i];
        if (!set.taken || set.stream != s) continue;
        cudaFree(set.partials);
        cudaFree(set.counters);
        set = ScratchSet();
    }
    return cudaSuccess;
}

int set_weight_prefetch(int on) { return g_weights_ahead.exchange(on ? 1 : 0); }

int set_schedule(int mode)
{
    if (mode < 0 || mode > 2) return -1;
    return g_schedule.exchange(mode);
}
void push_static_schedule() { ++t_static_depth; }
void pop_static_schedule() { --t_static_depth; }

cudaError_t reset_schedule_scratch()
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_scratch_mu);
    for (int i = 0; i < kScratchSets; ++i) {
        if (!g_scratch[dev][i].taken) continue;
        e = cudaMemset(g_scratch[dev][i].counters, 0, (size_t)(kCounterCap + 16) * sizeof(int));
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

int suggest_split_k(int M, int N, int K)
{
    DeviceInfo di = device_info();
    const int sms = di.ok ? di.sms : 148;
    const int row_blocks = (M / 64 + 1) / 2;
    const int kt = K / 64;
    const int npad = N <= 16 ? 16 : N <= 32 ? 32 : N <= 64 ? 64 : N <= 128 ? 128 : 256;   // as spmm_launch picks it
    const int n_tiles = (N + npad - 1) / npad;
    if (row_blocks <= 0 || kt <= 0) return 1;
    const bool may_balance = g_schedule.load() != 1 && t_static_depth == 0;
    int best = 1;
    double best_cost = static_cost(row_blocks, n_tiles, kt, 1, sms, npad);
    if (may_balance) {
        // Split_K = 1 with equal shares needs no fp16 partial sums and no reduction
        const double c = balanced_cost(row_blocks, n_tiles, kt, 1, sms, npad);
        if (c < best_cost) best_cost = c;
    }
    for (int sk = 2; sk <= 32 && sk <= kt; ++sk) {
        const int avg = (kt - 1) / sk + 1;
        if ((sk - 1) * avg >= kt) continue;  // would leave an empty last range
        if (avg < 4) break;
        const double cost = static_cost(row_blocks, n_tiles, kt, sk, sms, npad);
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
    // Activation tile width: the smallest of 16/32/64/128/256 that holds N; wider N (the prefill regime) is cut
    // into tiles of 256 columns, each of which re-reads and re-expands the weight: at 256 columns the tensor
    // core's time per k-tile (4 MMAs of 128 x 256 x 16) is about what the expansion of the k-tile takes.
    if (a.N <= 16) return launch_t<16>(s, a, di, status);
    if (a.N <= 32) return launch_t<32>(s, a, di, status);
    if (a.N <= 64) return launch_t<64>(s, a, di, status);
    if (a.N <= 128) return launch_t<128>(s, a, di, status);
    return launch_t<256>(s, a, di, status);
}

}  // namespace spb
