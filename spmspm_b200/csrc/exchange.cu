// Fused SpMM + all-gather over peer memory, for the M-split of tensor-parallel inference (the weight's rows are
// sharded over the GPUs, every GPU needs all output rows; FasterTransformer does this with an NCCL all-gather
// after the GEMM, third_party/ft_spinfer.patch:623-862).  The SpMM kernel's epilogue stores its output rows
// straight into every GPU's [N][M] buffer with plain stores through NVLink, and the last CTA to finish writes
// the launch's sequence number into every GPU's flag array.  A consumer waits, with a bounded number of polls,
// until its own flag array shows the current sequence number from every rank.  No load ever touches peer memory.
#include "../../include/spmm_b200.h"
#include "common.cuh"
#include <cuda_fp16.h>

namespace spb {
namespace {

constexpr uint32_t kPollLimit = 1u << 21;  // about half a second with the sleep below

// flags: [n] sequence numbers written by the n ranks, [n] this rank's own launch count (written by the SpMM
// kernel), [n + 1] how many exchanges this rank has waited for.
__global__ void wait_flags_kernel(uint32_t* flags, int n, int* status)
{
    __shared__ uint32_t want;
    if (threadIdx.x == 0) want = ++flags[n + 1];
    __syncthreads();
    const uint32_t w = want;
    bool ok = true;
    if ((int)threadIdx.x < n) {
        ok = false;
        for (uint32_t i = 0; i < kPollLimit; ++i) {
            uint32_t v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + threadIdx.x) : "memory");
            if ((int32_t)(v - w) >= 0) {
                ok = true;
                break;
            }
            __nanosleep(200);
        }
    }
    if (!ok) atomicOr(status, (int)kStatusWaitTimeout);
}

// Split-K reduction (the arithmetic of reduction.cu: fp32 sum of the fp16 partials in range order, one fp16
// rounding) whose result rows go to rows row0.. of every GPU's [N][ld] buffer; the last block numbers the
// exchange and writes the flags, like the SpMM kernel does when it gathers directly.
struct GatherOut {
    uint16_t* outs[8];
    uint32_t* flags[8];
    int n, flag_index;
    uint32_t* sequence;
    int* done;
};
__global__ void __launch_bounds__(256)
splitk_reduce_gather_kernel(const GatherOut g, const uint16_t* __restrict__ W, int M, size_t mn, int split_k, int ld,
                            int row0)
{
    const size_t e = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (e < mn) {
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        for (int s = 0; s < split_k; ++s) {
            const uint4 v = *reinterpret_cast<const uint4*>(W + (size_t)s * mn + e);
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
        const size_t col = e / (size_t)M, row = e - col * (size_t)M;  // 8 consecutive rows of one column
        const size_t at = col * (size_t)ld + (size_t)row0 + row;
        for (int q = 0; q < g.n; ++q) *reinterpret_cast<uint4*>(g.outs[q] + at) = o;
    }
    // one system-scope fence per block, behind the barrier that orders the other threads' stores before it
    __syncthreads();
    if (threadIdx.x != 0) return;
    const uint32_t seq = *reinterpret_cast<volatile uint32_t*>(g.sequence) + 1u;  // exchanges on a buffer are stream-ordered
    __threadfence_system();
    if (atomicAdd(g.done, 1) == (int)gridDim.x - 1) {
        *g.done = 0;
        __threadfence();
        *g.sequence = seq;
        for (int q = 0; q < g.n; ++q)
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(g.flags[q] + g.flag_index), "r"(seq) : "memory");
    }
}

}  // namespace

cudaError_t wait_flags_launch(cudaStream_t s, uint32_t* flags, int n, int* status)
{
    count_launch();
    wait_flags_kernel<<<1, 32, 0, s>>>(flags, n, status);
    return cudaGetLastError();
}

}  // namespace spb

extern "C" int spb_spmm_bitmap_v3_allgather(void* stream, const uint16_t* Compressed_A, const int* TileOffsets,
                                            const int* TileOffsets_Median, const uint64_t* bitmap,
                                            const int* max_nnz_intile, const uint16_t* B, uint16_t* const* C_peers,
                                            uint32_t* const* flag_peers, int n_peers, int rank, int M_shard,
                                            int N_Global, int K_Global, int M_full, int row_offset,
                                            uint32_t* B_flags, uint16_t* Reduction_Workspace, int Split_K)
{
    if (n_peers < 1 || n_peers > 8 || rank < 0 || rank >= n_peers || !C_peers || !flag_peers) {
        spb::set_error("spb_spmm_bitmap_v3_allgather: 1..8 peers, rank inside, pointer tables required");
        return (int)cudaErrorInvalidValue;
    }
    if (M_shard <= 0 || N_Global <= 0 || K_Global <= 0 || (M_shard % 64) || (K_Global % 64) || row_offset < 0 ||
        (row_offset % 8) || (M_full % 8) || row_offset + M_shard > M_full) {
        spb::set_error("spb_spmm_bitmap_v3_allgather: M_shard and K multiples of 64, the shard inside M_full, "
                       "row_offset and M_full multiples of 8 (M_shard=%d K=%d M_full=%d row_offset=%d)",
                       M_shard, K_Global, M_full, row_offset);
        return (int)cudaErrorInvalidValue;
    }
    {
        const cudaError_t chk = spb::check_spmm_args("spb_spmm_bitmap_v3_allgather", Compressed_A, TileOffsets, TileOffsets_Median,
                                                     bitmap, max_nnz_intile, B, M_shard, N_Global, K_Global, Reduction_Workspace,
                                                     Split_K);
        if (chk != cudaSuccess) return (int)chk;
    }
    spb::SpmmArgs a;
    a.vals = Compressed_A;
    a.gtile = TileOffsets;
    a.mtile = TileOffsets_Median;
    a.bitmap = bitmap;
    a.max_nnz = max_nnz_intile;
    a.B = B;
    a.out = nullptr;
    a.M = M_shard;
    a.N = N_Global;
    a.K = K_Global;
    a.split_k = Split_K;
    a.wait_flags = B_flags;
    a.wait_n = n_peers;
    for (int q = 0; q < n_peers; ++q) {
        if (!C_peers[q] || !flag_peers[q] || (reinterpret_cast<uintptr_t>(C_peers[q]) & 15u)) {
            spb::set_error("spb_spmm_bitmap_v3_allgather: peer %d: null or misaligned buffer", q);
            return (int)cudaErrorInvalidValue;
        }
        a.outs[q] = C_peers[q];
        a.flags[q] = flag_peers[q];
    }
    a.n_out = n_peers;
    a.n_flags = n_peers;
    a.ld_out = M_full;
    a.row0 = row_offset;
    a.flag_index = rank;
    a.sequence = flag_peers[rank] + n_peers;  // this rank's own array is local memory
    if (Split_K == 1) return (int)spb::spmm_launch((cudaStream_t)stream, a);
    // Split_K > 1: fp16 partials into the workspace as usual (the SpMM kernel still waits for B's exchange).  When
    // the kernel can fuse the reduction it also stores the rows into the peers' buffers and writes the flags;
    // otherwise the reduction kernel below does.
    bool fused = false;
    a.out = Reduction_Workspace;
    a.reduce_fused = &fused;
    spb::GatherOut g;
    for (int q = 0; q < 8; ++q) {
        g.outs[q] = q < n_peers ? C_peers[q] : nullptr;
        g.flags[q] = q < n_peers ? flag_peers[q] : nullptr;
    }
    g.n = n_peers;
    g.flag_index = rank;
    g.sequence = flag_peers[rank] + n_peers;
    cudaError_t e = spb::exchange_counter((cudaStream_t)stream, &g.done);
    if (e != cudaSuccess) return (int)e;
    e = spb::spmm_launch((cudaStream_t)stream, a);
    if (e != cudaSuccess || fused) return (int)e;
    const size_t mn = (size_t)M_shard * N_Global;
    const unsigned blocks = (unsigned)((mn / 8 + 255) / 256);
    spb::count_launch();
    spb::splitk_reduce_gather_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(g, Reduction_Workspace, M_shard, mn, Split_K,
                                                                             M_full, row_offset);
    return (int)cudaGetLastError();
}

extern "C" int spb_wait_flags(void* stream, uint32_t* flags, int n_peers)
{
    if (!flags || n_peers < 1 || n_peers > 8) {
        spb::set_error("spb_wait_flags: flags and 1..8 peers required");
        return (int)cudaErrorInvalidValue;
    }
    int* status = nullptr;
    cudaError_t e = spb::device_status_ptr(&status);
    if (e != cudaSuccess) return (int)e;
    return (int)spb::wait_flags_launch((cudaStream_t)stream, flags, n_peers, status);
}

// K-split of tensor-parallel inference (out-proj and FC2 in FasterTransformer: every rank holds a slice of the
// weight's columns and the matching slice of the activations, the partial products are summed over the ranks).
// One-shot all-reduce over peer stores: this rank's SpMM writes its fp16 partial [N][M] into slot `rank` of every
// rank's [n_peers][N][M] buffer (the fused all-gather above with the slot as the destination), and every rank then
// sums the n_peers slots of its own buffer.  Nothing is ever loaded from a peer.
extern "C" int spb_spmm_bitmap_v3_allreduce(void* stream, const uint16_t* Compressed_A, const int* TileOffsets,
                                            const int* TileOffsets_Median, const uint64_t* bitmap,
                                            const int* max_nnz_intile, const uint16_t* B, uint16_t* const* part_peers,
                                            uint32_t* const* flag_peers, int n_peers, int rank, int M_Global,
                                            int N_Global, int K_shard, uint32_t* B_flags, uint16_t* Reduction_Workspace,
                                            int Split_K)
{
    if (n_peers < 1 || n_peers > 8 || rank < 0 || rank >= n_peers || !part_peers || !flag_peers || M_Global <= 0 ||
        N_Global <= 0) {
        spb::set_error("spb_spmm_bitmap_v3_allreduce: 1..8 peers, rank inside, pointer tables and positive sizes required");
        return (int)cudaErrorInvalidValue;
    }
    uint16_t* slots[8];
    for (int q = 0; q < n_peers; ++q) {
        if (!part_peers[q]) {
            spb::set_error("spb_spmm_bitmap_v3_allreduce: peer %d: null buffer", q);
            return (int)cudaErrorInvalidValue;
        }
        slots[q] = part_peers[q] + (size_t)rank * M_Global * N_Global;
    }
    return spb_spmm_bitmap_v3_allgather(stream, Compressed_A, TileOffsets, TileOffsets_Median, bitmap, max_nnz_intile, B,
                                        slots, flag_peers, n_peers, rank, M_Global, N_Global, K_shard, M_Global, 0,
                                        B_flags, Reduction_Workspace, Split_K);
}

// Second half of the all-reduce: waits (bounded) until every rank's partial of the current exchange has arrived
// in this rank's buffer, then C = fp16(sum over the ranks, in rank order, of float(partial)), the arithmetic of
// the split-K reduction.
extern "C" int spb_linear_allreduce_finish(void* stream, uint16_t* C, const uint16_t* parts_local, uint32_t* flags_local,
                                           int n_peers, int M_Global, int N_Global, const uint16_t* bias,
                                           const uint16_t* residual, int activation)
{
    if (!flags_local || n_peers < 1 || n_peers > 8) {
        spb::set_error("spb_allreduce_finish: flags and 1..8 peers required");
        return (int)cudaErrorInvalidValue;
    }
    if (!C || !parts_local || M_Global <= 0 || N_Global <= 0 || (M_Global % 64) || !spb::aligned16(C) ||
        !spb::aligned16(parts_local) || !spb::aligned16(bias) || !spb::aligned16(residual) ||
        (activation != 0 && activation != 1)) {
        spb::set_error("spb_allreduce_finish: bad argument");
        return (int)cudaErrorInvalidValue;
    }
    int* status = nullptr;
    cudaError_t e = spb::device_status_ptr(&status);
    if (e != cudaSuccess) return (int)e;
    spb::Epilogue ep;
    ep.bias = bias;
    ep.residual = residual;
    ep.activation = activation;
    // one launch: every block first polls the flags, then sums its part of the slots
    return (int)spb::splitk_reduce((cudaStream_t)stream, C, parts_local, M_Global, N_Global, n_peers, ep, flags_local,
                                   n_peers, status);
}

extern "C" int spb_allreduce_finish(void* stream, uint16_t* C, const uint16_t* parts_local, uint32_t* flags_local,
                                    int n_peers, int M_Global, int N_Global)
{
    return spb_linear_allreduce_finish(stream, C, parts_local, flags_local, n_peers, M_Global, N_Global, nullptr, nullptr, 0);
}
