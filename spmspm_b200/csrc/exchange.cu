// Fused SpMM + all-gather over peer memory, for the M-split of tensor-parallel inference (the weight's rows are
// sharded over the GPUs, every GPU needs all output rows; FasterTransformer does this with an NCCL all-gather
// after the GEMM, third_party/ft_spinfer.patch:623-862).  The SpMM kernel's epilogue stores its output rows
// straight into every GPU's [N][M] buffer with plain stores through NVLink, and the last CTA to finish writes
// the launch's sequence number into every GPU's flag array.  A consumer waits, with a bounded number of polls,
// until its own flag array shows the current sequence number from every rank.  No load ever touches peer memory.
#include "../../include/spmm_b200.h"
#include "common.cuh"

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

}  // namespace

cudaError_t wait_flags_launch(cudaStream_t s, uint32_t* flags, int n, int* status)
{
    wait_flags_kernel<<<1, 32, 0, s>>>(flags, n, status);
    return cudaGetLastError();
}

}  // namespace spb

extern "C" int spb_spmm_bitmap_v3_allgather(void* stream, const uint16_t* Compressed_A, const int* TileOffsets,
                                            const int* TileOffsets_Median, const uint64_t* bitmap,
                                            const int* max_nnz_intile, const uint16_t* B, uint16_t* const* C_peers,
                                            uint32_t* const* flag_peers, int n_peers, int rank, int M_shard,
                                            int N_Global, int K_Global, int M_full, int row_offset,
                                            uint32_t* B_flags)
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
    if (!Compressed_A || !TileOffsets || !TileOffsets_Median || !bitmap || !max_nnz_intile || !B) {
        spb::set_error("spb_spmm_bitmap_v3_allgather: null device pointer");
        return (int)cudaErrorInvalidValue;
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
    a.split_k = 1;
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
    a.wait_flags = B_flags;
    a.wait_n = n_peers;
    return (int)spb::spmm_launch((cudaStream_t)stream, a);
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
