// Reference-style comparator: the SpInfer mma.sync / cp.async SpMM for a dense activation matrix, rebuilt from the
// reference's own device functions so that it can be timed on the same GPU and used as a second numerics pin.
//
// TEST AND BENCHMARK INFRASTRUCTURE ONLY.  Built into oracle/_ref/ by the Makefile beside this file, from the
// reference's headers where they lie (-I<reference>/csrc); never linked into the shipped library.
//
// Why glue is needed: the reference tree holds the kernel only in its work-in-progress form, where the
// activation matrix is bitmap-compressed too (reference csrc/SpMM_Kernel.cuh:18-199).  The 14-argument entry
// point that FasterTransformer calls takes a dense B, and every device function that version is made of is
// still in the tree.  This file puts them together the way the reference's loop does:
//   weight side, unchanged      bitmap and value copies   reference csrc/MatMulUtilities.cuh:111-137
//                               bitmap -> A fragments     reference csrc/MatMulUtilities.cuh:27-57
//                               split-K ranges            reference csrc/SpMM_Kernel.cuh:28-46
//                               C fragments -> smem -> C  reference csrc/MatMulUtilities.cuh:346-382, SpMM_Kernel.cuh:186-198
//   activation side, dense B    swizzled tile copy        addressing of reference csrc/MatMulUtilities.cuh:80-109
//                               ldmatrix B fragments      reference csrc/MMA_PTX.cuh:90-118
//                               k-step loop               reference csrc/MatMulUtilities.cuh:139-162 with the B
//                                                         fragments loaded as in :195-231
//   launcher                    tile configuration by N   reference csrc/SpMM_API.cuh:60-96, grid :33-36
//   reduction                   SplitK_Reduction          reference csrc/Reduction_Kernel.cuh:24-44
#include "MatMulUtilities.cuh"
#include "Reduction_Kernel.cuh"

#include <cstdio>

namespace {

// One 8-row copy unit per warp and pass, 16 bytes per lane, column index XOR-ed with the row (the layout
// B_FragLoadFromSharedToRegisters expects); the copies are only issued here, the caller commits and waits.
template <int Rows, typename TilingConfig>
__device__ __forceinline__ void issue_b_tile_copy(half* __restrict__ shared, const half* global, int stride, bool pred)
{
    const int lane = threadIdx.x % 32, warp = threadIdx.x / 32;
    const int col = lane % 8, row1 = lane / 8, row2 = lane / 8 + 4;
    constexpr int kUnits = Rows / COPY_UNIT_FP16_ROWS;
#pragma unroll
    for (int u = warp; u < kUnits; u += TilingConfig::BLOCK_WARPS) {
        const half* g = global + u * COPY_UNIT_FP16_ROWS * stride;
        half* s = shared + u * COPY_UNIT_FP16_ROWS * TILE_K;
        cp_async<16>(s + (col ^ row1) * HALF_PER_128B + row1 * TILE_K, g + col * HALF_PER_128B + row1 * stride, pred);
        cp_async<16>(s + (col ^ row2) * HALF_PER_128B + row2 * TILE_K, g + col * HALF_PER_128B + row2 * stride, pred);
    }
}

template <typename TilingConfig>
__global__ void ref_style_spmm_kernel(const half* Compressed_A, const int* TileOffsets, const int* TileOffsets_Median,
                                      const uint64_t* bitmap, const half* B, half* Reduction_Workspace, int M_Global,
                                      int N_Global, int K_Global, int Split_K, int a_halves)
{
    // split-K ranges: reference csrc/SpMM_Kernel.cuh:30-46
    const int BatchID = blockIdx.y / (M_Global / TilingConfig::TILE_M);
    const int IsLastBatch = (BatchID == (Split_K - 1));
    const int x = blockIdx.x;
    const int y = blockIdx.y % (M_Global / TilingConfig::TILE_M);
    const int NumKBlock = K_Global / TILE_K;
    const int AverageNumKBlock = (NumKBlock - 1) / Split_K + 1;
    const int PaddingKBlock = AverageNumKBlock * Split_K - NumKBlock;
    const int NumIter = IsLastBatch ? AverageNumKBlock - PaddingKBlock : AverageNumKBlock;
    const int BlockOffset = K_Global / TILE_K * y + BatchID * AverageNumKBlock;
    const int* TileOffsets_ThisBlock = TileOffsets + BlockOffset;

    extern __shared__ __align__(128) half smem[];
    half* smem_B = smem + a_halves;                                                    // two activation tiles
    uint64_t* smem_Bitmap = reinterpret_cast<uint64_t*>(smem_B + 2 * TilingConfig::TILE_N * TILE_K);

    const unsigned int warpId = threadIdx.x / WARP_SIZE;
    const int Tile_Start_M = y * TilingConfig::TILE_M;
    const int Tile_Start_N = x * TilingConfig::TILE_N;
    const int Warp_i = warpId / TilingConfig::BLOCK_COL_WARPS;
    uint32_t a[WARP_ROW_TENSORS_BITMAP_V3 * BLOCK_K_TENSORS][4];
    uint32_t b[TilingConfig::WARP_COL_TENSORS][4];
    uint64_t* smem_BitmapWarp = smem_Bitmap + Warp_i * 16;
    const int* TileOffsets_ThisWarp = TileOffsets_Median + BlockOffset * 4 + Warp_i;
    const uint64_t* BitmapTileGlobalPTR =
        bitmap + (size_t)y * TilingConfig::TILE_BITMAP_M_V3 * K_Global + BatchID * AverageNumKBlock * TilingConfig::TILE_BITMAP_K_V3;
    const half* BTileGlobalPTR = B + (size_t)Tile_Start_N * K_Global + BatchID * AverageNumKBlock * TILE_K;

    float c[WARP_ROW_TENSORS_BITMAP_V3 * TilingConfig::WARP_COL_TENSORS][REG_PER_C_TENSOR_16_16];
    for (int i = 0; i < WARP_ROW_TENSORS_BITMAP_V3 * TilingConfig::WARP_COL_TENSORS; i++)
        for (int j = 0; j < REG_PER_C_TENSOR_16_16; j++) c[i][j] = 0.0f;

    if (NumIter > 0) {
        // first k-tile: bitmaps and values of A, then the activation tile
        CopyTileFromGlobalToShared_Bitmap_1_64<TilingConfig::TILE_BITMAP_M_V3, TilingConfig>(smem_Bitmap, BitmapTileGlobalPTR);
        CopyTileFromGlobalToShared_Sparse<TilingConfig>(smem, Compressed_A + TileOffsets_ThisBlock[0],
                                                        TileOffsets_ThisBlock[1] - TileOffsets_ThisBlock[0]);
        cp_async_group_commit();
        issue_b_tile_copy<TilingConfig::TILE_N, TilingConfig>(smem_B, BTileGlobalPTR, K_Global, true);
        cp_async_group_commit();
        cp_async_wait_group<1>();
        __syncthreads();
        SpMM_LoadFragAwithBitmapFromShem(a, smem + TileOffsets_ThisWarp[0], smem_BitmapWarp);
        cp_async_wait_group<0>();
        __syncthreads();
    }
#pragma unroll(1)
    for (int tile_id_k = 0; tile_id_k < NumIter; tile_id_k++) {
        BitmapTileGlobalPTR += TilingConfig::TILE_BITMAP_K_V3;
        BTileGlobalPTR += TILE_K;
        const bool GlobalCopy = (tile_id_k + 1) < NumIter;
        // TileOffsets holds one entry more than there are global tiles, so [tile_id_k + 2] is in bounds whenever
        // the next k-tile exists; the loads are skipped otherwise
        const int next_start = GlobalCopy ? TileOffsets_ThisBlock[tile_id_k + 1] : 0;
        const int next_nnz = GlobalCopy ? TileOffsets_ThisBlock[tile_id_k + 2] - next_start : 0;
        half* smem_write_B = smem_B + ((tile_id_k + 1) % 2) * (TilingConfig::TILE_N * TILE_K);
        half* smem_read_B = smem_B + ((tile_id_k) % 2) * (TilingConfig::TILE_N * TILE_K);
        // next k-tile: A overwrites its buffer (its fragments are in registers), B goes to the other buffer
        CopyTileFromGlobalToShared_Bitmap_1_64<TilingConfig::TILE_BITMAP_M_V3, TilingConfig>(smem_Bitmap, BitmapTileGlobalPTR, GlobalCopy);
        CopyTileFromGlobalToShared_Sparse<TilingConfig>(smem, Compressed_A + next_start, next_nnz, GlobalCopy);
        cp_async_group_commit();
        issue_b_tile_copy<TilingConfig::TILE_N, TilingConfig>(smem_write_B, BTileGlobalPTR, K_Global, GlobalCopy);
        cp_async_group_commit();
        // the four k-steps of this k-tile
        uint32_t(*c_u)[REG_PER_C_TENSOR_16_16] = reinterpret_cast<uint32_t(*)[REG_PER_C_TENSOR_16_16]>(c);
#pragma unroll
        for (int k = 0; k < BLOCK_K_TENSORS; k++) {
            B_FragLoadFromSharedToRegisters<TilingConfig::WARP_COL_TENSORS, TilingConfig::N8>(b, smem_read_B, 0, k * MMA_K);
#pragma unroll
            for (int j = 0; j < TilingConfig::WARP_COL_TENSORS; j++) {
                MMA_FP16_M16N8K16(c_u[j * WARP_ROW_TENSORS_BITMAP_V3], a[k], b[j]);
                if (!TilingConfig::N8) MMA_FP16_M16N8K16(c_u[j * WARP_ROW_TENSORS_BITMAP_V3] + 4, a[k], b[j] + 2);
            }
        }
        cp_async_wait_group<1>();
        __syncthreads();
        SpMM_LoadFragAwithBitmapFromShem(a, smem + (GlobalCopy ? TileOffsets_ThisWarp[(tile_id_k + 1) * 4] : 0), smem_BitmapWarp, GlobalCopy);
        cp_async_wait_group<0>();
        __syncthreads();
    }
    // C fragments -> shared memory -> fp16, column-major: reference csrc/SpMM_Kernel.cuh:186-198
    float(*smem_CFrag)[TilingConfig::TILE_M + PADDING_SHARED_MEM_FOR_C] =
        reinterpret_cast<float(*)[TilingConfig::TILE_M + PADDING_SHARED_MEM_FOR_C]>(smem);
    StoreToSharedMemoryFromRegisterBitmapV3<TilingConfig>(smem_CFrag, c);
    __syncthreads();
    half* BlockGlobalPTR = Reduction_Workspace + (size_t)BatchID * M_Global * N_Global + Tile_Start_M + (size_t)Tile_Start_N * M_Global;
    for (int i = warpId; i < TilingConfig::TILE_N2; i += TilingConfig::BLOCK_WARPS)
        for (int j = threadIdx.x % WARP_SIZE; j < TilingConfig::TILE_M; j += WARP_SIZE)
            BlockGlobalPTR[j + (size_t)i * M_Global] = __float2half_rn((*(smem_CFrag + i))[j]);
}

template <typename TilingConfig>
cudaError_t launch(cudaStream_t stream, const half* vals, const int* gtile, const int* mtile, const uint64_t* bitmap,
                   const half* B, half* out, int M, int N, int K, int split_k, int max_nnz)
{
    const int a_halves = (max_nnz + 63) / 64 * 64;  // as the reference's file writer rounds it (csrc/SpMM_API.cuh:284-286)
    const int smem_main = a_halves * 2 + 2 * TilingConfig::TILE_N * TILE_K * 2 + 64 * 8;
    const int smem_c = (TilingConfig::TILE_M + PADDING_SHARED_MEM_FOR_C) * TilingConfig::TILE_N * 4;
    const int smem = smem_main > smem_c ? smem_main : smem_c;
    cudaError_t e = cudaFuncSetAttribute(ref_style_spmm_kernel<TilingConfig>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    const int dimN = N / TilingConfig::TILE_N > 1 ? N / TilingConfig::TILE_N : 1;  // reference csrc/SpMM_API.cuh:33
    dim3 grid(dimN, M * split_k / TilingConfig::TILE_M, 1), block(WARP_SIZE * TilingConfig::BLOCK_WARPS, 1, 1);
    ref_style_spmm_kernel<TilingConfig><<<grid, block, smem, stream>>>(vals, gtile, mtile, bitmap, B, out, M, N, K, split_k, a_halves);
    return cudaGetLastError();
}

}  // namespace

// Same arguments as the reference's 14-argument entry point without the unused A, plus max_nnz as a host value
// (the kernel's shared-memory carve-up needs it at launch; the reference hard-codes a bound, csrc/SpMM_API.cuh:28).
// N must be 8, 16, 32, 64 or a multiple of 128 (reference csrc/SpMM_API.cuh:60-96); for N = 8 the kernel copies a
// 16-row activation tile, so B must be readable for 16 rows.  Requires M % 64 == 0, K % 64 == 0 and, with
// Split_K > 1, M * N % 256 == 0, like the reference.
extern "C" int ref_style_spmm(void* stream, const void* vals, const int* gtile, const int* mtile, const uint64_t* bitmap,
                              const void* B, void* C, int M, int N, int K, void* workspace, int split_k, int max_nnz)
{
    cudaStream_t s = (cudaStream_t)stream;
    const half* v = (const half*)vals;
    const half* b = (const half*)B;
    half* out = split_k == 1 ? (half*)C : (half*)workspace;
    if (M % 64 || K % 64 || split_k < 1 || (split_k > 1 && (M * (long long)N) % 256)) return (int)cudaErrorInvalidValue;
    cudaError_t e;
    if (N == 8)
        e = launch<TilingConfigBitmapV3<4, 1, 1, 1>>(s, v, gtile, mtile, bitmap, b, out, M, N, K, split_k, max_nnz);
    else if (N == 16)
        e = launch<TilingConfigBitmapV3<4, 1, 1>>(s, v, gtile, mtile, bitmap, b, out, M, N, K, split_k, max_nnz);
    else if (N == 32)
        e = launch<TilingConfigBitmapV3<4, 1, 2>>(s, v, gtile, mtile, bitmap, b, out, M, N, K, split_k, max_nnz);
    else if (N == 64 || (N > 0 && N % 128 == 0))
        e = launch<TilingConfigBitmapV3<4, 1, 4>>(s, v, gtile, mtile, bitmap, b, out, M, N, K, split_k, max_nnz);
    else
        return (int)cudaErrorInvalidValue;
    if (e != cudaSuccess || split_k == 1) return (int)e;
    SplitK_Reduction<<<dim3((unsigned)((long long)M * N / 256)), dim3(WARP_SIZE), 0, s>>>((half*)C, (half*)workspace, M, N, split_k);
    return (int)cudaGetLastError();
}
