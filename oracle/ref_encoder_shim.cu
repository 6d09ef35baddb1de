// Builds the reference's own encoder, unmodified, into oracle/_ref/ so the
// test-suite can pin the C restatement (oracle.c) against it.  Nothing is
// copied: the reference header is included from where it lies (the Makefile
// passes its directory with -I) and only a thin extern "C" shim is added.
// Test infrastructure only; never linked into the shipped library.
#include "SpMM_API.cuh"  // reference: csrc/SpMM_API.cuh (InitSparseMatrixA_bitmap at :112)

extern "C" int ref_encode_bitmap_v3(const uint16_t* A, int M, int K, uint16_t** vals, int** tile_nnz,
                                    int** mtile, int** gtile, uint64_t** bitmap, int* max_nnz)
{
    half* v = nullptr;
    int mx = 0;
    // Tile shape arguments as passed by the reference's callers (csrc/SpMM_API.cuh:275).
    int g = InitSparseMatrixA_bitmap(reinterpret_cast<half*>(const_cast<uint16_t*>(A)), M, K, 8, 16, 64, 8, 64, 64,
                                     &v, tile_nnz, mtile, gtile, bitmap, mx);
    *vals = reinterpret_cast<uint16_t*>(v);
    *max_nnz = mx;
    return g;
}

extern "C" void ref_free(void* p) { free(p); }

extern "C" void ref_gen_bin_files(char* dense, int M, int K, char* val, char* gt, char* mt, char* lt, char* in, char* sz)
{
    Our_GenSparseMatrixBinFile(dense, M, K, val, gt, mt, lt, in, sz);
}
