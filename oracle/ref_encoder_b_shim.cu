// Builds the fork's encoder for a compressed second operand, unmodified, into oracle/_ref/ so that the test-suite can
// pin the C restatement (oracle_encode_bitmap_v6_b) and the library's GPU encoder against it.  Nothing is copied: the
// reference header is included from where it lies (the Makefile passes its directory with -I).
// Test infrastructure only; never linked into the shipped library.
#include "spmm_test_utils.h"  // reference: csrc/spmm_test_utils.h (InitSparseMatrixA_bitmap_v6_B at :523)

extern "C" int ref_encode_bitmap_v6_b(const uint16_t* A, int M, int K, uint16_t** vals, int** tile_nnz, int** mtile,
                                      int** gtile, uint64_t** bitmap, int* max_nnz)
{
    half* v = nullptr;
    int mx = 0;
    // Tile shape arguments as passed by the reference's caller (csrc/spmm_test.cu:205).
    int g = InitSparseMatrixA_bitmap_v6_B(reinterpret_cast<half*>(const_cast<uint16_t*>(A)), M, K, 8, 16, 64, 8, 16, 64, &v,
                                          tile_nnz, mtile, gtile, bitmap, mx);
    *vals = reinterpret_cast<uint16_t*>(v);
    *max_nnz = mx;
    return g;
}

extern "C" void ref_b_free(void* p) { free(p); }
