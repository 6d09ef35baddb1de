// A caller written against the reference's header, like its benchmark drivers
// (reference csrc/spmm_test.cu:146-191 encode and upload, :287-303 the SpMM call): it uses only the C++
// symbols SpMM_API.cuh declares and links -lSpMM_API, so it executes the mangled entry points
// FasterTransformer binds, not the extern "C" layer.
//
//   ref_api_caller A.bin B.bin out_prefix M K N Split_K
//
// A.bin: M*K fp16 row-major; B.bin: N*K fp16 ([N][K]).  Writes out_prefix.C.bin ([N][M] fp16) and the encoder's
// arrays out_prefix.{vals,gtile,mtile,bitmap,tile_nnz,max_nnz}.bin for the test to compare with the oracle.
#include "SpMM_API.cuh"

#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#define CHECK(x)                                                                         \
    do {                                                                                 \
        cudaError_t e_ = (x);                                                            \
        if (e_ != cudaSuccess) {                                                         \
            fprintf(stderr, "%s failed: %s\n", #x, cudaGetErrorString(e_));              \
            return 2;                                                                    \
        }                                                                                \
    } while (0)

static bool read_file(const char* path, void* dst, size_t bytes)
{
    FILE* f = fopen(path, "rb");
    if (!f) return false;
    const size_t got = fread(dst, 1, bytes, f);
    fclose(f);
    return got == bytes;
}
static bool write_file(const std::string& path, const void* src, size_t bytes)
{
    FILE* f = fopen(path.c_str(), "wb");
    if (!f) return false;
    const size_t put = bytes ? fwrite(src, 1, bytes, f) : 0;
    fclose(f);
    return put == bytes;
}

int main(int argc, char** argv)
{
    if (argc != 8) {
        fprintf(stderr, "usage: %s A.bin B.bin out_prefix M K N Split_K\n", argv[0]);
        return 1;
    }
    const std::string out = argv[3];
    const int M = atoi(argv[4]), K = atoi(argv[5]), N = atoi(argv[6]), split_k = atoi(argv[7]);
    std::vector<half> A((size_t)M * K), B((size_t)N * K);
    if (!read_file(argv[1], A.data(), A.size() * 2) || !read_file(argv[2], B.data(), B.size() * 2)) {
        fprintf(stderr, "cannot read the inputs\n");
        return 1;
    }
    half* vals = nullptr;
    int *tile_nnz = nullptr, *mtile = nullptr, *gtile = nullptr;
    uint64_t* bitmap = nullptr;
    int max_nnz = 0;
    const int G = InitSparseMatrixA_bitmap(A.data(), M, K, 8, 16, 64, 8, 64, 64, &vals, &tile_nnz, &mtile, &gtile,
                                           &bitmap, max_nnz);
    if (G != (M / 64) * (K / 64)) {
        fprintf(stderr, "InitSparseMatrixA_bitmap returned %d\n", G);
        return 3;
    }
    const size_t val_count = (size_t)gtile[G], nt = (size_t)M * K / 64;
    if (!write_file(out + ".vals.bin", vals, val_count * 2) || !write_file(out + ".gtile.bin", gtile, (size_t)(G + 1) * 4) ||
        !write_file(out + ".mtile.bin", mtile, (size_t)G * 16) || !write_file(out + ".bitmap.bin", bitmap, nt * 8) ||
        !write_file(out + ".tile_nnz.bin", tile_nnz, nt * 4) || !write_file(out + ".max_nnz.bin", &max_nnz, 4))
        return 4;

    half *d_vals, *d_B, *d_C, *d_ws;
    int *d_gtile, *d_mtile, *d_max;
    uint64_t* d_bitmap;
    CHECK(cudaMalloc(&d_vals, val_count ? val_count * 2 : 16));
    CHECK(cudaMalloc(&d_gtile, (size_t)(G + 1) * 4));
    CHECK(cudaMalloc(&d_mtile, (size_t)G * 16));
    CHECK(cudaMalloc(&d_bitmap, nt * 8));
    CHECK(cudaMalloc(&d_max, 4));
    CHECK(cudaMalloc(&d_B, B.size() * 2));
    CHECK(cudaMalloc(&d_C, (size_t)M * N * 2));
    CHECK(cudaMalloc(&d_ws, (size_t)M * N * 2 * (split_k > 1 ? split_k : 1)));
    CHECK(cudaMemcpy(d_vals, vals, val_count * 2, cudaMemcpyHostToDevice));
    CHECK(cudaMemcpy(d_gtile, gtile, (size_t)(G + 1) * 4, cudaMemcpyHostToDevice));
    CHECK(cudaMemcpy(d_mtile, mtile, (size_t)G * 16, cudaMemcpyHostToDevice));
    CHECK(cudaMemcpy(d_bitmap, bitmap, nt * 8, cudaMemcpyHostToDevice));
    CHECK(cudaMemcpy(d_max, &max_nnz, 4, cudaMemcpyHostToDevice));
    CHECK(cudaMemcpy(d_B, B.data(), B.size() * 2, cudaMemcpyHostToDevice));
    CHECK(cudaMemset(d_C, 0xff, (size_t)M * N * 2));
    free(vals);  // the encoder's arrays belong to the caller (reference csrc/spmm_test.cu:187-191)
    free(tile_nnz);
    free(mtile);
    free(gtile);
    free(bitmap);

    // stream 0, A = nullptr as FasterTransformer passes it (reference third_party/ft_spinfer.patch:3736-3749)
    CHECK(SpMM_SplitK_API_bitmap_v3(0, nullptr, d_vals, d_gtile, d_mtile, d_bitmap, d_max, d_B, d_C, M, N, K, d_ws,
                                    split_k));
    CHECK(cudaDeviceSynchronize());
    std::vector<half> C((size_t)M * N);
    CHECK(cudaMemcpy(C.data(), d_C, C.size() * 2, cudaMemcpyDeviceToHost));
    if (!write_file(out + ".C.bin", C.data(), C.size() * 2)) return 4;

    // an N the kernel cannot serve is impossible here (any N >= 1 works); a bad shape must fail without a launch
    if (SpMM_SplitK_API_bitmap_v3(0, nullptr, d_vals, d_gtile, d_mtile, d_bitmap, d_max, d_B, d_C, M + 1, N, K, d_ws, 1) ==
        cudaSuccess) {
        fprintf(stderr, "M = %d was accepted\n", M + 1);
        return 5;
    }
    printf("ok G=%d val_count=%zu max_nnz=%d\n", G, val_count, max_nnz);
    return 0;
}
