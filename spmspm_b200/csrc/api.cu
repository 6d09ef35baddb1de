// extern "C" layer of libSpMM_API.so (declared in include/spmm_b200.h) and the
// reference-compatible C++ symbols (declared in include/SpMM_API.cuh).
#include "../../include/SpMM_API.cuh"
#include "../../include/spmm_b200.h"
#include "common.cuh"

#include <cstdarg>
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <vector>

namespace spb {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

// One status word per device, living in the library's device image.
__device__ int g_device_status;

cudaError_t device_status_ptr(int** out)
{
    static int* cache[64] = {nullptr};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!cache[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_device_status);
        if (e != cudaSuccess) {
            set_error("cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            return e;
        }
        cache[dev] = static_cast<int*>(p);
    }
    *out = cache[dev];
    return cudaSuccess;
}

static std::atomic<unsigned long long> g_launches{0};
void count_launch(int n) { g_launches.fetch_add((unsigned long long)n, std::memory_order_relaxed); }

bool aligned16(const void* p)
{
    return (reinterpret_cast<uintptr_t>(p) & 15u) == 0;
}

// Shape, null and alignment checks shared by every SpMM entry point: the kernel hands Compressed_A, the median
// offsets and the bitmaps to bulk copies and B to a tensor map, all of which fault on the device when a pointer
// is not 16-byte aligned, so a bad pointer must be turned into an error code here and nothing launched.
cudaError_t check_spmm_args(const char* who, const void* vals, const void* gtile, const void* mtile, const void* bitmap,
                            const void* max_nnz, const void* B, int M, int N, int K, const void* ws, int split_k)
{
    if (M <= 0 || N <= 0 || K <= 0 || (M % 64) || (K % 64)) {
        set_error("%s: M and K must be positive multiples of 64, N positive (M=%d N=%d K=%d)", who, M, N, K);
        return cudaErrorInvalidValue;
    }
    if (split_k < 1 || split_k > K / 64) {
        set_error("%s: Split_K=%d out of range 1..%d", who, split_k, K / 64);
        return cudaErrorInvalidValue;
    }
    if (!vals || !gtile || !mtile || !bitmap || !max_nnz || !B || (split_k > 1 && !ws)) {
        set_error("%s: null device pointer", who);
        return cudaErrorInvalidValue;
    }
    if (!aligned16(vals) || !aligned16(mtile) || !aligned16(bitmap) || !aligned16(B) || (split_k > 1 && !aligned16(ws))) {
        set_error("%s: Compressed_A, TileOffsets_Median, bitmap, B and the workspace must be 16-byte aligned", who);
        return cudaErrorMisalignedAddress;
    }
    if (reinterpret_cast<uintptr_t>(gtile) & 3u) {
        set_error("%s: TileOffsets must be 4-byte aligned", who);
        return cudaErrorMisalignedAddress;
    }
    return cudaSuccess;
}

static cudaError_t spmm_checked(cudaStream_t stream, const uint16_t* vals, const int* gtile, const int* mtile,
                                const uint64_t* bitmap, const int* max_nnz, const uint16_t* B, uint16_t* C, int M,
                                int N, int K, uint16_t* ws, int split_k, const Epilogue& ep = Epilogue())
{
    cudaError_t chk = check_spmm_args("SpMM", vals, gtile, mtile, bitmap, max_nnz, B, M, N, K, ws, split_k);
    if (chk != cudaSuccess) return chk;
    if (ep.activation != 0 && ep.activation != 1) {
        set_error("SpMM: activation must be 0 (none) or 1 (ReLU), got %d", ep.activation);
        return cudaErrorInvalidValue;
    }
    if (!aligned16(ep.bias) || !aligned16(ep.residual)) {
        set_error("SpMM: bias and residual must be 16-byte aligned");
        return cudaErrorMisalignedAddress;
    }
    if (!C) {
        set_error("SpMM: null device pointer");
        return cudaErrorInvalidValue;
    }
    if (!aligned16(C)) {
        set_error("SpMM: C must be 16-byte aligned");
        return cudaErrorMisalignedAddress;
    }
    SpmmArgs a;
    a.vals = vals;
    a.gtile = gtile;
    a.mtile = mtile;
    a.bitmap = bitmap;
    a.max_nnz = max_nnz;
    a.B = B;
    a.out = split_k == 1 ? C : ws;  // reference csrc/SpMM_API.cuh:54-58
    a.M = M;
    a.N = N;
    a.K = K;
    a.split_k = split_k;
    bool fused = false;
    a.final_out = C;
    a.reduce_fused = &fused;
    a.ep = ep;
    cudaError_t e = spmm_launch(stream, a);
    if (e != cudaSuccess || split_k == 1 || fused) return e;
    return splitk_reduce(stream, C, ws, M, N, split_k, ep);
}

// SpMSpM: the compressed second operand (the stored [N][K] activation matrix in the second-operand layout) is
// expanded into a dense array from the stream's memory pool, then the SpMM runs as for a dense B.
static cudaError_t spmspm_checked(cudaStream_t stream, const uint16_t* vals, const int* gtile, const int* mtile,
                                  const uint64_t* bitmap, const int* max_nnz, const uint16_t* vals_b, const int* gtile_b,
                                  const uint64_t* bitmap_b, uint16_t* C, int M, int N, int K, uint16_t* ws, int split_k)
{
    if (!vals_b || !gtile_b || !bitmap_b) {
        set_error("SpMSpM: null pointer for the compressed second operand");
        return cudaErrorInvalidValue;
    }
    if (N <= 0 || K <= 0 || (N % 64) || (K % 64)) {
        set_error("SpMSpM: N and K must be positive multiples of 64 (the second operand is tiled 64 x 64), N=%d K=%d", N, K);
        return cudaErrorInvalidValue;
    }
    int* status = nullptr;
    cudaError_t e = device_status_ptr(&status);
    if (e != cudaSuccess) return e;
    void* dense = nullptr;
    e = cudaMallocAsync(&dense, (size_t)N * K * 2, stream);
    if (e != cudaSuccess) {
        set_error("SpMSpM: no memory for the expanded second operand (%zu bytes)", (size_t)N * K * 2);
        return e;
    }
    e = decode_operand_b(stream, vals_b, gtile_b, bitmap_b, N, K, (uint16_t*)dense, status);
    if (e == cudaSuccess)
        e = spmm_checked(stream, vals, gtile, mtile, bitmap, max_nnz, (const uint16_t*)dense, C, M, N, K, ws, split_k);
    const cudaError_t f = cudaFreeAsync(dense, stream);
    return e != cudaSuccess ? e : f;
}

struct DevBuf {
    void* p = nullptr;
    ~DevBuf()
    {
        if (p) cudaFree(p);
    }
    cudaError_t alloc(size_t n) { return cudaMalloc(&p, n ? n : 16); }
};

static int encode_host_impl(const uint16_t* A_h, int M, int K, uint16_t** vals, int** tile_nnz, int** mtile,
                            int** gtile, uint64_t** bitmap, int* max_nnz, int fmt = kFmtWeight)
{
    const size_t mt_per_g = fmt == kFmtWeight ? 4 : 16;   // median offsets per global tile
    if (!A_h || M <= 0 || K <= 0 || (M % 64) || (K % 64)) {
        set_error("encode: M and K must be positive multiples of 64 (M=%d K=%d)", M, K);
        return -(1000 + (int)cudaErrorInvalidValue);
    }
    const size_t MK = (size_t)M * K;
    const size_t G = (size_t)(M / 64) * (K / 64);
    const size_t nt = MK / 64;
    // Host arrays first, with the reference's sizes (csrc/SpMM_API.cuh:135-139); -1 when any fails (:141-144).
    *tile_nnz = (int*)malloc(nt * sizeof(int));
    *mtile = (int*)calloc(nt, sizeof(int));
    *gtile = (int*)malloc((G + 1) * sizeof(int));
    *bitmap = (uint64_t*)malloc(nt * sizeof(uint64_t));
    *vals = nullptr;
    if (!*tile_nnz || !*mtile || !*gtile || !*bitmap) return -1;

#define SPB_TRY(x)                                                          \
    do {                                                                    \
        cudaError_t e_ = (x);                                               \
        if (e_ != cudaSuccess) {                                            \
            set_error("encode: %s -> %s", #x, cudaGetErrorString(e_));      \
            return -(1000 + (int)e_);                                       \
        }                                                                   \
    } while (0)

    DevBuf dA, dtn, dmt, dgt, dbm, dmx, dscr, dvals, dst;
    SPB_TRY(dA.alloc(MK * 2));
    SPB_TRY(dtn.alloc(nt * 4));
    SPB_TRY(dmt.alloc(G * mt_per_g * 4));
    SPB_TRY(dgt.alloc((G + 1) * 4));
    SPB_TRY(dbm.alloc(nt * 8));
    SPB_TRY(dmx.alloc(4));
    SPB_TRY(dst.alloc(4));
    SPB_TRY(dscr.alloc(encode_scratch_bytes(M, K)));
    cudaStream_t s = 0;
    SPB_TRY(cudaMemcpyAsync(dA.p, A_h, MK * 2, cudaMemcpyHostToDevice, s));
    SPB_TRY(cudaMemsetAsync(dst.p, 0, 4, s));
    SPB_TRY(encode_count_and_scan(s, (const uint16_t*)dA.p, M, K, (int*)dtn.p, (int*)dmt.p, (int*)dgt.p,
                                  (uint64_t*)dbm.p, (int*)dmx.p, dscr.p, fmt));
    int val_count = 0, mx = 0;
    SPB_TRY(cudaMemcpyAsync(&val_count, (int*)dgt.p + G, 4, cudaMemcpyDeviceToHost, s));
    SPB_TRY(cudaMemcpyAsync(&mx, dmx.p, 4, cudaMemcpyDeviceToHost, s));
    SPB_TRY(cudaStreamSynchronize(s));
    *vals = (uint16_t*)malloc(val_count ? (size_t)val_count * 2 : 2);
    if (!*vals) return -1;
    SPB_TRY(dvals.alloc((size_t)val_count * 2));
    SPB_TRY(encode_pack(s, (const uint16_t*)dA.p, M, K, (const int*)dgt.p, (const uint64_t*)dbm.p,
                        (uint16_t*)dvals.p, (size_t)val_count, (int*)dst.p, fmt));
    SPB_TRY(cudaMemcpyAsync(*vals, dvals.p, (size_t)val_count * 2, cudaMemcpyDeviceToHost, s));
    SPB_TRY(cudaMemcpyAsync(*tile_nnz, dtn.p, nt * 4, cudaMemcpyDeviceToHost, s));
    SPB_TRY(cudaMemcpyAsync(*mtile, dmt.p, G * mt_per_g * 4, cudaMemcpyDeviceToHost, s));
    SPB_TRY(cudaMemcpyAsync(*gtile, dgt.p, (G + 1) * 4, cudaMemcpyDeviceToHost, s));
    SPB_TRY(cudaMemcpyAsync(*bitmap, dbm.p, nt * 8, cudaMemcpyDeviceToHost, s));
    SPB_TRY(cudaStreamSynchronize(s));
#undef SPB_TRY
    *max_nnz = mx;
    return (int)G;
}

static int gen_bin_files_impl(const char* dense, int M, int K, const char* valf, const char* gtf, const char* mtf,
                              const char* bmf, const char* mxf, const char* szf, bool exit_on_error)
{
    auto fail = [&](const char* msg) {
        if (exit_on_error) {
            printf("%s\n", msg);
            exit(-1);
        }
        set_error("%s", msg);
        return 1;
    };
    char msg[1024];
    std::vector<uint16_t> host((size_t)M * K);
    {
        std::ifstream in(dense, std::ios::in | std::ios::binary);
        if (!in.is_open()) {
            snprintf(msg, sizeof msg, "file %s cannot be opened, loadDataArrayFromBin fails. ", dense);
            return fail(msg);
        }
        const size_t want = host.size() * 2;
        in.read((char*)host.data(), (std::streamsize)want);
        const size_t got = (size_t)in.gcount();
        if (got != want) {
            snprintf(msg, sizeof msg, "file %s only has %ld, but request %ld, loading DenseMatrix fails! ", dense,
                     (long)got, (long)want);
            return fail(msg);
        }
    }
    uint16_t* vals = nullptr;
    int *tn = nullptr, *mt = nullptr, *gt = nullptr;
    uint64_t* bm = nullptr;
    int mx = 0;
    int G = encode_host_impl(host.data(), M, K, &vals, &tn, &mt, &gt, &bm, &mx);
    if (G < 0) {
        snprintf(msg, sizeof msg, "Our_GenSparseMatrixBinFile() ERROR: encoding failed (%d): %s", G, g_err);
        return fail(msg);
    }
    int val_count = gt[G];
    int num_mtiles = G * 4, num_ltiles = G * 64;
    if (mx % 64 != 0) mx = ((mx / 64) + 1) * 64;  // reference csrc/SpMM_API.cuh:284-286
    if (exit_on_error)
        printf("num_global_tiles: %d, bitmap v3 NNZ: %d, max_nnz_intilev3: %d \n", G, val_count, mx);
    std::ofstream o_sz(szf, std::ios::out | std::ios::binary), o_val(valf, std::ios::out | std::ios::binary),
        o_gt(gtf, std::ios::out | std::ios::binary), o_mt(mtf, std::ios::out | std::ios::binary),
        o_bm(bmf, std::ios::out | std::ios::binary), o_mx(mxf, std::ios::out | std::ios::binary);
    int rc = 0;
    if (!o_sz.is_open() || !o_val.is_open() || !o_gt.is_open() || !o_mt.is_open() || !o_bm.is_open() ||
        !o_mx.is_open()) {
        snprintf(msg, sizeof msg,
                 "Our_GenSparseMatrixBinFile() ERROR: file %s, %s, %s, %s, %s or %s cannot be opened or creaetd. ", szf,
                 valf, gtf, mtf, bmf, mxf);
        rc = fail(msg);
    } else {
        int g1 = G + 1;  // reference csrc/SpMM_API.cuh:304-308: [val_count, G+1, 4G, 64G]
        o_sz.write((char*)&val_count, 4);
        o_sz.write((char*)&g1, 4);
        o_sz.write((char*)&num_mtiles, 4);
        o_sz.write((char*)&num_ltiles, 4);
        o_val.write((char*)vals, (std::streamsize)val_count * 2);
        o_gt.write((char*)gt, (std::streamsize)g1 * 4);
        o_mt.write((char*)mt, (std::streamsize)num_mtiles * 4);
        o_bm.write((char*)bm, (std::streamsize)num_ltiles * 8);
        o_mx.write((char*)&mx, 4);
    }
    free(vals);
    free(tn);
    free(mt);
    free(gt);
    free(bm);
    return rc;
}

// Reads `count` items of `size` bytes from a file that must hold at least that many (the check
// FasterTransformer's loader makes, third_party/ft_spinfer.patch:4773-4810).
static bool read_exact(const char* path, void* dst, size_t size, size_t count, const char* what)
{
    std::ifstream in(path, std::ios::in | std::ios::binary);
    if (!in.is_open()) {
        set_error("load: file %s (%s) cannot be opened", path, what);
        return false;
    }
    in.read((char*)dst, (std::streamsize)(size * count));
    if ((size_t)in.gcount() != size * count) {
        set_error("load: file %s (%s) holds %ld bytes, %ld needed", path, what, (long)in.gcount(), (long)(size * count));
        return false;
    }
    return true;
}

static int load_bin_files_impl(const char* valf, const char* gtf, const char* mtf, const char* bmf, const char* mxf,
                               const char* szf, int M, int K, uint16_t** vals, int** mtile, int** gtile,
                               uint64_t** bitmap, int* max_nnz, int* val_count)
{
    *vals = nullptr;
    *mtile = *gtile = nullptr;
    *bitmap = nullptr;
    if (M <= 0 || K <= 0 || (M % 64) || (K % 64)) {
        set_error("load: M and K must be positive multiples of 64 (M=%d K=%d)", M, K);
        return (int)cudaErrorInvalidValue;
    }
    const long long G = (long long)(M / 64) * (K / 64);
    int sizes[4] = {0, 0, 0, 0};  // [val_count, G+1, 4G, 64G] (reference csrc/SpMM_API.cuh:304-308)
    if (!read_exact(szf, sizes, 4, 4, "OutputSizes")) return (int)cudaErrorInvalidValue;
    if (sizes[0] < 0 || sizes[1] != G + 1 || sizes[2] != 4 * G || sizes[3] != 64 * G) {
        set_error("load: %s says [%d, %d, %d, %d], a %d x %d matrix needs [n, %lld, %lld, %lld]", szf, sizes[0], sizes[1],
                  sizes[2], sizes[3], M, K, G + 1, 4 * G, 64 * G);
        return (int)cudaErrorInvalidValue;
    }
    const size_t n = (size_t)sizes[0];
    uint16_t* v = (uint16_t*)malloc(n ? n * 2 : 16);
    int* gt = (int*)malloc((size_t)(G + 1) * 4);
    int* mt = (int*)malloc((size_t)G * 16);
    uint64_t* bm = (uint64_t*)malloc((size_t)G * 512);
    int mx = 0;
    bool ok = v && gt && mt && bm;
    if (!ok) set_error("load: out of host memory");
    ok = ok && (n == 0 || read_exact(valf, v, 2, n, "NZWeights")) && read_exact(gtf, gt, 4, (size_t)(G + 1), "gtile") &&
         read_exact(mtf, mt, 4, (size_t)(4 * G), "mtile") && read_exact(bmf, bm, 8, (size_t)(64 * G), "ltile") &&
         read_exact(mxf, &mx, 4, 1, "intile");
    if (ok && (gt[0] != 0 || (size_t)gt[G] != n)) {
        set_error("load: global tile offsets run from %d to %d, the value file holds %ld", gt[0], gt[G], (long)n);
        ok = false;
    }
    if (!ok) {
        free(v);
        free(gt);
        free(mt);
        free(bm);
        return (int)cudaErrorInvalidValue;
    }
    *vals = v;
    *gtile = gt;
    *mtile = mt;
    *bitmap = bm;
    *max_nnz = mx;
    *val_count = (int)n;
    return 0;
}

}  // namespace spb

// ================================================================ extern "C" entry points
extern "C" {

int spb_version(void) { return 100; }

const char* spb_last_error(void) { return spb::g_err; }

int spb_encode_host(const uint16_t* A_h, int M, int K, uint16_t** vals, int** tile_nnz, int** mtile, int** gtile,
                    uint64_t** bitmap, int* max_nnz)
{
    if (!vals || !tile_nnz || !mtile || !gtile || !bitmap || !max_nnz) {
        spb::set_error("encode: null output pointer");
        return -(1000 + (int)cudaErrorInvalidValue);
    }
    return spb::encode_host_impl(A_h, M, K, vals, tile_nnz, mtile, gtile, bitmap, max_nnz);
}

int spb_encode_b_host(const uint16_t* B_h, int rows, int cols, uint16_t** vals, int** tile_nnz, int** mtile, int** gtile,
                      uint64_t** bitmap, int* max_nnz)
{
    if (!vals || !tile_nnz || !mtile || !gtile || !bitmap || !max_nnz) {
        spb::set_error("encode: null output pointer");
        return -(1000 + (int)cudaErrorInvalidValue);
    }
    return spb::encode_host_impl(B_h, rows, cols, vals, tile_nnz, mtile, gtile, bitmap, max_nnz, spb::kFmtOperandB);
}

int spb_spmspm_bitmap_v3(void* stream, const uint16_t* Compressed_A, const int* TileOffsets, const int* TileOffsets_Median,
                         const uint64_t* bitmap, const int* max_nnz_intile, const uint16_t* Compressed_B,
                         const int* TileOffsets_B, const uint64_t* bitmap_B, uint16_t* C, int M_Global, int N_Global,
                         int K_Global, uint16_t* Reduction_Workspace, int Split_K)
{
    return (int)spb::spmspm_checked((cudaStream_t)stream, Compressed_A, TileOffsets, TileOffsets_Median, bitmap,
                                    max_nnz_intile, Compressed_B, TileOffsets_B, bitmap_B, C, M_Global, N_Global, K_Global,
                                    Reduction_Workspace, Split_K);
}

void spb_free_host(void* p) { free(p); }

size_t spb_encode_scratch_bytes(int M, int K) { return spb::encode_scratch_bytes(M, K); }

int spb_encode_device(void* stream, const uint16_t* A_d, int M, int K, uint16_t* vals_d, size_t vals_capacity,
                      int* tile_nnz_d, int* mtile_d, int* gtile_d, uint64_t* bitmap_d, int* max_nnz_d, void* scratch_d,
                      int* status_d)
{
    if (M <= 0 || K <= 0 || (M % 64) || (K % 64) || !A_d || !vals_d || !tile_nnz_d || !mtile_d || !gtile_d ||
        !bitmap_d || !max_nnz_d || !scratch_d) {
        spb::set_error("encode_device: bad argument (M=%d K=%d)", M, K);
        return (int)cudaErrorInvalidValue;
    }
    if (!spb::aligned16(A_d) || !spb::aligned16(vals_d)) {
        spb::set_error("encode_device: A and vals must be 16-byte aligned");
        return (int)cudaErrorMisalignedAddress;
    }
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e = spb::encode_count_and_scan(s, A_d, M, K, tile_nnz_d, mtile_d, gtile_d, bitmap_d, max_nnz_d,
                                               scratch_d);
    if (e != cudaSuccess) return (int)e;
    return (int)spb::encode_pack(s, A_d, M, K, gtile_d, bitmap_d, vals_d, vals_capacity, status_d);
}

void Our_GenSparseMatrixBinFile(char* DenseMatrixFileName, int M, int K, char* Compressed_ValFileName,
                                char* bitmap_TileOffsets_globalFileName, char* bitmap_TileOffsets_medianFileName,
                                char* bitmapFileName, char* max_nnz_intileFileName, char* OutputSizesFileName)
{
    spb::gen_bin_files_impl(DenseMatrixFileName, M, K, Compressed_ValFileName, bitmap_TileOffsets_globalFileName,
                            bitmap_TileOffsets_medianFileName, bitmapFileName, max_nnz_intileFileName,
                            OutputSizesFileName, true);
}

int spb_gen_bin_files(const char* dense, int M, int K, const char* val, const char* gtile, const char* mtile,
                      const char* bitmap, const char* max_nnz, const char* sizes)
{
    return spb::gen_bin_files_impl(dense, M, K, val, gtile, mtile, bitmap, max_nnz, sizes, false);
}

int spb_load_bin_files(const char* val, const char* gtile, const char* mtile, const char* bitmap, const char* max_nnz,
                       const char* sizes, int M, int K, uint16_t** vals_out, int** mtile_out, int** gtile_out,
                       uint64_t** bitmap_out, int* max_nnz_out, int* val_count_out)
{
    if (!val || !gtile || !mtile || !bitmap || !max_nnz || !sizes || !vals_out || !mtile_out || !gtile_out ||
        !bitmap_out || !max_nnz_out || !val_count_out) {
        spb::set_error("load: null argument");
        return (int)cudaErrorInvalidValue;
    }
    return spb::load_bin_files_impl(val, gtile, mtile, bitmap, max_nnz, sizes, M, K, vals_out, mtile_out, gtile_out,
                                    bitmap_out, max_nnz_out, val_count_out);
}

int spb_spmm_bitmap_v3(void* stream, const uint16_t* A, const uint16_t* Compressed_A, const int* TileOffsets,
                       const int* TileOffsets_Median, const uint64_t* bitmap, const int* max_nnz_intile,
                       const uint16_t* B, uint16_t* C, int M_Global, int N_Global, int K_Global,
                       uint16_t* Reduction_Workspace, int Split_K)
{
    (void)A;
    return (int)spb::spmm_checked((cudaStream_t)stream, Compressed_A, TileOffsets, TileOffsets_Median, bitmap,
                                  max_nnz_intile, B, C, M_Global, N_Global, K_Global, Reduction_Workspace, Split_K);
}

int spb_linear_bitmap_v3(void* stream, const uint16_t* Compressed_A, const int* TileOffsets, const int* TileOffsets_Median,
                         const uint64_t* bitmap, const int* max_nnz_intile, const uint16_t* B, uint16_t* C, int M_Global,
                         int N_Global, int K_Global, const uint16_t* bias, const uint16_t* residual, int activation,
                         uint16_t* Reduction_Workspace, int Split_K)
{
    spb::Epilogue ep;
    ep.bias = bias;
    ep.residual = residual;
    ep.activation = activation;
    return (int)spb::spmm_checked((cudaStream_t)stream, Compressed_A, TileOffsets, TileOffsets_Median, bitmap,
                                  max_nnz_intile, B, C, M_Global, N_Global, K_Global, Reduction_Workspace, Split_K, ep);
}

int spb_splitk_reduce(void* stream, uint16_t* C, const uint16_t* Reduction_Workspace, int M_Global, int N_Global,
                      int Split_K)
{
    if (!C || !Reduction_Workspace || M_Global <= 0 || N_Global <= 0 || Split_K < 1 || (M_Global % 64) ||
        !spb::aligned16(C) || !spb::aligned16(Reduction_Workspace)) {
        spb::set_error("splitk_reduce: bad argument");
        return (int)cudaErrorInvalidValue;
    }
    return (int)spb::splitk_reduce((cudaStream_t)stream, C, Reduction_Workspace, M_Global, N_Global, Split_K);
}

int spb_suggest_split_k(int M, int N, int K) { return spb::suggest_split_k(M, N, K); }

unsigned long long spb_launch_count(void) { return spb::g_launches.load(); }

int spb_init(void* stream) { return (int)spb::init_stream((cudaStream_t)stream); }

int spb_release(void* stream) { return (int)spb::release_stream((cudaStream_t)stream); }

int spb_set_weight_prefetch(int on) { return spb::set_weight_prefetch(on); }

int spb_set_schedule(int mode)
{
    const int prev = spb::set_schedule(mode);
    if (prev < 0) spb::set_error("spb_set_schedule: mode must be SPB_SCHEDULE_AUTO, SPB_SCHEDULE_STATIC or SPB_SCHEDULE_BALANCED");
    return prev;
}

int spb_device_status(int* status_out)
{
    int* p = nullptr;
    cudaError_t e = spb::device_status_ptr(&p);
    if (e != cudaSuccess) return (int)e;
    e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return (int)e;
    return (int)cudaMemcpy(status_out, p, sizeof(int), cudaMemcpyDeviceToHost);
}

int spb_reset_device_status(void)
{
    int* p = nullptr;
    cudaError_t e = spb::device_status_ptr(&p);
    if (e != cudaSuccess) return (int)e;
    e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return (int)e;
    // a kernel that gave up may have left arrival counters of the balanced schedule behind
    e = spb::reset_schedule_scratch();
    if (e != cudaSuccess) return (int)e;
    return (int)cudaMemset(p, 0, sizeof(int));
}

}  // extern "C"

// ================================================================ reference C++ symbols
// Same signatures (hence the same mangled names) as the functions the reference defines
// inline in csrc/SpMM_API.cuh:47 and :112.

cudaError_t SpMM_SplitK_API_bitmap_v3(cudaStream_t stream, const half* A, const half* Compressed_A,
                                      const int* TileOffsets, const int* TileOffsets_Median, const uint64_t* bitmap,
                                      const int* max_nnz_intile, const half* B, half* C, const int M_Global,
                                      const int N_Global, const int K_Global, half* Reduction_Workspace, int Split_K)
{
    (void)A;
    cudaError_t e = spb::spmm_checked(stream, reinterpret_cast<const uint16_t*>(Compressed_A), TileOffsets,
                                      TileOffsets_Median, bitmap, max_nnz_intile,
                                      reinterpret_cast<const uint16_t*>(B), reinterpret_cast<uint16_t*>(C), M_Global,
                                      N_Global, K_Global, reinterpret_cast<uint16_t*>(Reduction_Workspace), Split_K);
    if (e == cudaErrorInvalidValue || e == cudaErrorMisalignedAddress)
        printf("MM_Sparse_API Error: %s\n", spb::g_err);  // the reference prints and returns an error (:91-94)
    return e;
}

int InitSparseMatrixA_bitmap(half* A_h, int M, int K, int tile_M, int tile_M_median, int tile_M_global, int tile_K,
                             int tile_K_median, int tile_K_global, half** Compressed_Val, int** TileOffsets,
                             int** TileOffsets_median, int** TileOffsets_global, uint64_t** bitmap, int& max_nnz_count)
{
    if (tile_M != 8 || tile_M_median != 16 || tile_M_global != 64 || tile_K != 8 || tile_K_median != 64 ||
        tile_K_global != 64) {
        spb::set_error("InitSparseMatrixA_bitmap: only the tile shape (8,16,64,8,64,64) is supported");
        printf("InitSparseMatrixA_bitmap Error: %s\n", spb::g_err);
        return -1;
    }
    int mx = 0;
    int g = spb::encode_host_impl(reinterpret_cast<const uint16_t*>(A_h), M, K,
                                  reinterpret_cast<uint16_t**>(Compressed_Val), TileOffsets, TileOffsets_median,
                                  TileOffsets_global, bitmap, &mx);
    max_nnz_count = mx;
    return g < 0 ? -1 : g;
}

// The fork's extension: the second operand compressed too (reference csrc/SpMM_API.cuh:47-53, 19 arguments).  The
// dense B passed beside its compressed form is ignored, like A.  The compressed B describes the stored [N][K] matrix
// (what InitSparseMatrixA_bitmap_v6_B makes of it with M = N_Global, K = K_Global).
cudaError_t SpMM_SplitK_API_bitmap_v3(cudaStream_t stream, const half* A, const half* Compressed_A, const int* TileOffsets,
                                      const int* TileOffsets_Median, const uint64_t* bitmap, const int* max_nnz_intile,
                                      const half* B, const half* Compressed_B, const int* TileOffsets_B,
                                      const int* TileOffsets_Median_B, const uint64_t* bitmap_B,
                                      const int* max_nnz_intile_B, half* C, const int M_Global, const int N_Global,
                                      const int K_Global, half* Reduction_Workspace, int Split_K)
{
    (void)A;
    (void)B;
    (void)TileOffsets_Median_B;   // the expansion takes the tile starts from the bitmaps
    (void)max_nnz_intile_B;
    cudaError_t e = spb::spmspm_checked(stream, reinterpret_cast<const uint16_t*>(Compressed_A), TileOffsets, TileOffsets_Median,
                                        bitmap, max_nnz_intile, reinterpret_cast<const uint16_t*>(Compressed_B), TileOffsets_B,
                                        bitmap_B, reinterpret_cast<uint16_t*>(C), M_Global, N_Global, K_Global,
                                        reinterpret_cast<uint16_t*>(Reduction_Workspace), Split_K);
    if (e == cudaErrorInvalidValue || e == cudaErrorMisalignedAddress) printf("MM_Sparse_API Error: %s\n", spb::g_err);
    return e;
}

// reference csrc/spmm_test_utils.h:523-652; only the tile shape its caller passes (csrc/spmm_test.cu:205) is supported
int InitSparseMatrixA_bitmap_v6_B(half* A_h, int M, int K, int tile_M, int tile_M_median, int tile_M_global, int tile_K,
                                  int tile_K_median, int tile_K_global, half** Compressed_Val, int** TileOffsets,
                                  int** TileOffsets_median, int** TileOffsets_global, uint64_t** bitmap, int& max_nnz_count)
{
    if (tile_M != 8 || tile_M_median != 16 || tile_M_global != 64 || tile_K != 8 || tile_K_median != 16 ||
        tile_K_global != 64) {
        spb::set_error("InitSparseMatrixA_bitmap_v6_B: only the tile shape (8,16,64,8,16,64) is supported");
        printf("InitSparseMatrixA_bitmap_v6_B Error: %s\n", spb::g_err);
        return -1;
    }
    int mx = 0;
    int g = spb::encode_host_impl(reinterpret_cast<const uint16_t*>(A_h), M, K,
                                  reinterpret_cast<uint16_t**>(Compressed_Val), TileOffsets, TileOffsets_median,
                                  TileOffsets_global, bitmap, &mx, spb::kFmtOperandB);
    max_nnz_count = mx;
    return g < 0 ? -1 : g;
}
