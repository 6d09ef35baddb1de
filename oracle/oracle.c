/*
 * CPU oracle for the bitmap-v3 sparse format and the SpMM that consumes it.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is a plain-C restatement of the
 * reference algorithm, used as the checker by the test-suite, the smoke test
 * and the CPU-baseline leg of the benchmark.  The shipped library never calls
 * into it and has no CPU fallback.
 *
 * Parity pin: the encoder restated here is compared bit-for-bit against the
 * reference's own InitSparseMatrixA_bitmap (compiled unmodified into
 * oracle/_ref by oracle/Makefile) and against the committed fixtures under
 * tests/golden/, which were produced by that compiled reference.  The SpMM
 * numerics have no golden vectors in the reference (its drivers only print a
 * summed error against cuBLAS), so for the floating-point part the pin is the
 * fp32 GEMM below: "parity unpinned by reference vectors" for that part.
 *
 * Each function cites the reference file:line it follows (paths are relative
 * to the reference project root).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* ---------------------------------------------------------------- fp16 --- */

/* IEEE binary16 -> binary32, exact (what host-side __half2float does). */
float oracle_h2f(uint16_t h)
{
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: normalise */
            int e = -1;
            do {
                man <<= 1;
                e++;
            } while (!(man & 0x400u));
            man &= 0x3ffu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* binary32 -> binary16, round-to-nearest-even (__float2half_rn). */
uint16_t oracle_f2h(float f)
{
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t absx = x & 0x7fffffffu;
    if (absx > 0x7f800000u) /* NaN */
        return (uint16_t)(sign | 0x7e00u | ((absx >> 13) & 0x3ffu));
    if (absx >= 0x477ff000u) /* 65520 and above (and inf) round to inf */
        return (uint16_t)(sign | 0x7c00u);
    if (absx < 0x33000001u) /* below half of the smallest subnormal */
        return (uint16_t)sign;
    int e = (int)(absx >> 23) - 127;
    uint32_t man = (absx & 0x7fffffu) | 0x800000u;
    int shift;
    uint32_t hexp;
    if (e < -14) { /* subnormal result */
        shift = 13 + (-14 - e);
        hexp = 0;
    } else {
        shift = 13;
        hexp = (uint32_t)(e + 15);
    }
    uint32_t q = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u)))
        q++;
    uint32_t out;
    if (hexp == 0)
        out = q; /* a carry into bit 10 correctly yields the smallest normal */
    else
        out = ((hexp - 1) << 10) + q; /* q carries the implicit 1 at bit 10 */
    return (uint16_t)(sign | out);
}

/* ------------------------------------------------------------- encoder --- */

/*
 * Position of the t-th 8x8 tile inside a 64x64 global tile, in the order the
 * reference encoder walks them (csrc/SpMM_API.cuh:162-176): four 16-row
 * "median" tiles top to bottom; inside each, four 16x16 groups left to right;
 * inside each group the 8x8 tiles go (rows 0-7,k 0-7), (rows 8-15,k 0-7),
 * (rows 0-7,k 8-15), (rows 8-15,k 8-15).
 */
static void tile_origin(int t, int *row, int *col)
{
    int m = t >> 4, g = (t >> 2) & 3, j = (t >> 1) & 1, i = t & 1;
    *row = 16 * m + 8 * i;
    *col = 16 * g + 8 * j;
}

/*
 * Restates InitSparseMatrixA_bitmap (csrc/SpMM_API.cuh:112-241) for the only
 * tile shape its callers use (8,16,64,8,64,64; csrc/SpMM_API.cuh:275).
 * M and K must be multiples of 64.
 *
 * Outputs (caller-allocated):
 *   vals        capacity M*K + 7*G halves is always enough
 *   tile_nnz    M*K/64 ints, non-zero count of each 8x8 tile   (ref "TileOffsets", :201)
 *   mtile       4*G ints, start of each median tile in its global tile (:160, :207-211)
 *   gtile       G+1 ints, exclusive prefix of padded global-tile counts (:231-235)
 *   bitmap      M*K/64 uint64, bit r*8+c of tile (:190)
 *   max_nnz     max padded count over global tiles (:224-226)
 * Returns G, the number of 64x64 global tiles (:240).
 */
int oracle_encode_bitmap_v3(const uint16_t *A, int M, int K, uint16_t *vals, int *tile_nnz,
                            int *mtile, int *gtile, uint64_t *bitmap, int *max_nnz)
{
    int GM = M / 64, GK = K / 64;
    int G = GM * GK;
    int val_count = 0;
    int mx = 0;
    gtile[0] = 0;
    for (int gm = 0; gm < GM; ++gm) {
        for (int gk = 0; gk < GK; ++gk) {
            int g = gm * GK + gk;
            int in_gtile = 0;
            for (int t = 0; t < 64; ++t) {
                if ((t & 15) == 0)
                    mtile[4 * g + (t >> 4)] = in_gtile;
                int r0, c0;
                tile_origin(t, &r0, &c0);
                uint64_t bm = 0;
                int cnt = 0;
                for (int r = 0; r < 8; ++r) {
                    const uint16_t *src = A + (size_t)(gm * 64 + r0 + r) * K + gk * 64 + c0;
                    for (int c = 0; c < 8; ++c) {
                        uint16_t h = src[c];
                        /* :189 keeps every value whose float image is != 0.0f:
                         * +-0 are dropped, NaN and subnormals are kept. */
                        if ((h & 0x7fffu) != 0) {
                            bm |= 1ull << (r * 8 + c);
                            vals[val_count++] = h;
                            cnt++;
                        }
                    }
                }
                bitmap[(size_t)g * 64 + t] = bm;
                tile_nnz[(size_t)g * 64 + t] = cnt;
                in_gtile += cnt;
            }
            /* :216-220 pad the global tile's values to a multiple of 8 halves */
            while (in_gtile & 7) {
                vals[val_count++] = 0;
                in_gtile++;
            }
            if (in_gtile > mx)
                mx = in_gtile;
            gtile[g + 1] = val_count;
        }
    }
    *max_nnz = mx;
    return G;
}

/*
 * Inverse of the encoder; follows the consumer side, i.e. the offset rules of
 * SpMM_LoadFragAwithBitmapFromShem / maskloadingv1
 * (csrc/MatMulUtilities.cuh:27-57): inside a median tile the 16 tiles' values
 * are consecutive, and element (r,c) of a tile sits at
 * popcount(bitmap & ((1<<(8r+c))-1)) from the tile's start.  The median tile's
 * start comes from mtile[], the global tile's start from gtile[]
 * (csrc/SpMM_Kernel.cuh:44-46, 77-79, 92-94).
 */
void oracle_decode_bitmap_v3(const uint16_t *vals, const int *mtile, const int *gtile,
                             const uint64_t *bitmap, int M, int K, uint16_t *A_out)
{
    int GM = M / 64, GK = K / 64;
#pragma omp parallel for schedule(static)
    for (int gm = 0; gm < GM; ++gm)
        for (int gk = 0; gk < GK; ++gk) {
            int g = gm * GK + gk;
            for (int m = 0; m < 4; ++m) {
                int pos = gtile[g] + mtile[4 * g + m];
                for (int u = 0; u < 16; ++u) {
                    int t = 16 * m + u;
                    int r0, c0;
                    tile_origin(t, &r0, &c0);
                    uint64_t bm = bitmap[(size_t)g * 64 + t];
                    for (int b = 0; b < 64; ++b) {
                        uint16_t h = 0;
                        if ((bm >> b) & 1ull)
                            h = vals[pos++];
                        A_out[(size_t)(gm * 64 + r0 + (b >> 3)) * K + gk * 64 + c0 + (b & 7)] = h;
                    }
                }
            }
        }
}

/* ---------------------------------------------- second-operand layout ---- */

/*
 * Position of the t-th 8x8 tile inside a 64x64 global tile in the order of the fork's encoder for a compressed
 * second operand, InitSparseMatrixA_bitmap_v6_B (csrc/spmm_test_utils.h:523-652) with the tile shape its caller
 * passes (8,16,64,8,16,64; csrc/spmm_test.cu:205): median tiles of 16 x 16, walked column by column (:566-567:
 * median_tile_k outer, median_tile_m inner); inside a median tile the four 8x8 tiles row-major (:575-578: i = row
 * half outer, j = column half inner).
 */
static void tile_origin_b(int t, int *row, int *col)
{
    int mk = t >> 4, mm = (t >> 2) & 3, i = (t >> 1) & 1, j = t & 1;
    *row = 16 * mm + 8 * i;
    *col = 16 * mk + 8 * j;
}

/*
 * Restates InitSparseMatrixA_bitmap_v6_B (csrc/spmm_test_utils.h:523-652).  Input row-major [M][K].  Outputs as
 * oracle_encode_bitmap_v3 except mtile: 16 ints per global tile, the first 0 (:564), then the running count after
 * every median tile but the last (:617-621).  Zero test (:589), bit position (:590), padding to 8 (:626-630),
 * max_nnz (:634-636), global offsets (:641-645) as in the weight encoder.
 */
int oracle_encode_bitmap_v6_b(const uint16_t *A, int M, int K, uint16_t *vals, int *tile_nnz, int *mtile, int *gtile,
                              uint64_t *bitmap, int *max_nnz)
{
    int GM = M / 64, GK = K / 64, G = GM * GK, val_count = 0, mx = 0;
    gtile[0] = 0;
    for (int gm = 0; gm < GM; ++gm)
        for (int gk = 0; gk < GK; ++gk) {
            int g = gm * GK + gk, in_gtile = 0;
            for (int t = 0; t < 64; ++t) {
                if ((t & 3) == 0)
                    mtile[16 * g + (t >> 2)] = in_gtile;
                int r0, c0;
                tile_origin_b(t, &r0, &c0);
                uint64_t bm = 0;
                int cnt = 0;
                for (int r = 0; r < 8; ++r) {
                    const uint16_t *src = A + (size_t)(gm * 64 + r0 + r) * K + gk * 64 + c0;
                    for (int c = 0; c < 8; ++c) {
                        uint16_t h = src[c];
                        if ((h & 0x7fffu) != 0) {
                            bm |= 1ull << (r * 8 + c);
                            vals[val_count++] = h;
                            cnt++;
                        }
                    }
                }
                bitmap[(size_t)g * 64 + t] = bm;
                tile_nnz[(size_t)g * 64 + t] = cnt;
                in_gtile += cnt;
            }
            while (in_gtile & 7) {
                vals[val_count++] = 0;
                in_gtile++;
            }
            if (in_gtile > mx)
                mx = in_gtile;
            gtile[g + 1] = val_count;
        }
    *max_nnz = mx;
    return G;
}

/* Inverse of the above: the tiles of a global tile are consecutive in storage order, element (r,c) of a tile sits
 * popcount(bitmap & ((1 << (8r+c)) - 1)) values after the tile's start. */
void oracle_decode_bitmap_v6_b(const uint16_t *vals, const int *gtile, const uint64_t *bitmap, int M, int K,
                               uint16_t *A_out)
{
    int GM = M / 64, GK = K / 64;
    for (int gm = 0; gm < GM; ++gm)
        for (int gk = 0; gk < GK; ++gk) {
            int g = gm * GK + gk, pos = gtile[g];
            for (int t = 0; t < 64; ++t) {
                int r0, c0;
                tile_origin_b(t, &r0, &c0);
                uint64_t bm = bitmap[(size_t)g * 64 + t];
                for (int b = 0; b < 64; ++b) {
                    uint16_t h = 0;
                    if ((bm >> b) & 1ull)
                        h = vals[pos++];
                    A_out[(size_t)(gm * 64 + r0 + (b >> 3)) * K + gk * 64 + c0 + (b & 7)] = h;
                }
            }
        }
}

/* --------------------------------------------------------------- GEMM ---- */

/*
 * fp32 host GEMM in the layouts of the reference kernel: A row-major [M][K]
 * fp16, B column-major K x N (stored [N][K], the cuBLAS call at
 * csrc/spmm_test.cu:101-102 uses ldb = K), C column-major M x N (stored
 * [N][M], csrc/SpMM_Kernel.cuh:192-198).  The reference itself validates
 * against cuBLAS, not a host GEMM; this restates the same product in fp32
 * (products exact in fp32, summed in double to make the checker's own error
 * negligible).
 */
void oracle_gemm_f32(const uint16_t *A, const uint16_t *B, float *C, int M, int N, int K)
{
    float *Bf = (float *)malloc((size_t)N * K * sizeof(float));
    for (size_t i = 0; i < (size_t)N * K; ++i)
        Bf[i] = oracle_h2f(B[i]);
#pragma omp parallel
    {
        float *row = (float *)malloc((size_t)K * sizeof(float));
#pragma omp for schedule(static)
        for (int m = 0; m < M; ++m) {
            for (int k = 0; k < K; ++k)
                row[k] = oracle_h2f(A[(size_t)m * K + k]);
            for (int n = 0; n < N; ++n) {
                const float *b = Bf + (size_t)n * K;
                double acc = 0.0;
                for (int k = 0; k < K; ++k)
                    acc += (double)(row[k] * b[k]);
                C[(size_t)n * M + m] = (float)acc;
            }
        }
        free(row);
    }
    free(Bf);
}

/* Same product, computed straight from the compressed form (skips zeros). */
void oracle_spmm_f32(const uint16_t *vals, const int *mtile, const int *gtile,
                     const uint64_t *bitmap, const uint16_t *B, float *C, int M, int N, int K)
{
    uint16_t *A = (uint16_t *)malloc((size_t)M * K * sizeof(uint16_t));
    oracle_decode_bitmap_v3(vals, mtile, gtile, bitmap, M, K, A);
    oracle_gemm_f32(A, B, C, M, N, K);
    free(A);
}

/*
 * The reference's split-K arithmetic: k-tiles of 64 are cut into Split_K
 * ranges of ceil((K/64)/Split_K) tiles, the last one shorter
 * (csrc/SpMM_Kernel.cuh:35-43); each range is accumulated in fp32 and rounded
 * to fp16 (:198); the partials are then summed in fp32 in range order and
 * rounded to fp16 (csrc/Reduction_Kernel.cuh:24-44).  With split_k == 1 the
 * single range is rounded once.  Output is fp16, column-major M x N.
 */
void oracle_spmm_splitk_f16(const uint16_t *A, const uint16_t *B, uint16_t *C, int M, int N, int K,
                            int split_k)
{
    int kt = K / 64;
    int avg = (kt - 1) / split_k + 1;
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m)
        for (int n = 0; n < N; ++n) {
            float total = 0.f;
            for (int s = 0; s < split_k; ++s) {
                int k0 = s * avg * 64, k1 = (s + 1) * avg * 64;
                if (k1 > K)
                    k1 = K;
                double acc = 0.0;
                for (int k = k0; k < k1; ++k)
                    acc += (double)(oracle_h2f(A[(size_t)m * K + k]) * oracle_h2f(B[(size_t)n * K + k]));
                if (split_k == 1)
                    total = (float)acc;
                else
                    total += oracle_h2f(oracle_f2h((float)acc));
            }
            C[(size_t)n * M + m] = oracle_f2h(total);
        }
}

/* Reduction alone (csrc/Reduction_Kernel.cuh:24-44): fp16 partials
 * [split_k][N*M] summed in fp32 in index order, rounded to fp16. */
void oracle_splitk_reduce(const uint16_t *partials, uint16_t *C, int M, int N, int split_k)
{
    size_t mn = (size_t)M * N;
    for (size_t e = 0; e < mn; ++e) {
        float acc = 0.f;
        for (int s = 0; s < split_k; ++s)
            acc += oracle_h2f(partials[(size_t)s * mn + e]);
        C[e] = oracle_f2h(acc);
    }
}

/* The reference drivers' only correctness figure: sum |a-b| over fp16 outputs
 * (csrc/spmm_test_utils.h:110-115). */
double oracle_total_error(const uint16_t *a, const uint16_t *b, size_t n)
{
    double e = 0.0;
    for (size_t i = 0; i < n; ++i)
        e += fabs((double)oracle_h2f(a[i]) - (double)oracle_h2f(b[i]));
    return e;
}

/* Number of OpenMP threads the GEMMs of this file use from now on (a launcher may have exported
 * OMP_NUM_THREADS=1 for its children; the timed CPU baseline wants all cores of the box). */
void oracle_set_num_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int oracle_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
