/*
 * CPU oracle for the cute-rs GEMM / elementwise hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain C, the arithmetic
 * that the reference's CPU simulator (Kernel::simulate) performs for the four
 * kernels on the hot path.  It is the checker the CUDA kernels are compared
 * against and the timed CPU baseline; it is never linked into, loaded by or
 * called from the product library.
 *
 * The reference is a Rust crate and no Rust toolchain exists in the build
 * image, so the reference itself cannot be compiled.  Parity is pinned on the
 * reference's own known-answer tests (integer-valued inputs whose results are
 * exact, see tests/test_oracle.py) and on its published conversion rules.
 *
 * Every function cites the reference file:line (paths inside the cute-rs
 * repository) whose behaviour it follows.
 */
#include <immintrin.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))
#define CLONES __attribute__((target_clones("avx512f", "avx2,fma", "default")))

enum { ORACLE_F16 = 0, ORACLE_BF16 = 1, ORACLE_F32 = 2 };

/* ------------------------------------------------------------------------ */
/* Scalar conversions                                                        */
/* ------------------------------------------------------------------------ */

static inline uint32_t f32_bits(float x) { uint32_t b; memcpy(&b, &x, 4); return b; }
static inline float bits_f32(uint32_t b) { float x; memcpy(&x, &b, 4); return x; }

/* The NaN a single-precision PTX instruction returns: the simulator maps
 * every NaN result of an f32 add, mul or fma to the canonical 0x7fffffff
 * (ptx_nan, src/sim/float.rs:416-428; applied at src/sim/exec.rs:351, 1229). */
static inline float ptx_nan_f32(float r) { return r != r ? bits_f32(0x7fffffffu) : r; }

/* bf16 -> f32: the 16 bits become the high half.  src/value.rs:88-90 */
static inline float bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

/* f32 -> bf16, round to nearest even, NaN keeps its sign and gets the quiet
 * bit.  src/value.rs:92-99 */
static inline uint16_t f32_to_bf16(float x) {
    uint32_t bits = f32_bits(x);
    uint16_t high = (uint16_t)(bits >> 16);
    uint32_t low = bits & 0xffffu;
    if (x != x) return high | 0x40;
    return (uint16_t)(high + ((low > 0x8000u || (low == 0x8000u && (high & 1))) ? 1 : 0));
}

/* f32 -> bf16 as a kernel's own narrowing conversion does it: the same
 * rounding, but a NaN becomes the canonical 0x7fff (cast, src/sim/exec.rs:
 * 430-449). */
static inline uint16_t f32_to_bf16_device(float x) { return x != x ? (uint16_t)0x7fff : f32_to_bf16(x); }

/* f32 -> f16, round to nearest even with subnormals, overflow to infinity and
 * NaN payload kept.  src/value.rs:101-134 */
static inline uint16_t f32_to_f16(float x) {
    uint32_t b = f32_bits(x);
    uint16_t sign = (uint16_t)((b >> 16) & 0x8000u);
    int32_t exp = (int32_t)((b >> 23) & 0xff);
    uint32_t mant = b & 0x7fffffu;
    if (exp == 0xff) {
        uint16_t payload = mant ? (uint16_t)(0x200u | (mant >> 13)) : 0;
        return sign | 0x7c00 | payload;
    }
    int32_t e = exp - 127 + 15;
    if (e >= 0x1f) return sign | 0x7c00;
    if (e <= 0) {
        if (e < -10) return sign;
        uint32_t m = mant | 0x800000u;
        uint32_t shift = (uint32_t)(14 - e);
        uint32_t half = 1u << (shift - 1);
        uint32_t rem = m & ((1u << shift) - 1);
        uint32_t r = m >> shift;
        if (rem > half || (rem == half && (r & 1))) r += 1;
        return sign | (uint16_t)r;
    }
    uint32_t r = ((uint32_t)e << 10) | (mant >> 13);
    uint32_t rem = mant & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (r & 1))) r += 1;
    return sign | (uint16_t)r;
}

/* f16 -> f32, exact.  src/value.rs:136-158 */
static inline float f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)(h & 0x8000u)) << 16;
    uint32_t exp = (h >> 10) & 0x1f;
    uint32_t mant = h & 0x3ff;
    uint32_t bits;
    if (exp == 0) {
        if (mant == 0) {
            bits = sign;
        } else {
            uint32_t e = 127 - 15 + 1, m = mant;
            while ((m & 0x400) == 0) { m <<= 1; e -= 1; }
            bits = sign | (e << 23) | ((m & 0x3ff) << 13);
        }
    } else if (exp == 0x1f) {
        bits = sign | 0x7f800000u | (mant << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (mant << 13);
    }
    return bits_f32(bits);
}

ORACLE_API void oracle_f32_to_f16(const float *src, uint16_t *dst, size_t n) {
    for (size_t i = 0; i < n; i++) dst[i] = f32_to_f16(src[i]);
}
ORACLE_API void oracle_f16_to_f32(const uint16_t *src, float *dst, size_t n) {
    for (size_t i = 0; i < n; i++) dst[i] = f16_to_f32(src[i]);
}
ORACLE_API void oracle_f32_to_bf16(const float *src, uint16_t *dst, size_t n) {
    for (size_t i = 0; i < n; i++) dst[i] = f32_to_bf16(src[i]);
}
ORACLE_API void oracle_bf16_to_f32(const uint16_t *src, float *dst, size_t n) {
    for (size_t i = 0; i < n; i++) dst[i] = bf16_to_f32(src[i]);
}

/* torchrun exports OMP_NUM_THREADS=1; the timed CPU baseline asks for the
 * host's cores explicitly. */
ORACLE_API void oracle_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

ORACLE_API int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ------------------------------------------------------------------------ */
/* elementwise_add                                                           */
/* ------------------------------------------------------------------------ */

/* out[i] = x[i] + y[i] in IEEE binary32, round to nearest even, subnormals
 * kept.  The simulator evaluates BinaryOp::Add on f32 as a host f32 add
 * (src/sim/exec.rs:342-351); the kernel adds every in-bounds element once
 * (examples/elementwise_add.rs:66-78). */
ORACLE_API void oracle_elementwise_add_f32(const float *x, const float *y, float *out, size_t n) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) out[i] = ptx_nan_f32(x[i] + y[i]);
}

/* ------------------------------------------------------------------------ */
/* Epilogue                                                                  */
/* ------------------------------------------------------------------------ */

/* alpha * acc + beta * c with three separate roundings: the sgemm example
 * writes `alpha * acc + beta * c` as two multiplies and an add
 * (examples/sgemm.rs:75-79) and each is a rounded f32 binary op in the
 * simulator (src/sim/exec.rs:342-351).  volatile keeps the compiler from
 * contracting them into an fma. */
static inline float epilogue(float alpha, float acc, float beta, float c_old) {
    volatile float p = ptx_nan_f32(alpha * acc);
    volatile float q = ptx_nan_f32(beta * c_old);
    return ptx_nan_f32(p + q);
}

/* ------------------------------------------------------------------------ */
/* Tensor-core GEMM (tensorop_gemm / runtime_gemm)                           */
/* ------------------------------------------------------------------------ */

#define GT_MR 6   /* rows of C per micro-tile   */
#define GT_NR 64  /* columns of C per micro-tile */

/* One GT_MR x GT_NR block of accumulators over the whole K range.  `ap` is
 * the A block as (k, GT_MR) floats, `bp` the B panel as (k, GT_NR) floats.
 * For every output, acc = acc + a*b with k strictly ascending and one f32
 * rounding per step: the simulator's mma() folds
 * `acc + (a*b as f32)` over kk in order (src/sim/exec.rs:2138) and the kernel
 * feeds it K blocks in ascending order (examples/tensorop_gemm.rs:136-159,
 * src/atom/mma.rs:497-511).  The product of two f16 or two bf16 values is
 * exact in f32, so the rounding of the product is a no-op and only the add
 * rounds. */
typedef float vf16 __attribute__((vector_size(64), aligned(4)));

CLONES static void gemm_tn_micro(const float *ap, const float *bp, size_t k, float *acc /* GT_MR*GT_NR */) {
    vf16 t[GT_MR][GT_NR / 16];
    for (int i = 0; i < GT_MR; i++)
        for (int j = 0; j < GT_NR / 16; j++) t[i][j] = (vf16){0};
    for (size_t kk = 0; kk < k; kk++) {
        const vf16 *b = (const vf16 *)(bp + kk * GT_NR);
        const float *a = ap + kk * GT_MR;
        vf16 b0 = b[0], b1 = b[1], b2 = b[2], b3 = b[3];
#pragma GCC unroll 8
        for (int i = 0; i < GT_MR; i++) {
            float av = a[i];
            t[i][0] = t[i][0] + av * b0;
            t[i][1] = t[i][1] + av * b1;
            t[i][2] = t[i][2] + av * b2;
            t[i][3] = t[i][3] + av * b3;
        }
    }
    memcpy(acc, t, sizeof(t));
}

static inline float load_ab(const void *p, int dtype, size_t idx) {
    const uint16_t *h = (const uint16_t *)p;
    return dtype == ORACLE_F16 ? f16_to_f32(h[idx]) : bf16_to_f32(h[idx]);
}

/* C[m,n] = epilogue(sum_k A[m,k] * B[n,k]).
 *   A: (M, K) row-major (K contiguous), f16 or bf16 bits.
 *   B: (N, K) row-major (K contiguous), same type.
 *   C: (M, N) row-major, f32 or bf16.
 * With alpha == 1 and beta == 0 the accumulator is stored as is and C is
 * never read, like tensorop_gemm's epilogue (examples/tensorop_gemm.rs:161-162).
 * A bf16 C is the f32 result rounded to nearest even, NaN -> 0x7fff (the
 * kernel-side cast, src/sim/exec.rs:430-449; rounding as src/value.rs:92-99).
 * Rows [row_begin, row_end) of C are produced; pass 0, M for all of them.
 * Returns 0, or -1 for an unsupported dtype. */
ORACLE_API int oracle_gemm_tn(int ab_dtype, int c_dtype, size_t M, size_t N, size_t K, const void *A,
                              const void *B, void *C, float alpha, float beta, size_t row_begin,
                              size_t row_end) {
    if ((ab_dtype != ORACLE_F16 && ab_dtype != ORACLE_BF16) || (c_dtype != ORACLE_F32 && c_dtype != ORACLE_BF16))
        return -1;
    if (row_end > M) row_end = M;
    if (row_begin >= row_end || N == 0) return 0;
    const int plain = (alpha == 1.0f && beta == 0.0f);
    size_t n_panels = (N + GT_NR - 1) / GT_NR;
    size_t kpad = K ? K : 1;
    /* B as f32 panels: panel p holds (k, GT_NR) with zero padding past N. */
    float *bpanels = (float *)aligned_alloc(64, n_panels * kpad * GT_NR * sizeof(float));
    if (!bpanels) return -2;
#pragma omp parallel for schedule(static)
    for (size_t p = 0; p < n_panels; p++) {
        float *dst = bpanels + p * kpad * GT_NR;
        for (size_t kk = 0; kk < K; kk++)
            for (size_t j = 0; j < GT_NR; j++) {
                size_t col = p * GT_NR + j;
                dst[kk * GT_NR + j] = col < N ? load_ab(B, ab_dtype, col * K + kk) : 0.0f;
            }
    }
    size_t rows = row_end - row_begin;
    size_t m_blocks = (rows + GT_MR - 1) / GT_MR;
#pragma omp parallel
    {
        float *ap = (float *)aligned_alloc(64, kpad * GT_MR * sizeof(float));
        float acc[GT_MR * GT_NR];
#pragma omp for schedule(dynamic, 4)
        for (size_t mb = 0; mb < m_blocks; mb++) {
            size_t r0 = row_begin + mb * GT_MR;
            for (size_t kk = 0; kk < K; kk++)
                for (size_t i = 0; i < GT_MR; i++)
                    ap[kk * GT_MR + i] = (r0 + i < row_end) ? load_ab(A, ab_dtype, (r0 + i) * K + kk) : 0.0f;
            for (size_t p = 0; p < n_panels; p++) {
                gemm_tn_micro(ap, bpanels + p * kpad * GT_NR, K, acc);
                for (size_t i = 0; i < GT_MR && r0 + i < row_end; i++)
                    for (size_t j = 0; j < GT_NR && p * GT_NR + j < N; j++) {
                        size_t idx = (r0 + i) * N + p * GT_NR + j;
                        float v = acc[i * GT_NR + j];
                        if (c_dtype == ORACLE_F32) {
                            float *c = (float *)C;
                            c[idx] = plain ? v : epilogue(alpha, v, beta, c[idx]);
                        } else {
                            uint16_t *c = (uint16_t *)C;
                            c[idx] = f32_to_bf16_device(plain ? v : epilogue(alpha, v, beta, bf16_to_f32(c[idx])));
                        }
                    }
            }
        }
        free(ap);
    }
    free(bpanels);
    return 0;
}

/* sum_k |A[m,k]| * |B[n,k]| accumulated like oracle_gemm_tn, as f32 (M, N):
 * the magnitude the reference's tolerance is scaled by.  Its GPU test runs
 * the same kernel on |A| and |B| (tests/gpu.rs:159-175). */
ORACLE_API int oracle_gemm_tn_abs(int ab_dtype, size_t M, size_t N, size_t K, const void *A, const void *B,
                                  float *mag, size_t row_begin, size_t row_end) {
    size_t na = M * K, nb = N * K;
    uint16_t *a2 = (uint16_t *)malloc((na ? na : 1) * 2), *b2 = (uint16_t *)malloc((nb ? nb : 1) * 2);
    if (!a2 || !b2) { free(a2); free(b2); return -2; }
    const uint16_t *a = (const uint16_t *)A, *b = (const uint16_t *)B;
    for (size_t i = 0; i < na; i++) a2[i] = a[i] & 0x7fff;
    for (size_t i = 0; i < nb; i++) b2[i] = b[i] & 0x7fff;
    int rc = oracle_gemm_tn(ab_dtype, ORACLE_F32, M, N, K, a2, b2, mag, 1.0f, 0.0f, row_begin, row_end);
    free(a2);
    free(b2);
    return rc;
}

/* ------------------------------------------------------------------------ */
/* SIMT sgemm (sgemm_nt)                                                     */
/* ------------------------------------------------------------------------ */

#define SG_MR 64 /* rows (contiguous in memory) per micro-tile */
#define SG_NR 4  /* columns per micro-tile */

/* acc = fma(a, b, acc), k ascending, one rounding per step:
 * MmaOp::UniversalFma lowers to Op::Fma (src/atom/mma.rs:522-526), which the
 * simulator evaluates with f32::mul_add (src/sim/exec.rs:1214-1231). */
__attribute__((target("avx512f"))) static void sgemm_micro_avx512(const float *A, const float *B, size_t M,
                                                                  size_t N, size_t K, size_t i0, size_t j0,
                                                                  float *acc) {
    __m512 t[SG_NR][SG_MR / 16];
    for (int j = 0; j < SG_NR; j++)
        for (int i = 0; i < SG_MR / 16; i++) t[j][i] = _mm512_setzero_ps();
    for (size_t kk = 0; kk < K; kk++) {
        const float *a = A + kk * M + i0;
        const float *b = B + kk * N + j0;
        __m512 a0 = _mm512_loadu_ps(a), a1 = _mm512_loadu_ps(a + 16), a2 = _mm512_loadu_ps(a + 32),
               a3 = _mm512_loadu_ps(a + 48);
#pragma GCC unroll 8
        for (int j = 0; j < SG_NR; j++) {
            __m512 bv = _mm512_set1_ps(b[j]);
            t[j][0] = _mm512_fmadd_ps(a0, bv, t[j][0]);
            t[j][1] = _mm512_fmadd_ps(a1, bv, t[j][1]);
            t[j][2] = _mm512_fmadd_ps(a2, bv, t[j][2]);
            t[j][3] = _mm512_fmadd_ps(a3, bv, t[j][3]);
        }
    }
    for (int j = 0; j < SG_NR; j++)
        for (int i = 0; i < SG_MR / 16; i++) _mm512_storeu_ps(acc + j * SG_MR + i * 16, t[j][i]);
}

__attribute__((target("avx2,fma"))) static void sgemm_micro_avx2(const float *A, const float *B, size_t M, size_t N,
                                                                 size_t K, size_t i0, size_t j0, float *acc) {
    /* two passes of 32 rows keep the accumulators in the 16 ymm registers */
    for (int half = 0; half < 2; half++) {
        __m256 t[SG_NR][4];
        for (int j = 0; j < SG_NR; j++)
            for (int i = 0; i < 4; i++) t[j][i] = _mm256_setzero_ps();
        for (size_t kk = 0; kk < K; kk++) {
            const float *a = A + kk * M + i0 + half * 32;
            const float *b = B + kk * N + j0;
            __m256 a0 = _mm256_loadu_ps(a), a1 = _mm256_loadu_ps(a + 8), a2 = _mm256_loadu_ps(a + 16),
                   a3 = _mm256_loadu_ps(a + 24);
#pragma GCC unroll 8
            for (int j = 0; j < SG_NR; j++) {
                __m256 bv = _mm256_set1_ps(b[j]);
                t[j][0] = _mm256_fmadd_ps(a0, bv, t[j][0]);
                t[j][1] = _mm256_fmadd_ps(a1, bv, t[j][1]);
                t[j][2] = _mm256_fmadd_ps(a2, bv, t[j][2]);
                t[j][3] = _mm256_fmadd_ps(a3, bv, t[j][3]);
            }
        }
        for (int j = 0; j < SG_NR; j++)
            for (int i = 0; i < 4; i++) _mm256_storeu_ps(acc + j * SG_MR + half * 32 + i * 8, t[j][i]);
    }
}

static void sgemm_micro_scalar(const float *A, const float *B, size_t M, size_t N, size_t K, size_t i0, size_t j0,
                               float *acc) {
    for (int j = 0; j < SG_NR; j++)
        for (int i = 0; i < SG_MR; i++) {
            float t = 0.0f;
            for (size_t kk = 0; kk < K; kk++) t = fmaf(A[kk * M + i0 + i], B[kk * N + j0 + j], t);
            acc[j * SG_MR + i] = t;
        }
}

static void sgemm_micro(const float *A, const float *B, size_t M, size_t N, size_t K, size_t i0, size_t j0,
                        float *acc /* SG_NR*SG_MR, column-major */) {
    if (__builtin_cpu_supports("avx512f")) sgemm_micro_avx512(A, B, M, N, K, i0, j0, acc);
    else if (__builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma")) sgemm_micro_avx2(A, B, M, N, K, i0, j0, acc);
    else sgemm_micro_scalar(A, B, M, N, K, i0, j0, acc);
}

/* C = alpha * (A * B^T) + beta * C, everything f32 and column-major:
 * A (M, K) with a[i + k*M], B (N, K) with b[j + k*N], C (M, N) with
 * c[i + j*M] (examples/sgemm.rs:28-33).  The epilogue always reads C
 * (examples/sgemm.rs:75-79).  M must be a multiple of 64 and N of 4 (the
 * reference kernel needs multiples of 128).  Returns 0 or -1. */
ORACLE_API int oracle_sgemm_nt(size_t M, size_t N, size_t K, float alpha, float beta, const float *A,
                               const float *B, float *C) {
    if (M % SG_MR || N % SG_NR) return -1;
    size_t mt = M / SG_MR, nt = N / SG_NR;
#pragma omp parallel
    {
        float acc[SG_NR * SG_MR];
#pragma omp for schedule(dynamic, 8) collapse(2)
        for (size_t jb = 0; jb < nt; jb++)
            for (size_t ib = 0; ib < mt; ib++) {
                sgemm_micro(A, B, M, N, K, ib * SG_MR, jb * SG_NR, acc);
                for (size_t j = 0; j < SG_NR; j++)
                    for (size_t i = 0; i < SG_MR; i++) {
                        size_t idx = (ib * SG_MR + i) + (jb * SG_NR + j) * M;
                        /* a NaN accumulator is the canonical one: every fma step maps NaN to it */
                        C[idx] = epilogue(alpha, ptx_nan_f32(acc[j * SG_MR + i]), beta, C[idx]);
                    }
            }
    }
    return 0;
}

/* ------------------------------------------------------------------------ */
/* Deliberately naive forms, used only to cross-check the blocked ones       */
/* ------------------------------------------------------------------------ */

/* The reference examples' own host check: `(0..k).map(|l| a*b).sum()` in f32
 * (examples/tensorop_gemm.rs:180-185).  One output element. */
ORACLE_API float oracle_gemm_tn_naive_elem(int ab_dtype, size_t K, const void *A, const void *B, size_t i,
                                           size_t j) {
    volatile float acc = 0.0f;
    for (size_t kk = 0; kk < K; kk++) {
        volatile float p = load_ab(A, ab_dtype, i * K + kk) * load_ab(B, ab_dtype, j * K + kk);
        acc = acc + p;
    }
    return acc;
}

ORACLE_API float oracle_sgemm_nt_naive_elem(size_t M, size_t N, size_t K, float alpha, float beta,
                                            const float *A, const float *B, float c_old, size_t i, size_t j) {
    float acc = 0.0f;
    for (size_t kk = 0; kk < K; kk++) acc = ptx_nan_f32(fmaf(A[i + kk * M], B[j + kk * N], acc));
    return epilogue(alpha, acc, beta, c_old);
}
