// sgemm_nt for sm_100a: C = alpha * A * B^T + beta * C, all f32, column-major
// (a[i + l*m], b[j + l*n], c[i + j*m]).
//
// This is a CUDA-core kernel on purpose.  The reference accumulates every
// output with fma.rn.f32 in ascending l and finishes with mul, mul, add
// (examples/sgemm.rs:23-81; UniversalFma -> Op::Fma, src/atom/mma.rs:522-526),
// and its GPU test demands the bits of the simulator (tests/gpu.rs:249-253).
// Tensor cores cannot reproduce that rounding sequence, so the arithmetic
// stays on the FP32 pipe and the bound is the FFMA rate, not HBM:
// 2*m*n*k flops against 4*(m*k + n*k + 2*m*n) bytes.
//
// Shape: a CTA of 256 threads owns a BM x BN tile of C; both operand tiles are
// contiguous along m / n in global memory, so they stream into shared memory
// as (BK, BM) and (BK, BN) panels with 16-byte cp.async through a multi-stage
// ring, and each thread keeps a (TM x TN) block of accumulators as two 4-wide
// strips per dimension so that every shared-memory read is a conflict-free
// 128-bit load.
#include "common.cuh"

namespace cb {
namespace {

constexpr int BM = 128, BN = 128, BK = 16, STAGES = 3, THREADS = 256;
constexpr int TM = 8, TN = 8;
constexpr int A_STAGE = BK * BM, B_STAGE = BK * BN;  // floats
constexpr int SMEM_BYTES = STAGES * (A_STAGE + B_STAGE) * 4;

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, bool valid) {
    // src-size 0 writes 16 zero bytes: rows of the K tail contribute
    // fma(0, 0, acc) == acc (acc is never -0: it starts at +0).
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(valid ? 16 : 0));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__global__ void __launch_bounds__(THREADS, 2)
    sgemm_nt_kernel(int M, int N, int K, float alpha, float beta, const float *__restrict__ A,
                    const float *__restrict__ B, float *__restrict__ C) {
    extern __shared__ __align__(16) float smem[];
    float *sA = smem;                     // [STAGES][BK][BM]
    float *sB = smem + STAGES * A_STAGE;  // [STAGES][BK][BN]

    const int tid = threadIdx.x;
    const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
    const int tx = tid % 16, ty = tid / 16;  // 16 x 16 threads, 8 x 8 outputs each
    const int k_tiles = (K + BK - 1) / BK;

    // Loader mapping: a (BK, 128) panel is 16 rows of 32 float4; 256 threads
    // move two float4 each.
    const int ld_row = tid / 32, ld_col = (tid % 32) * 4;
    const uint32_t sA_u32 = (uint32_t)__cvta_generic_to_shared(sA);
    const uint32_t sB_u32 = (uint32_t)__cvta_generic_to_shared(sB);

    auto load_tile = [&](int kt, int stage) {
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int kr = ld_row + h * 8;
            const int kg = kt * BK + kr;
            const bool ok = kg < K;
            const size_t kk = ok ? size_t(kg) : 0;
            cp_async16(sA_u32 + 4u * (stage * A_STAGE + kr * BM + ld_col), A + kk * M + m0 + ld_col, ok);
            cp_async16(sB_u32 + 4u * (stage * B_STAGE + kr * BN + ld_col), B + kk * N + n0 + ld_col, ok);
        }
    };

    // acc2[p][j] holds rows 2p and 2p+1 of column j: the packed form feeds
    // fma.rn.f32x2, two IEEE fused multiply-adds per issue slot (measured on
    // 4096^3: 59.0 TFLOP/s against 55.8 with scalar fma.rn.f32; same bits).
    float2 acc2[TM / 2][TN];
#pragma unroll
    for (int i = 0; i < TM / 2; i++)
#pragma unroll
        for (int j = 0; j < TN; j++) acc2[i][j] = make_float2(0.0f, 0.0f);

#pragma unroll
    for (int s = 0; s < STAGES - 1; s++) {
        if (s < k_tiles) load_tile(s, s);
        cp_async_commit();
    }

    for (int kt = 0; kt < k_tiles; kt++) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();
        const int next = kt + STAGES - 1;
        if (next < k_tiles) load_tile(next, next % STAGES);
        cp_async_commit();

        const float *a_s = sA + (kt % STAGES) * A_STAGE;
        const float *b_s = sB + (kt % STAGES) * B_STAGE;
#pragma unroll
        for (int kk = 0; kk < BK; kk++) {
            const float4 a0 = *reinterpret_cast<const float4 *>(a_s + kk * BM + tx * 4);
            const float4 a1 = *reinterpret_cast<const float4 *>(a_s + kk * BM + 64 + tx * 4);
            const float4 b0 = *reinterpret_cast<const float4 *>(b_s + kk * BN + ty * 4);
            const float4 b1 = *reinterpret_cast<const float4 *>(b_s + kk * BN + 64 + ty * 4);
            const float2 a2[TM / 2] = {make_float2(a0.x, a0.y), make_float2(a0.z, a0.w), make_float2(a1.x, a1.y),
                                       make_float2(a1.z, a1.w)};
            const float b[TN] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int j = 0; j < TN; j++) {
                const float2 bb = make_float2(b[j], b[j]);
#pragma unroll
                for (int i = 0; i < TM / 2; i++) {
                    acc2[i][j] = __ffma2_rn(a2[i], bb, acc2[i][j]);
                }
            }
        }
    }
    cp_async_wait<0>();

    // Epilogue: alpha * acc + beta * c as mul, mul, add (three roundings).
#pragma unroll
    for (int j = 0; j < TN; j++) {
        const int col = n0 + (j / 4) * 64 + ty * 4 + (j % 4);
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int row = m0 + h * 64 + tx * 4;
            float4 *p = reinterpret_cast<float4 *>(C + size_t(col) * M + row);
            const float4 c = *p;
            float4 r;
            r.x = __fadd_rn(__fmul_rn(alpha, acc2[h * 2][j].x), __fmul_rn(beta, c.x));
            r.y = __fadd_rn(__fmul_rn(alpha, acc2[h * 2][j].y), __fmul_rn(beta, c.y));
            r.z = __fadd_rn(__fmul_rn(alpha, acc2[h * 2 + 1][j].x), __fmul_rn(beta, c.z));
            r.w = __fadd_rn(__fmul_rn(alpha, acc2[h * 2 + 1][j].y), __fmul_rn(beta, c.w));
            *p = r;
        }
    }
}

}  // namespace

cute_b200_status sgemm_nt_init(const DeviceState &) {
    CB_CUDA(cudaFuncSetAttribute(sgemm_nt_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    return CUTE_B200_OK;
}

cute_b200_status sgemm_nt(int m, int n, int k, float alpha, float beta, const float *a, const float *b, float *c,
                          cudaStream_t stream, const DeviceState &) {
    if (m <= 0 || n <= 0 || k < 0)
        return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "sgemm_nt: invalid size %dx%dx%d", m, n, k);
    if (m % BM || n % BN)
        return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "sgemm_nt: problem size must be a multiple of the tile size (%d x %d), got %d x %d",
                    BM, BN, m, n);
    if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c)) & 15u)
        return fail(CUTE_B200_ERR_MISALIGNED, "sgemm_nt: buffers must be 16-byte aligned");
    if (n / BN > 65535) return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "sgemm_nt: n too large");
    sgemm_nt_kernel<<<dim3(m / BM, n / BN), THREADS, SMEM_BYTES, stream>>>(m, n, k, alpha, beta, a, b, c);
    CB_CUDA(cudaGetLastError());
    count_launch();
    return CUTE_B200_OK;
}

}  // namespace cb
