/*
 * Restated reference GPU kernel: the structure of cute-rs's tensorop_gemm,
 * written by hand so that it can be timed on a B200 beside the sm_100a kernel.
 *
 * MEASUREMENT BASELINE / TEST INFRASTRUCTURE ONLY, never part of the product.
 * The reference produces this kernel as PTX through an external `mlir-opt`
 * (src/backend/toolchain.rs:195-209), which does not exist in the build
 * image, so its own PTX cannot be generated.  This file follows the kernel's
 * description in examples/tensorop_gemm.rs:51-164 instead:
 *   - grid (M/128, N/128), 128 threads = 2 x 2 warps (:66, :107);
 *   - three stages of a 128 x 32 A tile and a 128 x 32 B tile in shared memory,
 *     49 152 bytes, 16-byte chunks XOR-swizzled with the row (Swizzle<2,3,3>
 *     over 8 x 32 atoms, :83-95);
 *   - global -> shared with 16-byte cp.async.cg, 32 x 4 threads (:98-104);
 *   - shared -> registers with ldmatrix.x4 (A) and ldmatrix.x2 (B) (:117-124);
 *   - mma.sync.m16n8k16, f32 accumulate, each warp 4 x 8 instruction tiles
 *     interleaved over the CTA tile (:107-113, src/atom/mma.rs:289-301);
 *   - one cp.async.wait_group + one barrier per k tile (:136-159);
 *   - two f32 per store in the epilogue, no alpha/beta (:161-162).
 * It is compiled to compute_80 PTX and JIT-compiled by the driver at load, the
 * way the reference's launcher treats its PTX (src/cuda.rs:258-274).
 */
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

constexpr int BM = 128, BN = 128, BK = 32, STAGES = 3, THREADS = 128;
constexpr int TILE = BM * BK;  // elements per operand per stage

// Element offset of (row, k) inside one stage: 64-byte rows, the 16-byte chunk
// index XORed with bits 1-2 of the row.
__device__ __forceinline__ int swz(int row, int k) { return row * BK + ((((k >> 3) ^ (row >> 1)) & 3) << 3) + (k & 7); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t (&r)[2], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
template <bool BF16>
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    if constexpr (BF16)
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
    else
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

template <bool BF16>
__global__ void __launch_bounds__(THREADS) ref_tensorop_gemm_kernel(const uint16_t *__restrict__ A,
                                                                    const uint16_t *__restrict__ B, float *__restrict__ C,
                                                                    int N, int K) {
    __shared__ __align__(128) uint16_t sA[STAGES * TILE];
    __shared__ __align__(128) uint16_t sB[STAGES * TILE];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = warp % 2, wn = warp / 2;
    const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
    const int k_tiles = K / BK;
    const uint32_t sA_u32 = (uint32_t)__cvta_generic_to_shared(sA), sB_u32 = (uint32_t)__cvta_generic_to_shared(sB);

    auto issue = [&](int kt, int stage) {
        const int chunk = tid % 4, row = tid / 4;
#pragma unroll
        for (int g = 0; g < 4; g++) {
            const int r = row + 32 * g;
            cp_async16(sA_u32 + 2u * (stage * TILE + swz(r, chunk * 8)), A + size_t(m0 + r) * K + kt * BK + chunk * 8);
            cp_async16(sB_u32 + 2u * (stage * TILE + swz(r, chunk * 8)), B + size_t(n0 + r) * K + kt * BK + chunk * 8);
        }
    };

    float acc[4][8][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 8; j++)
#pragma unroll
            for (int e = 0; e < 4; e++) acc[i][j][e] = 0.0f;

#pragma unroll
    for (int s = 0; s < STAGES - 1; s++) {
        if (s < k_tiles) issue(s, s);
        asm volatile("cp.async.commit_group;\n" ::);
    }
    for (int kt = 0; kt < k_tiles; kt++) {
        asm volatile("cp.async.wait_group %0;\n" ::"n"(STAGES - 2));
        __syncthreads();
        const int next = kt + STAGES - 1;
        if (next < k_tiles) issue(next, next % STAGES);
        asm volatile("cp.async.commit_group;\n" ::);
        const int stage = kt % STAGES;
#pragma unroll
        for (int kb = 0; kb < BK / 16; kb++) {
            uint32_t a[4][4], b[8][2];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int row = 32 * i + 16 * wm + (lane % 8) + 8 * ((lane / 8) % 2);
                ldmatrix_x4(a[i], sA_u32 + 2u * (stage * TILE + swz(row, kb * 16 + 8 * (lane / 16))));
            }
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const int row = 16 * j + 8 * wn + (lane % 8);
                ldmatrix_x2(b[j], sB_u32 + 2u * (stage * TILE + swz(row, kb * 16 + 8 * ((lane / 8) % 2))));
            }
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int jj = 0; jj < 8; jj++) {
                    const int j = (i & 1) ? 7 - jj : jj;  // serpentine over n (src/atom/mma.rs:503-506)
                    mma16816<BF16>(acc[i][j], a[i], b[j]);
                }
        }
    }
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int row = m0 + 32 * i + 16 * wm + lane / 4, col = n0 + 16 * j + 8 * wn + 2 * (lane % 4);
            *reinterpret_cast<float2 *>(C + size_t(row) * N + col) = make_float2(acc[i][j][0], acc[i][j][1]);
            *reinterpret_cast<float2 *>(C + size_t(row + 8) * N + col) = make_float2(acc[i][j][2], acc[i][j][3]);
        }
}

}  // namespace

/* C (m, n) f32 row-major = A (m, k) * B (n, k)^T, A and B f16 (bf16 = 0) or bf16
 * (bf16 = 1), K-major.  m, n multiples of 128, k of 32, as the reference
 * requires.  Returns the cudaError_t of the launch. */
extern "C" __attribute__((visibility("default"))) int ref_tensorop_gemm(int bf16, int m, int n, int k, const void *dA,
                                                                          const void *dB, void *dC, void *stream) {
    if (m <= 0 || n <= 0 || k <= 0 || m % BM || n % BN || k % BK) return int(cudaErrorInvalidValue);
    const dim3 grid(m / BM, n / BN);
    if (bf16)
        ref_tensorop_gemm_kernel<true><<<grid, THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
            static_cast<const uint16_t *>(dA), static_cast<const uint16_t *>(dB), static_cast<float *>(dC), n, k);
    else
        ref_tensorop_gemm_kernel<false><<<grid, THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
            static_cast<const uint16_t *>(dA), static_cast<const uint16_t *>(dB), static_cast<float *>(dC), n, k);
    return int(cudaGetLastError());
}
