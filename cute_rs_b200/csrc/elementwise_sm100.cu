// elementwise_add for sm_100a: out[i] = x[i] + y[i], f32.
//
// The kernel is bound by HBM traffic (12 bytes per element), so the whole
// design is about keeping enough wide requests in flight per SM: every thread
// issues all of its loads (64 bytes from x, 64 from y) before the first add,
// accesses are fully coalesced (256-bit per lane where the pointers share a
// 32-byte phase, 128-bit otherwise) and the streaming cache policy keeps the
// three 1 GiB arrays of the headline case from evicting each other in L2.
//
// Arithmetic: one add.rn.f32 per element, no flush-to-zero (this file is
// built without fast-math), which is what the reference kernel computes
// (examples/elementwise_add.rs:23-80; simulator add src/sim/exec.rs:342-351).
// Elements at index >= n are never read or written: the role the identity
// tensor predicate plays in the reference's tiled kernel
// (examples/elementwise_add.rs:66-78).
#include "common.cuh"

namespace cb {
namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;  // float4 per thread per array
constexpr uint64_t kVecPerBlock = uint64_t(kThreads) * kUnroll;

// Vector body: x4/y4/o4 are 16-byte aligned and n4 float4 long.  The scalar
// head (elements before the first aligned one) and tail (n % 4 leftovers)
// are done by block 0, at most 3 + 3 elements.
__global__ void __launch_bounds__(kThreads) add_f32_vec(const float4 *__restrict__ x4, const float4 *__restrict__ y4,
                                                        float4 *__restrict__ o4, uint64_t n4, const float *xs,
                                                        const float *ys, float *os, uint32_t head, uint64_t tail_begin,
                                                        uint64_t n) {
    const uint64_t base = uint64_t(blockIdx.x) * kVecPerBlock + threadIdx.x;
    if (base + uint64_t(kUnroll - 1) * kThreads < n4) {
        float4 a[kUnroll], b[kUnroll];
#pragma unroll
        for (int j = 0; j < kUnroll; j++) a[j] = __ldcs(x4 + base + uint64_t(j) * kThreads);
#pragma unroll
        for (int j = 0; j < kUnroll; j++) b[j] = __ldcs(y4 + base + uint64_t(j) * kThreads);
#pragma unroll
        for (int j = 0; j < kUnroll; j++) {
            float4 r;
            r.x = __fadd_rn(a[j].x, b[j].x);
            r.y = __fadd_rn(a[j].y, b[j].y);
            r.z = __fadd_rn(a[j].z, b[j].z);
            r.w = __fadd_rn(a[j].w, b[j].w);
            __stcs(o4 + base + uint64_t(j) * kThreads, r);
        }
    } else {
#pragma unroll
        for (int j = 0; j < kUnroll; j++) {
            const uint64_t i = base + uint64_t(j) * kThreads;
            if (i < n4) {
                const float4 a = __ldcs(x4 + i), b = __ldcs(y4 + i);
                float4 r;
                r.x = __fadd_rn(a.x, b.x);
                r.y = __fadd_rn(a.y, b.y);
                r.z = __fadd_rn(a.z, b.z);
                r.w = __fadd_rn(a.w, b.w);
                __stcs(o4 + i, r);
            }
        }
    }
    if (blockIdx.x == 0) {
        if (threadIdx.x < head) os[threadIdx.x] = __fadd_rn(xs[threadIdx.x], ys[threadIdx.x]);
        const uint64_t t = tail_begin + threadIdx.x;
        if (threadIdx.x < 4 && t < n) os[t] = __fadd_rn(xs[t], ys[t]);
    }
}

// 256-bit variant (sm_100 ld/st.global.v8): half as many requests for the same
// bytes.  x8/y8/o8 are 32-byte aligned and n8 groups of eight floats long; the
// head (up to 7 elements) and the tail (n % 8) are done by block 0.
struct alignas(32) float8 {
    float v[8];
};
__device__ __forceinline__ float8 ld_cs_v8(const float8 *p) {
    float8 r;
    asm volatile("ld.global.cs.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=f"(r.v[0]), "=f"(r.v[1]), "=f"(r.v[2]), "=f"(r.v[3]), "=f"(r.v[4]), "=f"(r.v[5]), "=f"(r.v[6]), "=f"(r.v[7])
                 : "l"(p));
    return r;
}
__device__ __forceinline__ void st_cs_v8(float8 *p, const float8 &a, const float8 &b) {
    asm volatile("st.global.cs.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "f"(__fadd_rn(a.v[0], b.v[0])),
                 "f"(__fadd_rn(a.v[1], b.v[1])), "f"(__fadd_rn(a.v[2], b.v[2])), "f"(__fadd_rn(a.v[3], b.v[3])),
                 "f"(__fadd_rn(a.v[4], b.v[4])), "f"(__fadd_rn(a.v[5], b.v[5])), "f"(__fadd_rn(a.v[6], b.v[6])),
                 "f"(__fadd_rn(a.v[7], b.v[7]))
                 : "memory");
}
constexpr int kUnroll8 = 2;  // float8 per thread per array: the same 64 bytes per array as the 128-bit kernel
__global__ void __launch_bounds__(kThreads) add_f32_vec8(const float8 *__restrict__ x8, const float8 *__restrict__ y8,
                                                         float8 *__restrict__ o8, uint64_t n8, const float *xs,
                                                         const float *ys, float *os, uint32_t head, uint64_t tail_begin,
                                                         uint64_t n) {
    const uint64_t base = uint64_t(blockIdx.x) * (uint64_t(kThreads) * kUnroll8) + threadIdx.x;
    if (base + uint64_t(kUnroll8 - 1) * kThreads < n8) {
        float8 a[kUnroll8], b[kUnroll8];
#pragma unroll
        for (int j = 0; j < kUnroll8; j++) a[j] = ld_cs_v8(x8 + base + uint64_t(j) * kThreads);
#pragma unroll
        for (int j = 0; j < kUnroll8; j++) b[j] = ld_cs_v8(y8 + base + uint64_t(j) * kThreads);
#pragma unroll
        for (int j = 0; j < kUnroll8; j++) st_cs_v8(o8 + base + uint64_t(j) * kThreads, a[j], b[j]);
    } else {
#pragma unroll
        for (int j = 0; j < kUnroll8; j++) {
            const uint64_t i = base + uint64_t(j) * kThreads;
            if (i < n8) st_cs_v8(o8 + i, ld_cs_v8(x8 + i), ld_cs_v8(y8 + i));
        }
    }
    if (blockIdx.x == 0) {
        if (threadIdx.x < head) os[threadIdx.x] = __fadd_rn(xs[threadIdx.x], ys[threadIdx.x]);
        const uint64_t t = tail_begin + threadIdx.x;
        if (threadIdx.x < 8 && t < n) os[t] = __fadd_rn(xs[t], ys[t]);
    }
}

// Used only when the three pointers do not share their offset within a
// 16-byte line, so no common vector alignment exists.
__global__ void __launch_bounds__(kThreads) add_f32_scalar(const float *__restrict__ x, const float *__restrict__ y,
                                                           float *__restrict__ o, uint64_t n) {
    const uint64_t base = uint64_t(blockIdx.x) * (kThreads * 8ull) + threadIdx.x;
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const uint64_t i = base + uint64_t(j) * kThreads;
        if (i < n) o[i] = __fadd_rn(x[i], y[i]);
    }
}

}  // namespace

cute_b200_status elementwise_add_f32(const float *x, const float *y, float *out, uint64_t n, cudaStream_t stream,
                                     const DeviceState &) {
    if (n == 0) return CUTE_B200_OK;
    const uintptr_t px = reinterpret_cast<uintptr_t>(x), py = reinterpret_cast<uintptr_t>(y),
                    po = reinterpret_cast<uintptr_t>(out);
    if ((px | py | po) & 3u)
        return fail(CUTE_B200_ERR_MISALIGNED, "elementwise_add: buffers must be 4-byte aligned");
    // 256-bit accesses when the pointers allow them (2^28 elements: 6 975 against 6 910 GB/s with 128-bit ones).
    if ((px & 31u) == (py & 31u) && (px & 31u) == (po & 31u)) {
        uint64_t head = ((32u - (px & 31u)) & 31u) / 4u;
        if (head > n) head = n;
        const uint64_t n8 = (n - head) / 8;
        const uint64_t tail_begin = head + n8 * 8;
        const uint64_t per_block = uint64_t(kThreads) * kUnroll8;
        uint64_t blocks = (n8 + per_block - 1) / per_block;
        if (blocks == 0) blocks = 1;
        if (blocks > 0x7fffffffull) return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "elementwise_add: n too large");
        add_f32_vec8<<<dim3(unsigned(blocks)), kThreads, 0, stream>>>(
            reinterpret_cast<const float8 *>(x + head), reinterpret_cast<const float8 *>(y + head),
            reinterpret_cast<float8 *>(out + head), n8, x, y, out, uint32_t(head), tail_begin, n);
    } else if ((px & 15u) == (py & 15u) && (px & 15u) == (po & 15u)) {
        uint64_t head = ((16u - (px & 15u)) & 15u) / 4u;
        if (head > n) head = n;
        const uint64_t n4 = (n - head) / 4;
        const uint64_t tail_begin = head + n4 * 4;
        uint64_t blocks = (n4 + kVecPerBlock - 1) / kVecPerBlock;
        if (blocks == 0) blocks = 1;
        if (blocks > 0x7fffffffull) return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "elementwise_add: n too large");
        add_f32_vec<<<dim3(unsigned(blocks)), kThreads, 0, stream>>>(
            reinterpret_cast<const float4 *>(x + head), reinterpret_cast<const float4 *>(y + head),
            reinterpret_cast<float4 *>(out + head), n4, x, y, out, uint32_t(head), tail_begin, n);
    } else {
        const uint64_t per_block = kThreads * 8ull;
        const uint64_t blocks = (n + per_block - 1) / per_block;
        if (blocks > 0x7fffffffull) return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "elementwise_add: n too large");
        add_f32_scalar<<<dim3(unsigned(blocks)), kThreads, 0, stream>>>(x, y, out, n);
    }
    CB_CUDA(cudaGetLastError());
    count_launch();
    return CUTE_B200_OK;
}

}  // namespace cb
