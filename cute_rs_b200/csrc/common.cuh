// Shared host-side plumbing of libcute_b200: error reporting, per-device
// state, launch accounting.  Internal; the public surface is include/cute_b200.h.
#pragma once

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <string>

#include "../../include/cute_b200.h"

namespace cb {

// Message of the calling thread's last failure; worded like the reference's
// CudaError / check_launch messages (src/cuda.rs:532-546, src/sim/mod.rs:328-385).
std::string &last_error();
cute_b200_status fail(cute_b200_status code, const char *fmt, ...) __attribute__((format(printf, 2, 3)));
cute_b200_status cuda_fail(cudaError_t err, const char *what);

#define CB_CUDA(call)                                                  \
    do {                                                               \
        cudaError_t err__ = (call);                                    \
        if (err__ != cudaSuccess) return ::cb::cuda_fail(err__, #call); \
    } while (0)

#define CB_TRY(call)                                   \
    do {                                               \
        cute_b200_status st__ = (call);                \
        if (st__ != CUTE_B200_OK) return st__;         \
    } while (0)

// Per-device state created by cute_b200_init.
struct DeviceState {
    bool ready = false;
    int sm_count = 0;
    uint32_t *status_word = nullptr;  // 4 x u32 in device memory, zero when healthy
};

// State of the current device, initialising it on first use.
cute_b200_status current_device(DeviceState **out);

void count_launch(uint64_t n = 1);

// Kernels, one translation unit each.
cute_b200_status elementwise_add_f32(const float *x, const float *y, float *out, uint64_t n, cudaStream_t stream,
                                     const DeviceState &dev);
cute_b200_status sgemm_nt(int m, int n, int k, float alpha, float beta, const float *a, const float *b, float *c,
                          cudaStream_t stream, const DeviceState &dev);
cute_b200_status gemm_tn(const cute_b200_gemm_desc &desc, uint64_t a, uint64_t b, uint64_t c, cudaStream_t stream,
                         const DeviceState &dev);
// signal_list: null, or `count` addresses of which [1..] are counters that receive +1 when the launch is complete.
cute_b200_status gemm_tn_multi(const cute_b200_gemm_desc &desc, uint64_t a, uint64_t b, const uint64_t *c_list, int count,
                               const uint64_t *signal_list, cudaStream_t stream, const DeviceState &dev);
cute_b200_status wait_signal(uint64_t counter, uint32_t mask, uint32_t at_least, uint32_t timeout_ms, cudaStream_t stream,
                             const DeviceState &dev);
// The same GEMM writing an m x n block of a wider row-major C: ldc elements between rows (>= n).
// Never splits k (the second pass of a split assumes a dense C); k must be positive.
cute_b200_status gemm_tn_strided(const cute_b200_gemm_desc &desc, uint64_t a, uint64_t b, uint64_t c, int ldc,
                                 cudaStream_t stream, const DeviceState &dev);
cute_b200_status gemm_layout_info(int cta_group, int tile_n, int tile_m, int ab_dtype, int c_dtype, uint32_t smem_addr,
                                  cute_b200_gemm_layout *out);
cute_b200_status gemm_plan(const cute_b200_gemm_desc &desc, int sm_count, int32_t out[4]);
cute_b200_status gemm_tn_init(const DeviceState &dev);
void gemm_tn_release_scratch();
cute_b200_status gemm_tn_static(const cute_b200_gemm_desc &desc, uint64_t a, uint64_t b, uint64_t c, cudaStream_t stream,
                                uint32_t *shared_status);
// Device address of the status words gemm_tn_static owns on `device`, null until that entry point has run there.
uint32_t *gemm_tn_static_status_words(int device);
cute_b200_status sgemm_nt_init(const DeviceState &dev);
// Waits for the current device and turns a kernel's bounded-wait report into CUTE_B200_ERR_DEVICE_TIMEOUT.
cute_b200_status sync_and_check();
// The launcher for several GPUs (multi_gpu.cu).
cute_b200_status comm_create(int ngpus, const int *ordinals, void **comm_out);
cute_b200_status comm_destroy(void *comm);
cute_b200_status comm_info(void *comm, int32_t out[4]);
cute_b200_status gemm_tn_sharded(void *comm, const cute_b200_gemm_desc *desc, const uint64_t *dA_shard, const uint64_t *dB,
                                 const uint64_t *dC, int replicate_c);
cute_b200_status gemm_tn_sharded_host(void *comm, const cute_b200_gemm_desc *desc, const void *hA, const void *hB, void *hC,
                                      double *seconds);

}  // namespace cb
