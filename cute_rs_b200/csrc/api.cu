// C ABI of libcute_b200 (include/cute_b200.h): status handling, device set-up,
// the per-kernel entry points and the launch-by-name front end that mirrors
// the reference launcher's argument and error conventions.
#include <atomic>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "common.cuh"

namespace cb {

std::string &last_error() {
    static thread_local std::string msg;
    return msg;
}

cute_b200_status fail(cute_b200_status code, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    last_error() = buf;
    return code;
}

// "<call> failed: <name>" like check() in the reference (src/cuda.rs:532-546).
cute_b200_status cuda_fail(cudaError_t err, const char *what) {
    std::string call(what);
    const size_t paren = call.find('(');
    if (paren != std::string::npos) call.resize(paren);
    if (err == cudaErrorNoDevice || err == cudaErrorInsufficientDriver)
        return fail(CUTE_B200_ERR_NO_DEVICE, "%s failed: %s", call.c_str(), cudaGetErrorName(err));
    return fail(CUTE_B200_ERR_CUDA, "%s failed: %s", call.c_str(), cudaGetErrorName(err));
}

static std::atomic<uint64_t> g_launches{0};
void count_launch(uint64_t n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

static constexpr int kMaxDevices = 64;
static DeviceState g_devices[kMaxDevices];
static std::mutex g_device_mu;

static cute_b200_status init_device(int ordinal) {
    if (ordinal < 0 || ordinal >= kMaxDevices)
        return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "device ordinal %d out of range", ordinal);
    int count = 0;
    cudaError_t err = cudaGetDeviceCount(&count);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail(CUTE_B200_ERR_NO_DEVICE, "cudaGetDeviceCount failed: %s", cudaGetErrorName(err));
    }
    if (ordinal >= count) return fail(CUTE_B200_ERR_NO_DEVICE, "device %d requested, %d present", ordinal, count);
    CB_CUDA(cudaSetDevice(ordinal));
    std::lock_guard<std::mutex> lock(g_device_mu);
    DeviceState &d = g_devices[ordinal];
    if (d.ready) return CUTE_B200_OK;
    cudaDeviceProp prop;
    CB_CUDA(cudaGetDeviceProperties(&prop, ordinal));
    if (prop.major != 10)
        return fail(CUTE_B200_ERR_NO_DEVICE, "device %d is sm_%d%d; this library is built for sm_100a only", ordinal,
                    prop.major, prop.minor);
    d.sm_count = prop.multiProcessorCount;
    CB_CUDA(cudaMalloc(&d.status_word, 64));
    CB_CUDA(cudaMemset(d.status_word, 0, 64));
    CB_TRY(gemm_tn_init(d));
    CB_TRY(sgemm_nt_init(d));
    d.ready = true;
    return CUTE_B200_OK;
}

cute_b200_status current_device(DeviceState **out) {
    int ordinal = 0;
    cudaError_t err = cudaGetDevice(&ordinal);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail(CUTE_B200_ERR_NO_DEVICE, "cudaGetDevice failed: %s", cudaGetErrorName(err));
    }
    if (ordinal < 0 || ordinal >= kMaxDevices) return fail(CUTE_B200_ERR_NO_DEVICE, "no current device");
    if (!g_devices[ordinal].ready) CB_TRY(init_device(ordinal));
    *out = &g_devices[ordinal];
    return CUTE_B200_OK;
}

// Status word of `ordinal` if cute_b200_init has set that device up, else null.
static uint32_t *status_word_if_ready(int ordinal) {
    if (ordinal < 0 || ordinal >= kMaxDevices) return nullptr;
    std::lock_guard<std::mutex> lock(g_device_mu);
    return g_devices[ordinal].ready ? g_devices[ordinal].status_word : nullptr;
}

// Read and clear the bounded-wait report of the current device.  A device that
// only cute_b200_gemm_tn_static has touched is not initialised here (that would
// allocate): its report lives in the words that entry point owns.
static cute_b200_status read_status(uint32_t out[4]) {
    int ordinal = 0;
    cudaError_t err = cudaGetDevice(&ordinal);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail(CUTE_B200_ERR_NO_DEVICE, "cudaGetDevice failed: %s", cudaGetErrorName(err));
    }
    uint32_t *word = status_word_if_ready(ordinal);
    uint32_t *static_word = gemm_tn_static_status_words(ordinal);
    if (!word && !static_word) {
        DeviceState *dev;
        CB_TRY(current_device(&dev));
        word = dev->status_word;
    }
    CB_CUDA(cudaDeviceSynchronize());
    out[0] = out[1] = out[2] = out[3] = 0;
    if (word) {
        CB_CUDA(cudaMemcpy(out, word, 16, cudaMemcpyDeviceToHost));
        if (out[0] != 0) CB_CUDA(cudaMemset(word, 0, 16));
    }
    if (out[0] == 0 && static_word && static_word != word) {
        CB_CUDA(cudaMemcpy(out, static_word, 16, cudaMemcpyDeviceToHost));
        if (out[0] != 0) CB_CUDA(cudaMemset(static_word, 0, 16));
    }
    return CUTE_B200_OK;
}

cute_b200_status sync_and_check() {
    uint32_t st[4];
    CB_TRY(read_status(st));
    if (st[0] != 0)
        return fail(CUTE_B200_ERR_DEVICE_TIMEOUT,
                    "kernel execution failed: a bounded wait gave up (where %u, detail %u, block %u, parity %u)", st[0],
                    st[1], st[2], st[3]);
    return CUTE_B200_OK;
}

// ---- launch by name ---------------------------------------------------------

static const char *dtype_name(int dt) {
    switch (dt) {
        case CUTE_B200_F16: return "f16";
        case CUTE_B200_BF16: return "bf16";
        case CUTE_B200_F32: return "f32";
        case CUTE_B200_I32: return "i32";
        default: return "?";
    }
}

static std::string describe(const cute_b200_arg &a) {
    char buf[96];
    if (a.is_scalar) snprintf(buf, sizeof(buf), "%s %s scalar", a.dtype == CUTE_B200_F32 ? "an" : "a", dtype_name(a.dtype));
    else
        snprintf(buf, sizeof(buf), "%s %s buffer of %llu", (a.dtype == CUTE_B200_F32 || a.dtype == CUTE_B200_F16 || a.dtype == CUTE_B200_I32) ? "an" : "a",
                 dtype_name(a.dtype), (unsigned long long)a.len);
    return buf;
}

struct ParamSpec {
    const char *name;
    bool scalar;
    int dtype;
    uint64_t multiple_of;  // scalars
};

enum class Kind { TensorOp, RuntimeGemm, Sgemm, Add };

struct KernelSpec {
    const char *name;
    Kind kind;
    int ab_dtype;
    uint32_t block;  // block_dim the reference kernel is built for
    std::vector<ParamSpec> params;
};

static const std::vector<KernelSpec> &kernel_specs() {
    static const std::vector<KernelSpec> specs = {
        {"tensorop_gemm", Kind::TensorOp, CUTE_B200_F16, 128,
         {{"a", false, CUTE_B200_F16, 0}, {"b", false, CUTE_B200_F16, 0}, {"c", false, CUTE_B200_F32, 0}}},
        {"tensorop_gemm_unswizzled", Kind::TensorOp, CUTE_B200_F16, 128,
         {{"a", false, CUTE_B200_F16, 0}, {"b", false, CUTE_B200_F16, 0}, {"c", false, CUTE_B200_F32, 0}}},
        {"tensorop_gemm_bf16", Kind::TensorOp, CUTE_B200_BF16, 128,
         {{"a", false, CUTE_B200_BF16, 0}, {"b", false, CUTE_B200_BF16, 0}, {"c", false, CUTE_B200_F32, 0}}},
        {"tensorop_gemm_bf16_unswizzled", Kind::TensorOp, CUTE_B200_BF16, 128,
         {{"a", false, CUTE_B200_BF16, 0}, {"b", false, CUTE_B200_BF16, 0}, {"c", false, CUTE_B200_F32, 0}}},
        {"runtime_gemm", Kind::RuntimeGemm, CUTE_B200_F16, 128,
         {{"a", false, CUTE_B200_F16, 0}, {"b", false, CUTE_B200_F16, 0}, {"c", false, CUTE_B200_F32, 0},
          {"n", true, CUTE_B200_I32, 128}, {"k", true, CUTE_B200_I32, 32}}},
        {"sgemm_nt", Kind::Sgemm, CUTE_B200_F32, 256,
         {{"a", false, CUTE_B200_F32, 0}, {"b", false, CUTE_B200_F32, 0}, {"c", false, CUTE_B200_F32, 0},
          {"alpha", true, CUTE_B200_F32, 1}, {"beta", true, CUTE_B200_F32, 1}}},
        {"elementwise_add_naive", Kind::Add, CUTE_B200_F32, 256,
         {{"a", false, CUTE_B200_F32, 0}, {"b", false, CUTE_B200_F32, 0}, {"c", false, CUTE_B200_F32, 0}}},
        {"elementwise_add_tiled", Kind::Add, CUTE_B200_F32, 128,
         {{"a", false, CUTE_B200_F32, 0}, {"b", false, CUTE_B200_F32, 0}, {"c", false, CUTE_B200_F32, 0}}},
    };
    return specs;
}

static float scalar_f32(const cute_b200_arg &a) {
    const uint32_t bits = uint32_t(a.value);
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

// The size-independent checks of check_launch (src/sim/mod.rs:328-385), in the
// same order and with the same wording.
static cute_b200_status check_launch(const KernelSpec &spec, const cute_b200_launch_config &cfg,
                                     const cute_b200_arg *args, int num_args) {
    if (size_t(num_args) != spec.params.size())
        return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "kernel `%s` takes %zu arguments, %d were given", spec.name,
                    spec.params.size(), num_args);
    const uint64_t threads = uint64_t(cfg.block[0]) * cfg.block[1] * cfg.block[2];
    if (threads == 0 || threads > 1024)
        return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "invalid block size [%u, %u, %u]", cfg.block[0], cfg.block[1],
                    cfg.block[2]);
    if (cfg.grid[0] == 0 || cfg.grid[1] == 0 || cfg.grid[2] == 0)
        return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "invalid grid size [%u, %u, %u]", cfg.grid[0], cfg.grid[1],
                    cfg.grid[2]);
    bool clusters_ok = cfg.cluster[0] && cfg.cluster[1] && cfg.cluster[2];
    for (int i = 0; clusters_ok && i < 3; i++) clusters_ok = cfg.grid[i] % cfg.cluster[i] == 0;
    if (!clusters_ok)
        return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "grid [%u, %u, %u] is not a whole number of clusters of [%u, %u, %u]",
                    cfg.grid[0], cfg.grid[1], cfg.grid[2], cfg.cluster[0], cfg.cluster[1], cfg.cluster[2]);
    if (cfg.block[0] != spec.block || cfg.block[1] != 1 || cfg.block[2] != 1)
        return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "kernel `%s` was built for blocks of [%u, 1, 1], launched with [%u, %u, %u]",
                    spec.name, spec.block, cfg.block[0], cfg.block[1], cfg.block[2]);
    for (int i = 0; i < num_args; i++) {
        const ParamSpec &p = spec.params[i];
        const cute_b200_arg &a = args[i];
        if (!p.scalar) {
            if (a.is_scalar || a.dtype != p.dtype)
                return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "argument %d (`%s`) must be a %s buffer, got %s", i, p.name,
                            dtype_name(p.dtype), describe(a).c_str());
        } else {
            if (!a.is_scalar || a.dtype != p.dtype)
                return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "argument %d (`%s`) must be a %s scalar, got %s", i, p.name,
                            dtype_name(p.dtype), describe(a).c_str());
            if (p.dtype == CUTE_B200_I32 && p.multiple_of > 1 && (a.value & 0xffffffffull) % p.multiple_of != 0)
                return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "argument %d (`%s`) must be a multiple of %llu, got %llu", i,
                            p.name, (unsigned long long)p.multiple_of, (unsigned long long)(a.value & 0xffffffffull));
        }
    }
    return CUTE_B200_OK;
}

static cute_b200_status need_len(const KernelSpec &spec, const cute_b200_arg *args, int i, uint64_t need) {
    if (args[i].len < need)
        return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "argument %d (`%s`) needs at least %llu elements, got %llu", i,
                    spec.params[i].name, (unsigned long long)need, (unsigned long long)args[i].len);
    return CUTE_B200_OK;
}

static const KernelSpec *find_spec(const char *name) {
    for (const KernelSpec &s : kernel_specs())
        if (strcmp(s.name, name) == 0) return &s;
    return nullptr;
}

// Validate and launch with DEVICE pointers in the buffer slots.
static cute_b200_status launch_named(const KernelSpec &spec, const cute_b200_launch_config &cfg,
                                     const cute_b200_arg *args, int num_args, cudaStream_t stream) {
    CB_TRY(check_launch(spec, cfg, args, num_args));
    DeviceState *dev;
    CB_TRY(current_device(&dev));
    switch (spec.kind) {
        case Kind::TensorOp:
        case Kind::RuntimeGemm: {
            // The kernels tile C 128 x 128 per block: m and n follow from the
            // grid (examples/tensorop_gemm.rs:177, examples/runtime_gemm.rs:119).
            if (cfg.grid[2] != 1)
                return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "kernel `%s` takes a two-dimensional grid", spec.name);
            const uint64_t m = uint64_t(cfg.grid[0]) * 128, n = uint64_t(cfg.grid[1]) * 128;
            uint64_t k;
            if (spec.kind == Kind::RuntimeGemm) {
                const uint64_t n_arg = args[3].value & 0xffffffffull;
                k = args[4].value & 0xffffffffull;
                if (n_arg != n)
                    return fail(CUTE_B200_ERR_INVALID_ARGUMENT,
                                "argument 3 (`n`) is %llu but the grid covers %llu columns", (unsigned long long)n_arg,
                                (unsigned long long)n);
            } else {
                // Sizes are baked into the reference kernel; here k follows
                // from the length of `a` (m * k elements).
                if (args[0].len == 0 || args[0].len % m)
                    return fail(CUTE_B200_ERR_INVALID_ARGUMENT,
                                "argument 0 (`a`) has %llu elements, not a multiple of the %llu rows the grid covers",
                                (unsigned long long)args[0].len, (unsigned long long)m);
                k = args[0].len / m;
                if (k % 32)
                    return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "problem size must be a multiple of the tile size");
            }
            if (m > 0x7fffffffull || n > 0x7fffffffull || k > 0x7fffffffull)
                return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "problem too large");
            CB_TRY(need_len(spec, args, 0, m * k));
            CB_TRY(need_len(spec, args, 1, n * k));
            CB_TRY(need_len(spec, args, 2, m * n));
            cute_b200_gemm_desc d = {};
            d.m = int(m);
            d.n = int(n);
            d.k = int(k);
            d.ab_dtype = spec.ab_dtype;
            d.c_dtype = CUTE_B200_F32;
            d.alpha = 1.0f;
            d.beta = 0.0f;
            return gemm_tn(d, args[0].value, args[1].value, args[2].value, stream, *dev);
        }
        case Kind::Sgemm: {
            if (cfg.grid[2] != 1)
                return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "kernel `%s` takes a two-dimensional grid", spec.name);
            const uint64_t m = uint64_t(cfg.grid[0]) * 128, n = uint64_t(cfg.grid[1]) * 128;
            if (args[0].len % m)
                return fail(CUTE_B200_ERR_INVALID_ARGUMENT,
                            "argument 0 (`a`) has %llu elements, not a multiple of the %llu rows the grid covers",
                            (unsigned long long)args[0].len, (unsigned long long)m);
            const uint64_t k = args[0].len / m;
            if (k % 8) return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "problem size must be a multiple of the tile size");
            if (m > 0x7fffffffull || n > 0x7fffffffull || k > 0x7fffffffull)
                return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "problem too large");
            CB_TRY(need_len(spec, args, 1, n * k));
            CB_TRY(need_len(spec, args, 2, m * n));
            return sgemm_nt(int(m), int(n), int(k), scalar_f32(args[3]), scalar_f32(args[4]),
                            reinterpret_cast<const float *>(args[0].value), reinterpret_cast<const float *>(args[1].value),
                            reinterpret_cast<float *>(args[2].value), stream, *dev);
        }
        case Kind::Add: {
            // Every element of the (M, N) tensors is added once; the grid only
            // has to cover them (examples/elementwise_add.rs:92-93).
            const uint64_t count = args[2].len;
            const uint64_t covered = spec.block == 256 ? uint64_t(cfg.grid[0]) * cfg.grid[1] * cfg.grid[2] * 256
                                                       : uint64_t(cfg.grid[0]) * cfg.grid[1] * cfg.grid[2] * 16 * 128;
            if (covered < count)
                return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "grid [%u, %u, %u] covers %llu of the %llu elements",
                            cfg.grid[0], cfg.grid[1], cfg.grid[2], (unsigned long long)covered,
                            (unsigned long long)count);
            CB_TRY(need_len(spec, args, 0, count));
            CB_TRY(need_len(spec, args, 1, count));
            return elementwise_add_f32(reinterpret_cast<const float *>(args[0].value),
                                       reinterpret_cast<const float *>(args[1].value),
                                       reinterpret_cast<float *>(args[2].value), count, stream, *dev);
        }
    }
    return fail(CUTE_B200_ERR_UNSUPPORTED, "kernel `%s` is not implemented", spec.name);
}

static size_t dtype_bytes(int dt) { return (dt == CUTE_B200_F16 || dt == CUTE_B200_BF16) ? 2 : 4; }

}  // namespace cb

using namespace cb;

extern "C" {

const char *cute_b200_status_string(cute_b200_status status) {
    switch (status) {
        case CUTE_B200_OK: return "CUTE_B200_OK";
        case CUTE_B200_ERR_INVALID_ARGUMENT: return "CUTE_B200_ERR_INVALID_ARGUMENT";
        case CUTE_B200_ERR_MISALIGNED: return "CUTE_B200_ERR_MISALIGNED";
        case CUTE_B200_ERR_UNSUPPORTED: return "CUTE_B200_ERR_UNSUPPORTED";
        case CUTE_B200_ERR_NO_DEVICE: return "CUTE_B200_ERR_NO_DEVICE";
        case CUTE_B200_ERR_DEVICE_TIMEOUT: return "CUTE_B200_ERR_DEVICE_TIMEOUT";
        case CUTE_B200_ERR_CUDA: return "CUTE_B200_ERR_CUDA";
        case CUTE_B200_ERR_NULL_POINTER: return "CUTE_B200_ERR_NULL_POINTER";
        default: return "CUTE_B200_ERR_UNKNOWN";
    }
}

const char *cute_b200_last_error(void) { return last_error().c_str(); }

cute_b200_status cute_b200_init(int32_t device_ordinal) { return init_device(device_ordinal); }

cute_b200_status cute_b200_gemm_tn(const cute_b200_gemm_desc *desc, uint64_t dA, uint64_t dB, uint64_t dC,
                                   void *stream) {
    if (!desc) return fail(CUTE_B200_ERR_NULL_POINTER, "gemm_tn: desc is null");
    DeviceState *dev;
    CB_TRY(current_device(&dev));
    return gemm_tn(*desc, dA, dB, dC, static_cast<cudaStream_t>(stream), *dev);
}

// Grow-only device staging buffers of the host-buffer entry points, per device.
struct Workspace {
    void *ptr[3] = {nullptr, nullptr, nullptr};
    size_t bytes[3] = {0, 0, 0};
};
static Workspace g_workspace[kMaxDevices];

static cute_b200_status workspace_get(int device, int slot, size_t bytes, void **out) {
    Workspace &w = g_workspace[device];
    if (w.bytes[slot] < bytes) {
        if (w.ptr[slot]) cudaFree(w.ptr[slot]);
        w.ptr[slot] = nullptr;
        w.bytes[slot] = 0;
        CB_CUDA(cudaMalloc(&w.ptr[slot], bytes));
        w.bytes[slot] = bytes;
    }
    *out = w.ptr[slot];
    return CUTE_B200_OK;
}

// Streams and events of the host-buffer GEMM, created once per device.
struct Pipeline {
    static constexpr int kMaxPanels = 24;            // per operand
    static constexpr int kMaxSteps = 2 * kMaxPanels;  // one upload per step
    bool ready = false;
    cudaStream_t up = nullptr, compute = nullptr, down = nullptr;
    cudaEvent_t uploaded[kMaxSteps], computed[kMaxSteps], t0[kMaxSteps], t1[kMaxSteps];
};
static Pipeline g_pipeline[kMaxDevices];

static cute_b200_status pipeline_get(int device, Pipeline **out) {
    Pipeline &p = g_pipeline[device];
    if (!p.ready) {
        CB_CUDA(cudaStreamCreateWithFlags(&p.up, cudaStreamNonBlocking));
        CB_CUDA(cudaStreamCreateWithFlags(&p.compute, cudaStreamNonBlocking));
        CB_CUDA(cudaStreamCreateWithFlags(&p.down, cudaStreamNonBlocking));
        for (int i = 0; i < Pipeline::kMaxSteps; i++) {
            CB_CUDA(cudaEventCreateWithFlags(&p.uploaded[i], cudaEventDisableTiming));
            CB_CUDA(cudaEventCreateWithFlags(&p.computed[i], cudaEventDisableTiming));
            CB_CUDA(cudaEventCreate(&p.t0[i]));
            CB_CUDA(cudaEventCreate(&p.t1[i]));
        }
        p.ready = true;
    }
    *out = &p;
    return CUTE_B200_OK;
}

cute_b200_status cute_b200_release_workspace(void) {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) {
        cudaGetLastError();
        return CUTE_B200_OK;
    }
    gemm_tn_release_scratch();
    Workspace &w = g_workspace[device];
    for (int i = 0; i < 3; i++) {
        if (w.ptr[i]) cudaFree(w.ptr[i]);
        w.ptr[i] = nullptr;
        w.bytes[i] = 0;
    }
    return CUTE_B200_OK;
}

// Cuts `dim` rows of `row_bytes` each into panels for the host-buffer GEMM: about eight of equal size (a
// multiple of 256 rows, at least 2 MiB); with `tail` the end halves down to the smallest panel worth a
// copy of its own (1 MiB, at least 256 rows).  row0[i] is the first row of panel i, row0[count] = dim.
static int split_panels(int dim, size_t row_bytes, bool tail, int *row0) {
    size_t min_rows = (((size_t(1) << 20) / (row_bytes ? row_bytes : 1) + 255) / 256) * 256;
    if (min_rows < 256) min_rows = 256;
    if (min_rows > size_t(dim)) min_rows = size_t(dim);
    int big = ((dim / 8 + 255) / 256) * 256;
    if (size_t(big) < 2 * min_rows) big = int(2 * min_rows);
    int count = 0;
    row0[0] = 0;
    while (row0[count] < dim) {
        const int left = dim - row0[count];
        int take;
        if (left > big + big / 2) take = big;
        else if (tail && size_t(left) >= 2 * min_rows) take = ((left / 2 + 255) / 256) * 256;
        else take = left;
        if (count == Pipeline::kMaxPanels - 1) take = left;
        row0[count + 1] = row0[count] + take;
        count++;
    }
    return count;
}

cute_b200_status cute_b200_gemm_tn_host(const cute_b200_gemm_desc *desc, const void *hA, const void *hB, void *hC,
                                        double *seconds) {
    if (!desc) return fail(CUTE_B200_ERR_NULL_POINTER, "gemm_tn_host: desc is null");
    if (desc->m <= 0 || desc->n <= 0 || desc->k < 0)
        return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "gemm_tn: invalid size %dx%dx%d", desc->m, desc->n, desc->k);
    if (!hC || (desc->k > 0 && (!hA || !hB))) return fail(CUTE_B200_ERR_NULL_POINTER, "gemm_tn_host: null buffer");
    DeviceState *dev;
    CB_TRY(current_device(&dev));
    int device = 0;
    CB_CUDA(cudaGetDevice(&device));
    const size_t a_bytes = size_t(desc->m) * desc->k * 2, b_bytes = size_t(desc->n) * desc->k * 2;
    const size_t c_bytes = size_t(desc->m) * desc->n * (desc->c_dtype == CUTE_B200_BF16 ? 2 : 4);
    void *dA, *dB, *dC;
    CB_TRY(workspace_get(device, 0, a_bytes ? a_bytes : 16, &dA));
    CB_TRY(workspace_get(device, 1, b_bytes ? b_bytes : 16, &dB));
    CB_TRY(workspace_get(device, 2, c_bytes, &dC));
    // Three streams pipeline the call.  PCIe carries about 54 GB/s up or 57 GB/s down alone but only
    // about 78 GB/s both ways together, so the way down has to start long before the way up ends: A and B
    // go up alternately in panels of rows, and each new panel unlocks a block of C (its rows or columns
    // against everything of the other operand that is already there), which is multiplied at once and
    // sent down while the next panels come up.  The area of C that can be computed then grows as early
    // as the data allows (with the product of the rows of A and B on the device).  The last uploads are
    // small panels of A: what the last upload unlocks is the part that nothing hides, and rows of C
    // come down as one contiguous copy, while a block of columns is a pitched copy that PCIe carries
    // less well the narrower it is (52 against 57 GB/s at 2 KiB per row), so B has no small panels.
    Pipeline *pipe = nullptr;
    CB_TRY(pipeline_get(device, &pipe));
    const size_t c_elem = desc->c_dtype == CUTE_B200_BF16 ? 2 : 4;
    const bool reads_c = !(desc->alpha == 1.0f && desc->beta == 0.0f);
    int steps = 0;
    // Everything that is queued below reads or writes the caller's buffers asynchronously, so whatever
    // happens while queueing, the call only returns after the device-wide wait that follows.
    auto issue = [&]() -> cute_b200_status {
        cute_b200_status st = CUTE_B200_OK;
        if (desc->k == 0) {
            if (reads_c) CB_CUDA(cudaMemcpyAsync(dC, hC, c_bytes, cudaMemcpyHostToDevice, pipe->compute));
            st = gemm_tn(*desc, 0, 0, reinterpret_cast<uint64_t>(dC), pipe->compute, *dev);
            if (st == CUTE_B200_OK) CB_CUDA(cudaMemcpyAsync(hC, dC, c_bytes, cudaMemcpyDeviceToHost, pipe->compute));
        } else {
            int a_row0[Pipeline::kMaxPanels + 1], b_row0[Pipeline::kMaxPanels + 1];
            const size_t row_bytes = size_t(desc->k) * 2, c_pitch = size_t(desc->n) * c_elem;
            const int a_panels = split_panels(desc->m, row_bytes, true, a_row0);
            const int b_panels = split_panels(desc->n, row_bytes, false, b_row0);
            int ia = 0, ib = 0;  // panels of A and B on their way or on the device
            while ((ia < a_panels || ib < b_panels) && st == CUTE_B200_OK) {
                const bool is_a = ib >= b_panels || (ia < a_panels && a_row0[ia] <= b_row0[ib]);  // keep the rows level
                // The panel going up, and the block of C it unlocks: rows [r0, r1) x columns [c0, c1).
                int r0, r1, c0, c1;
                if (is_a) {
                    r0 = a_row0[ia], r1 = a_row0[ia + 1], c0 = 0, c1 = b_row0[ib];
                    CB_CUDA(cudaMemcpyAsync(static_cast<char *>(dA) + r0 * row_bytes, static_cast<const char *>(hA) + r0 * row_bytes,
                                            (r1 - r0) * row_bytes, cudaMemcpyHostToDevice, pipe->up));
                    ia++;
                } else {
                    c0 = b_row0[ib], c1 = b_row0[ib + 1], r0 = 0, r1 = a_row0[ia];
                    CB_CUDA(cudaMemcpyAsync(static_cast<char *>(dB) + c0 * row_bytes, static_cast<const char *>(hB) + c0 * row_bytes,
                                            (c1 - c0) * row_bytes, cudaMemcpyHostToDevice, pipe->up));
                    ib++;
                }
                if (r1 == r0 || c1 == c0) continue;  // nothing of the other operand is up yet
                const size_t c_off = size_t(r0) * c_pitch + size_t(c0) * c_elem;
                const size_t width = size_t(c1 - c0) * c_elem;
                if (reads_c)
                    CB_CUDA(cudaMemcpy2DAsync(static_cast<char *>(dC) + c_off, c_pitch, static_cast<const char *>(hC) + c_off, c_pitch,
                                              width, size_t(r1 - r0), cudaMemcpyHostToDevice, pipe->up));
                const int i = steps++;
                CB_CUDA(cudaEventRecord(pipe->uploaded[i], pipe->up));
                CB_CUDA(cudaStreamWaitEvent(pipe->compute, pipe->uploaded[i], 0));
                cute_b200_gemm_desc d = *desc;
                d.m = r1 - r0;
                d.n = c1 - c0;
                if (seconds) CB_CUDA(cudaEventRecord(pipe->t0[i], pipe->compute));
                st = gemm_tn_strided(d, reinterpret_cast<uint64_t>(dA) + r0 * row_bytes, reinterpret_cast<uint64_t>(dB) + c0 * row_bytes,
                                     reinterpret_cast<uint64_t>(dC) + c_off, desc->n, pipe->compute, *dev);
                if (st != CUTE_B200_OK) break;
                if (seconds) CB_CUDA(cudaEventRecord(pipe->t1[i], pipe->compute));
                CB_CUDA(cudaEventRecord(pipe->computed[i], pipe->compute));
                CB_CUDA(cudaStreamWaitEvent(pipe->down, pipe->computed[i], 0));
                CB_CUDA(cudaMemcpy2DAsync(static_cast<char *>(hC) + c_off, c_pitch, static_cast<char *>(dC) + c_off, c_pitch, width,
                                          size_t(r1 - r0), cudaMemcpyDeviceToHost, pipe->down));
            }
        }
        return st;
    };
    cute_b200_status st = issue();
    {
        const cute_b200_status sync = sync_and_check();  // waits for all three streams (device-wide)
        if (st == CUTE_B200_OK) st = sync;
    }
    if (seconds && st == CUTE_B200_OK) {
        double total = 0.0;
        for (int i = 0; i < steps; i++) {
            float ms = 0.0f;
            if (cudaEventElapsedTime(&ms, pipe->t0[i], pipe->t1[i]) == cudaSuccess) total += double(ms) * 1e-3;
        }
        *seconds = total;
    }
    return st;
}

cute_b200_status cute_b200_gemm_tn_multi(const cute_b200_gemm_desc *desc, uint64_t dA, uint64_t dB, const uint64_t *dC_list,
                                         int32_t count, void *stream) {
    if (!desc) return fail(CUTE_B200_ERR_NULL_POINTER, "gemm_tn_multi: desc is null");
    DeviceState *dev;
    CB_TRY(current_device(&dev));
    return gemm_tn_multi(*desc, dA, dB, dC_list, count, nullptr, static_cast<cudaStream_t>(stream), *dev);
}

cute_b200_status cute_b200_gemm_tn_multi_signal(const cute_b200_gemm_desc *desc, uint64_t dA, uint64_t dB, const uint64_t *dC_list,
                                                const uint64_t *dSignal_list, int32_t count, void *stream) {
    if (!desc) return fail(CUTE_B200_ERR_NULL_POINTER, "gemm_tn_multi_signal: desc is null");
    if (!dSignal_list) return fail(CUTE_B200_ERR_NULL_POINTER, "gemm_tn_multi_signal: the list of counters is null");
    DeviceState *dev;
    CB_TRY(current_device(&dev));
    return gemm_tn_multi(*desc, dA, dB, dC_list, count, dSignal_list, static_cast<cudaStream_t>(stream), *dev);
}

cute_b200_status cute_b200_wait_signal(uint64_t dSignals, uint32_t mask, uint32_t at_least, uint32_t timeout_ms, void *stream) {
    DeviceState *dev;
    CB_TRY(current_device(&dev));
    return wait_signal(dSignals, mask, at_least, timeout_ms, static_cast<cudaStream_t>(stream), *dev);
}

cute_b200_status cute_b200_gemm_tn_static(const cute_b200_gemm_desc *desc, uint64_t dA, uint64_t dB, uint64_t dC,
                                          void *stream) {
    if (!desc) return fail(CUTE_B200_ERR_NULL_POINTER, "gemm_tn_static: desc is null");
    // A device already set up through cute_b200_init shares its status word; otherwise
    // the entry point uses status words of its own, which cute_b200_synchronize and
    // cute_b200_device_status read as well.  Nothing is initialised here.
    int device = 0;
    uint32_t *shared = nullptr;
    if (cudaGetDevice(&device) == cudaSuccess) shared = status_word_if_ready(device);
    return gemm_tn_static(*desc, dA, dB, dC, static_cast<cudaStream_t>(stream), shared);
}

cute_b200_status cute_b200_sgemm_nt(int32_t m, int32_t n, int32_t k, float alpha, float beta, uint64_t dA, uint64_t dB,
                                    uint64_t dC, void *stream) {
    DeviceState *dev;
    CB_TRY(current_device(&dev));
    if (!dC || (k > 0 && (!dA || !dB))) return fail(CUTE_B200_ERR_NULL_POINTER, "sgemm_nt: null buffer");
    return sgemm_nt(m, n, k, alpha, beta, reinterpret_cast<const float *>(dA), reinterpret_cast<const float *>(dB),
                    reinterpret_cast<float *>(dC), static_cast<cudaStream_t>(stream), *dev);
}

cute_b200_status cute_b200_elementwise_add_f32(uint64_t dX, uint64_t dY, uint64_t dOut, uint64_t n, void *stream) {
    DeviceState *dev;
    CB_TRY(current_device(&dev));
    if (n && (!dX || !dY || !dOut)) return fail(CUTE_B200_ERR_NULL_POINTER, "elementwise_add: null buffer");
    return elementwise_add_f32(reinterpret_cast<const float *>(dX), reinterpret_cast<const float *>(dY),
                               reinterpret_cast<float *>(dOut), n, static_cast<cudaStream_t>(stream), *dev);
}

cute_b200_status cute_b200_launch(const char *kernel_name, const cute_b200_launch_config *cfg,
                                  const cute_b200_arg *args, int32_t num_args, void *stream) {
    if (!kernel_name || !cfg || (!args && num_args)) return fail(CUTE_B200_ERR_NULL_POINTER, "launch: null argument");
    const KernelSpec *spec = find_spec(kernel_name);
    if (!spec) return fail(CUTE_B200_ERR_UNSUPPORTED, "kernel `%s` is not one of this library's kernels", kernel_name);
    return launch_named(*spec, *cfg, args, num_args, static_cast<cudaStream_t>(stream));
}

cute_b200_status cute_b200_launch_host(const char *kernel_name, const cute_b200_launch_config *cfg,
                                       const cute_b200_arg *args, int32_t num_args, double *seconds) {
    if (!kernel_name || !cfg || (!args && num_args)) return fail(CUTE_B200_ERR_NULL_POINTER, "launch: null argument");
    const KernelSpec *spec = find_spec(kernel_name);
    if (!spec) return fail(CUTE_B200_ERR_UNSUPPORTED, "kernel `%s` is not one of this library's kernels", kernel_name);
    // Check before anything is allocated, as the reference does.
    CB_TRY(check_launch(*spec, *cfg, args, num_args));
    DeviceState *dev;
    CB_TRY(current_device(&dev));

    std::vector<cute_b200_arg> dargs(args, args + num_args);
    std::vector<void *> owned;
    auto cleanup = [&] {
        for (void *p : owned) cudaFree(p);
    };
    cudaStream_t stream = nullptr;  // the reference launches on the null stream (src/cuda.rs:382)
    for (int i = 0; i < num_args; i++) {
        if (args[i].is_scalar) continue;
        const size_t bytes = size_t(args[i].len) * dtype_bytes(args[i].dtype);
        void *p = nullptr;
        cudaError_t err = cudaMalloc(&p, bytes ? bytes : 1);  // cuMemAlloc(bytes.max(1)), src/cuda.rs:288
        if (err != cudaSuccess) {
            cleanup();
            return cuda_fail(err, "cudaMalloc");
        }
        owned.push_back(p);
        if (bytes) {
            if (!args[i].value) {
                cleanup();
                return fail(CUTE_B200_ERR_NULL_POINTER, "argument %d is a null host buffer", i);
            }
            err = cudaMemcpyAsync(p, reinterpret_cast<const void *>(args[i].value), bytes, cudaMemcpyHostToDevice, stream);
            if (err != cudaSuccess) {
                cleanup();
                return cuda_fail(err, "cudaMemcpyAsync");
            }
        }
        dargs[i].value = reinterpret_cast<uint64_t>(p);
    }
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    if (seconds) {
        cudaEventCreate(&e0);
        cudaEventCreate(&e1);
        cudaEventRecord(e0, stream);
    }
    cute_b200_status st = launch_named(*spec, *cfg, dargs.data(), num_args, stream);
    if (seconds) cudaEventRecord(e1, stream);
    if (st == CUTE_B200_OK) st = sync_and_check();
    if (st == CUTE_B200_OK) {
        int j = 0;
        for (int i = 0; i < num_args && st == CUTE_B200_OK; i++) {
            if (args[i].is_scalar) continue;
            const size_t bytes = size_t(args[i].len) * dtype_bytes(args[i].dtype);
            if (bytes) {
                cudaError_t err = cudaMemcpy(reinterpret_cast<void *>(args[i].value), owned[j], bytes, cudaMemcpyDeviceToHost);
                if (err != cudaSuccess) st = cuda_fail(err, "cudaMemcpy");
            }
            j++;
        }
    }
    if (seconds) {
        float ms = 0.0f;
        if (st == CUTE_B200_OK && cudaEventElapsedTime(&ms, e0, e1) == cudaSuccess) *seconds = double(ms) * 1e-3;
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
    }
    cleanup();
    return st;
}

cute_b200_status cute_b200_upload(const void *host, uint64_t bytes, uint64_t *device_out) {
    if (!device_out || (bytes && !host)) return fail(CUTE_B200_ERR_NULL_POINTER, "upload: null argument");
    DeviceState *dev;
    CB_TRY(current_device(&dev));
    void *p = nullptr;
    CB_CUDA(cudaMalloc(&p, bytes ? bytes : 1));
    if (bytes) {
        cudaError_t err = cudaMemcpy(p, host, bytes, cudaMemcpyHostToDevice);
        if (err != cudaSuccess) {
            cudaFree(p);
            return cuda_fail(err, "cudaMemcpy");
        }
    }
    *device_out = reinterpret_cast<uint64_t>(p);
    return CUTE_B200_OK;
}

cute_b200_status cute_b200_download(uint64_t device, void *host, uint64_t bytes) {
    if (bytes && (!device || !host)) return fail(CUTE_B200_ERR_NULL_POINTER, "download: null argument");
    if (bytes) CB_CUDA(cudaMemcpy(host, reinterpret_cast<const void *>(device), bytes, cudaMemcpyDeviceToHost));
    return CUTE_B200_OK;
}

cute_b200_status cute_b200_free(uint64_t device) {
    if (device) CB_CUDA(cudaFree(reinterpret_cast<void *>(device)));
    return CUTE_B200_OK;
}

cute_b200_status cute_b200_synchronize(void) { return sync_and_check(); }

cute_b200_status cute_b200_alloc(uint64_t bytes, uint64_t *device_out) {
    if (!device_out) return fail(CUTE_B200_ERR_NULL_POINTER, "alloc: null output");
    DeviceState *dev;
    CB_TRY(current_device(&dev));
    // Large buffers are made a whole number of 2 MiB: a 2 GiB + 256 byte allocation, exported by CUDA IPC,
    // took the stores of peer GPUs at less than half the rate of a 2 GiB one (measured on eight B200s).
    constexpr uint64_t kGranule = uint64_t(2) << 20;
    if (bytes > kGranule) bytes = (bytes + kGranule - 1) / kGranule * kGranule;
    void *p = nullptr;
    CB_CUDA(cudaMalloc(&p, bytes ? bytes : 1));
    *device_out = reinterpret_cast<uint64_t>(p);
    return CUTE_B200_OK;
}

cute_b200_status cute_b200_ipc_export(uint64_t device, uint8_t handle_out[64]) {
    if (!device || !handle_out) return fail(CUTE_B200_ERR_NULL_POINTER, "ipc_export: null argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t h;
    CB_CUDA(cudaIpcGetMemHandle(&h, reinterpret_cast<void *>(device)));
    memcpy(handle_out, &h, 64);
    return CUTE_B200_OK;
}

cute_b200_status cute_b200_ipc_open(const uint8_t handle[64], uint64_t *device_out) {
    if (!handle || !device_out) return fail(CUTE_B200_ERR_NULL_POINTER, "ipc_open: null argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    void *p = nullptr;
    CB_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    *device_out = reinterpret_cast<uint64_t>(p);
    return CUTE_B200_OK;
}

cute_b200_status cute_b200_ipc_close(uint64_t device) {
    if (device) CB_CUDA(cudaIpcCloseMemHandle(reinterpret_cast<void *>(device)));
    return CUTE_B200_OK;
}

cute_b200_status cute_b200_copy_async(uint64_t dst, uint64_t src, uint64_t bytes, void *stream) {
    if (bytes && (!dst || !src)) return fail(CUTE_B200_ERR_NULL_POINTER, "copy_async: null argument");
    if (bytes)
        CB_CUDA(cudaMemcpyAsync(reinterpret_cast<void *>(dst), reinterpret_cast<const void *>(src), bytes,
                                cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream)));
    return CUTE_B200_OK;
}

cute_b200_status cute_b200_shard_rows(int32_t m, int32_t world, int32_t rank, int32_t *row_begin, int32_t *rows) {
    if (!row_begin || !rows) return fail(CUTE_B200_ERR_NULL_POINTER, "shard_rows: null output");
    if (m < 0 || world <= 0 || rank < 0 || rank >= world)
        return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "shard_rows: invalid m %d, world %d, rank %d", m, world, rank);
    // Blocks are whole 128-row tiles; the first (tiles % world) ranks take one
    // extra tile and the last block absorbs a ragged end.
    const int tiles = (m + 127) / 128;
    const int base = tiles / world, extra = tiles % world;
    const int first_tile = rank * base + (rank < extra ? rank : extra);
    const int my_tiles = base + (rank < extra ? 1 : 0);
    long long begin = (long long)first_tile * 128, end = (long long)(first_tile + my_tiles) * 128;
    if (begin > m) begin = m;
    if (end > m) end = m;
    *row_begin = int32_t(begin);
    *rows = int32_t(end - begin);
    return CUTE_B200_OK;
}

cute_b200_status cute_b200_gemm_tn_shard(const cute_b200_gemm_desc *desc, int32_t world, int32_t rank,
                                         uint64_t dA_shard, uint64_t dB, uint64_t dC_base, int32_t c_is_full,
                                         void *stream) {
    if (!desc) return fail(CUTE_B200_ERR_NULL_POINTER, "gemm_tn_shard: desc is null");
    int32_t begin = 0, rows = 0;
    CB_TRY(cute_b200_shard_rows(desc->m, world, rank, &begin, &rows));
    if (rows == 0) return CUTE_B200_OK;
    cute_b200_gemm_desc d = *desc;
    d.m = rows;
    const uint64_t c_elem = desc->c_dtype == CUTE_B200_BF16 ? 2 : 4;
    const uint64_t dC = c_is_full ? dC_base + uint64_t(begin) * uint64_t(desc->n) * c_elem : dC_base;
    return cute_b200_gemm_tn(&d, dA_shard, dB, dC, stream);
}

cute_b200_status cute_b200_comm_create(int32_t ngpus, const int32_t *ordinals, void **comm_out) {
    return comm_create(ngpus, ordinals, comm_out);
}

cute_b200_status cute_b200_comm_destroy(void *comm) { return comm_destroy(comm); }

cute_b200_status cute_b200_comm_info(void *comm, int32_t out[4]) { return comm_info(comm, out); }

cute_b200_status cute_b200_gemm_tn_sharded(void *comm, const cute_b200_gemm_desc *desc, const uint64_t *dA_shard,
                                           const uint64_t *dB, const uint64_t *dC, int32_t replicate_c) {
    return gemm_tn_sharded(comm, desc, dA_shard, dB, dC, replicate_c);
}

cute_b200_status cute_b200_gemm_tn_sharded_host(void *comm, const cute_b200_gemm_desc *desc, const void *hA, const void *hB,
                                                void *hC, double *seconds) {
    return gemm_tn_sharded_host(comm, desc, hA, hB, hC, seconds);
}

cute_b200_status cute_b200_device_status(uint32_t out[4]) {
    if (!out) return fail(CUTE_B200_ERR_NULL_POINTER, "device_status: null output");
    return read_status(out);
}

cute_b200_status cute_b200_gemm_layout_info(int32_t cta_group, int32_t tile_n, int32_t tile_m, int32_t ab_dtype,
                                            int32_t c_dtype, uint32_t smem_addr, cute_b200_gemm_layout *out) {
    return gemm_layout_info(cta_group, tile_n, tile_m, ab_dtype, c_dtype, smem_addr, out);
}

cute_b200_status cute_b200_gemm_plan(const cute_b200_gemm_desc *desc, int32_t sm_count, int32_t out[4]) {
    if (!desc || !out) return fail(CUTE_B200_ERR_NULL_POINTER, "gemm_plan: null argument");
    return gemm_plan(*desc, sm_count, out);
}

uint64_t cute_b200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

}  // extern "C"
