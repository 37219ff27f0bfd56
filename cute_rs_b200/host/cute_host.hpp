// C++ mirror of the cute-rs launch surface for the hot-path kernels, on top of
// the C ABI of libcute_b200.so (include/cute_b200.h).
//
// The reference crate is Rust; where a Rust toolchain is not available this
// header gives compiled-language callers the same names, argument meaning and
// error behaviour:
//   Kernel::builder(name).block_dim({..}).build(closure) with param_tensor /
//   param_ptr / param_extent / param_scalar inside the closure
//   (src/builder.rs:747-824, src/tensor.rs:401-431, 526-539);
//   KernelArg, LaunchConfig (src/sim/mod.rs:41-216);
//   CudaContext::{upload, download, launch, launch_on_device, launch_async,
//   synchronize}, Kernel::run_cuda (src/cuda.rs:204-488, 570-593).
// Like the reference's launcher (src/cuda.rs:88-196) it binds its native
// library with dlopen at run time, so building needs no CUDA installation.
//
// Only launching is mirrored: the closure declares parameters, the kernel that
// runs is the sm_100a kernel of that name.  There is no CPU path.
#pragma once

#include <dlfcn.h>

#include <cmath>
#include <cstdint>
#include <cstring>
#include <functional>
#include <memory>
#include <optional>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/cute_b200.h"

namespace cute {

enum class DType { F16 = CUTE_B200_F16, BF16 = CUTE_B200_BF16, F32 = CUTE_B200_F32, I32 = CUTE_B200_I32 };

inline const char *dtype_name(DType t) {
    switch (t) {
        case DType::F16: return "f16";
        case DType::BF16: return "bf16";
        case DType::F32: return "f32";
        default: return "i32";
    }
}
inline size_t dtype_bytes(DType t) { return (t == DType::F16 || t == DType::BF16) ? 2 : 4; }

// ---- host conversions (src/value.rs:88-158) ---------------------------------
inline uint16_t f32_to_bf16_bits(float x) {
    uint32_t bits;
    std::memcpy(&bits, &x, 4);
    const uint16_t high = uint16_t(bits >> 16);
    const uint32_t low = bits & 0xffffu;
    if (x != x) return high | 0x40;
    return uint16_t(high + ((low > 0x8000u || (low == 0x8000u && (high & 1))) ? 1 : 0));
}
inline float bf16_bits_to_f32(uint16_t h) {
    const uint32_t bits = uint32_t(h) << 16;
    float x;
    std::memcpy(&x, &bits, 4);
    return x;
}
inline uint16_t f32_to_f16_bits(float x) {
    uint32_t b;
    std::memcpy(&b, &x, 4);
    const uint16_t sign = uint16_t((b >> 16) & 0x8000u);
    const int32_t exp = int32_t((b >> 23) & 0xff);
    const uint32_t mant = b & 0x7fffffu;
    if (exp == 0xff) return sign | 0x7c00 | (mant ? uint16_t(0x200u | (mant >> 13)) : 0);
    const int32_t e = exp - 127 + 15;
    if (e >= 0x1f) return sign | 0x7c00;
    if (e <= 0) {
        if (e < -10) return sign;
        const uint32_t m = mant | 0x800000u, shift = uint32_t(14 - e), half = 1u << (shift - 1);
        const uint32_t rem = m & ((1u << shift) - 1);
        uint32_t r = m >> shift;
        if (rem > half || (rem == half && (r & 1))) r += 1;
        return sign | uint16_t(r);
    }
    uint32_t r = (uint32_t(e) << 10) | (mant >> 13);
    const uint32_t rem = mant & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (r & 1))) r += 1;
    return sign | uint16_t(r);
}

// ---- errors --------------------------------------------------------------------
struct CudaError : std::runtime_error {
    std::string message;
    int status;
    CudaError(std::string msg, int st = CUTE_B200_ERR_CUDA)
        : std::runtime_error("CUDA: " + msg), message(std::move(msg)), status(st) {}
};

// ---- the native library, bound with dlopen ---------------------------------------
struct Api {
    void *handle = nullptr;
    decltype(&cute_b200_init) init = nullptr;
    decltype(&cute_b200_last_error) last_error = nullptr;
    decltype(&cute_b200_launch) launch = nullptr;
    decltype(&cute_b200_launch_host) launch_host = nullptr;
    decltype(&cute_b200_upload) upload = nullptr;
    decltype(&cute_b200_download) download = nullptr;
    decltype(&cute_b200_free) free_ = nullptr;
    decltype(&cute_b200_synchronize) synchronize = nullptr;
    decltype(&cute_b200_comm_create) comm_create = nullptr;
    decltype(&cute_b200_comm_destroy) comm_destroy = nullptr;
    decltype(&cute_b200_comm_info) comm_info = nullptr;
    decltype(&cute_b200_gemm_tn_sharded) gemm_tn_sharded = nullptr;
    decltype(&cute_b200_gemm_tn_sharded_host) gemm_tn_sharded_host = nullptr;

    static const Api &get(const char *path = nullptr) {
        static Api api = load(path);
        return api;
    }

   private:
    template <class F>
    static void bind(void *h, F &fn, const char *name) {
        fn = reinterpret_cast<F>(dlsym(h, name));
        if (!fn) throw CudaError(std::string("symbol ") + name + " not found in libcute_b200.so");
    }
    static Api load(const char *path) {
        const char *env = std::getenv("CUTE_B200_LIB");
        const char *file = path ? path : (env ? env : "libcute_b200.so");
        Api a;
        a.handle = dlopen(file, RTLD_NOW);
        if (!a.handle) throw CudaError(std::string("could not load ") + file + ": " + dlerror(), CUTE_B200_ERR_NO_DEVICE);
        bind(a.handle, a.init, "cute_b200_init");
        bind(a.handle, a.last_error, "cute_b200_last_error");
        bind(a.handle, a.launch, "cute_b200_launch");
        bind(a.handle, a.launch_host, "cute_b200_launch_host");
        bind(a.handle, a.upload, "cute_b200_upload");
        bind(a.handle, a.download, "cute_b200_download");
        bind(a.handle, a.free_, "cute_b200_free");
        bind(a.handle, a.synchronize, "cute_b200_synchronize");
        bind(a.handle, a.comm_create, "cute_b200_comm_create");
        bind(a.handle, a.comm_destroy, "cute_b200_comm_destroy");
        bind(a.handle, a.comm_info, "cute_b200_comm_info");
        bind(a.handle, a.gemm_tn_sharded, "cute_b200_gemm_tn_sharded");
        bind(a.handle, a.gemm_tn_sharded_host, "cute_b200_gemm_tn_sharded_host");
        return a;
    }
};

inline void check(int status) {
    if (status != CUTE_B200_OK) throw CudaError(Api::get().last_error(), status);
}

// ---- layouts: what param_tensor needs -----------------------------------------------
struct Layout {
    std::vector<int64_t> shape, stride;
    static Layout row_major(std::vector<int64_t> s) {
        Layout l{s, std::vector<int64_t>(s.size())};
        int64_t acc = 1;
        for (size_t i = s.size(); i-- > 0;) l.stride[i] = acc, acc *= s[i];
        return l;
    }
    static Layout col_major(std::vector<int64_t> s) {
        Layout l{s, std::vector<int64_t>(s.size())};
        int64_t acc = 1;
        for (size_t i = 0; i < s.size(); i++) l.stride[i] = acc, acc *= s[i];
        return l;
    }
    int64_t size() const {
        int64_t n = 1;
        for (int64_t s : shape) n *= s;
        return n;
    }
    // One past the largest offset the layout produces.
    int64_t cosize() const {
        if (size() == 0) return 0;
        int64_t n = 1;
        for (size_t i = 0; i < shape.size(); i++) n += (shape[i] - 1) * stride[i];
        return n;
    }
};

// ---- launch configuration and arguments (src/sim/mod.rs:41-216) -------------------------
struct LaunchConfig {
    uint32_t grid[3], block[3], cluster[3] = {1, 1, 1};
    static LaunchConfig make(std::initializer_list<uint32_t> g, std::initializer_list<uint32_t> b) {
        LaunchConfig c{};
        std::copy(g.begin(), g.end(), c.grid);
        std::copy(b.begin(), b.end(), c.block);
        c.cluster[0] = c.cluster[1] = c.cluster[2] = 1;
        return c;
    }
    LaunchConfig with_cluster(std::initializer_list<uint32_t> cl) const {
        LaunchConfig c = *this;
        std::copy(cl.begin(), cl.end(), c.cluster);
        return c;
    }
    size_t threads_per_block() const { return size_t(block[0]) * block[1] * block[2]; }
};

// A buffer per tensor parameter or a scalar per scalar parameter.
struct KernelArg {
    DType dtype = DType::F32;
    bool is_scalar = false;
    std::vector<uint8_t> bytes;  // buffers, little-endian elements
    uint64_t bits = 0;           // scalars

    static KernelArg f32(const std::vector<float> &v) { return raw(DType::F32, v.data(), v.size() * 4); }
    static KernelArg i32(const std::vector<int32_t> &v) { return raw(DType::I32, v.data(), v.size() * 4); }
    static KernelArg f16_from_f32(const std::vector<float> &v) {
        std::vector<uint16_t> h(v.size());
        for (size_t i = 0; i < v.size(); i++) h[i] = f32_to_f16_bits(v[i]);
        return raw(DType::F16, h.data(), h.size() * 2);
    }
    static KernelArg bf16_from_f32(const std::vector<float> &v) {
        std::vector<uint16_t> h(v.size());
        for (size_t i = 0; i < v.size(); i++) h[i] = f32_to_bf16_bits(v[i]);
        return raw(DType::BF16, h.data(), h.size() * 2);
    }
    // Elements of any type as raw bytes (KernelArg::Bytes, src/sim/mod.rs:80-84).
    static KernelArg Bytes(DType t, const void *p, size_t nbytes) { return raw(t, p, nbytes); }
    static KernelArg ScalarF32(float x) {
        KernelArg a;
        a.dtype = DType::F32, a.is_scalar = true;
        uint32_t b;
        std::memcpy(&b, &x, 4);
        a.bits = b;
        return a;
    }
    static KernelArg ScalarI32(int32_t x) {
        KernelArg a;
        a.dtype = DType::I32, a.is_scalar = true, a.bits = uint32_t(x);
        return a;
    }
    size_t len() const { return bytes.size() / dtype_bytes(dtype); }
    std::string describe() const {
        const char *article = (dtype == DType::BF16) ? "a" : "an";
        if (is_scalar) return std::string(article) + " " + dtype_name(dtype) + " scalar";
        return std::string(article) + " " + dtype_name(dtype) + " buffer of " + std::to_string(len());
    }
    // The contents of an f32 buffer (KernelArg::as_f32).
    const float *as_f32() const {
        if (is_scalar || dtype != DType::F32) throw std::logic_error("argument is " + describe() + ", not an f32 buffer");
        return reinterpret_cast<const float *>(bytes.data());
    }
    bool operator==(const KernelArg &o) const {
        return dtype == o.dtype && is_scalar == o.is_scalar && bytes == o.bytes && bits == o.bits;
    }

   private:
    static KernelArg raw(DType t, const void *p, size_t n) {
        KernelArg a;
        a.dtype = t;
        a.bytes.assign(static_cast<const uint8_t *>(p), static_cast<const uint8_t *>(p) + n);
        return a;
    }
};

// ---- kernel builder ---------------------------------------------------------------------
struct Param {
    std::string name;
    DType dtype;
    bool is_scalar;
    std::optional<int64_t> length;  // buffers: minimum element count; none for param_ptr
    int64_t multiple_of = 1;
};

namespace detail {
inline std::vector<Param> *&current_params() {
    static thread_local std::vector<Param> *p = nullptr;
    return p;
}
inline void declare(Param p) {
    auto *params = current_params();
    if (!params) throw std::logic_error("kernel parameters can only be declared inside Kernel::builder(..).build(closure)");
    for (const Param &q : *params)
        if (q.name == p.name) throw std::logic_error("duplicate kernel parameter `" + p.name + "`");
    params->push_back(std::move(p));
}
}  // namespace detail

inline void param_tensor(DType t, const std::string &name, const Layout &layout) {
    detail::declare({name, t, false, layout.cosize(), 1});
}
inline void param_ptr(DType t, const std::string &name) { detail::declare({name, t, false, std::nullopt, 1}); }
inline void param_extent(const std::string &name, int64_t multiple_of = 1) {
    detail::declare({name, DType::I32, true, std::nullopt, multiple_of});
}
inline void param_scalar(DType t, const std::string &name) { detail::declare({name, t, true, std::nullopt, 1}); }

struct LaunchStats {
    double kernel_seconds;
};

class CudaContext;

class Kernel {
   public:
    class Options {
       public:
        explicit Options(std::string name) : name_(std::move(name)) {}
        Options &block_dim(std::initializer_list<uint32_t> d) {
            block_.assign(d.begin(), d.end());
            return *this;
        }
        Kernel build(const std::function<void()> &closure) {
            if (detail::current_params()) throw std::logic_error("Kernel builds cannot be nested");
            std::vector<Param> params;
            detail::current_params() = &params;
            try {
                closure();
            } catch (...) {
                detail::current_params() = nullptr;
                throw;
            }
            detail::current_params() = nullptr;
            return Kernel(name_, block_, std::move(params));
        }

       private:
        std::string name_;
        std::vector<uint32_t> block_;
    };
    static Options builder(const std::string &name) { return Options(name); }
    const std::string &name() const { return name_; }
    const std::vector<Param> &params() const { return params_; }
    const std::vector<uint32_t> &block_dim() const { return block_; }
    // Upload, run, wait, download (Kernel::run_cuda, src/cuda.rs:574-592).
    LaunchStats run_cuda(CudaContext &ctx, const LaunchConfig &cfg, std::vector<KernelArg> &args) const;

   private:
    Kernel(std::string n, std::vector<uint32_t> b, std::vector<Param> p)
        : name_(std::move(n)), block_(std::move(b)), params_(std::move(p)) {}
    std::string name_;
    std::vector<uint32_t> block_;
    std::vector<Param> params_;
};

// ---- launcher (src/cuda.rs:204-488) --------------------------------------------------------
// Device memory owned by the object and freed with it (DeviceBuffer, src/cuda.rs:491-502).
class DeviceBuffer {
   public:
    DeviceBuffer(uint64_t ptr, size_t bytes, DType t, size_t len) : ptr_(ptr), bytes_(bytes), dtype_(t), len_(len) {}
    DeviceBuffer(const DeviceBuffer &) = delete;
    DeviceBuffer &operator=(const DeviceBuffer &) = delete;
    DeviceBuffer(DeviceBuffer &&o) noexcept : ptr_(o.ptr_), bytes_(o.bytes_), dtype_(o.dtype_), len_(o.len_) { o.ptr_ = 0; }
    ~DeviceBuffer() {
        if (ptr_) Api::get().free_(ptr_);
    }
    uint64_t ptr() const { return ptr_; }
    size_t bytes() const { return bytes_; }
    DType dtype() const { return dtype_; }
    size_t len() const { return len_; }

   private:
    uint64_t ptr_;
    size_t bytes_;
    DType dtype_;
    size_t len_;
};

// A launch argument already on the device (DeviceArg, src/cuda.rs:505-509).
struct DeviceArg {
    const DeviceBuffer *buffer = nullptr;
    KernelArg scalar;
    static DeviceArg Buffer(const DeviceBuffer &b) {
        DeviceArg a;
        a.buffer = &b;
        return a;
    }
    static DeviceArg Scalar(const KernelArg &s) {
        DeviceArg a;
        a.scalar = s;
        return a;
    }
};

class CudaContext {
   public:
    explicit CudaContext(int ordinal = 0) : ordinal_(ordinal) { check(Api::get().init(ordinal)); }

    DeviceBuffer upload(const KernelArg &arg) const {
        if (arg.is_scalar) throw std::logic_error("only buffers can be uploaded");
        uint64_t ptr = 0;
        check(Api::get().upload(arg.bytes.data(), arg.bytes.size(), &ptr));
        return DeviceBuffer(ptr, arg.bytes.size(), arg.dtype, arg.len());
    }
    void download(const DeviceBuffer &buffer, KernelArg &arg) const {
        if (arg.bytes.size() != buffer.bytes())
            throw CudaError("downloading " + std::to_string(buffer.bytes()) + " bytes into " + std::to_string(arg.bytes.size()));
        check(Api::get().download(buffer.ptr(), arg.bytes.data(), buffer.bytes()));
    }
    void synchronize() const { check(Api::get().synchronize()); }

    // Host buffers in, results copied back in place (CudaContext::launch).
    LaunchStats launch(const Kernel &kernel, const LaunchConfig &cfg, std::vector<KernelArg> &args) const {
        check_count(kernel, args.size());
        std::vector<cute_b200_arg> slots;
        for (size_t i = 0; i < args.size(); i++) {
            KernelArg &a = args[i];
            check_length(kernel, i, a.is_scalar, a.len());
            slots.push_back({a.is_scalar ? 1 : 0, int32_t(a.dtype),
                             a.is_scalar ? a.bits : reinterpret_cast<uint64_t>(a.bytes.data()), a.is_scalar ? 0 : a.len()});
        }
        double seconds = 0.0;
        const cute_b200_launch_config c = to_c(cfg);
        check(Api::get().launch_host(kernel.name().c_str(), &c, slots.data(), int32_t(slots.size()), &seconds));
        return {seconds};
    }
    // Submit without waiting, arguments already on the device (launch_async).
    void launch_async(const Kernel &kernel, const LaunchConfig &cfg, const std::vector<DeviceArg> &args,
                      void *stream = nullptr) const {
        check_count(kernel, args.size());
        std::vector<cute_b200_arg> slots;
        for (size_t i = 0; i < args.size(); i++) {
            const DeviceArg &a = args[i];
            if (a.buffer) {
                check_length(kernel, i, false, a.buffer->len());
                slots.push_back({0, int32_t(a.buffer->dtype()), a.buffer->ptr(), a.buffer->len()});
            } else {
                slots.push_back({1, int32_t(a.scalar.dtype), a.scalar.bits, 0});
            }
        }
        const cute_b200_launch_config c = to_c(cfg);
        check(Api::get().launch(kernel.name().c_str(), &c, slots.data(), int32_t(slots.size()), stream));
    }
    // Submit and wait (launch_on_device).
    void launch_on_device(const Kernel &kernel, const LaunchConfig &cfg, const std::vector<DeviceArg> &args) const {
        launch_async(kernel, cfg, args);
        synchronize();
    }

   private:
    static cute_b200_launch_config to_c(const LaunchConfig &cfg) {
        cute_b200_launch_config c;
        for (int i = 0; i < 3; i++) c.grid[i] = cfg.grid[i], c.block[i] = cfg.block[i], c.cluster[i] = cfg.cluster[i];
        return c;
    }
    static void check_count(const Kernel &k, size_t n) {
        if (n != k.params().size())
            throw CudaError("kernel `" + k.name() + "` takes " + std::to_string(k.params().size()) + " arguments, " +
                                std::to_string(n) + " were given",
                            CUTE_B200_ERR_INVALID_ARGUMENT);
    }
    // The statically declared size of a param_tensor (src/sim/mod.rs:350-357).
    static void check_length(const Kernel &k, size_t i, bool is_scalar, size_t len) {
        const Param &p = k.params()[i];
        if (!p.is_scalar && !is_scalar && p.length && int64_t(len) < *p.length)
            throw CudaError("argument " + std::to_string(i) + " (`" + p.name + "`) needs at least " +
                                std::to_string(*p.length) + " elements, got " + std::to_string(len),
                            CUTE_B200_ERR_INVALID_ARGUMENT);
    }
    int ordinal_;
};

inline LaunchStats Kernel::run_cuda(CudaContext &ctx, const LaunchConfig &cfg, std::vector<KernelArg> &args) const {
    return ctx.launch(*this, cfg, args);
}

// ---- the reference's example kernels, declared through the builder --------------------------
namespace examples {

struct GemmConfig {  // examples/tensorop_gemm.rs:22-40
    int64_t m, n, k, bm = 128, bn = 128, bk = 32, stages = 3;
    bool swizzle = true;
    DType ab = DType::F16;
};

inline Kernel tensorop_gemm(const GemmConfig &cfg) {  // examples/tensorop_gemm.rs:42-164
    if (cfg.ab != DType::F16 && cfg.ab != DType::BF16) throw std::invalid_argument("tensorop_gemm takes f16 or bf16 inputs");
    if (cfg.m % cfg.bm || cfg.n % cfg.bn || cfg.k % cfg.bk)
        throw std::invalid_argument("problem size must be a multiple of the tile size");
    const bool bf = cfg.ab == DType::BF16;
    const char *name = cfg.swizzle ? (bf ? "tensorop_gemm_bf16" : "tensorop_gemm")
                                   : (bf ? "tensorop_gemm_bf16_unswizzled" : "tensorop_gemm_unswizzled");
    return Kernel::builder(name).block_dim({128, 1, 1}).build([&] {
        param_tensor(cfg.ab, "a", Layout::row_major({cfg.m, cfg.k}));
        param_tensor(cfg.ab, "b", Layout::row_major({cfg.n, cfg.k}));
        param_tensor(DType::F32, "c", Layout::row_major({cfg.m, cfg.n}));
    });
}

inline Kernel runtime_gemm() {  // examples/runtime_gemm.rs:22-33
    return Kernel::builder("runtime_gemm").block_dim({128, 1, 1}).build([] {
        param_ptr(DType::F16, "a");
        param_ptr(DType::F16, "b");
        param_ptr(DType::F32, "c");
        param_extent("n", 128);
        param_extent("k", 32);
    });
}

inline Kernel sgemm(int64_t m, int64_t n, int64_t k) {  // examples/sgemm.rs:23-33
    if (m % 128 || n % 128 || k % 8) throw std::invalid_argument("problem size must be a multiple of the tile size");
    return Kernel::builder("sgemm_nt").block_dim({256, 1, 1}).build([&] {
        param_tensor(DType::F32, "a", Layout::col_major({m, k}));
        param_tensor(DType::F32, "b", Layout::col_major({n, k}));
        param_tensor(DType::F32, "c", Layout::col_major({m, n}));
        param_scalar(DType::F32, "alpha");
        param_scalar(DType::F32, "beta");
    });
}

inline Kernel elementwise_add(bool tiled, int64_t m = 300, int64_t n = 512) {  // examples/elementwise_add.rs:23-80
    return Kernel::builder(tiled ? "elementwise_add_tiled" : "elementwise_add_naive")
        .block_dim({tiled ? 128u : 256u, 1, 1})
        .build([&] {
            for (const char *p : {"a", "b", "c"}) param_tensor(DType::F32, p, Layout::row_major({m, n}));
        });
}

}  // namespace examples
// ---- several GPUs behind one call -------------------------------------------------------
// What a `CudaContext` over all the GPUs of a box looks like: the launcher the library adds next
// to src/cuda.rs.  One object, one call per GEMM; the library cuts the rows among the GPUs.
class MultiGpuContext {
   public:
    explicit MultiGpuContext(const std::vector<int> &ordinals) {
        std::vector<int32_t> o(ordinals.begin(), ordinals.end());
        check(Api::get().comm_create(int32_t(o.size()), o.data(), &comm_));
        n_ = int(o.size());
    }
    MultiGpuContext(const MultiGpuContext &) = delete;
    MultiGpuContext &operator=(const MultiGpuContext &) = delete;
    ~MultiGpuContext() {
        if (comm_) Api::get().comm_destroy(comm_);
    }
    int gpus() const { return n_; }
    bool has_collective_library() const {
        int32_t out[4] = {0, 0, 0, 0};
        check(Api::get().comm_info(comm_, out));
        return out[3] != 0;
    }
    // Host matrices in, C back in place: CudaContext::launch for the row-sharded GEMM.
    LaunchStats gemm(const cute_b200_gemm_desc &desc, const KernelArg &a, const KernelArg &b, KernelArg &c) const {
        double seconds = 0.0;
        check(Api::get().gemm_tn_sharded_host(comm_, &desc, a.bytes.data(), b.bytes.data(), c.bytes.data(), &seconds));
        return {seconds};
    }
    // Device buffers, one per GPU (launch_on_device): returns when every GPU is done.
    void gemm_on_devices(const cute_b200_gemm_desc &desc, const std::vector<uint64_t> &a_shards, const std::vector<uint64_t> &b,
                         const std::vector<uint64_t> &c, int replicate_c) const {
        if (int(a_shards.size()) != n_ || int(b.size()) != n_ || int(c.size()) != n_)
            throw CudaError("one buffer per GPU is needed", CUTE_B200_ERR_INVALID_ARGUMENT);
        check(Api::get().gemm_tn_sharded(comm_, &desc, a_shards.data(), b.data(), c.data(), replicate_c));
    }

   private:
    void *comm_ = nullptr;
    int n_ = 0;
};

}  // namespace cute
