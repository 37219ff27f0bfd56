// C++ counterpart of the reference's GPU tests (tests/gpu.rs) written against
// cute_host.hpp: the same kernels, inputs and acceptance rules, with the CPU
// oracle (liboracle.so, test infrastructure) in the simulator's place.
//
//   test_host_mirror cpu   checks that need no device (builder, launch checks)
//   test_host_mirror gpu   runs every kernel on device 0 and compares
#include <cstdio>
#include <cstdlib>
#include <string>

#include "../../cute_rs_b200/host/cute_host.hpp"

extern "C" {
int oracle_gemm_tn(int ab, int c, size_t M, size_t N, size_t K, const void *A, const void *B, void *C, float alpha,
                   float beta, size_t r0, size_t r1);
int oracle_gemm_tn_abs(int ab, size_t M, size_t N, size_t K, const void *A, const void *B, float *mag, size_t r0, size_t r1);
int oracle_sgemm_nt(size_t M, size_t N, size_t K, float alpha, float beta, const float *A, const float *B, float *C);
void oracle_elementwise_add_f32(const float *x, const float *y, float *out, size_t n);
}

using namespace cute;
static int failures = 0;
#define EXPECT(cond)                                                          \
    do {                                                                      \
        if (!(cond)) {                                                        \
            std::printf("FAIL %s:%d: %s\n", __FILE__, __LINE__, #cond);       \
            failures++;                                                       \
        }                                                                     \
    } while (0)

template <class F>
static std::string error_of(F &&f) {
    try {
        f();
    } catch (const CudaError &e) {
        return e.message;
    } catch (const std::exception &e) {
        return std::string("other: ") + e.what();
    }
    return "";
}

// One input per kernel parameter from the LCG of tests/gpu.rs:55-83.
struct Lcg {
    uint64_t state = 1;
    uint64_t next() {
        state = state * 6364136223846793005ull + 1442695040888963407ull;
        return state >> 40;
    }
};
static std::vector<KernelArg> inputs(const Kernel &kernel, bool small, const std::vector<size_t> &ptr_lens = {}) {
    Lcg g;
    const float scalars[2] = {1.5f, -0.5f};
    int next_scalar = 0;
    size_t next_ptr = 0;
    std::vector<KernelArg> out;
    for (const Param &p : kernel.params()) {
        if (p.is_scalar) {
            out.push_back(KernelArg::ScalarF32(scalars[next_scalar++ % 2]));
            continue;
        }
        const size_t n = p.length ? size_t(*p.length) : ptr_lens.at(next_ptr++);
        std::vector<float> v(n);
        for (float &x : v) x = small ? float(g.next() % 17) - 8.0f : float(g.next()) / float(1 << 23) - 1.0f;
        out.push_back(p.dtype == DType::F16 ? KernelArg::f16_from_f32(v)
                                            : p.dtype == DType::BF16 ? KernelArg::bf16_from_f32(v) : KernelArg::f32(v));
    }
    return out;
}

static void cpu_checks() {
    Kernel k = examples::tensorop_gemm({256, 128, 96});
    EXPECT(k.name() == "tensorop_gemm" && k.params().size() == 3 && *k.params()[0].length == 256 * 96);
    EXPECT(examples::tensorop_gemm({256, 128, 96, 128, 128, 32, 3, false, DType::BF16}).name() == "tensorop_gemm_bf16_unswizzled");
    EXPECT(examples::runtime_gemm().params()[4].multiple_of == 32);
    EXPECT(Layout::col_major({128, 8}).stride[1] == 128 && Layout::row_major({300, 512}).cosize() == 300 * 512);
    EXPECT(f32_to_f16_bits(1.0f) == 0x3c00 && f32_to_f16_bits(65520.0f) == 0x7c00 && f32_to_bf16_bits(1.00390625f) == 0x3f80);
    bool threw = false;
    try {
        param_tensor(DType::F32, "x", Layout::row_major({4}));
    } catch (const std::logic_error &) {
        threw = true;
    }
    EXPECT(threw);
    // check_launch messages (src/sim/mod.rs:328-385) come back before any device is touched
    CudaContext *no_ctx = nullptr;
    (void)no_ctx;
    std::vector<KernelArg> args = inputs(examples::elementwise_add(true, 16, 128), true);
    const Api &api = Api::get();
    auto call = [&](const Kernel &kern, LaunchConfig cfg, std::vector<KernelArg> &a) {
        std::vector<cute_b200_arg> slots;
        for (KernelArg &x : a)
            slots.push_back({x.is_scalar ? 1 : 0, int32_t(x.dtype), x.is_scalar ? x.bits : uint64_t(0), x.is_scalar ? 0 : x.len()});
        cute_b200_launch_config c;
        for (int i = 0; i < 3; i++) c.grid[i] = cfg.grid[i], c.block[i] = cfg.block[i], c.cluster[i] = cfg.cluster[i];
        return api.launch_host(kern.name().c_str(), &c, slots.data(), int32_t(slots.size()), nullptr) == 0
                   ? std::string()
                   : std::string(api.last_error());
    };
    Kernel add = examples::elementwise_add(true, 16, 128);
    EXPECT(call(add, LaunchConfig::make({1, 1, 1}, {256, 1, 1}), args) ==
           "kernel `elementwise_add_tiled` was built for blocks of [128, 1, 1], launched with [256, 1, 1]");
    EXPECT(call(add, LaunchConfig::make({0, 1, 1}, {128, 1, 1}), args) == "invalid grid size [0, 1, 1]");
    EXPECT(call(add, LaunchConfig::make({3, 1, 1}, {128, 1, 1}).with_cluster({2, 1, 1}), args) ==
           "grid [3, 1, 1] is not a whole number of clusters of [2, 1, 1]");
    Kernel rt = examples::runtime_gemm();
    std::vector<KernelArg> rargs = inputs(rt, true, {128 * 32, 128 * 32, 128 * 128});
    rargs[3] = KernelArg::ScalarI32(128);
    rargs[4] = KernelArg::ScalarI32(40);
    EXPECT(call(rt, LaunchConfig::make({1, 1, 1}, {128, 1, 1}), rargs) == "argument 4 (`k`) must be a multiple of 32, got 40");
    args.pop_back();
    EXPECT(call(add, LaunchConfig::make({1, 1, 1}, {128, 1, 1}), args) ==
           "kernel `elementwise_add_tiled` takes 3 arguments, 2 were given");
}

static size_t output_index(const Kernel &k) {
    size_t last = 0;
    for (size_t i = 0; i < k.params().size(); i++)
        if (!k.params()[i].is_scalar) last = i;
    return last;
}

// Run on the GPU from `input`; inputs other than the output must come back unchanged (tests/gpu.rs:92-109).
static std::vector<float> run_gpu(CudaContext &ctx, const Kernel &k, const LaunchConfig &cfg, const std::vector<KernelArg> &input) {
    std::vector<KernelArg> on_gpu = input;
    const LaunchStats st = k.run_cuda(ctx, cfg, on_gpu);
    EXPECT(st.kernel_seconds > 0.0);
    const size_t out = output_index(k);
    for (size_t i = 0; i < input.size(); i++)
        if (i != out) EXPECT(on_gpu[i] == input[i]);
    const float *p = on_gpu[out].as_f32();
    return std::vector<float>(p, p + on_gpu[out].len());
}

static bool identical(const std::vector<float> &a, const std::vector<float> &b) {
    return a.size() == b.size() && std::memcmp(a.data(), b.data(), a.size() * 4) == 0;
}

// Bit-exact on small integers, within 2 * terms * 2^-23 * sum|a*b| on data that rounds (tests/gpu.rs:146-176).
static void check_tensor_core(CudaContext &ctx, const Kernel &k, const LaunchConfig &cfg, size_t m, size_t n, size_t kk,
                              const std::vector<size_t> &ptr_lens = {}) {
    const int ab = k.params()[0].dtype == DType::BF16 ? 1 : 0;
    for (bool small : {true, false}) {
        std::vector<KernelArg> in = inputs(k, small, ptr_lens);
        if (k.name() == "runtime_gemm") in[3] = KernelArg::ScalarI32(int32_t(n)), in[4] = KernelArg::ScalarI32(int32_t(kk));
        const std::vector<float> gpu = run_gpu(ctx, k, cfg, in);
        std::vector<float> sim(m * n, 0.0f), mag(m * n, 0.0f);
        oracle_gemm_tn(ab, 2, m, n, kk, in[0].bytes.data(), in[1].bytes.data(), sim.data(), 1.0f, 0.0f, 0, m);
        if (small) {
            EXPECT(identical(std::vector<float>(gpu.begin(), gpu.begin() + m * n), sim));
        } else {
            oracle_gemm_tn_abs(ab, m, n, kk, in[0].bytes.data(), in[1].bytes.data(), mag.data(), 0, m);
            size_t bad = 0;
            for (size_t i = 0; i < m * n; i++)
                if (std::fabs(double(gpu[i]) - double(sim[i])) > 2.0 * double(kk) * std::ldexp(1.0, -23) * double(mag[i])) bad++;
            EXPECT(bad == 0);
        }
    }
}

static void gpu_checks() {
    CudaContext ctx(0);
    // elementwise_add, naive and tiled: bit-exact on both data sets (tests/gpu.rs:243-247)
    for (bool tiled : {false, true}) {
        Kernel k = examples::elementwise_add(tiled);
        const LaunchConfig cfg = tiled ? LaunchConfig::make({19, 4, 1}, {128, 1, 1}) : LaunchConfig::make({600, 1, 1}, {256, 1, 1});
        for (bool small : {true, false}) {
            std::vector<KernelArg> in = inputs(k, small);
            std::vector<float> sim(300 * 512);
            oracle_elementwise_add_f32(in[0].as_f32(), in[1].as_f32(), sim.data(), sim.size());
            EXPECT(identical(run_gpu(ctx, k, cfg, in), sim));
        }
    }
    // sgemm: two 128 x 128 tiles of C (tests/gpu.rs:249-253)
    {
        Kernel k = examples::sgemm(256, 128, 32);
        for (bool small : {true, false}) {
            std::vector<KernelArg> in = inputs(k, small);
            std::vector<float> sim(in[2].as_f32(), in[2].as_f32() + 256 * 128);
            oracle_sgemm_nt(256, 128, 32, 1.5f, -0.5f, in[0].as_f32(), in[1].as_f32(), sim.data());
            EXPECT(identical(run_gpu(ctx, k, LaunchConfig::make({2, 1, 1}, {256, 1, 1}), in), sim));
        }
    }
    // tensorop_gemm: grid and short pipeline, long k loop, unswizzled name, bf16 (tests/gpu.rs:260-284)
    check_tensor_core(ctx, examples::tensorop_gemm({256, 128, 96}), LaunchConfig::make({2, 1, 1}, {128, 1, 1}), 256, 128, 96);
    check_tensor_core(ctx, examples::tensorop_gemm({256, 256, 256}), LaunchConfig::make({2, 2, 1}, {128, 1, 1}), 256, 256, 256);
    check_tensor_core(ctx, examples::tensorop_gemm({256, 256, 256, 128, 128, 32, 3, false}), LaunchConfig::make({2, 2, 1}, {128, 1, 1}),
                      256, 256, 256);
    check_tensor_core(ctx, examples::tensorop_gemm({256, 128, 96, 128, 128, 32, 3, true, DType::BF16}),
                      LaunchConfig::make({2, 1, 1}, {128, 1, 1}), 256, 128, 96);
    // runtime_gemm: one kernel, several sizes (tests/gpu.rs:212-241)
    Kernel rt = examples::runtime_gemm();
    const size_t sizes[][3] = {{128, 128, 32}, {256, 128, 96}, {128, 256, 160}, {512, 512, 512}};
    for (auto &s : sizes)
        check_tensor_core(ctx, rt, LaunchConfig::make({uint32_t(s[0] / 128), uint32_t(s[1] / 128), 1}, {128, 1, 1}), s[0], s[1], s[2],
                          {s[0] * s[2], s[1] * s[2], s[0] * s[1]});
    // device-resident relaunch x3
    {
        std::vector<KernelArg> in = inputs(rt, true, {256 * 64, 256 * 64, 256 * 256});
        in[3] = KernelArg::ScalarI32(256), in[4] = KernelArg::ScalarI32(64);
        DeviceBuffer ua = ctx.upload(in[0]), ub = ctx.upload(in[1]), uc = ctx.upload(in[2]);
        const std::vector<DeviceArg> dargs = {DeviceArg::Buffer(ua), DeviceArg::Buffer(ub), DeviceArg::Buffer(uc),
                                              DeviceArg::Scalar(in[3]), DeviceArg::Scalar(in[4])};
        for (int i = 0; i < 3; i++) ctx.launch_async(rt, LaunchConfig::make({2, 2, 1}, {128, 1, 1}), dargs);
        ctx.synchronize();
        ctx.download(uc, in[2]);
        std::vector<float> sim(256 * 256);
        oracle_gemm_tn(0, 2, 256, 256, 64, in[0].bytes.data(), in[1].bytes.data(), sim.data(), 1.0f, 0.0f, 0, 256);
        EXPECT(std::memcmp(in[2].bytes.data(), sim.data(), sim.size() * 4) == 0);
    }
    // errors through the context
    {
        std::vector<KernelArg> in = inputs(rt, true, {128 * 32, 128 * 32, 128 * 128});
        in[3] = KernelArg::ScalarI32(128), in[4] = KernelArg::ScalarI32(40);
        EXPECT(error_of([&] { ctx.launch(rt, LaunchConfig::make({1, 1, 1}, {128, 1, 1}), in); }) ==
               "argument 4 (`k`) must be a multiple of 32, got 40");
        Kernel t = examples::tensorop_gemm({128, 128, 64});
        std::vector<KernelArg> small_in = inputs(examples::tensorop_gemm({128, 128, 32}), true);
        EXPECT(error_of([&] { ctx.launch(t, LaunchConfig::make({1, 1, 1}, {128, 1, 1}), small_in); }) ==
               "argument 0 (`a`) needs at least 8192 elements, got 4096");
    }
}

// The launcher for several GPUs: one call, host matrices in, C back; rows cut among the GPUs of
// the communicator.  {0, 0} runs a two-GPU partition on one device; {0, 1} needs a second GPU and
// is skipped without one.  Integer data: bit-exact against the oracle.
static void multi_gpu_checks() {
    const size_t m = 1000, n = 264, k = 136;
    Lcg g;
    std::vector<uint16_t> a(m * k), b(n * k);
    for (auto &x : a) x = f32_to_bf16_bits(float(int(g.next() % 17) - 8));
    for (auto &x : b) x = f32_to_bf16_bits(float(int(g.next() % 17) - 8));
    std::vector<float> sim(m * n);
    oracle_gemm_tn(1, 2, m, n, k, a.data(), b.data(), sim.data(), 1.0f, 0.0f, 0, m);
    cute_b200_gemm_desc d = {};
    d.m = int(m), d.n = int(n), d.k = int(k), d.ab_dtype = CUTE_B200_BF16, d.c_dtype = CUTE_B200_F32, d.alpha = 1.0f;
    const KernelArg ka = KernelArg::Bytes(DType::BF16, a.data(), a.size() * 2), kb = KernelArg::Bytes(DType::BF16, b.data(), b.size() * 2);
    for (const std::vector<int> &devices : {std::vector<int>{0, 0}, std::vector<int>{0, 1}, std::vector<int>{0, 0, 0}}) {
        try {
            MultiGpuContext ctx(devices);
            KernelArg kc = KernelArg::f32(std::vector<float>(m * n, -1.0f));
            const LaunchStats stats = ctx.gemm(d, ka, kb, kc);
            EXPECT(stats.kernel_seconds > 0.0);
            EXPECT(std::memcmp(kc.bytes.data(), sim.data(), sim.size() * 4) == 0);
            // device buffers, C replicated by the kernel's own stores: both copies hold every row
            CudaContext first(devices[0]);
            std::vector<DeviceBuffer> keep;
            std::vector<uint64_t> pa, pb, pc;
            for (size_t i = 0; i < devices.size(); i++) {
                CudaContext here(devices[i]);
                const size_t tiles = (m + 127) / 128, base = tiles / devices.size(), extra = tiles % devices.size();
                const size_t t0 = i * base + (i < extra ? i : extra), t1 = t0 + base + (i < extra ? 1 : 0);
                const size_t lo = std::min(t0 * 128, m), hi = std::min(t1 * 128, m);
                keep.push_back(here.upload(KernelArg::Bytes(DType::BF16, a.data() + lo * k, std::max<size_t>(hi - lo, 1) * k * 2)));
                pa.push_back(keep.back().ptr());
                keep.push_back(here.upload(kb));
                pb.push_back(keep.back().ptr());
                keep.push_back(here.upload(KernelArg::f32(std::vector<float>(m * n, 0.0f))));
                pc.push_back(keep.back().ptr());
            }
            ctx.gemm_on_devices(d, pa, pb, pc, CUTE_B200_REPLICATE_AUTO);
            for (size_t i = 0; i < devices.size(); i++) {
                CudaContext here(devices[i]);
                KernelArg back = KernelArg::f32(std::vector<float>(m * n, -1.0f));
                here.download(keep[3 * i + 2], back);
                EXPECT(std::memcmp(back.bytes.data(), sim.data(), sim.size() * 4) == 0);
            }
        } catch (const CudaError &e) {
            if (e.status == CUTE_B200_ERR_NO_DEVICE && devices.size() == 2 && devices[1] == 1) {
                std::printf("skipped {0, 1}: %s\n", e.message.c_str());
                continue;
            }
            throw;
        }
    }
    EXPECT(error_of([] { MultiGpuContext none(std::vector<int>{}); }) == "comm_create: 1 to 8 GPUs, got 0");
}

int main(int argc, char **argv) {
    const std::string mode = argc > 1 ? argv[1] : "cpu";
    try {
        cpu_checks();
        if (mode == "gpu") {
            gpu_checks();
            multi_gpu_checks();
        }
    } catch (const std::exception &e) {
        std::printf("FAIL: exception: %s\n", e.what());
        return 2;
    }
    if (failures) std::printf("%d check(s) failed\n", failures);
    else std::printf("all checks passed (%s)\n", mode.c_str());
    return failures ? 1 : 0;
}
