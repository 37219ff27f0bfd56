// The launcher for several GPUs of one box, behind the C ABI: one process, one
// host thread and one set of streams per GPU, peer access enabled between every
// pair.  A large GEMM is cut into contiguous blocks of whole 128-row tiles of A
// and C, one per GPU, with B whole in every GPU's memory; nothing crosses
// between GPUs while the blocks are computed.  A caller that asks for a
// replicated C gets it from the GEMM kernel itself (its pusher warp stores every
// finished tile into the peers' C over NVLink) whenever the result qualifies,
// else from an all-gather by the collective library (NCCL, loaded at run time
// like the reference loads libcuda, src/cuda.rs:88-196) or, without it, from
// device-to-device copies.  Peer memory is only ever the target of plain
// stores and copies; no load reads it.
//
// The reference has one GPU and one entry, CudaContext::launch (src/cuda.rs:
// 443-473): buffers in, a wait, buffers back.  cute_b200_gemm_tn_sharded keeps
// that shape for device buffers, cute_b200_gemm_tn_sharded_host for host
// buffers (every GPU uploads its rows of A and only its share of B, the shares
// are exchanged over NVLink, and every GPU sends its rows of C back).
#include <dlfcn.h>

#include <chrono>
#include <condition_variable>
#include <cstring>
#include <mutex>
#include <thread>
#include <vector>

#include "common.cuh"

namespace cb {
namespace {

constexpr uint32_t kCommMagic = 0xC0B200C0u;
constexpr int kMaxGpus = 8;
constexpr int kMaxPanels = 16;
constexpr int kMaxBlocks = 8;  // column blocks of C in the host-buffer call (B goes up block by block)

// The few entry points of the collective library that the fallback needs, resolved at run time.
struct Nccl {
    void *handle = nullptr;
    int (*CommInitAll)(void **, int, const int *) = nullptr;
    int (*CommDestroy)(void *) = nullptr;
    int (*AllGather)(const void *, void *, size_t, int, void *, cudaStream_t) = nullptr;
    int (*Broadcast)(const void *, void *, size_t, int, int, void *, cudaStream_t) = nullptr;
    int (*GroupStart)() = nullptr;
    int (*GroupEnd)() = nullptr;
    const char *(*GetErrorString)(int) = nullptr;
    bool load() {
        if (handle) return true;
        for (const char *name : {"libnccl.so.2", "libnccl.so"}) {
            handle = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
            if (handle) break;
        }
        if (!handle) return false;
        CommInitAll = reinterpret_cast<decltype(CommInitAll)>(dlsym(handle, "ncclCommInitAll"));
        CommDestroy = reinterpret_cast<decltype(CommDestroy)>(dlsym(handle, "ncclCommDestroy"));
        AllGather = reinterpret_cast<decltype(AllGather)>(dlsym(handle, "ncclAllGather"));
        Broadcast = reinterpret_cast<decltype(Broadcast)>(dlsym(handle, "ncclBroadcast"));
        GroupStart = reinterpret_cast<decltype(GroupStart)>(dlsym(handle, "ncclGroupStart"));
        GroupEnd = reinterpret_cast<decltype(GroupEnd)>(dlsym(handle, "ncclGroupEnd"));
        GetErrorString = reinterpret_cast<decltype(GetErrorString)>(dlsym(handle, "ncclGetErrorString"));
        return CommInitAll && CommDestroy && AllGather && Broadcast && GroupStart && GroupEnd && GetErrorString;
    }
};
constexpr int kNcclInt8 = 0;  // ncclInt8: the blocks travel as bytes, whatever C's type

// Rendezvous of the per-GPU host threads of one call.  Every thread passes whether it is still
// healthy; all of them learn whether everybody is, so that none waits for a thread that gave up.
class HostBarrier {
public:
    void reset(int n) {
        count_ = n, waiting_ = 0, generation_ = 0, all_ok_ = true, result_ = true;
    }
    bool arrive(bool ok) {
        std::unique_lock<std::mutex> lock(mu_);
        all_ok_ = all_ok_ && ok;
        const uint64_t gen = generation_;
        if (++waiting_ == count_) {
            result_ = all_ok_;
            waiting_ = 0;
            generation_++;
            cv_.notify_all();
            return result_;
        }
        cv_.wait(lock, [&] { return generation_ != gen; });
        return result_;
    }

private:
    std::mutex mu_;
    std::condition_variable cv_;
    int count_ = 0, waiting_ = 0;
    uint64_t generation_ = 0;
    bool all_ok_ = true, result_ = true;
};

struct GpuState {
    int ordinal = 0;
    cudaStream_t compute = nullptr, up = nullptr, down = nullptr, spread[2] = {nullptr, nullptr};
    cudaEvent_t b_up[kMaxBlocks] = {}, spread_join[kMaxBlocks] = {}, b_spread[kMaxBlocks] = {}, a_up[kMaxPanels] = {}, c_done = nullptr;
    void *buf[3] = {nullptr, nullptr, nullptr};  // staging of the host-buffer call: A rows, B, C rows
    size_t bytes[3] = {0, 0, 0};
};

struct Comm {
    uint32_t magic = kCommMagic;
    int n = 0;
    bool distinct = true;   // no ordinal twice
    bool peers_ok = true;   // every pair of different devices can reach each other's memory
    GpuState gpu[kMaxGpus];
    Nccl nccl;
    bool nccl_tried = false, nccl_ok = false;
    void *nccl_comm[kMaxGpus] = {};
    HostBarrier barrier;
    std::mutex call_mu;  // one call at a time per communicator
};

Comm *as_comm(void *p) {
    Comm *c = static_cast<Comm *>(p);
    return (c && c->magic == kCommMagic) ? c : nullptr;
}

struct Outcome {
    cute_b200_status status = CUTE_B200_OK;
    std::string message;
};

// Runs fn(g) on one host thread per GPU, that GPU current, and returns the first failure
// (with its message moved into the caller's thread).
template <class F>
cute_b200_status on_every_gpu(Comm &comm, F &&fn) {
    std::vector<Outcome> out(comm.n);
    std::vector<std::thread> threads;
    comm.barrier.reset(comm.n);
    for (int g = 0; g < comm.n; g++)
        threads.emplace_back([&, g] {
            cudaError_t err = cudaSetDevice(comm.gpu[g].ordinal);
            cute_b200_status st = err == cudaSuccess ? fn(g) : cuda_fail(err, "cudaSetDevice");
            out[g].status = st;
            if (st != CUTE_B200_OK) out[g].message = last_error();
        });
    for (auto &t : threads) t.join();
    for (int g = 0; g < comm.n; g++)
        if (out[g].status != CUTE_B200_OK) return fail(out[g].status, "GPU %d (device %d): %s", g, comm.gpu[g].ordinal, out[g].message.c_str());
    return CUTE_B200_OK;
}

cute_b200_status ensure_nccl(Comm &comm) {
    if (comm.nccl_tried) return comm.nccl_ok ? CUTE_B200_OK : fail(CUTE_B200_ERR_UNSUPPORTED, "the collective library is not available");
    comm.nccl_tried = true;
    if (!comm.distinct) return fail(CUTE_B200_ERR_UNSUPPORTED, "the collective library needs distinct devices");
    if (!comm.nccl.load()) return fail(CUTE_B200_ERR_UNSUPPORTED, "libnccl.so.2 could not be loaded: %s", dlerror() ? dlerror() : "symbols missing");
    int devs[kMaxGpus];
    for (int g = 0; g < comm.n; g++) devs[g] = comm.gpu[g].ordinal;
    const int rc = comm.nccl.CommInitAll(comm.nccl_comm, comm.n, devs);
    if (rc != 0) return fail(CUTE_B200_ERR_CUDA, "ncclCommInitAll failed: %s", comm.nccl.GetErrorString(rc));
    comm.nccl_ok = true;
    return CUTE_B200_OK;
}

cute_b200_status grow(GpuState &gs, int slot, size_t bytes) {
    if (gs.bytes[slot] >= bytes) return CUTE_B200_OK;
    if (gs.buf[slot]) CB_CUDA(cudaFree(gs.buf[slot]));
    gs.buf[slot] = nullptr;
    gs.bytes[slot] = 0;
    CB_CUDA(cudaMalloc(&gs.buf[slot], bytes ? bytes : 16));
    gs.bytes[slot] = bytes;
    return CUTE_B200_OK;
}

size_t c_elem_bytes(const cute_b200_gemm_desc &d) { return d.c_dtype == CUTE_B200_BF16 ? 2 : 4; }

cute_b200_status check_desc(const cute_b200_gemm_desc *desc, const char *who) {
    if (!desc) return fail(CUTE_B200_ERR_NULL_POINTER, "%s: desc is null", who);
    if (desc->m <= 0 || desc->n <= 0 || desc->k < 0)
        return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "%s: invalid size %dx%dx%d", who, desc->m, desc->n, desc->k);
    if ((desc->ab_dtype != CUTE_B200_F16 && desc->ab_dtype != CUTE_B200_BF16) ||
        (desc->c_dtype != CUTE_B200_F32 && desc->c_dtype != CUTE_B200_BF16))
        return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "%s: f16/bf16 inputs and f32/bf16 output only", who);
    return CUTE_B200_OK;
}

}  // namespace

cute_b200_status comm_create(int ngpus, const int *ordinals, void **comm_out) {
    if (!comm_out) return fail(CUTE_B200_ERR_NULL_POINTER, "comm_create: null output");
    *comm_out = nullptr;
    if (ngpus < 1 || ngpus > kMaxGpus)
        return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "comm_create: 1 to %d GPUs, got %d", kMaxGpus, ngpus);
    int count = 0;
    cudaError_t err = cudaGetDeviceCount(&count);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail(CUTE_B200_ERR_NO_DEVICE, "cudaGetDeviceCount failed: %s", cudaGetErrorName(err));
    }
    Comm *comm = new Comm();
    comm->n = ngpus;
    for (int g = 0; g < ngpus; g++) {
        const int ord = ordinals ? ordinals[g] : g;
        if (ord < 0 || ord >= count) {
            delete comm;
            return fail(CUTE_B200_ERR_NO_DEVICE, "comm_create: device %d requested, %d present", ord, count);
        }
        comm->gpu[g].ordinal = ord;
        for (int h = 0; h < g; h++)
            if (comm->gpu[h].ordinal == ord) comm->distinct = false;
    }
    int previous = 0;
    cudaGetDevice(&previous);
    auto setup = [&]() -> cute_b200_status {
        for (int g = 0; g < ngpus; g++) {
            GpuState &gs = comm->gpu[g];
            CB_TRY(cute_b200_init(gs.ordinal));  // selects the device
            for (int h = 0; h < ngpus; h++) {
                const int other = comm->gpu[h].ordinal;
                if (other == gs.ordinal) continue;
                int can = 0;
                CB_CUDA(cudaDeviceCanAccessPeer(&can, gs.ordinal, other));
                if (!can) {
                    comm->peers_ok = false;
                    continue;
                }
                err = cudaDeviceEnablePeerAccess(other, 0);
                if (err == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
                else if (err != cudaSuccess) return cuda_fail(err, "cudaDeviceEnablePeerAccess");
            }
            CB_CUDA(cudaStreamCreateWithFlags(&gs.compute, cudaStreamNonBlocking));
            CB_CUDA(cudaStreamCreateWithFlags(&gs.up, cudaStreamNonBlocking));
            CB_CUDA(cudaStreamCreateWithFlags(&gs.down, cudaStreamNonBlocking));
            for (auto &s : gs.spread) CB_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
            for (int j = 0; j < kMaxBlocks; j++) {
                CB_CUDA(cudaEventCreateWithFlags(&gs.b_up[j], cudaEventDisableTiming));
                CB_CUDA(cudaEventCreateWithFlags(&gs.b_spread[j], cudaEventDisableTiming));
                CB_CUDA(cudaEventCreateWithFlags(&gs.spread_join[j], cudaEventDisableTiming));
            }
            for (int i = 0; i < kMaxPanels; i++) CB_CUDA(cudaEventCreateWithFlags(&gs.a_up[i], cudaEventDisableTiming));
            CB_CUDA(cudaEventCreateWithFlags(&gs.c_done, cudaEventDisableTiming));
        }
        return CUTE_B200_OK;
    };
    const cute_b200_status st = setup();
    cudaSetDevice(previous);
    if (st != CUTE_B200_OK) {
        const std::string msg = last_error();
        comm_destroy(comm);
        return fail(st, "%s", msg.c_str());
    }
    *comm_out = comm;
    return CUTE_B200_OK;
}

cute_b200_status comm_destroy(void *p) {
    if (!p) return CUTE_B200_OK;
    Comm *comm = as_comm(p);
    if (!comm) return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "comm_destroy: not a communicator of this library");
    int previous = 0;
    cudaGetDevice(&previous);
    for (int g = 0; g < comm->n; g++) {
        GpuState &gs = comm->gpu[g];
        if (cudaSetDevice(gs.ordinal) != cudaSuccess) continue;
        cudaDeviceSynchronize();
        if (comm->nccl_ok && comm->nccl_comm[g]) comm->nccl.CommDestroy(comm->nccl_comm[g]);
        for (cudaStream_t s : {gs.compute, gs.up, gs.down, gs.spread[0], gs.spread[1]})
            if (s) cudaStreamDestroy(s);
        for (int j = 0; j < kMaxBlocks; j++)
            for (cudaEvent_t e : {gs.b_up[j], gs.b_spread[j], gs.spread_join[j]})
                if (e) cudaEventDestroy(e);
        for (int i = 0; i < kMaxPanels; i++)
            if (gs.a_up[i]) cudaEventDestroy(gs.a_up[i]);
        if (gs.c_done) cudaEventDestroy(gs.c_done);
        for (void *b : gs.buf)
            if (b) cudaFree(b);
    }
    cudaSetDevice(previous);
    comm->magic = 0;
    delete comm;
    return CUTE_B200_OK;
}

cute_b200_status comm_info(void *p, int32_t out[4]) {
    Comm *comm = as_comm(p);
    if (!comm || !out) return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "comm_info: not a communicator of this library, or null output");
    std::lock_guard<std::mutex> lock(comm->call_mu);
    // "usable" = the library loads and the devices are distinct; its communicators are only made by the first
    // call that needs them (ncclCommInitAll takes seconds and talks to every GPU)
    const bool nccl = comm->nccl_ok || (!comm->nccl_tried && comm->distinct && comm->nccl.load());
    out[0] = comm->n, out[1] = comm->distinct ? 1 : 0, out[2] = comm->peers_ok ? 1 : 0, out[3] = nccl ? 1 : 0;
    return CUTE_B200_OK;
}

cute_b200_status gemm_tn_sharded(void *p, const cute_b200_gemm_desc *desc, const uint64_t *dA_shard, const uint64_t *dB,
                                 const uint64_t *dC, int replicate_c) {
    Comm *comm = as_comm(p);
    if (!comm) return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "gemm_tn_sharded: not a communicator of this library");
    CB_TRY(check_desc(desc, "gemm_tn_sharded"));
    if (!dA_shard || !dB || !dC) return fail(CUTE_B200_ERR_NULL_POINTER, "gemm_tn_sharded: null pointer list");
    if (replicate_c < 0 || replicate_c > CUTE_B200_REPLICATE_COPIES)
        return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "gemm_tn_sharded: replicate_c must be 0 to %d, got %d", CUTE_B200_REPLICATE_COPIES, replicate_c);
    std::lock_guard<std::mutex> lock(comm->call_mu);
    const int n = comm->n;
    const size_t esize = c_elem_bytes(*desc), row_bytes = size_t(desc->n) * esize;
    int begin[kMaxGpus], rows[kMaxGpus];
    bool even = true;
    for (int g = 0; g < n; g++) {
        CB_TRY(cute_b200_shard_rows(desc->m, n, g, &begin[g], &rows[g]));
        if (!dC[g] || (desc->k > 0 && rows[g] > 0 && (!dA_shard[g] || !dB[g])))
            return fail(CUTE_B200_ERR_NULL_POINTER, "gemm_tn_sharded: null buffer for GPU %d", g);
        if (rows[g] != rows[0]) even = false;
    }
    // How the blocks reach the other GPUs.
    int how = replicate_c;
    if (n == 1) how = CUTE_B200_REPLICATE_NONE;
    const bool plain = desc->alpha == 1.0f && desc->beta == 0.0f;
    const bool can_fuse = plain && desc->k > 0 && (comm->peers_ok || !comm->distinct);
    if (how == CUTE_B200_REPLICATE_AUTO) {
        bool tma_ok = row_bytes % 16 == 0;
        for (int g = 0; g < n; g++) tma_ok = tma_ok && (dC[g] & 15u) == 0;
        if (can_fuse && tma_ok) how = CUTE_B200_REPLICATE_FUSED;
        else how = ensure_nccl(*comm) == CUTE_B200_OK ? CUTE_B200_REPLICATE_COLLECTIVE : CUTE_B200_REPLICATE_COPIES;
    }
    if (how == CUTE_B200_REPLICATE_FUSED && !can_fuse)
        return fail(CUTE_B200_ERR_INVALID_ARGUMENT,
                    "gemm_tn_sharded: the fused form needs alpha = 1, beta = 0, k > 0 and peer access between all GPUs");
    if (how == CUTE_B200_REPLICATE_COLLECTIVE) CB_TRY(ensure_nccl(*comm));

    return on_every_gpu(*comm, [&](int g) -> cute_b200_status {
        GpuState &gs = comm->gpu[g];
        DeviceState *dev;
        CB_TRY(current_device(&dev));
        cute_b200_gemm_desc d = *desc;
        d.m = rows[g];
        const uint64_t off = uint64_t(begin[g]) * row_bytes;
        cute_b200_status st = CUTE_B200_OK;
        if (how == CUTE_B200_REPLICATE_NONE) {
            // replicate_c == 0: dC[g] is the block itself; a single GPU asked for a full C holds all of it anyway
            if (rows[g] > 0) st = gemm_tn(d, dA_shard[g], dB[g], dC[g], gs.compute, *dev);
        } else if (how == CUTE_B200_REPLICATE_FUSED) {
            if (rows[g] > 0) {
                uint64_t dests[kMaxGpus];
                dests[0] = dC[g] + off;
                for (int s = 1; s < n; s++) dests[s] = dC[(g + s) % n] + off;  // every link carries one peer's tiles
                d.split_k = 1;
                st = gemm_tn_multi(d, dA_shard[g], dB[g], dests, n, nullptr, gs.compute, *dev);
            }
        } else {
            if (rows[g] > 0) st = gemm_tn(d, dA_shard[g], dB[g], dC[g] + off, gs.compute, *dev);
            if (how == CUTE_B200_REPLICATE_COLLECTIVE) {
                // Every thread has to join the collective, healthy or not, or the others would wait for it.
                const Nccl &nc = comm->nccl;
                int rc = 0;
                if (even) {
                    rc = nc.AllGather(reinterpret_cast<const void *>(dC[g] + off), reinterpret_cast<void *>(dC[g]),
                                      size_t(rows[g]) * row_bytes, kNcclInt8, comm->nccl_comm[g], gs.compute);
                } else {
                    nc.GroupStart();
                    for (int r = 0; r < n && rc == 0; r++)
                        if (rows[r] > 0) {
                            void *blk = reinterpret_cast<void *>(dC[g] + uint64_t(begin[r]) * row_bytes);
                            rc = nc.Broadcast(blk, blk, size_t(rows[r]) * row_bytes, kNcclInt8, r, comm->nccl_comm[g], gs.compute);
                        }
                    const int rc2 = nc.GroupEnd();
                    if (rc == 0) rc = rc2;
                }
                if (rc != 0 && st == CUTE_B200_OK) st = fail(CUTE_B200_ERR_CUDA, "the all-gather failed: %s", nc.GetErrorString(rc));
            } else if (st == CUTE_B200_OK && rows[g] > 0) {
                for (int s = 1; s < n; s++) {
                    const int peer = (g + s) % n;
                    CB_CUDA(cudaMemcpyPeerAsync(reinterpret_cast<void *>(dC[peer] + off), comm->gpu[peer].ordinal,
                                                reinterpret_cast<const void *>(dC[g] + off), gs.ordinal,
                                                size_t(rows[g]) * row_bytes, gs.compute));
                }
            }
        }
        // The call returns when every GPU's kernels, pushes and copies are complete: each thread
        // waits for its device here and the caller joins all threads.
        const cute_b200_status sync = sync_and_check();
        return st != CUTE_B200_OK ? st : sync;
    });
}

cute_b200_status gemm_tn_sharded_host(void *p, const cute_b200_gemm_desc *desc, const void *hA, const void *hB, void *hC,
                                      double *seconds) {
    Comm *comm = as_comm(p);
    if (!comm) return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "gemm_tn_sharded_host: not a communicator of this library");
    CB_TRY(check_desc(desc, "gemm_tn_sharded_host"));
    if (!hC || (desc->k > 0 && (!hA || !hB))) return fail(CUTE_B200_ERR_NULL_POINTER, "gemm_tn_sharded_host: null buffer");
    std::lock_guard<std::mutex> lock(comm->call_mu);
    const auto t_start = std::chrono::steady_clock::now();
    const int n = comm->n;
    const size_t esize = c_elem_bytes(*desc), c_pitch = size_t(desc->n) * esize, k_bytes = size_t(desc->k) * 2;
    const bool reads_c = !(desc->alpha == 1.0f && desc->beta == 0.0f);
    int begin[kMaxGpus], rows[kMaxGpus];
    for (int g = 0; g < n; g++) CB_TRY(cute_b200_shard_rows(desc->m, n, g, &begin[g], &rows[g]));
    // The way down to the host is the slowest leg (every GPU sends m/N x n elements of C back against
    // m/N + n/N rows of k elements that it fetches, and the host takes writes from several GPUs more
    // slowly than it serves their reads), so it should start as early as possible and never wait.  C is
    // cut into blocks of columns and B goes up block by block: of block j every GPU fetches 1/N of the
    // rows of B and passes them to the others over NVLink.  The first block is multiplied panel by panel
    // of A's rows as they arrive, the later ones against all of this GPU's rows at once, and every
    // finished block of C goes down while the uploads and products of the next ones run ahead.
    int blocks = desc->k > 0 ? desc->n / 4096 : 1;
    blocks = blocks < 1 ? 1 : (blocks > kMaxBlocks ? kMaxBlocks : blocks);
    int col0[kMaxBlocks + 1];
    for (int j = 0; j <= blocks; j++) col0[j] = j == blocks ? desc->n : int(int64_t(desc->n) * j / blocks / 256 * 256);
    // rows [piece(j, g), piece(j, g + 1)) of B: what GPU g fetches of block j
    auto piece = [&](int j, int g) { return col0[j] + int(int64_t(col0[j + 1] - col0[j]) * g / n); };
    const cute_b200_status st = on_every_gpu(*comm, [&](int g) -> cute_b200_status {
        GpuState &gs = comm->gpu[g];
        DeviceState *dev = nullptr;
        // phase 1: staging memory, so that every GPU's B exists before anybody copies into it
        cute_b200_status st = current_device(&dev);
        if (st == CUTE_B200_OK) st = grow(gs, 0, size_t(rows[g]) * k_bytes);
        if (st == CUTE_B200_OK) st = grow(gs, 1, size_t(desc->n) * k_bytes);
        if (st == CUTE_B200_OK) st = grow(gs, 2, size_t(rows[g]) * c_pitch);
        if (!comm->barrier.arrive(st == CUTE_B200_OK)) return st != CUTE_B200_OK ? st : fail(CUTE_B200_ERR_CUDA, "another GPU of the call failed");

        char *dA = static_cast<char *>(gs.buf[0]), *dB = static_cast<char *>(gs.buf[1]), *dC = static_cast<char *>(gs.buf[2]);
        int panels = 8;
        while (panels > 1 && (rows[g] / panels < 256 || size_t(rows[g] / panels) * c_pitch < (size_t(4) << 20))) panels /= 2;
        const int per = rows[g] > 0 ? ((rows[g] + panels - 1) / panels + 127) / 128 * 128 : 128;
        panels = (rows[g] + per - 1) / per;
#ifdef CB_TRACE_SHARDED
        cudaEvent_t tr[8];
        for (auto &e : tr) cudaEventCreate(&e);
        const auto host_p2 = std::chrono::steady_clock::now();
        cudaEventRecord(tr[0], gs.up);
#endif
        // phase 2: everything that goes up, in the order in which it unlocks blocks of C: the first
        // panel of A, this GPU's piece of the first block of B, the other panels of A, the other pieces
        // of B.  Every piece of B goes on to every other GPU as soon as it is here.
        auto b_piece = [&](int j) -> cute_b200_status {
            const int r0 = piece(j, g), r1 = piece(j, g + 1);
            if (desc->k > 0 && r1 > r0) {
                const size_t off = size_t(r0) * k_bytes, bytes = size_t(r1 - r0) * k_bytes;
                CB_CUDA(cudaMemcpyAsync(dB + off, static_cast<const char *>(hB) + off, bytes, cudaMemcpyHostToDevice, gs.up));
                CB_CUDA(cudaEventRecord(gs.b_up[j], gs.up));
                for (auto &s : gs.spread) CB_CUDA(cudaStreamWaitEvent(s, gs.b_up[j], 0));
                for (int s = 1; s < n; s++) {  // two streams, so that two copy engines and two links work at a time
                    const int peer = (g + s) % n;
                    CB_CUDA(cudaMemcpyPeerAsync(static_cast<char *>(comm->gpu[peer].buf[1]) + off, comm->gpu[peer].ordinal,
                                                dB + off, gs.ordinal, bytes, gs.spread[s & 1]));
                }
            }
            // b_spread[j]: this GPU's piece of block j is in its own memory and in every peer's
            CB_CUDA(cudaEventRecord(gs.spread_join[j], gs.spread[0]));
            CB_CUDA(cudaStreamWaitEvent(gs.spread[1], gs.spread_join[j], 0));
            CB_CUDA(cudaEventRecord(gs.b_spread[j], gs.spread[1]));
            return CUTE_B200_OK;
        };
        auto a_panel = [&](int i) -> cute_b200_status {
            const int r0 = i * per, r = rows[g] - r0 < per ? rows[g] - r0 : per;
            const size_t grow0 = size_t(begin[g]) + r0;
            if (desc->k > 0)
                CB_CUDA(cudaMemcpyAsync(dA + size_t(r0) * k_bytes, static_cast<const char *>(hA) + grow0 * k_bytes, size_t(r) * k_bytes,
                                        cudaMemcpyHostToDevice, gs.up));
            if (reads_c)  // the old values of these rows of C, all columns
                CB_CUDA(cudaMemcpyAsync(dC + size_t(r0) * c_pitch, static_cast<const char *>(hC) + grow0 * c_pitch, size_t(r) * c_pitch,
                                        cudaMemcpyHostToDevice, gs.up));
            CB_CUDA(cudaEventRecord(gs.a_up[i], gs.up));
            return CUTE_B200_OK;
        };
        auto phase2 = [&]() -> cute_b200_status {
            if (panels > 0) CB_TRY(a_panel(0));
            CB_TRY(b_piece(0));
            for (int i = 1; i < panels; i++) CB_TRY(a_panel(i));
            for (int j = 1; j < blocks; j++) CB_TRY(b_piece(j));
            return CUTE_B200_OK;
        };
        st = phase2();
#ifdef CB_TRACE_SHARDED
        cudaEventRecord(tr[1], gs.up);  // everything is queued for the way up
        cudaEventRecord(tr[2], gs.spread[1]);                // and every piece of B is with every peer
#endif
        if (!comm->barrier.arrive(st == CUTE_B200_OK)) {
            cudaDeviceSynchronize();
            return st != CUTE_B200_OK ? st : fail(CUTE_B200_ERR_CUDA, "another GPU of the call failed");
        }

        // phase 3 (every GPU has recorded its events by now): block (panel i, columns of block 0) as
        // soon as panel i and all pieces of block 0 are here, then block j of all rows as soon as all
        // pieces of block j are; each goes down behind its product.
        auto product = [&](int r0, int r, int j) -> cute_b200_status {
            const int c0 = col0[j], w = col0[j + 1] - c0;
            char *c_at = dC + size_t(r0) * c_pitch + size_t(c0) * esize;
            cute_b200_gemm_desc d = *desc;
            d.m = r, d.n = w;
            if (blocks == 1)  // all columns: a dense C, which may also split k (and takes k = 0)
                CB_TRY(gemm_tn(d, reinterpret_cast<uint64_t>(dA + size_t(r0) * k_bytes), reinterpret_cast<uint64_t>(dB),
                               reinterpret_cast<uint64_t>(c_at), gs.compute, *dev));
            else
                CB_TRY(gemm_tn_strided(d, reinterpret_cast<uint64_t>(dA + size_t(r0) * k_bytes),
                                       reinterpret_cast<uint64_t>(dB + size_t(c0) * k_bytes), reinterpret_cast<uint64_t>(c_at), desc->n,
                                       gs.compute, *dev));
            CB_CUDA(cudaEventRecord(gs.c_done, gs.compute));
            CB_CUDA(cudaStreamWaitEvent(gs.down, gs.c_done, 0));
            char *h_at = static_cast<char *>(hC) + (size_t(begin[g]) + r0) * c_pitch + size_t(c0) * esize;
            if (blocks == 1)
                CB_CUDA(cudaMemcpyAsync(h_at, c_at, size_t(r) * c_pitch, cudaMemcpyDeviceToHost, gs.down));
            else
                CB_CUDA(cudaMemcpy2DAsync(h_at, c_pitch, c_at, c_pitch, size_t(w) * esize, size_t(r), cudaMemcpyDeviceToHost, gs.down));
            return CUTE_B200_OK;
        };
        auto phase3 = [&]() -> cute_b200_status {
            if (rows[g] == 0) return CUTE_B200_OK;
            for (int j = 0; j < blocks; j++) {
                for (int peer = 0; peer < n; peer++) CB_CUDA(cudaStreamWaitEvent(gs.compute, comm->gpu[peer].b_spread[j], 0));
                if (j > 0) {
                    CB_TRY(product(0, rows[g], j));
                    continue;
                }
                for (int i = 0; i < panels; i++) {
                    CB_CUDA(cudaStreamWaitEvent(gs.compute, gs.a_up[i], 0));
                    CB_TRY(product(i * per, rows[g] - i * per < per ? rows[g] - i * per : per, 0));
#ifdef CB_TRACE_SHARDED
                    if (i == 0) cudaEventRecord(tr[3], gs.compute), cudaEventRecord(tr[4], gs.down);  // first product done, first way down begins
#endif
                }
            }
            return CUTE_B200_OK;
        };
        st = phase3();
#ifdef CB_TRACE_SHARDED
        cudaEventRecord(tr[5], gs.up);
        cudaEventRecord(tr[6], gs.compute);
        cudaEventRecord(tr[7], gs.down);
#endif
        const cute_b200_status sync = sync_and_check();  // everything queued reads or writes the caller's buffers
#ifdef CB_TRACE_SHARDED
        {
            float ms[8] = {};
            for (int i = 1; i < 8; i++) cudaEventElapsedTime(&ms[i], tr[0], tr[i]);
            const double h0 = std::chrono::duration<double, std::milli>(host_p2 - t_start).count();
            const double h1 = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t_start).count();
            fprintf(stderr, "trace gpu %d: host->phase2 %.2f | all up %.2f spread %.2f gemm0 %.2f d2h0-start %.2f up-end %.2f gemm-all %.2f d2h-all %.2f | host end %.2f ms\n",
                    g, h0, ms[1], ms[2], ms[3], ms[4], ms[5], ms[6], ms[7], h1);
            for (auto &e : tr) cudaEventDestroy(e);
        }
#endif
        // nobody's B may be overwritten by the next call while a slower GPU still multiplies: leave together
        comm->barrier.arrive(true);
        return st != CUTE_B200_OK ? st : sync;
    });
    if (seconds) *seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - t_start).count();
    return st;
}

}  // namespace cb
