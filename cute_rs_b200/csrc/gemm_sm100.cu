// Tensor-core GEMM for sm_100a: C = alpha * A * B^T + beta * C with A (m, k)
// and B (n, k) both K-major f16/bf16, f32 accumulation, C (m, n) row-major in
// f32 or bf16.  Takes the place of the kernels the reference generates for
// tensorop_gemm (examples/tensorop_gemm.rs:51-164) and runtime_gemm
// (examples/runtime_gemm.rs:22-105), which are mma.sync.m16n8k16 kernels with
// a cp.async ring; nothing of their structure is kept.
//
// Structure (one persistent CTA, or CTA pair, per SM):
//   warp 0   TMA producer: cp.async.bulk.tensor.2d loads of a (128 MH x 64) A
//            block and a (BN/pair x 64) B block per stage into 128-byte
//            swizzled shared memory, completion counted on the stage's `full`
//            mbarrier.
//   warp 1   MMA issuer: one thread issues tcgen05.mma (M = 128 per CTA,
//            N = BN, K = 16, four per stage) into a TMEM accumulator and
//            releases the stage with tcgen05.commit on its `empty` mbarrier.
//            Also owns the TMEM allocation.
//   warps 2-9  epilogue: tcgen05.ld of the finished accumulator (each warp
//            its own 32 TMEM lanes and every other 32-column chunk),
//            alpha/beta, conversion, global stores.
//   warp 10  pusher, only in the several-destination form (gemm_tn_multi): one
//            thread copies every finished tile from C, still in L2, into the
//            further copies of C (other GPUs' memory over NVLink) with a TMA
//            load and one bulk tensor store per copy, behind the epilogue and
//            beside the main loop of the following tiles.
// Each CTA keeps one (MH = 1) or two (MH = 2) 128-row accumulators of BN f32
// columns in TMEM.  When two sets fit in the 512 columns they are double
// buffered and the epilogue of tile i overlaps the main loop of tile i+1; the
// largest tile (256 rows x 256 columns per CTA) fills TMEM on its own, and the
// next tile's MMAs restart half by half as the epilogue drains each half.
//
// With CTA_GROUP == 2 two CTAs of a cluster work on one tile of 256 MH rows:
// each loads its own rows of A and its own half of the B rows, the leader CTA
// issues tcgen05.mma.cta_group::2 reading both shared memories, and each CTA
// ends up with its rows of the result in its own TMEM.  That halves the
// B traffic per output.  Every CTA issues its own loads; none is shared.
//
// A long k with few tiles can be cut into ranges (work units): their f32 partial
// sums are added by a second kernel through planes in global memory, or - for
// single-CTA 128-row tiles cut in two or four - inside this kernel by the CTAs
// of a cluster through each other's shared memory (GemmParams::kc).  Every
// launch is a programmatic dependent of the kernel before it in the stream:
// the set-up overlaps that kernel's tail, griddepcontrol.wait guards the
// first global access.
//
// Every mbarrier wait has a time limit.  A waiter that gives up raises the
// CTA's abort flag, writes a report to the device status word and all roles
// fall through to the common teardown, so a protocol error ends the kernel
// with an error code instead of hanging the GPU.
#include <cuda.h>
#include <cuda_bf16.h>

#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"
#include "ptx_sm100.cuh"

namespace cb {
namespace {

constexpr int BM = 128;        // rows of C per CTA = TMEM lanes
constexpr int BK = 64;         // k per stage: 64 x 2 B = one 128-byte swizzle row
constexpr int UMMA_K = 16;     // k per tcgen05.mma for 16-bit inputs
constexpr uint32_t RING_BYTES = 192 * 1024;
constexpr uint32_t PUSH_BUF_BYTES = 16 * 1024;  // one chunk of a finished tile on its way to the other GPUs
constexpr uint32_t STAGING_BYTES = 2 * PUSH_BUF_BYTES;
constexpr uint32_t BAR_BYTES = 512;
constexpr int MAX_STAGES = 12;
constexpr uint32_t DESC_K_STEP = (UMMA_K * 2) >> 4;  // one MMA's k (16 elements = 32 bytes) in units of the descriptor's address field
// Rows of one pusher chunk: whole tile rows of bn columns filling one staging buffer.
__host__ __device__ constexpr int push_rows(int bn, bool c_bf16) { return int(PUSH_BUF_BYTES) / (bn * (c_bf16 ? 2 : 4)); }
constexpr uint64_t WAIT_LIMIT_NS = 4ull * 1000 * 1000 * 1000;

// Report codes written to the status word.
enum : uint32_t {
    WHERE_PRODUCER = 1,
    WHERE_MMA_FULL = 2,
    WHERE_MMA_TMEM = 3,
    WHERE_EPILOGUE = 4,
    WHERE_DRAIN = 5,
    WHERE_PUSHER = 6,
    WHERE_SIGNAL = 7  // cute_b200_wait_signal: the counter did not reach the expected value in time
};

#ifndef CB_FAST_DRAIN
#define CB_FAST_DRAIN 1  // 0 builds the epilogue without the read-everything-then-store path (measurements)
#endif
#ifndef EPI_GROUPS_BIG
#define EPI_GROUPS_BIG 2  // measured: four groups (16 warps) are no faster than two on 8192^3 (0.699 vs 0.695 ms)
#endif
// warp 0 TMA, warp 1 MMA + TMEM, then EG groups of four epilogue warps, then the warp that pushes
// finished tiles to other GPUs (idle unless the launch has several destinations).
__host__ __device__ constexpr int epilogue_groups(int bn, int mh) { return (bn == 256 && mh == 2) ? EPI_GROUPS_BIG : 2; }
__host__ __device__ constexpr int num_threads(int bn, int mh) { return 64 + 128 * epilogue_groups(bn, mh) + 32; }

// CTA_GROUP: CTAs per MMA (1, or 2 = a cluster pair).  BN: columns of C per
// tile (the MMA's N).  MH: 128-row accumulators per CTA (1 or 2); with MH == 2
// a CTA owns 256 rows of C, reuses every B block for two MMAs and so moves a
// quarter less operand data per flop, at the price of a single-buffered
// accumulator when BN == 256 (2 x 256 columns fill the 512 columns of TMEM).
// MH == 0 is the 64-rows-per-CTA tile of a pair: one cta_group::2 MMA of
// M = 128 whose accumulator keeps all 128 TMEM lanes busy with 64 rows - lanes
// 0-63 hold columns [0, BN/2) of the CTA's rows, lanes 64-127 columns
// [BN/2, BN) - in BN/2 TMEM columns.  Its stages are small (16 KiB at BN = 128),
// so the ring is deep: the tile for problems with few row tiles and a long k,
// which are bound by how fast A streams in from HBM.
template <int CTA_GROUP, int BN, int MH>
struct Cfg {
    static constexpr bool HALF = MH == 0;
    static_assert(!HALF || CTA_GROUP == 2, "the 64-row tile is a pair tile");
    static constexpr int HALVES = HALF ? 1 : MH;                  // 128-lane accumulators per CTA
    static constexpr int A_ROWS = HALF ? 64 : BM * MH;           // A rows this CTA loads per stage
    static constexpr int B_ROWS = BN / CTA_GROUP;                 // B rows this CTA loads per stage
    static constexpr int UMMA_M = (HALF ? 64 : BM) * CTA_GROUP;   // rows of one MMA over the whole group
    static constexpr uint32_t A_BYTES = A_ROWS * BK * 2;
    static constexpr uint32_t B_BYTES = B_ROWS * BK * 2;
    static constexpr uint32_t KB_BYTES = A_BYTES + B_BYTES;  // one k block (64 of k) of both operands
    // k blocks per ring stage.  The thread that issues the MMAs pays a fixed price per stage (a wait on
    // the stage's barrier, a fence, the commits that free it: about 175 clocks during which the tensor
    // core runs dry, measured with one thread issuing M 128 x N 128 MMAs), so a stage has to hold
    // enough MMA time to make that small: tiles whose k block is short on math (128 columns, or 64
    // rows) put several k blocks behind one barrier.  The ring holds the same bytes either way.
    static constexpr int KPS = HALF ? (BN == 128 ? 4 : 2) : ((MH == 1 && BN == 128) ? 2 : 1);
    static constexpr uint32_t STAGE_BYTES = KPS * KB_BYTES;
    static constexpr int STAGES = (RING_BYTES / STAGE_BYTES) > MAX_STAGES ? MAX_STAGES : int(RING_BYTES / STAGE_BYTES);
    static constexpr int HALF_COLS = HALF ? BN / 2 : BN;             // TMEM columns of one 128-lane accumulator
    static constexpr int ACC_COLS = HALVES * HALF_COLS;              // TMEM columns of one accumulator set
    static constexpr int ACC_BUFS = (2 * ACC_COLS <= 512) ? 2 : 1;  // double buffered when it fits
    static constexpr uint32_t TMEM_COLS = (ACC_COLS * ACC_BUFS <= 128) ? 128 : ((ACC_COLS * ACC_BUFS <= 256) ? 256 : 512);
    static constexpr uint32_t SMEM_BYTES = STAGES * STAGE_BYTES + STAGING_BYTES + 1024 + BAR_BYTES;
    // Arrival counts of the mbarriers: the producer's arrive.expect_tx fills a stage, one tcgen05.commit
    // frees it and one publishes an accumulator, every epilogue warp of the group hands a half back.
    static constexpr uint32_t FULL_ARRIVALS = 1, EMPTY_ARRIVALS = 1, TFULL_ARRIVALS = 1;
    static constexpr uint32_t TEMPTY_ARRIVALS = 4 * epilogue_groups(BN, MH) * CTA_GROUP;
    static constexpr uint32_t EXPECT_TX_PER_KB = CTA_GROUP * KB_BYTES;  // bytes the (leader's) full barrier counts per k block of a stage
    // Row pitch of a CTA's partial sums in shared memory when a cluster adds its k ranges (GemmParams::kc):
    // 16 bytes more than a row of BN floats, so that the 32 lanes' 16-byte stores of a column group spread over the banks.
    static constexpr uint32_t KC_PITCH = BN * 4 + 16;
    static_assert(uint32_t(BM) * KC_PITCH <= STAGES * STAGE_BYTES, "the partial sums reuse the ring");
    static_assert(STAGES >= 2 && STAGES <= MAX_STAGES, "ring depth");
    static_assert(ACC_COLS * ACC_BUFS <= 512, "accumulators exceed TMEM");
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory");
};

// Instruction descriptor of tcgen05.mma.kind::f16: f32 accumulator (bit 4), A and B format (0 = f16,
// 1 = bf16) at bits 7 and 10, both operands K-major (bits 15, 16 clear), N >> 3 at bit 17, M >> 4 at
// bit 24, M counting the rows of the whole CTA group.
__host__ __device__ constexpr uint32_t make_idesc(bool bf16, int umma_m, int bn) {
    return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | (uint32_t(bn >> 3) << 17) |
           (uint32_t(umma_m >> 4) << 24);
}

struct GemmParams {
    void *C;
    int M, N, K, ldc;
    float alpha, beta;
    uint32_t idesc;
    int m_tiles, n_tiles, group_m;
    int c_vec_ok;  // C base and row pitch allow 16-byte (1) or 32-byte (2) accesses
    int debug;     // measurements and tests only: bit 0 skips the TMA loads, bit 1 the stores, bit 2 makes the
                   // producer issue nothing at all (every consumer wait then runs out), bit 3 shortens the limit
    int splits;              // k is cut into this many ranges, one work unit each (1 = no split)
    size_t split_stride;     // bytes between the partial-sum planes of consecutive ranges
    // kc > 1 (single-CTA 128-row tiles only): the `splits` = kc ranges of a tile are computed by the kc CTAs
    // of one cluster, which then add their partial sums through each other's shared memory and write C
    // themselves - no planes in global memory, no second kernel.  One unit per CTA: the grid is tiles x kc.
    int kc;
    uint32_t *status;
    // Further copies of C that receive the same result (other GPUs' C over NVLink peer mappings).
    // Plain epilogue, no k split.  push = 1: the pusher warp copies every finished tile from C to
    // each of them by TMA (load from C, which is still in L2, then one bulk tensor store per copy);
    // push = 0: the epilogue warps store every chunk to each of them from registers as well.
    int extra_count;
    void *extra_c[7];
    int push;
    // Completion signal of the several-destination form: when every CTA of the launch has finished
    // (all stores and pushes to every destination complete), the last one adds 1 to each of these
    // counters, which live in the memory of the GPUs that own the destinations (release, system scope).
    // `done_counter` is this GPU's count of finished CTAs; the last CTA sets it back to zero.
    int signal_count;
    uint32_t *signal[7];
    uint32_t *done_counter;
};

// Tensor maps of C ([0]) and of its further copies, for the pusher warp: boxes of BN columns by
// PUSH_BUF_BYTES / (BN * element size) rows, not swizzled.
struct CMaps {
    CUtensorMap m[8];
};

// Shared-memory matrix descriptor of a K-major tile stored as 128-byte rows
// with the 128B swizzle (what TMA writes with CU_TENSOR_MAP_SWIZZLE_128B):
// start address >> 4, leading byte offset 1 (unused by swizzled K-major),
// stride byte offset 1024 (eight rows), descriptor version 1, layout 2.
__host__ __device__ __forceinline__ constexpr uint64_t sw128_desc(uint32_t saddr) {
    return uint64_t((saddr & 0x3FFFFu) >> 4) | (uint64_t(1) << 16) | (uint64_t(1024 >> 4) << 32) |
           (uint64_t(1) << 46) | (uint64_t(2) << 61);
}

__device__ __noinline__ void report_timeout(uint32_t *status, uint32_t where, uint32_t detail, uint32_t parity) {
    if (atomicCAS(status, 0u, where) == 0u) {
        status[1] = detail;
        status[2] = blockIdx.x;
        status[3] = parity;
        __threadfence();
    }
}

// Wait for phase `parity` of `bar`.  false = gave up (limit or CTA abort).
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag,
                                         uint32_t *status, uint32_t where, uint32_t detail,
                                         uint64_t limit_ns = WAIT_LIMIT_NS) {
    if (ptx::mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = ptx::globaltimer_ns();
    uint32_t spins = 0;
    for (;;) {
        if (ptx::mbar_try_wait(bar, parity)) return true;
        if ((++spins & 255u) == 0u) {
            if (*abort_flag) return false;
            if (ptx::globaltimer_ns() - t0 > limit_ns) {
                *abort_flag = 1u;
                report_timeout(status, where, detail, parity);
                return false;
            }
        }
    }
}

struct TileCoord {
    int tm, tn;
};
// Tiles are numbered so that `group_m` row tiles are walked before the column
// advances: the CTAs running at one time then share a compact set of A and B
// panels in L2.
__device__ __forceinline__ TileCoord tile_coord(int t, const GemmParams &p) {
    const int group_size = p.group_m * p.n_tiles;
    const int g = t / group_size;
    const int first = g * p.group_m;
    const int gm = min(p.group_m, p.m_tiles - first);
    const int r = t - g * group_size;
    return {first + r % gm, r / gm};
}

// A work unit is one k range of one tile: unit u = tile * splits + range.
struct Unit {
    int tile, range, kb0, kb1;
};
__device__ __forceinline__ Unit unit_of(int u, const GemmParams &p, int k_blocks) {
    const int range = u % p.splits, per = (k_blocks + p.splits - 1) / p.splits;
    const int kb0 = min(range * per, k_blocks);
    return {u / p.splits, range, kb0, min(kb0 + per, k_blocks)};
}

template <bool C_BF16>
__device__ __forceinline__ void store_chunk(const GemmParams &p, void *cbase, int row, int col0,
                                            const uint32_t (&v)[32], bool plain) {
    if (row >= p.M || col0 >= p.N) return;
    const float alpha = p.alpha, beta = p.beta;
    auto epi = [&](uint32_t acc_bits, float c_old) {
        return __fadd_rn(__fmul_rn(alpha, __uint_as_float(acc_bits)), __fmul_rn(beta, c_old));
    };
    if constexpr (!C_BF16) {
        float *crow = reinterpret_cast<float *>(cbase) + size_t(row) * p.ldc + col0;
        if (p.c_vec_ok == 2 && plain && col0 + 32 <= p.N) {
#pragma unroll
            for (int g = 0; g < 4; g++)
                ptx::st_global_v8(crow + 8 * g, v[8 * g], v[8 * g + 1], v[8 * g + 2], v[8 * g + 3], v[8 * g + 4],
                                  v[8 * g + 5], v[8 * g + 6], v[8 * g + 7]);
        } else if (p.c_vec_ok && col0 + 32 <= p.N) {
#pragma unroll
            for (int g = 0; g < 8; g++) {
                float4 o;
                if (plain) {
                    o = make_float4(__uint_as_float(v[4 * g]), __uint_as_float(v[4 * g + 1]),
                                    __uint_as_float(v[4 * g + 2]), __uint_as_float(v[4 * g + 3]));
                } else {
                    const float4 c = *reinterpret_cast<const float4 *>(crow + 4 * g);
                    o = make_float4(epi(v[4 * g], c.x), epi(v[4 * g + 1], c.y), epi(v[4 * g + 2], c.z),
                                    epi(v[4 * g + 3], c.w));
                }
                *reinterpret_cast<float4 *>(crow + 4 * g) = o;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; j++)
                if (col0 + j < p.N) crow[j] = plain ? __uint_as_float(v[j]) : epi(v[j], crow[j]);
        }
    } else {
        __nv_bfloat16 *crow = reinterpret_cast<__nv_bfloat16 *>(cbase) + size_t(row) * p.ldc + col0;
        if (p.c_vec_ok == 2 && plain && col0 + 32 <= p.N) {
            uint32_t w[16];
#pragma unroll
            for (int j = 0; j < 16; j++) {
                const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
                w[j] = *reinterpret_cast<const uint32_t *>(&h);
            }
            ptx::st_global_v8(crow, w[0], w[1], w[2], w[3], w[4], w[5], w[6], w[7]);
            ptx::st_global_v8(crow + 16, w[8], w[9], w[10], w[11], w[12], w[13], w[14], w[15]);
        } else if (p.c_vec_ok && col0 + 32 <= p.N) {
#pragma unroll
            for (int g = 0; g < 4; g++) {
                float f[8];
                if (plain) {
#pragma unroll
                    for (int j = 0; j < 8; j++) f[j] = __uint_as_float(v[8 * g + j]);
                } else {
                    const uint4 c = *reinterpret_cast<const uint4 *>(crow + 8 * g);
                    const uint32_t cw[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        f[2 * j] = epi(v[8 * g + 2 * j], __uint_as_float(cw[j] << 16));
                        f[2 * j + 1] = epi(v[8 * g + 2 * j + 1], __uint_as_float(cw[j] & 0xffff0000u));
                    }
                }
                uint32_t w[4];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
                    w[j] = *reinterpret_cast<const uint32_t *>(&h);
                }
                *reinterpret_cast<uint4 *>(crow + 8 * g) = make_uint4(w[0], w[1], w[2], w[3]);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; j++)
                if (col0 + j < p.N) {
                    const float r = plain ? __uint_as_float(v[j]) : epi(v[j], __bfloat162float(crow[j]));
                    crow[j] = __float2bfloat16_rn(r);
                }
        }
    }
}

template <int CTA_GROUP, int BN, int MH, bool C_BF16>
__global__ void __launch_bounds__(num_threads(BN, MH), 1)
    gemm_tn_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                   const __grid_constant__ CMaps tmC, const GemmParams p) {
    using C = Cfg<CTA_GROUP, BN, MH>;
    constexpr int EG = epilogue_groups(BN, MH);
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = ptx::smem_u32(smem_raw);
    const uint32_t ring = (raw + 1023u) & ~1023u;  // swizzle atoms need 1024-byte alignment
    const uint32_t staging = ring + C::STAGES * C::STAGE_BYTES;  // 1024-byte aligned: stages are multiples of 1 KiB
    const uint32_t bars = staging + STAGING_BYTES;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (C::STAGES + s); };
    auto tfull_bar = [&](int buf) { return bars + 8u * (2 * C::STAGES + buf); };
    auto tempty_bar = [&](int buf, int h) { return bars + 8u * (2 * C::STAGES + 2 + buf * 2 + h); };
    const uint32_t drain_bar = bars + 8u * (2 * C::STAGES + 6);
    auto push_bar = [&](int b) { return bars + 8u * (2 * C::STAGES + 7 + b); };
    uint8_t *tail = smem_raw + (bars - raw) + 8u * (2 * C::STAGES + 9);
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(tail);
    volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(tail + 4);
    // tiles_stored[w]: how many tiles epilogue warp w has stored to C.  One slot per warp, not one shared
    // count: a warp may run a tile or two ahead of another, and a sum could not tell whose parts are in.
    volatile uint32_t *tiles_stored = reinterpret_cast<volatile uint32_t *>(tail + 8);
    static_assert(8u * (2 * C::STAGES + 9) + 8u + 4u * 4 * EG <= BAR_BYTES, "barrier area");
    constexpr int HALVES = C::HALVES;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = CTA_GROUP == 1 ? 0u : ptx::cluster_ctarank();
    bool kc_mode = false;
    if constexpr (CTA_GROUP == 1 && MH == 1) kc_mode = p.kc > 1;
    const uint32_t kc_rank = kc_mode ? ptx::cluster_ctarank() : 0u;
    const int cluster_id = kc_mode ? int(blockIdx.x) / p.kc : int(blockIdx.x) / CTA_GROUP;
    const int num_clusters = kc_mode ? int(gridDim.x) / p.kc : int(gridDim.x) / CTA_GROUP;
    const int num_units = p.m_tiles * p.n_tiles * p.splits;
    // Units of this CTA: first, first + step, ...  (With kc the cluster's CTAs take the kc ranges of one tile.)
    const int unit_first = kc_mode ? cluster_id * p.kc + int(kc_rank) : cluster_id;
    const int unit_step = kc_mode ? num_clusters * p.kc : num_clusters;
    const int k_blocks = (p.K + BK - 1) / BK;
    constexpr int nstages = C::STAGES;
    const uint64_t wait_limit = (p.debug & 8) ? 20ull * 1000 * 1000 : WAIT_LIMIT_NS;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; s++) {
            ptx::mbar_init(full_bar(s), C::FULL_ARRIVALS);
            ptx::mbar_init(empty_bar(s), C::EMPTY_ARRIVALS);
        }
        for (int buf = 0; buf < 2; buf++) {
            ptx::mbar_init(tfull_bar(buf), C::TFULL_ARRIVALS);
            for (int h = 0; h < 2; h++)
                ptx::mbar_init(tempty_bar(buf, h), C::TEMPTY_ARRIVALS);  // one arrival per epilogue warp of the pair
        }
        ptx::mbar_init(drain_bar, 1);
        ptx::mbar_init(push_bar(0), 1);
        ptx::mbar_init(push_bar(1), 1);
        *abort_flag = 0u;
        for (int w = 0; w < 4 * EG; w++) tiles_stored[w] = 0u;
        ptx::fence_mbar_init();
    }
    if (warp == 1) {
        ptx::tmem_alloc<CTA_GROUP>(ptx::smem_u32(const_cast<uint32_t *>(tmem_slot)), C::TMEM_COLS);
        ptx::tmem_relinquish<CTA_GROUP>();
    }
    ptx::tc_fence_before();
    __syncthreads();
    if constexpr (CTA_GROUP == 2) {  // the peer's barriers must exist before anything arrives on them
        ptx::cluster_arrive();
        ptx::cluster_wait();
    }
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Programmatic dependent launch, both ways.  This kernel may have been scheduled while the kernel
    // before it in the stream was still running (only another launch of this library lets that happen):
    // everything so far touched only this CTA's shared memory and TMEM; nothing below may read or write
    // global memory before that kernel has completed.  And whatever is queued behind this kernel as a
    // programmatic dependent (the kernel that adds the planes of a split GEMM, or the next GEMM) may be
    // scheduled from now on; it waits the same way.
    ptx::griddep_wait();
    if (threadIdx.x == 0) ptx::griddep_launch_dependents();

    if (warp == 0) {
        // ------------------------------------------------------------ producer
        if (lane == 0) {
            ptx::prefetch_tensormap(&tmA);
            ptx::prefetch_tensormap(&tmB);
            int s = 0;
            uint32_t ph = 0;
            uint32_t filled = 0, filled_parity = 0;  // per stage: was it filled, and in which phase
            bool ok = true;
            for (int t = unit_first; t < num_units && ok && !(p.debug & 4); t += unit_step) {
                const Unit u = unit_of(t, p, k_blocks);
                const TileCoord tc = tile_coord(u.tile, p);
                const int row_a = (tc.tm * CTA_GROUP + int(rank)) * C::A_ROWS;
                const int row_b = tc.tn * BN + int(rank) * C::B_ROWS;
                const int nkb = u.kb1 - u.kb0;
                for (int i0 = 0; i0 < nkb; i0 += C::KPS) {
                    const int nk = nkb - i0 < C::KPS ? nkb - i0 : C::KPS;  // k blocks of this stage (the last may be short)
                    if (!wait_bar(empty_bar(s), ph ^ 1u, abort_flag, p.status, WHERE_PRODUCER, uint32_t(s), wait_limit)) {
                        ok = false;
                        break;
                    }
                    const uint32_t dst0 = ring + uint32_t(s) * C::STAGE_BYTES;
                    const int k0 = (u.kb0 + i0) * BK;
                    if (p.debug & 1) {
                        if (rank == 0) ptx::mbar_arrive(full_bar(s));
                    } else if constexpr (CTA_GROUP == 1) {
                        ptx::mbar_arrive_expect_tx(full_bar(s), uint32_t(nk) * C::EXPECT_TX_PER_KB);
#pragma unroll
                        for (int kk = 0; kk < C::KPS; kk++)
                            if (kk < nk) {
                                ptx::tma_load_2d(dst0 + uint32_t(kk) * C::KB_BYTES, &tmA, full_bar(s), k0 + kk * BK, row_a);
                                ptx::tma_load_2d(dst0 + uint32_t(kk) * C::KB_BYTES + C::A_BYTES, &tmB, full_bar(s), k0 + kk * BK, row_b);
                            }
                    } else {
                        // Both CTAs' bytes are counted on the leader's barrier,
                        // which is the one the MMA issuer waits on.
                        if (rank == 0) ptx::mbar_arrive_expect_tx(full_bar(s), uint32_t(nk) * C::EXPECT_TX_PER_KB);
                        const uint32_t leader_full = ptx::mapa(full_bar(s), 0);
#pragma unroll
                        for (int kk = 0; kk < C::KPS; kk++)
                            if (kk < nk) {
                                ptx::tma_load_2d_pair(dst0 + uint32_t(kk) * C::KB_BYTES, &tmA, leader_full, k0 + kk * BK, row_a);
                                ptx::tma_load_2d_pair(dst0 + uint32_t(kk) * C::KB_BYTES + C::A_BYTES, &tmB, leader_full, k0 + kk * BK, row_b);
                            }
                    }
                    filled |= 1u << s;
                    filled_parity = (filled_parity & ~(1u << s)) | (ph << s);
                    if (++s == nstages) {
                        s = 0;
                        ph ^= 1u;
                    }
                }
            }
            if (!ok && (CTA_GROUP == 1 || rank == 0)) {
                // Giving up: let this CTA's copies in flight land before the
                // shared memory is handed back (bounded by the same limit).
                for (int i = 0; i < C::STAGES; i++)
                    if (filled & (1u << i)) {
                        const uint64_t t0 = ptx::globaltimer_ns();
                        while (!ptx::mbar_try_wait(full_bar(i), (filled_parity >> i) & 1u))
                            if (ptx::globaltimer_ns() - t0 > WAIT_LIMIT_NS / 4) break;
                    }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------------------------------------------------- MMA issuer
        if (lane == 0 && rank == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true, issued = false;
            int it = 0;
            for (int t = unit_first; t < num_units && ok; t += unit_step) {
                const Unit u = unit_of(t, p, k_blocks);
                if (u.kb0 >= u.kb1) continue;  // an empty k range uses no accumulator
                const int buf = it % C::ACC_BUFS;
                const uint32_t aph = uint32_t(it / C::ACC_BUFS) & 1u;
                it++;
                const uint32_t d_tmem = tmem_base + uint32_t(buf * C::ACC_COLS);
                const int nkb = u.kb1 - u.kb0;
                for (int i0 = 0; i0 < nkb && ok; i0 += C::KPS) {
                    const int nk = nkb - i0 < C::KPS ? nkb - i0 : C::KPS;
                    if (!wait_bar(full_bar(s), ph, abort_flag, p.status, WHERE_MMA_FULL, uint32_t(s), wait_limit)) {
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
                    const uint32_t stage = ring + uint32_t(s) * C::STAGE_BYTES;
#pragma unroll
                    for (int kk = 0; kk < C::KPS; kk++) {
                        if (kk >= nk) break;
                        const bool first = (i0 == 0 && kk == 0);  // the unit's first k block overwrites the accumulator
                        const uint32_t a_src = stage + uint32_t(kk) * C::KB_BYTES;
                        const uint64_t b_desc = sw128_desc(a_src + C::A_BYTES);
#pragma unroll
                        for (int h = 0; h < HALVES; h++) {
                            if (first) {
                                // The epilogue must have drained this half of the buffer
                                // (a fresh barrier passes at once).
                                if (!wait_bar(tempty_bar(buf, h), aph ^ 1u, abort_flag, p.status, WHERE_MMA_TMEM,
                                              uint32_t(buf * 2 + h), wait_limit)) {
                                    ok = false;
                                    break;
                                }
                                ptx::tc_fence_after();
                            }
                            const uint64_t a_desc = sw128_desc(a_src + uint32_t(h) * (BM * BK * 2));
#pragma unroll
                            for (int j = 0; j < BK / UMMA_K; j++) {
                                ptx::umma_f16<CTA_GROUP>(d_tmem + uint32_t(h * C::HALF_COLS), a_desc + DESC_K_STEP * j, b_desc + DESC_K_STEP * j,
                                                         p.idesc, (!first || j > 0) ? 1u : 0u);
                            }
                            issued = true;
                        }
                        if (!ok) break;
                    }
                    if (!ok) break;
                    ptx::umma_commit<CTA_GROUP>(empty_bar(s));
                    if constexpr (CTA_GROUP == 2) ptx::umma_commit<CTA_GROUP>(ptx::mapa(empty_bar(s), 1));
                    if (++s == nstages) {
                        s = 0;
                        ph ^= 1u;
                    }
                }
                if (!ok) break;
                ptx::umma_commit<CTA_GROUP>(tfull_bar(buf));
                if constexpr (CTA_GROUP == 2) ptx::umma_commit<CTA_GROUP>(ptx::mapa(tfull_bar(buf), 1));
            }
            if (!ok && issued) {
                // Giving up: wait (bounded) until the tensor core is done with
                // shared memory and TMEM before they are released.
                ptx::umma_commit<CTA_GROUP>(drain_bar);
                const uint64_t t0 = ptx::globaltimer_ns();
                while (!ptx::mbar_try_wait(drain_bar, 0u))
                    if (ptx::globaltimer_ns() - t0 > WAIT_LIMIT_NS / 4) break;
            }
        }
        __syncwarp();
    } else if (warp < 2 + 4 * EG) {
        // ------------------------------------------------------------ epilogue
        // EG groups of four warps: warp w reads TMEM lane quarter w % 4 (the only one
        // it may address) and, of every 128-lane accumulator, every EG-th 32-column chunk.
        // In the 64-row tile lanes 64-127 hold the same rows as lanes 0-63, for the upper
        // half of the tile's columns.
        const uint32_t q = uint32_t(warp) & 3u;
        const int e = (warp - 2) >> 2;
        constexpr int CH = C::HALF_COLS / 32 / EG;  // chunks per accumulator per warp
        constexpr int ITEMS = HALVES * CH;
        static_assert(CH >= 1, "every epilogue warp needs a chunk");
        const bool plain = (p.alpha == 1.0f && p.beta == 0.0f);
        bool ok = true;
        int it = 0;
        uint32_t tiles_done = 0;
        for (int t = unit_first; t < num_units && ok; t += unit_step) {
            const Unit u = unit_of(t, p, k_blocks);
            const TileCoord tc = tile_coord(u.tile, p);
            const bool have_acc = u.kb0 < u.kb1;  // else this range contributes zeros
            const int buf = it % C::ACC_BUFS;
            const uint32_t aph = uint32_t(it / C::ACC_BUFS) & 1u;
            void *cbase = reinterpret_cast<uint8_t *>(p.C) + size_t(u.range) * p.split_stride;
            if (have_acc) {
                it++;
                if (!wait_bar(tfull_bar(buf), aph, abort_flag, p.status, WHERE_EPILOGUE, uint32_t(buf), wait_limit)) {
                    ok = false;
                    break;
                }
                ptx::tc_fence_after();
            }
            const int row0 = (tc.tm * CTA_GROUP + int(rank)) * C::A_ROWS + (C::HALF ? int(q & 1u) : int(q)) * 32 + lane;
            const int col_base = tc.tn * BN + (C::HALF ? int(q >> 1) * C::HALF_COLS : 0);
            const uint32_t taddr0 = tmem_base + ((q * 32u) << 16) + uint32_t(buf * C::ACC_COLS);
            auto col_of = [&](int i) { return ((i % CH) * EG + e) * 32; };  // within the accumulator's columns
            if constexpr (CTA_GROUP == 1 && MH == 1) {
                if (kc_mode) {
                    // This CTA's partial sums go to its shared memory (the ring is idle: the CTA's only unit
                    // has been multiplied), row r of the tile at r * KC_PITCH; the cluster adds them below.
                    ptx::fence_proxy_async_shared();
                    const uint32_t row_addr = ring + (q * 32u + uint32_t(lane)) * C::KC_PITCH;
#pragma unroll 1
                    for (int i = 0; i < ITEMS; i++) {
                        uint32_t v[32];
                        if (have_acc) {
                            ptx::tmem_ld_32x32(taddr0 + uint32_t(col_of(i)), v);
                            ptx::tmem_ld_wait(v);
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; j++) v[j] = 0u;
                        }
#pragma unroll
                        for (int g = 0; g < 8; g++)
                            ptx::st_shared_v4(row_addr + uint32_t(col_of(i) + 4 * g) * 4u, v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3]);
                    }
                    continue;
                }
            }
            auto load = [&](int i, uint32_t(&v)[32]) {
                if (have_acc) {
                    ptx::tmem_ld_32x32(taddr0 + uint32_t((i / CH) * C::HALF_COLS + col_of(i)), v);
                } else {
#pragma unroll
                    for (int j = 0; j < 32; j++) v[j] = 0u;
                }
            };
            // Item i has landed in v: release its half if it was this warp's last
            // read of it, then convert and store.
            auto finish = [&](int i, uint32_t(&v)[32]) {
                if (have_acc && (i % CH) == CH - 1) {
                    ptx::tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        if constexpr (CTA_GROUP == 1) ptx::mbar_arrive(tempty_bar(buf, i / CH));
                        else ptx::mbar_arrive_cluster(ptx::mapa(tempty_bar(buf, i / CH), 0));
                    }
                }
                if (p.debug & 2) return;
                store_chunk<C_BF16>(p, cbase, row0 + (i / CH) * BM, col_base + col_of(i), v, plain);
                if (!p.push)
                    for (int d = 0; d < p.extra_count; d++)
                        store_chunk<C_BF16>(p, p.extra_c[d], row0 + (i / CH) * BM, col_base + col_of(i), v, true);
            };
#if CB_FAST_DRAIN
            // The single-buffered accumulator (two halves of 256 columns fill TMEM): the MMA issuer
            // of the NEXT tile waits for each half to be handed back, so what counts is how soon
            // after the tile's last MMA a half is out of TMEM.  For the common result (whole tile
            // inside C, bf16, 32-byte aligned rows, plain epilogue, one destination written here)
            // a warp reads all its chunks of a half into registers with back-to-back tcgen05.ld,
            // hands the half back, and only then converts and stores.
            if constexpr (C_BF16 && C::ACC_BUFS == 1 && CH == 4) {
                const bool whole = (tc.tm * CTA_GROUP + int(rank) + 1) * C::A_ROWS <= p.M && (tc.tn + 1) * BN <= p.N;
                if (have_acc && plain && whole && p.c_vec_ok == 2 && !(p.debug & 2) && (p.push || p.extra_count == 0)) {
#pragma unroll 1
                    for (int h = 0; h < HALVES; h++) {
                        uint32_t v[CH][32];
#pragma unroll
                        for (int c = 0; c < CH; c++) ptx::tmem_ld_32x32(taddr0 + uint32_t(h * C::HALF_COLS + col_of(c)), v[c]);
                        ptx::tmem_ld_wait_all();
#pragma unroll
                        for (int c = 0; c < CH; c++) ptx::pin(v[c]);
                        ptx::tc_fence_before();
                        __syncwarp();
                        if (lane == 0) {
                            if constexpr (CTA_GROUP == 1) ptx::mbar_arrive(tempty_bar(buf, h));
                            else ptx::mbar_arrive_cluster(ptx::mapa(tempty_bar(buf, h), 0));
                        }
                        __nv_bfloat16 *crow = reinterpret_cast<__nv_bfloat16 *>(cbase) + size_t(row0 + h * BM) * p.ldc + col_base;
#pragma unroll
                        for (int c = 0; c < CH; c++) {
                            uint32_t w[16];
#pragma unroll
                            for (int j = 0; j < 16; j++) {
                                const __nv_bfloat162 hh = __floats2bfloat162_rn(__uint_as_float(v[c][2 * j]), __uint_as_float(v[c][2 * j + 1]));
                                w[j] = *reinterpret_cast<const uint32_t *>(&hh);
                            }
                            ptx::st_global_v8(crow + col_of(c), w[0], w[1], w[2], w[3], w[4], w[5], w[6], w[7]);
                            ptx::st_global_v8(crow + col_of(c) + 16, w[8], w[9], w[10], w[11], w[12], w[13], w[14], w[15]);
                        }
                    }
                    goto tile_stored;
                }
            }
#endif
            {
            // Two register buffers: the TMEM read of the next chunk is in flight
            // while the current one is converted and stored.
            uint32_t va[32], vb[32];
            load(0, va);
#pragma unroll 1
            for (int i = 0; i < ITEMS; i += 2) {
                if (have_acc) ptx::tmem_ld_wait(va);
                if (i + 1 < ITEMS) load(i + 1, vb);
                finish(i, va);
                if (i + 1 < ITEMS) {
                    if (have_acc) ptx::tmem_ld_wait(vb);
                    if (i + 2 < ITEMS) load(i + 2, va);
                    finish(i + 1, vb);
                }
            }
            }
#if CB_FAST_DRAIN
        tile_stored:
#endif
            if (p.push) {
                // This warp's part of the tile is in C: make the stores visible to the TMA unit
                // (async proxy) and publish the warp's tile count for the pusher.
                ptx::fence_proxy_async_global();
                __syncwarp();
                tiles_done++;
                if (lane == 0)
                    ptx::st_release_shared(ptx::smem_u32(const_cast<uint32_t *>(tiles_stored + (warp - 2))), tiles_done);
            }
        }
    } else {
        // -------------------------------------------------------------- pusher
        // One thread copies every tile this CTA has finished from C (still in L2) to the further
        // copies of C on other GPUs: a TMA load of a chunk of whole tile rows (BN columns, 512 bytes
        // or more per row, the segments NVLink carries best) into one of two buffers, then one bulk
        // tensor store per destination.  It runs behind the epilogue and beside the main loop of
        // the following tiles; nothing but the end of the kernel waits for it.
        if (p.push && lane == 0) {
            constexpr int PUSH_ROWS = push_rows(BN, C_BF16);
            constexpr int CHUNKS = C::A_ROWS / PUSH_ROWS;
            static_assert(PUSH_ROWS >= 8 && C::A_ROWS % PUSH_ROWS == 0, "push chunk shape");
            for (int d = 0; d <= p.extra_count; d++) ptx::prefetch_tensormap(&tmC.m[d]);
            const int my_tiles = cluster_id < num_units ? (num_units - cluster_id + num_clusters - 1) / num_clusters : 0;
            const int total = my_tiles * CHUNKS;
            const uint32_t stored_addr = ptx::smem_u32(const_cast<uint32_t *>(tiles_stored));
            auto coords = [&](int g, int &row, int &col) {
                const TileCoord tc = tile_coord(unit_of(cluster_id + (g / CHUNKS) * num_clusters, p, k_blocks).tile, p);
                row = (tc.tm * CTA_GROUP + int(rank)) * C::A_ROWS + (g % CHUNKS) * PUSH_ROWS;
                col = tc.tn * BN;
            };
            // All epilogue warps have stored tile number `j` of this CTA.  false = gave up.
            auto tile_stored = [&](int j) -> bool {
                const uint32_t want = uint32_t(j + 1);
                const uint64_t t0 = ptx::globaltimer_ns();
                uint32_t spins = 0;
                for (int w = 0; w < 4 * EG; w++) {
                    while (ptx::ld_acquire_shared(stored_addr + 4u * uint32_t(w)) < want) {
                        if ((++spins & 63u) == 0u) {
                            if (*abort_flag) return false;
                            if (ptx::globaltimer_ns() - t0 > wait_limit) {
                                *abort_flag = 1u;
                                report_timeout(p.status, WHERE_PUSHER, want, uint32_t(w));
                                return false;
                            }
                        }
                    }
                }
                ptx::fence_proxy_async_global();
                return true;
            };
            auto load = [&](int g) -> bool {
                if (g % CHUNKS == 0 && !tile_stored(g / CHUNKS)) return false;
                int row, col;
                coords(g, row, col);
                ptx::mbar_arrive_expect_tx(push_bar(g & 1), PUSH_BUF_BYTES);
                ptx::tma_load_2d(staging + uint32_t(g & 1) * PUSH_BUF_BYTES, &tmC.m[0], push_bar(g & 1), col, row);
                return true;
            };
            bool ok = total > 0 && load(0);
            for (int g = 0; g < total && ok; g++) {
                if (!wait_bar(push_bar(g & 1), uint32_t(g >> 1) & 1u, abort_flag, p.status, WHERE_PUSHER, uint32_t(g), wait_limit))
                    break;
                int row, col;
                coords(g, row, col);
                if (row < p.M)  // rows past the end of C are clipped by the TMA unit, whole chunks are skipped here
                    for (int d = 1; d <= p.extra_count; d++)
                        ptx::tma_store_2d(&tmC.m[d], staging + uint32_t(g & 1) * PUSH_BUF_BYTES, col, row);
                ptx::bulk_commit();
                ptx::bulk_wait_read<1>();  // the stores of chunk g - 1 have read the buffer that chunk g + 1 fills
                if (g + 1 < total) ok = load(g + 1);
            }
            ptx::bulk_wait_all();
        }
        __syncwarp();
    }

    // ------------------------------------------- sum of the k ranges inside a cluster
    if constexpr (CTA_GROUP == 1 && MH == 1) {
        if (kc_mode) {
            ptx::cluster_arrive();  // every CTA of the cluster has its partial sums in shared memory (or has given up)
            ptx::cluster_wait();
            if (warp >= 2 && warp < 2 + 4 * EG && unit_first < num_units && !*abort_flag) {
                // CTA r of the cluster finishes rows [r, r + 1) * 128 / kc of the tile: a warp per row, a lane per
                // four columns, the ranges added in ascending order (as the second kernel of the two-pass form does).
                const TileCoord tc = tile_coord(unit_of(unit_first, p, k_blocks).tile, p);
                const int rows_per = BM / p.kc;
                const bool plain = (p.alpha == 1.0f && p.beta == 0.0f);
                for (int r = warp - 2; r < rows_per; r += 4 * EG) {
                    const int trow = int(kc_rank) * rows_per + r;
                    const int grow = tc.tm * BM + trow;
                    if (grow >= p.M) continue;
#pragma unroll
                    for (int seg = 0; seg < BN / 128; seg++) {
                        const int tcol = seg * 128 + 4 * lane;
                        const int gcol = tc.tn * BN + tcol;
                        if (gcol >= p.N) continue;
                        const uint32_t local = ring + uint32_t(trow) * C::KC_PITCH + uint32_t(tcol) * 4u;
                        float4 acc = ptx::ld_shared_cluster_v4(ptx::mapa(local, 0));
                        for (int c = 1; c < p.kc; c++) {
                            const float4 b = ptx::ld_shared_cluster_v4(ptx::mapa(local, uint32_t(c)));
                            acc.x = __fadd_rn(acc.x, b.x);
                            acc.y = __fadd_rn(acc.y, b.y);
                            acc.z = __fadd_rn(acc.z, b.z);
                            acc.w = __fadd_rn(acc.w, b.w);
                        }
                        const float a4[4] = {acc.x, acc.y, acc.z, acc.w};
                        auto epi = [&](float a, float c_old) { return __fadd_rn(__fmul_rn(p.alpha, a), __fmul_rn(p.beta, c_old)); };
                        if constexpr (C_BF16) {
                            __nv_bfloat16 *c = reinterpret_cast<__nv_bfloat16 *>(p.C) + size_t(grow) * p.ldc + gcol;
                            if (p.c_vec_ok && gcol + 4 <= p.N) {
                                float f[4];
                                if (plain) {
#pragma unroll
                                    for (int j = 0; j < 4; j++) f[j] = a4[j];
                                } else {
                                    const uint2 old = *reinterpret_cast<const uint2 *>(c);
                                    f[0] = epi(a4[0], __uint_as_float(old.x << 16));
                                    f[1] = epi(a4[1], __uint_as_float(old.x & 0xffff0000u));
                                    f[2] = epi(a4[2], __uint_as_float(old.y << 16));
                                    f[3] = epi(a4[3], __uint_as_float(old.y & 0xffff0000u));
                                }
                                const __nv_bfloat162 h0 = __floats2bfloat162_rn(f[0], f[1]), h1 = __floats2bfloat162_rn(f[2], f[3]);
                                *reinterpret_cast<uint2 *>(c) = make_uint2(*reinterpret_cast<const uint32_t *>(&h0), *reinterpret_cast<const uint32_t *>(&h1));
                            } else {
                                for (int j = 0; j < 4 && gcol + j < p.N; j++)
                                    c[j] = __float2bfloat16_rn(plain ? a4[j] : epi(a4[j], __bfloat162float(c[j])));
                            }
                        } else {
                            float *c = reinterpret_cast<float *>(p.C) + size_t(grow) * p.ldc + gcol;
                            if (p.c_vec_ok && gcol + 4 <= p.N) {
                                float4 o = acc;
                                if (!plain) {
                                    const float4 old = *reinterpret_cast<const float4 *>(c);
                                    o = make_float4(epi(acc.x, old.x), epi(acc.y, old.y), epi(acc.z, old.z), epi(acc.w, old.w));
                                }
                                *reinterpret_cast<float4 *>(c) = o;
                            } else {
                                for (int j = 0; j < 4 && gcol + j < p.N; j++) c[j] = plain ? a4[j] : epi(a4[j], c[j]);
                            }
                        }
                    }
                }
            }
            __syncwarp();
        }
    }

    // ---------------------------------------------------------------- teardown
    ptx::tc_fence_before();
    __syncthreads();
    if (CTA_GROUP == 2 || kc_mode) {  // the peer may still arrive on our barriers or read our shared memory
        ptx::cluster_arrive();
        ptx::cluster_wait();
    }
    if (warp == 1) ptx::tmem_dealloc<CTA_GROUP>(tmem_base, C::TMEM_COLS);
    // Everything this CTA stored, to its own C and to the other destinations (the pusher's thread has
    // waited for its bulk stores), is ordered before this point by the barrier above.  The last CTA
    // of the launch tells the owners of the destinations.  Every CTA counts itself (low half of the
    // word), one that gave up also in the high half; if any did, nothing is signalled, so that the
    // owners' waits run out and report as well.
    if (p.signal_count > 0 && threadIdx.x == 0) {
        ptx::fence_proxy_async_global();
        __threadfence();
        const uint32_t mine = 1u + (*abort_flag ? 0x10000u : 0u);
        const uint32_t all = atomicAdd(p.done_counter, mine) + mine;
        if ((all & 0xffffu) == gridDim.x) {
            *p.done_counter = 0u;  // the next launch on this device counts from zero again
            if ((all >> 16) == 0u) {
                __threadfence_system();
                for (int i = 0; i < p.signal_count; i++) ptx::red_release_sys_add(p.signal[i], 1u);
            }
        }
    }
}

// Waits until every counter[i] with bit i of `mask` set has reached at_least (acquire, system scope,
// compared as wrapping 32-bit counts) or the limit runs out; then reports {WHERE_SIGNAL, at_least,
// index of the counter that was short, its value} in the status word and returns.
__global__ void wait_signal_kernel(const uint32_t *counter, uint32_t mask, uint32_t at_least, uint64_t limit_ns, uint32_t *status) {
    if (threadIdx.x != 0) return;
    const uint64_t t0 = ptx::globaltimer_ns();
    for (int i = 0; i < 32; i++) {
        if (!((mask >> i) & 1u)) continue;
        uint32_t seen = ptx::ld_acquire_sys(counter + i);
        while (int32_t(seen - at_least) < 0) {
            if (ptx::globaltimer_ns() - t0 > limit_ns) {
                if (atomicCAS(status, 0u, uint32_t(WHERE_SIGNAL)) == 0u) {
                    status[1] = at_least;
                    status[2] = uint32_t(i);
                    status[3] = seen;
                    __threadfence();
                }
                return;
            }
            __nanosleep(200);
            seen = ptx::ld_acquire_sys(counter + i);
        }
    }
}

// out = alpha * 0 + beta * c (or 0 when C is write-only): the k == 0 case.
template <bool C_BF16>
__global__ void gemm_k0_kernel(void *C, size_t count, float alpha, float beta) {
    const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const bool plain = (alpha == 1.0f && beta == 0.0f);
    if constexpr (C_BF16) {
        __nv_bfloat16 *c = reinterpret_cast<__nv_bfloat16 *>(C);
        const float r = plain ? 0.0f : __fadd_rn(__fmul_rn(alpha, 0.0f), __fmul_rn(beta, __bfloat162float(c[i])));
        c[i] = __float2bfloat16_rn(r);
    } else {
        float *c = reinterpret_cast<float *>(C);
        c[i] = plain ? 0.0f : __fadd_rn(__fmul_rn(alpha, 0.0f), __fmul_rn(beta, c[i]));
    }
}

// Second pass of a split-k GEMM: C = alpha * (P_0 + P_1 + ... ) + beta * C over
// the f32 partial planes, ranges added in ascending order.
template <bool C_BF16>
__global__ void __launch_bounds__(256) gemm_splitk_reduce(const float *__restrict__ partial, int splits, size_t plane,
                                                          size_t count, void *C, float alpha, float beta) {
    ptx::griddep_wait();  // launched as a programmatic dependent of the first pass: wait for its planes
    const size_t i4 = (size_t(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
    if (i4 >= count) return;
    const bool plain = (alpha == 1.0f && beta == 0.0f);
    float acc[4];
    const int n = int(min(size_t(4), count - i4));
    if (n == 4 && (plane & 3) == 0) {  // planes 16 bytes apart in phase: else their float4 loads would be misaligned
        float4 a = *reinterpret_cast<const float4 *>(partial + i4);
        for (int s = 1; s < splits; s++) {
            const float4 b = *reinterpret_cast<const float4 *>(partial + s * plane + i4);
            a.x = __fadd_rn(a.x, b.x);
            a.y = __fadd_rn(a.y, b.y);
            a.z = __fadd_rn(a.z, b.z);
            a.w = __fadd_rn(a.w, b.w);
        }
        acc[0] = a.x, acc[1] = a.y, acc[2] = a.z, acc[3] = a.w;
    } else {
        for (int j = 0; j < n; j++) {
            float a = partial[i4 + j];
            for (int s = 1; s < splits; s++) a = __fadd_rn(a, partial[s * plane + i4 + j]);
            acc[j] = a;
        }
    }
    for (int j = 0; j < n; j++) {
        if constexpr (C_BF16) {
            __nv_bfloat16 *c = reinterpret_cast<__nv_bfloat16 *>(C) + i4 + j;
            const float r = plain ? acc[j] : __fadd_rn(__fmul_rn(alpha, acc[j]), __fmul_rn(beta, __bfloat162float(*c)));
            *c = __float2bfloat16_rn(r);
        } else {
            float *c = reinterpret_cast<float *>(C) + i4 + j;
            *c = plain ? acc[j] : __fadd_rn(__fmul_rn(alpha, acc[j]), __fmul_rn(beta, *c));
        }
    }
}

// ---------------------------------------------------------------------- host
using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

cute_b200_status encode_fn(EncodeTiledFn *out) {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    static cudaError_t err = cudaSuccess;
    std::call_once(once, [] {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        err = cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &sym, 12000, cudaEnableDefault, &q);
        if (err == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = reinterpret_cast<EncodeTiledFn>(sym);
    });
    if (!fn) return fail(CUTE_B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    *out = fn;
    return CUTE_B200_OK;
}

// K-major (rows, k) 16-bit matrix, box (box_rows, 64), 128-byte swizzle,
// out-of-range elements read as zero.
cute_b200_status make_tensor_map(CUtensorMap *tm, uint64_t base, int dtype, int rows, int k, int box_rows) {
    using Key = std::tuple<uint64_t, int, int, int, int, int>;
    static std::map<Key, CUtensorMap> cache;
    static std::mutex mu;
    int device = 0;
    cudaGetDevice(&device);
    const Key key{base, dtype, rows, k, box_rows, device};
    {
        std::lock_guard<std::mutex> lock(mu);
        auto it = cache.find(key);
        if (it != cache.end()) {
            *tm = it->second;
            return CUTE_B200_OK;
        }
    }
    EncodeTiledFn encode;
    CB_TRY(encode_fn(&encode));
    const cuuint64_t dims[2] = {cuuint64_t(k), cuuint64_t(rows)};
    const cuuint64_t strides[1] = {cuuint64_t(k) * 2};
    const cuuint32_t box[2] = {cuuint32_t(BK), cuuint32_t(box_rows)};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = encode(tm, dtype == CUTE_B200_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                              2, reinterpret_cast<void *>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(CUTE_B200_ERR_CUDA, "cuTensorMapEncodeTiled failed: CUresult %d (rows %d, k %d, box %d)", int(r), rows, k,
                    box_rows);
    std::lock_guard<std::mutex> lock(mu);
    if (cache.size() > 4096) cache.clear();
    cache[key] = *tm;
    return CUTE_B200_OK;
}

// Row-major (m, n) C, f32 or bf16, in boxes of box_cols x box_rows elements, not swizzled.
cute_b200_status make_tensor_map_c(CUtensorMap *tm, uint64_t base, bool bf16, int m, int n, int box_cols, int box_rows) {
    EncodeTiledFn encode;
    CB_TRY(encode_fn(&encode));
    const cuuint64_t esize = bf16 ? 2 : 4;
    const cuuint64_t dims[2] = {cuuint64_t(n), cuuint64_t(m)};
    const cuuint64_t strides[1] = {cuuint64_t(n) * esize};
    const cuuint32_t box[2] = {cuuint32_t(box_cols), cuuint32_t(box_rows)};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = encode(tm, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2,
                              reinterpret_cast<void *>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(CUTE_B200_ERR_CUDA, "cuTensorMapEncodeTiled (C) failed: CUresult %d (m %d, n %d, box %d x %d)", int(r), m, n,
                    box_cols, box_rows);
    return CUTE_B200_OK;
}

template <int CTA_GROUP, int BN, int MH, bool C_BF16>
cute_b200_status launch(const CUtensorMap &tmA, const CUtensorMap &tmB, const CMaps &tmC, GemmParams p,
                        int sm_count, cudaStream_t stream) {
    using C = Cfg<CTA_GROUP, BN, MH>;
    const int tile_rows = C::A_ROWS * CTA_GROUP;
    p.m_tiles = (p.M + tile_rows - 1) / tile_rows;
    p.n_tiles = (p.N + BN - 1) / BN;
    const long long tiles = (long long)p.m_tiles * p.n_tiles * p.splits;
    int clusters = sm_count / CTA_GROUP;
    if (tiles < clusters) clusters = int(tiles);
    const bool kc = CTA_GROUP == 1 && MH == 1 && p.kc > 1;
    if (kc) {  // one unit per CTA, the kc ranges of a tile in one cluster
        if (tiles > (1 << 20)) return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "gemm_tn: too many tiles for the in-cluster k split");
        clusters = int(tiles);
    }
    // Walk about sqrt(#concurrent tiles) row tiles before moving to the next
    // column so that a wave of CTAs covers a near-square patch of C.
    int gm = 1;
    while (gm * gm * 2 <= clusters) gm *= 2;
    if (p.group_m > 0) gm = p.group_m;  // caller's override
    p.group_m = gm < p.m_tiles ? gm : p.m_tiles;
    if (p.group_m < 1) p.group_m = 1;

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(clusters * CTA_GROUP));
    cfg.blockDim = dim3(num_threads(BN, MH));
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kc ? unsigned(p.kc) : unsigned(CTA_GROUP);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    // Queued behind another launch of this library, the kernel is set up (barriers, TMEM) while that one
    // drains; its griddepcontrol.wait keeps every global access behind the predecessor's completion.
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = (p.debug & 32) ? 0 : 1;  // bit 5: plain stream order (measurements)
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    CB_CUDA(cudaLaunchKernelEx(&cfg, gemm_tn_kernel<CTA_GROUP, BN, MH, C_BF16>, tmA, tmB, tmC, p));
    count_launch();
    return CUTE_B200_OK;
}

template <int CTA_GROUP, int BN, int MH, bool C_BF16>
cute_b200_status set_smem_limit() {
    CB_CUDA(cudaFuncSetAttribute(gemm_tn_kernel<CTA_GROUP, BN, MH, C_BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Cfg<CTA_GROUP, BN, MH>::SMEM_BYTES));
    return CUTE_B200_OK;
}

// Every (cta_group, tile_n, rows-per-CTA, C type) the library instantiates.
#define CB_GEMM_VARIANTS(X) \
    X(1, 128, 1, false) X(1, 128, 1, true) X(1, 256, 1, false) X(1, 256, 1, true) \
    X(2, 128, 1, false) X(2, 128, 1, true) X(2, 256, 1, false) X(2, 256, 1, true) \
    X(1, 128, 2, false) X(1, 128, 2, true) X(1, 256, 2, false) X(1, 256, 2, true) \
    X(2, 128, 2, false) X(2, 128, 2, true) X(2, 256, 2, false) X(2, 256, 2, true) \
    X(2, 128, 0, false) X(2, 128, 0, true) X(2, 256, 0, false) X(2, 256, 0, true)

// Relative mainloop efficiency of a tiling, measured on 8192^3 bf16 (the 512 x 256
// pair tile is the reference point); used only to rank candidates.  mh counts the
// 128-row accumulators per CTA, 0 = the 64-row pair tile.
double tiling_efficiency(int group, int bn, int mh) {
    // The 64-row pair tile is bound by the rate at which one thread can issue cta_group::2 MMAs
    // (about 115 clocks each, whatever their size): 8192 x 128 x 8192 runs 0.23 us per k block,
    // 8192 x 256 x 8192 0.31 us.
    if (mh == 0) return bn == 128 ? 0.40 : 0.67;
    double e = 1.0;
    if (group == 1) e *= (mh == 2 ? 0.96 : 0.86);
    else if (mh == 1) e *= 0.92;
    if (bn == 128) e *= (mh == 2 ? 0.85 : (group == 1 ? 0.82 : 0.72));
    return e;
}

// Pick tiling and k split with the smallest estimated time.  A launch runs
// whole waves of work units (tile x k range) over the clusters that fit; a
// unit costs its MMA time plus a fixed start/drain latency, or the time its
// share of HBM bandwidth needs to bring its rows of A in, whichever is longer;
// a split GEMM also pays a second pass over the f32 partial planes.
//
// want_* != 0 fixes that choice (want_rows: rows of C per CTA, 64, 128 or 256).
// A caller's want_splits > 1 is honoured as it is (cut down to the number of k
// blocks and to max_splits), whether or not the cost model would have picked
// it; with want_splits == 0 the splits min_splits..max_splits compete, and a
// split above min_splits must leave each range at least four k blocks.
// *mh receives the 128-row accumulators per CTA, 0 for the 64-row pair tile.
// Returns the estimate in seconds.
// Whether a k split is summed inside the kernel by the CTAs of a cluster (GemmParams::kc): single-CTA
// 128-row tiles, two or four ranges, all units in one wave.
bool kc_applies(int m, int n, int g, int b, int h, int s, int sm_count) {
    if (g != 1 || h != 1 || (s != 2 && s != 4)) return false;
    const long long units = (long long)((m + BM - 1) / BM) * ((n + b - 1) / b) * s;
    return units <= sm_count;
}

double choose_tiling(int m, int n, int k, int c_bytes, int sm_count, int want_group, int want_bn, int want_rows,
                     int want_splits, int min_splits, int max_splits, bool allow_kc, int *group, int *bn, int *mh, int *splits) {
    const double sm_rate = 1.0e13;       // dense 16-bit flop/s of one SM at the clocks a GEMM sustains
    const double unit_latency = 2.5e-6;  // fill the ring, drain the accumulator
    // A launch of CTA pairs starts about 2 us later than one of single CTAs (cluster scheduling and the
    // cluster barrier around the TMEM set-up); measured on one-wave problems: 1024^3 12.7 / 10.6 us,
    // 2048^3 20.7 / 18.6, 3072^3 41.2 / 39.6 (pair / single), equal from 4096^3 on.
    const double pair_start = 2.0e-6;
    const double hbm = 4.5e12;  // what rows of A read as 128-byte pieces, 16 KiB apart, reach (cuBLAS: 4.7e12 on the same shape)
    const int k_blocks = (k + BK - 1) / BK;
    if (max_splits > 16) max_splits = 16;
    if (max_splits > k_blocks) max_splits = k_blocks;
    if (max_splits < 1) max_splits = 1;
    if (min_splits < 1) min_splits = 1;
    if (min_splits > max_splits) min_splits = max_splits;
    int s_lo = min_splits, s_hi = max_splits;
    if (want_splits > 0) {
        s_lo = s_hi = want_splits < min_splits ? min_splits : (want_splits > max_splits ? max_splits : want_splits);
    }
    if (want_rows == 64) want_group = 2;  // the 64-row tile exists as a pair tile only
    double best = 1e300;
    for (int g = 1; g <= 2; g++)
        for (int b = 128; b <= 256; b += 128)
            for (int h = 0; h <= 2; h++)
                for (int s = s_lo; s <= s_hi; s++) {
                    const int cta_rows = h == 0 ? 64 : 128 * h;
                    if (h == 0 && g != 2) continue;
                    if ((want_group && g != want_group) || (want_bn && b != want_bn) || (want_rows && cta_rows != want_rows)) continue;
                    if (want_splits == 0 && s > min_splits && (s > k_blocks / 4 || double(s) * m * n * 4 > 512e6)) continue;
                    const long long rows = (long long)cta_rows * g;
                    const long long units = ((m + rows - 1) / rows) * ((n + b - 1) / b) * s;
                    const long long clusters = sm_count / g;
                    const long long waves = (units + clusters - 1) / clusters;
                    const int kb_per = (k_blocks + s - 1) / s;
                    double unit_time = 2.0 * rows * b * kb_per * BK / (g * sm_rate * tiling_efficiency(g, b, h));
                    // With a single column of tiles every row of A is read by one unit only: the units of a
                    // wave share the HBM bandwidth for their rows (B stays in L2).
                    if ((n + b - 1) / b == 1) {
                        const long long in_wave = units < clusters ? units : clusters;
                        const double stream_time = double(in_wave) * rows * kb_per * BK * 2 / hbm;
                        if (stream_time > unit_time) unit_time = stream_time;
                    }
                    double t = waves * (unit_time + unit_latency);
                    if (g == 2) t += pair_start;
                    if (s > 1) {
                        if (allow_kc && kc_applies(m, n, g, b, h, s, sm_count)) t += 3.0e-6;  // the exchange through shared memory
                        else t += (double(s + 1) * m * n * 4 + double(m) * n * c_bytes) / hbm + 3.5e-6;  // planes + the second launch (a programmatic dependent)
                    }
                    if (t < best) {
                        best = t;
                        *group = g, *bn = b, *mh = h, *splits = s;
                    }
                }
    return best;
}

// Grow-only scratch of the split-k path, one per device, shared by every
// stream.  `idle` is recorded behind the second pass of each split GEMM and the
// next split GEMM's stream waits for it before its first pass, so two calls on
// different streams take turns on the planes instead of racing.
struct Scratch {
    void *ptr = nullptr;
    size_t size = 0;
    cudaEvent_t idle = nullptr;
};
Scratch g_scratch[64];
std::mutex g_scratch_mu;

// Hands out the device's scratch (grown if needed) after making `stream` wait
// for the previous user.  The caller queues its kernels and then calls
// scratch_release on the same stream.
cute_b200_status scratch_acquire(size_t bytes, cudaStream_t stream, void **out) {
    int device = 0;
    CB_CUDA(cudaGetDevice(&device));
    if (device < 0 || device >= 64) return fail(CUTE_B200_ERR_NO_DEVICE, "no current device");
    std::lock_guard<std::mutex> lock(g_scratch_mu);
    Scratch &sc = g_scratch[device];
    if (!sc.idle) CB_CUDA(cudaEventCreateWithFlags(&sc.idle, cudaEventDisableTiming));
    if (sc.size < bytes) {
        if (sc.ptr) CB_CUDA(cudaFree(sc.ptr));  // waits for the device: no user of the old planes is left
        sc.ptr = nullptr;
        sc.size = 0;
        CB_CUDA(cudaMalloc(&sc.ptr, bytes));
        sc.size = bytes;
    }
    CB_CUDA(cudaStreamWaitEvent(stream, sc.idle, 0));  // an event never recorded counts as complete
    *out = sc.ptr;
    return CUTE_B200_OK;
}

cute_b200_status scratch_release(cudaStream_t stream) {
    int device = 0;
    CB_CUDA(cudaGetDevice(&device));
    std::lock_guard<std::mutex> lock(g_scratch_mu);
    CB_CUDA(cudaEventRecord(g_scratch[device].idle, stream));
    return CUTE_B200_OK;
}

}  // namespace

// ---- split-k GEMM without any allocation -------------------------------------
// Scratch and status words of cute_b200_gemm_tn_static: part of the library
// image, so every GPU that loads the library holds them until the process ends.
constexpr size_t kStaticScratchBytes = size_t(32) << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
static __device__ __align__(16) uint32_t g_static_status[4];

namespace {
struct StaticSetup {
    bool ready = false;
    void *scratch = nullptr;      // device address of g_static_scratch on this device
    uint32_t *status = nullptr;   // device address of g_static_status on this device
    int sm_count = 0;
};
StaticSetup g_static_setup[64];
std::mutex g_static_mu;

// Once per device, with that device current: resolve the device addresses of
// the two arrays (their names are host-side stand-ins, not device pointers)
// and raise the kernels' shared-memory limit.  Allocates nothing.
cute_b200_status static_setup(int device, StaticSetup **out) {
    std::lock_guard<std::mutex> lock(g_static_mu);
    StaticSetup &st = g_static_setup[device];
    if (!st.ready) {
        int major = 0;
        CB_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
        if (major != 10)
            return fail(CUTE_B200_ERR_NO_DEVICE, "device %d is not sm_100; this library is built for sm_100a only", device);
        CB_CUDA(cudaDeviceGetAttribute(&st.sm_count, cudaDevAttrMultiProcessorCount, device));
        void *p = nullptr;
        CB_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
        st.scratch = p;
        CB_CUDA(cudaGetSymbolAddress(&p, g_static_status));
        st.status = static_cast<uint32_t *>(p);
#define CB_SET(G, N_, H, BF) CB_TRY((set_smem_limit<G, N_, H, BF>()));
        CB_GEMM_VARIANTS(CB_SET)
#undef CB_SET
        st.ready = true;
    }
    *out = &st;
    return CUTE_B200_OK;
}
}  // namespace

uint32_t *gemm_tn_static_status_words(int device) {
    if (device < 0 || device >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(g_static_mu);
    return g_static_setup[device].ready ? g_static_setup[device].status : nullptr;
}

cute_b200_status gemm_tn_static(const cute_b200_gemm_desc &d, uint64_t a, uint64_t b, uint64_t c, cudaStream_t stream,
                                uint32_t *shared_status) {
    if (d.m <= 0 || d.n <= 0 || d.k <= 0)
        return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "gemm_tn_static: invalid size %dx%dx%d (k must be positive)", d.m,
                    d.n, d.k);
    if ((d.ab_dtype != CUTE_B200_F16 && d.ab_dtype != CUTE_B200_BF16) ||
        (d.c_dtype != CUTE_B200_F32 && d.c_dtype != CUTE_B200_BF16))
        return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "gemm_tn_static: f16/bf16 inputs and f32/bf16 output only");
    if (d.k % 8) return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "gemm_tn_static: k must be a multiple of 8, got %d", d.k);
    if ((d.tile_n != 0 && d.tile_n != 128 && d.tile_n != 256) || d.cta_group < 0 || d.cta_group > 2 ||
        (d.tile_m != 0 && d.tile_m != 64 && d.tile_m != 128 && d.tile_m != 256) || (d.tile_m == 64 && d.cta_group == 1))
        return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "gemm_tn_static: invalid tile_n, tile_m or cta_group");
    if (d.split_k == 1 || d.split_k < 0 || d.split_k > 16)
        return fail(CUTE_B200_ERR_INVALID_ARGUMENT,
                    "gemm_tn_static is the split-k GEMM: split_k must be 0 (choose) or 2..16, got %d", d.split_k);
    if (!a || !b || !c) return fail(CUTE_B200_ERR_NULL_POINTER, "gemm_tn_static: null buffer");
    const bool c_bf16 = d.c_dtype == CUTE_B200_BF16;
    if ((a | b) & 15u) return fail(CUTE_B200_ERR_MISALIGNED, "gemm_tn_static: A and B must be 16-byte aligned");
    if (c & (c_bf16 ? 1u : 3u)) return fail(CUTE_B200_ERR_MISALIGNED, "gemm_tn_static: C is not aligned to its element size");
    const int k_blocks = (d.k + BK - 1) / BK;
    if (k_blocks < 2) return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "gemm_tn_static: k = %d is too short to split", d.k);

    int device = 0;
    CB_CUDA(cudaGetDevice(&device));
    if (device < 0 || device >= 64) return fail(CUTE_B200_ERR_NO_DEVICE, "no current device");
    StaticSetup *setup = nullptr;
    CB_TRY(static_setup(device, &setup));

    const size_t plane = size_t(d.m) * d.n;
    const size_t max_splits_by_scratch = kStaticScratchBytes / (plane * 4);
    if (max_splits_by_scratch < 2 || (d.split_k && size_t(d.split_k) > max_splits_by_scratch))
        return fail(CUTE_B200_ERR_INVALID_ARGUMENT,
                    "gemm_tn_static: %d x %d with %d k ranges needs %zu bytes of scratch, the built-in buffer holds %zu",
                    d.m, d.n, d.split_k ? d.split_k : 2, plane * 4 * size_t(d.split_k ? d.split_k : 2), kStaticScratchBytes);

    // The tiling comes from the same cost model as the allocating path, asked for at least
    // two ranges and at most what the built-in array (and k) allow.
    int group = 2, bn = 256, mh = 2, splits = 2;
    choose_tiling(d.m, d.n, d.k, c_bf16 ? 2 : 4, setup->sm_count, d.cta_group, d.tile_n, d.tile_m, d.split_k, 2,
                  int(max_splits_by_scratch < 16 ? max_splits_by_scratch : 16), false, &group, &bn, &mh, &splits);

    GemmParams p = {};
    p.C = setup->scratch;
    p.M = d.m;
    p.N = d.n;
    p.K = d.k;
    p.ldc = d.n;
    p.alpha = 1.0f;
    p.beta = 0.0f;
    p.status = shared_status ? shared_status : setup->status;
    p.debug = d.tuning[0] & (4 | 8);  // the two test knobs of the bounded waits; the measurement knobs stay off
    p.group_m = d.tuning[1];
    p.splits = splits;
    p.split_stride = plane * 4;
    p.c_vec_ok = (size_t(d.n) * 4) % 32 == 0 ? 2 : ((size_t(d.n) * 4) % 16 == 0 ? 1 : 0);
    const int cta_rows = mh == 0 ? 64 : BM * mh;
    p.idesc = make_idesc(d.ab_dtype == CUTE_B200_BF16, (mh == 0 ? 64 : BM) * group, bn);

    CUtensorMap tmA, tmB;
    CB_TRY(make_tensor_map(&tmA, a, d.ab_dtype, d.m, d.k, cta_rows));
    CB_TRY(make_tensor_map(&tmB, b, d.ab_dtype, d.n, d.k, bn / group));
    cute_b200_status st = CUTE_B200_ERR_UNSUPPORTED;
#define CB_CASE(G, N_, H, BF) \
    if (group == G && bn == N_ && mh == H && !BF) st = launch<G, N_, H, false>(tmA, tmB, CMaps{}, p, setup->sm_count, stream);
    CB_GEMM_VARIANTS(CB_CASE)
#undef CB_CASE
    CB_TRY(st);
    const unsigned blocks = unsigned((plane + 1023) / 1024);
    if (c_bf16)
        gemm_splitk_reduce<true><<<blocks, 256, 0, stream>>>(static_cast<const float *>(setup->scratch), splits, plane, plane,
                                                             reinterpret_cast<void *>(c), d.alpha, d.beta);
    else
        gemm_splitk_reduce<false><<<blocks, 256, 0, stream>>>(static_cast<const float *>(setup->scratch), splits, plane, plane,
                                                              reinterpret_cast<void *>(c), d.alpha, d.beta);
    CB_CUDA(cudaGetLastError());
    count_launch();
    return CUTE_B200_OK;
}

void gemm_tn_release_scratch() {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return;
    std::lock_guard<std::mutex> lock(g_scratch_mu);
    if (g_scratch[device].ptr) cudaFree(g_scratch[device].ptr);
    g_scratch[device].ptr = nullptr;
    g_scratch[device].size = 0;
}

cute_b200_status gemm_tn_init(const DeviceState &) {
#define CB_SET(G, N_, H, BF) CB_TRY((set_smem_limit<G, N_, H, BF>()));
    CB_GEMM_VARIANTS(CB_SET)
#undef CB_SET
    return CUTE_B200_OK;
}

// What the plain entry point does not take: further destinations, a row pitch of C.
struct GemmExtras {
    const uint64_t *extra_c = nullptr;
    int extra_count = 0;
    int ldc = 0;  // 0 = n
    const uint64_t *signal = nullptr;  // extra_count counters to add 1 to when the launch is complete, or null
};
static cute_b200_status gemm_tn_ex(const cute_b200_gemm_desc &d, uint64_t a, uint64_t b, uint64_t c, cudaStream_t stream,
                                   const DeviceState &dev, const GemmExtras &ex);

cute_b200_status wait_signal(uint64_t counter, uint32_t mask, uint32_t at_least, uint32_t timeout_ms, cudaStream_t stream,
                             const DeviceState &dev) {
    if (!counter || (counter & 3u)) return fail(CUTE_B200_ERR_MISALIGNED, "wait_signal: the counters are null or not 4-byte aligned");
    if (timeout_ms == 0 || timeout_ms > 600000u)
        return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "wait_signal: the limit must be 1 ms to 10 min, got %u ms", timeout_ms);
    wait_signal_kernel<<<1, 32, 0, stream>>>(reinterpret_cast<const uint32_t *>(counter), mask, at_least,
                                             uint64_t(timeout_ms) * 1000000ull, dev.status_word);
    CB_CUDA(cudaGetLastError());
    count_launch();
    return CUTE_B200_OK;
}

cute_b200_status gemm_tn_multi(const cute_b200_gemm_desc &d, uint64_t a, uint64_t b, const uint64_t *c_list, int count,
                               const uint64_t *signal_list, cudaStream_t stream, const DeviceState &dev) {
    if (!c_list || count < 1 || count > 8)
        return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "gemm_tn_multi: 1 to 8 destinations, got %d", count);
    if (count > 1) {
        if (!(d.alpha == 1.0f && d.beta == 0.0f))
            return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "gemm_tn_multi: several destinations need alpha = 1, beta = 0");
        if (d.split_k > 1)
            return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "gemm_tn_multi: several destinations cannot be combined with split_k");
        const uint64_t mask = d.c_dtype == CUTE_B200_BF16 ? 1u : 3u;
        for (int i = 1; i < count; i++)
            if (!c_list[i] || ((c_list[i] ^ c_list[0]) & 31u) || (c_list[i] & mask))
                return fail(CUTE_B200_ERR_MISALIGNED, "gemm_tn_multi: destination %d is null or aligned differently from the first", i);
    }
    if (signal_list) {
        if (d.k == 0) return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "gemm_tn_multi: the completion signal needs k > 0");
        for (int i = 1; i < count; i++)
            if (!signal_list[i] || (signal_list[i] & 3u))
                return fail(CUTE_B200_ERR_MISALIGNED, "gemm_tn_multi: signal counter %d is null or not 4-byte aligned", i);
    }
    cute_b200_gemm_desc dd = d;
    if (count > 1 && d.k == 0) {  // nothing to multiply: every destination is filled with zeros by its own launch
        for (int i = 0; i < count; i++) CB_TRY(gemm_tn(dd, a, b, c_list[i], stream, dev));
        return CUTE_B200_OK;
    }
    if (count > 1) {
        dd.split_k = 1;
    }
    GemmExtras ex;
    ex.extra_c = c_list + 1;
    ex.extra_count = count - 1;
    ex.signal = signal_list ? signal_list + 1 : nullptr;
    return gemm_tn_ex(dd, a, b, c_list[0], stream, dev, ex);
}

cute_b200_status gemm_tn(const cute_b200_gemm_desc &d, uint64_t a, uint64_t b, uint64_t c, cudaStream_t stream,
                         const DeviceState &dev) {
    return gemm_tn_ex(d, a, b, c, stream, dev, GemmExtras{});
}

cute_b200_status gemm_tn_strided(const cute_b200_gemm_desc &d, uint64_t a, uint64_t b, uint64_t c, int ldc,
                                 cudaStream_t stream, const DeviceState &dev) {
    if (ldc < d.n) return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "gemm_tn: row pitch %d of C is below n = %d", ldc, d.n);
    if (d.k <= 0) return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "gemm_tn: a block of a wider C needs k > 0");
    GemmExtras ex;
    ex.ldc = ldc;
    cute_b200_gemm_desc dd = d;
    dd.split_k = 1;
    return gemm_tn_ex(dd, a, b, c, stream, dev, ex);
}

static cute_b200_status gemm_tn_ex(const cute_b200_gemm_desc &d, uint64_t a, uint64_t b, uint64_t c, cudaStream_t stream,
                                   const DeviceState &dev, const GemmExtras &ex) {
    if (d.m <= 0 || d.n <= 0 || d.k < 0)
        return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "gemm_tn: invalid size %dx%dx%d", d.m, d.n, d.k);
    if (d.ab_dtype != CUTE_B200_F16 && d.ab_dtype != CUTE_B200_BF16)
        return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "gemm_tn takes f16 or bf16 inputs, not dtype %d", d.ab_dtype);
    if (d.c_dtype != CUTE_B200_F32 && d.c_dtype != CUTE_B200_BF16)
        return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "gemm_tn writes f32 or bf16, not dtype %d", d.c_dtype);
    if (d.k % 8) return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "gemm_tn: k must be a multiple of 8, got %d", d.k);
    if (d.tile_n != 0 && d.tile_n != 128 && d.tile_n != 256)
        return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "gemm_tn: tile_n must be 0, 128 or 256, got %d", d.tile_n);
    if (d.cta_group < 0 || d.cta_group > 2)
        return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "gemm_tn: cta_group must be 0, 1 or 2, got %d", d.cta_group);
    if (d.tile_m != 0 && d.tile_m != 64 && d.tile_m != 128 && d.tile_m != 256)
        return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "gemm_tn: tile_m must be 0, 64, 128 or 256, got %d", d.tile_m);
    if (d.tile_m == 64 && d.cta_group == 1)
        return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "gemm_tn: the 64-row tile needs a CTA pair (cta_group 0 or 2)");
    if (!c) return fail(CUTE_B200_ERR_NULL_POINTER, "gemm_tn: C is null");
    const bool c_bf16 = d.c_dtype == CUTE_B200_BF16;
    if (c & (c_bf16 ? 1u : 3u)) return fail(CUTE_B200_ERR_MISALIGNED, "gemm_tn: C is not aligned to its element size");

    if (d.k == 0) {
        const size_t count = size_t(d.m) * d.n;
        const unsigned blocks = unsigned((count + 255) / 256);
        if (c_bf16) gemm_k0_kernel<true><<<blocks, 256, 0, stream>>>(reinterpret_cast<void *>(c), count, d.alpha, d.beta);
        else gemm_k0_kernel<false><<<blocks, 256, 0, stream>>>(reinterpret_cast<void *>(c), count, d.alpha, d.beta);
        CB_CUDA(cudaGetLastError());
        count_launch();
        return CUTE_B200_OK;
    }
    if (!a || !b) return fail(CUTE_B200_ERR_NULL_POINTER, "gemm_tn: A or B is null");
    if ((a | b) & 15u) return fail(CUTE_B200_ERR_MISALIGNED, "gemm_tn: A and B must be 16-byte aligned");

    if (d.split_k < 0 || d.split_k > 16)
        return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "gemm_tn: split_k must be 0 (choose) to 16, got %d", d.split_k);
    int group = 2, bn = 256, mh = 2, splits = 1;
    // tuning[0] bit 7 keeps a k split in its two-kernel form (measurements, and the test that the two forms agree)
    const bool allow_kc = ex.extra_count == 0 && !(d.tuning[0] & 128);
    choose_tiling(d.m, d.n, d.k, c_bf16 ? 2 : 4, dev.sm_count, d.cta_group, d.tile_n, d.tile_m, d.split_k, 1, 16, allow_kc,
                  &group, &bn, &mh, &splits);

    GemmParams p = {};
    p.C = reinterpret_cast<void *>(c);
    p.M = d.m;
    p.N = d.n;
    p.K = d.k;
    const int ldc = ex.ldc ? ex.ldc : d.n;
    p.ldc = ldc;
    p.alpha = d.alpha;
    p.beta = d.beta;
    p.status = dev.status_word;
    p.debug = d.tuning[0];
    p.group_m = d.tuning[1];
    p.splits = splits;
    p.split_stride = 0;
    p.extra_count = ex.extra_count;
    for (int i = 0; i < ex.extra_count; i++) p.extra_c[i] = reinterpret_cast<void *>(ex.extra_c[i]);
    if (ex.signal && ex.extra_count > 0) {
        p.signal_count = ex.extra_count;
        for (int i = 0; i < ex.extra_count; i++) p.signal[i] = reinterpret_cast<uint32_t *>(ex.signal[i]);
        p.done_counter = dev.status_word + 8;  // words 8.. of the device's 64-byte status block are the library's own counters
    }
    const size_t c_elem = c_bf16 ? 2 : 4;
    p.c_vec_ok = ((c & 15u) == 0 && (size_t(ldc) * c_elem) % 16 == 0) ? 1 : 0;
    if ((c & 31u) == 0 && (size_t(ldc) * c_elem) % 32 == 0) p.c_vec_ok = 2;
    const int cta_rows = mh == 0 ? 64 : BM * mh;
    p.idesc = make_idesc(d.ab_dtype == CUTE_B200_BF16, (mh == 0 ? 64 : BM) * group, bn);

    CUtensorMap tmA, tmB;
    CB_TRY(make_tensor_map(&tmA, a, d.ab_dtype, d.m, d.k, cta_rows));
    CB_TRY(make_tensor_map(&tmB, b, d.ab_dtype, d.n, d.k, bn / group));
    // Several destinations: the pusher warp copies finished tiles by TMA when every C is 16-byte
    // aligned with a 16-byte row pitch; otherwise the epilogue stores to each of them from registers.
    CMaps tmC = {};
    if (p.extra_count > 0 && splits == 1 && ldc == d.n && (c & 15u) == 0 && (size_t(d.n) * c_elem) % 16 == 0 &&
        !(d.tuning[0] & 16)) {
        const int box_rows = push_rows(bn, c_bf16);
        CB_TRY(make_tensor_map_c(&tmC.m[0], c, c_bf16, d.m, d.n, bn, box_rows));
        for (int i = 0; i < p.extra_count; i++)
            CB_TRY(make_tensor_map_c(&tmC.m[i + 1], reinterpret_cast<uint64_t>(p.extra_c[i]), c_bf16, d.m, d.n, bn, box_rows));
        p.push = 1;
    }

    // A split in two or four of single-CTA 128-row tiles can be summed inside the kernel: the CTAs of a
    // cluster take a tile's k ranges and add their partial sums through shared memory.
    if (allow_kc && kc_applies(d.m, d.n, group, bn, mh, splits, dev.sm_count)) {
        p.kc = splits;
#define CB_CASE(G, N_, H, BF) \
    if (G == 1 && H == 1 && bn == N_ && c_bf16 == BF) return launch<G, N_, H, BF>(tmA, tmB, tmC, p, dev.sm_count, stream);
        CB_GEMM_VARIANTS(CB_CASE)
#undef CB_CASE
    }
    if (splits > 1) {
        // First pass: every k range writes an f32 plane of partial sums into the
        // library's scratch buffer; second pass adds the planes and applies the
        // epilogue.  The scratch is allocated on first need and kept.
        const size_t plane = size_t(d.m) * d.n;
        void *scratch = nullptr;
        CB_TRY(scratch_acquire(plane * 4 * splits, stream, &scratch));
        GemmParams q = p;
        q.C = scratch;
        q.alpha = 1.0f;
        q.beta = 0.0f;
        q.split_stride = plane * 4;
        q.c_vec_ok = (size_t(d.n) * 4) % 32 == 0 ? 2 : ((size_t(d.n) * 4) % 16 == 0 ? 1 : 0);
        cute_b200_status st = CUTE_B200_ERR_UNSUPPORTED;
#define CB_CASE(G, N_, H, BF) \
    if (group == G && bn == N_ && mh == H && !BF) st = launch<G, N_, H, false>(tmA, tmB, tmC, q, dev.sm_count, stream);
        CB_GEMM_VARIANTS(CB_CASE)
#undef CB_CASE
        CB_TRY(st);
        // The second pass is a programmatic dependent of the first: it is scheduled while the first still
        // runs and waits (griddepcontrol.wait) for the planes, which hides its launch behind the first pass.
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(unsigned((plane + 1023) / 1024));
        cfg.blockDim = dim3(256);
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = (d.tuning[0] & 32) ? 0 : 1;  // bit 5: plain stream order (measurements)
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        const float *planes = static_cast<const float *>(scratch);
        if (c_bf16) CB_CUDA(cudaLaunchKernelEx(&cfg, gemm_splitk_reduce<true>, planes, splits, plane, plane, p.C, d.alpha, d.beta));
        else CB_CUDA(cudaLaunchKernelEx(&cfg, gemm_splitk_reduce<false>, planes, splits, plane, plane, p.C, d.alpha, d.beta));
        count_launch();
        return scratch_release(stream);
    }
#define CB_CASE(G, N_, H, BF) \
    if (group == G && bn == N_ && mh == H && c_bf16 == BF) return launch<G, N_, H, BF>(tmA, tmB, tmC, p, dev.sm_count, stream);
    CB_GEMM_VARIANTS(CB_CASE)
#undef CB_CASE
    return fail(CUTE_B200_ERR_UNSUPPORTED, "gemm_tn: no kernel for cta_group %d, tile %d x %d", group, cta_rows, bn);
}

cute_b200_status gemm_plan(const cute_b200_gemm_desc &d, int sm_count, int32_t out[4]) {
    if (d.m <= 0 || d.n <= 0 || d.k <= 0) return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "gemm_plan: invalid size %dx%dx%d", d.m, d.n, d.k);
    if (sm_count <= 0) sm_count = 148;
    int group = 2, bn = 256, mh = 2, splits = 1;
    choose_tiling(d.m, d.n, d.k, d.c_dtype == CUTE_B200_BF16 ? 2 : 4, sm_count, d.cta_group, d.tile_n, d.tile_m, d.split_k, 1, 16,
                  !(d.tuning[0] & 128), &group, &bn, &mh, &splits);
    out[0] = group, out[1] = bn, out[2] = mh == 0 ? 64 : 128 * mh, out[3] = splits;
    return CUTE_B200_OK;
}

template <int CTA_GROUP, int BN, int MH>
static void fill_layout(bool ab_bf16, bool c_bf16, uint32_t smem_addr, cute_b200_gemm_layout *o) {
    using C = Cfg<CTA_GROUP, BN, MH>;
    o->instruction_descriptor = make_idesc(ab_bf16, C::UMMA_M, BN);
    o->umma_m = C::UMMA_M, o->umma_n = BN, o->umma_k = UMMA_K;
    o->block_k = BK;
    o->cta_rows = C::A_ROWS;
    o->a_block_bytes = C::A_BYTES, o->b_block_bytes = C::B_BYTES, o->k_blocks_per_stage = C::KPS;
    o->stage_bytes = C::STAGE_BYTES, o->stages = C::STAGES;
    o->accumulator_halves = C::HALVES, o->half_columns = C::HALF_COLS, o->accumulator_buffers = C::ACC_BUFS;
    o->tmem_columns = C::TMEM_COLS;
    o->threads = num_threads(BN, MH), o->epilogue_warps = 4 * epilogue_groups(BN, MH);
    o->full_arrivals = C::FULL_ARRIVALS, o->empty_arrivals = C::EMPTY_ARRIVALS, o->tmem_full_arrivals = C::TFULL_ARRIVALS;
    o->tmem_empty_arrivals = C::TEMPTY_ARRIVALS;
    o->full_expect_tx_bytes_per_k_block = C::EXPECT_TX_PER_KB;
    o->push_chunk_bytes = PUSH_BUF_BYTES, o->push_chunk_rows = push_rows(BN, c_bf16);
    o->push_chunks_per_tile = C::A_ROWS / push_rows(BN, c_bf16);
    o->shared_memory_bytes = C::SMEM_BYTES;
    o->descriptor_k_step = DESC_K_STEP;
    o->smem_descriptor = sw128_desc(smem_addr);
}

cute_b200_status gemm_layout_info(int cta_group, int tile_n, int tile_m, int ab_dtype, int c_dtype, uint32_t smem_addr,
                                  cute_b200_gemm_layout *out) {
    if (!out) return fail(CUTE_B200_ERR_NULL_POINTER, "gemm_layout_info: null output");
    if ((ab_dtype != CUTE_B200_F16 && ab_dtype != CUTE_B200_BF16) || (c_dtype != CUTE_B200_F32 && c_dtype != CUTE_B200_BF16))
        return fail(CUTE_B200_ERR_INVALID_ARGUMENT, "gemm_layout_info: f16/bf16 inputs and f32/bf16 output only");
    const int mh = tile_m == 64 ? 0 : tile_m / 128;
    *out = cute_b200_gemm_layout{};
#define CB_CASE(G, N_, H, BF)                                                                       \
    if (cta_group == G && tile_n == N_ && mh == H && !BF && (tile_m == 64 || tile_m == 128 * H)) { \
        fill_layout<G, N_, H>(ab_dtype == CUTE_B200_BF16, c_dtype == CUTE_B200_BF16, smem_addr, out); \
        return CUTE_B200_OK;                                                                        \
    }
    CB_GEMM_VARIANTS(CB_CASE)
#undef CB_CASE
    return fail(CUTE_B200_ERR_UNSUPPORTED, "gemm_layout_info: no kernel for cta_group %d, tile %d x %d", cta_group, tile_m, tile_n);
}

}  // namespace cb
