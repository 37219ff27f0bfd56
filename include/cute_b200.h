/*
 * cute_b200.h - C ABI of libcute_b200.so
 *
 * A B200 (sm_100a) implementation of the kernels the cute-rs crate exists to
 * run: the tensor-core GEMMs `tensorop_gemm` / `runtime_gemm`, the SIMT
 * `sgemm_nt`, and `elementwise_add`.  The library sits beside the crate's
 * CUDA launcher (src/cuda.rs) and takes over the launch of those kernels;
 * everything else keeps going through the crate's own PTX path.
 *
 * Conventions (those of src/cuda.rs, so a Rust shim can bind this 1:1):
 *   - device pointers travel as uint64_t, like `CuDevicePtr` (src/cuda.rs:35);
 *   - the caller owns every buffer; the library owns only cached TMA
 *     descriptors, a small per-device status word and optional workspaces;
 *   - every entry point returns a status code and never throws or aborts;
 *     `cute_b200_last_error()` gives the message a `CudaError` would carry
 *     (src/cuda.rs:71-86, 532-546);
 *   - launches are asynchronous on `stream` (a CUstream/cudaStream_t; NULL is
 *     the legacy default stream the reference launches on, src/cuda.rs:382);
 *   - one host thread per device at a time, no internal locking beyond the
 *     descriptor cache (the reference's types are !Send + !Sync).
 *
 * There is no CPU fallback: without a CUDA device every compute entry point
 * returns CUTE_B200_ERR_NO_DEVICE.
 */
#ifndef CUTE_B200_H
#define CUTE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

typedef int32_t cute_b200_status;

enum {
    CUTE_B200_OK = 0,
    CUTE_B200_ERR_INVALID_ARGUMENT = -1, /* a size, count, dtype or launch shape the kernel cannot take */
    CUTE_B200_ERR_MISALIGNED = -2,       /* a pointer or pitch breaks the 16-byte rule of param_tensor / TMA */
    CUTE_B200_ERR_UNSUPPORTED = -3,      /* a kernel name or option this library does not implement */
    CUTE_B200_ERR_NO_DEVICE = -4,        /* no usable sm_100 device */
    CUTE_B200_ERR_DEVICE_TIMEOUT = -5,   /* a bounded wait inside a kernel gave up; see cute_b200_device_status */
    CUTE_B200_ERR_CUDA = -6,             /* a CUDA runtime/driver call failed; message in cute_b200_last_error */
    CUTE_B200_ERR_NULL_POINTER = -7
};

typedef enum { CUTE_B200_F16 = 0, CUTE_B200_BF16 = 1, CUTE_B200_F32 = 2, CUTE_B200_I32 = 3 } cute_b200_dtype;

/* Static name of a status code.  Counterpart of cuGetErrorName as used by
 * check() in src/cuda.rs:532-546. */
const char *cute_b200_status_string(cute_b200_status status);

/* Message of the calling thread's most recent failure ("" if none), worded
 * like the reference's errors ("argument 3 (`n`) must be a multiple of 128,
 * got 100", src/sim/mod.rs:328-385; "<call> failed: <name>", src/cuda.rs:540). */
const char *cute_b200_last_error(void);

/* Make `device_ordinal` usable by this library on the calling thread: selects
 * the device (its primary context, which CudaContext::new retains too,
 * src/cuda.rs:210-224), checks that it is sm_100, raises the kernels'
 * dynamic shared-memory limit and allocates the status word.  Idempotent.
 * Other entry points call it lazily for the current device. */
cute_b200_status cute_b200_init(int32_t device_ordinal);

/* ---- tensor-core GEMM ------------------------------------------------------
 * C = alpha * (A * B^T) + beta * C
 *   A: (m, k) row-major, k contiguous ("K-major"), f16 or bf16
 *   B: (n, k) row-major, k contiguous, same type as A
 *   C: (m, n) row-major, f32 or bf16
 * f32 accumulation on the tcgen05 tensor cores.  With alpha == 1 and
 * beta == 0 C is write-only, as in tensorop_gemm (examples/tensorop_gemm.rs:
 * 161-162); otherwise the epilogue is the three-rounding form of sgemm
 * (examples/sgemm.rs:75-79).  Replaces the kernels built by
 * tensorop_gemm::build_typed (examples/tensorop_gemm.rs:51-164) and
 * runtime_gemm::build (examples/runtime_gemm.rs:22-105).
 *
 * m, n >= 1; k >= 0 (k == 0 stores the beta term only); k must be a multiple
 * of 8 and A, B 16-byte aligned (TMA row pitch); C needs only the alignment
 * of its element type (16- or 32-byte alignment of its base and row pitch
 * selects the wider stores).
 * The reference's own limits (multiples of 128 / 128 / 32) are enforced by
 * cute_b200_launch, which mirrors its launch checks. */
typedef struct {
    int32_t m, n, k;
    int32_t ab_dtype; /* CUTE_B200_F16 or CUTE_B200_BF16 */
    int32_t c_dtype;  /* CUTE_B200_F32 or CUTE_B200_BF16 */
    float alpha, beta;
    int32_t tile_n;    /* columns of C per tile: 0 = choose; 128 or 256 */
    int32_t cta_group; /* 0 = choose; 1 = one CTA per tile; 2 = a CTA pair shares each tile's MMAs */
    int32_t tile_m;    /* rows of C per CTA: 0 = choose; 128 or 256; 64 = the pair tile for few row tiles and a long
                          k (needs cta_group 0 or 2): 16 KiB stages, a 12-deep ring */
    int32_t split_k;   /* k ranges computed as separate work units and summed in ascending order, either inside the
                          kernel (single-CTA 128-row tiles cut in two or four ranges that fit one wave: the CTAs of a
                          cluster take a tile's ranges and add their partial sums through shared memory) or by a second
                          kernel through an f32 scratch buffer the library allocates on first need - the same sums in
                          the same order, hence the same bits: 0 = choose, 1 = never,
                          2..16 = exactly that many (cut down to the number of 64-wide k blocks when k is shorter;
                          ranges left without a block contribute zeros).  The scratch is one buffer per device shared
                          by all streams: the library orders split launches on different streams one behind the
                          other with an event, so they do not race, but they do not overlap either */
    int32_t tuning[2]; /* zero.  Measurement and test knobs: [0] bit 0 skips the loads, bit 1 the stores (results
                          are then meaningless), bits 2+3 make every in-kernel wait run out after 20 ms so that
                          the bounded-wait report can be tested, bit 4 makes cute_b200_gemm_tn_multi store to its
                          destinations from registers instead of by TMA, bit 5 queues the GEMM's kernels in plain
                          stream order instead of as programmatic dependents of the kernel before them,
                          bit 7 keeps every k split in its two-kernel form;
                          [1] row tiles walked per column step */
} cute_b200_gemm_desc;

cute_b200_status cute_b200_gemm_tn(const cute_b200_gemm_desc *desc, uint64_t dA, uint64_t dB, uint64_t dC,
                                   void *stream);

/* The same GEMM on HOST buffers, the convention of CudaContext::launch
 * (src/cuda.rs:443-473): A and B are uploaded, the kernel runs, the call waits
 * and C is copied back (C is uploaded first only when beta != 0).  Device
 * staging memory is kept by the library between calls and grows on demand;
 * cute_b200_release_workspace frees it.  Pinned host memory makes the copies
 * faster but is not required.  `seconds`, if not NULL, receives the kernel's
 * device time. */
cute_b200_status cute_b200_gemm_tn_host(const cute_b200_gemm_desc *desc, const void *hA, const void *hB, void *hC,
                                        double *seconds);
cute_b200_status cute_b200_release_workspace(void);

/* The split-k GEMM for callers that must not allocate device memory.  It has
 * no counterpart in the reference crate.
 *
 * Who needs it: a process whose GPU memory is handed out by a pool it does not
 * control (an inference server with a fixed memory budget, a framework that
 * forbids raw cudaMalloc), a latency-critical loop that cannot afford the
 * device-wide synchronisation cudaMalloc and cudaFree imply, or code that is
 * already inside a region where allocation is not permitted.  For them the
 * ordinary entry point is unsuitable as soon as the library decides to split
 * k, because that path creates its scratch buffer on first need.
 *
 * This variant computes the same result (the tiling comes from the same cost
 * model and the k ranges are added in the same order, so with the same
 * split_k >= 2 it returns the same bits as cute_b200_gemm_tn; with split_k = 0
 * the ordinary entry point may decide not to split at all, this one always
 * uses at least two ranges) but takes its scratch from a 32 MiB array that is
 * part of the library image.  Every GPU that loads the library holds those 32 MiB until
 * the process exits.  It calls no cudaMalloc, cudaFree or other allocating
 * routine, and it does not need cute_b200_init.
 *
 *   - split_k: 0 = choose, or 2..16; 1 is rejected (use cute_b200_gemm_tn).
 *   - limit: m * n * 4 bytes * split_k must fit in 32 MiB (33 554 432 bytes),
 *     e.g. 8192 x 128 in up to 8 ranges, 1024 x 1024 in up to 8; larger requests
 *     return CUTE_B200_ERR_INVALID_ARGUMENT with the sizes in the message.
 *     k must exceed 64 (two 64-wide k blocks are the least that can be split).
 *   - the first call on each device resolves the array's device address and
 *     raises the kernels' shared-memory limit (no allocation either); make that
 *     first call before any stream capture begins.
 *   - all calls share the one array and it keeps the previous call's partial
 *     sums; every element a call reads was written by that same call, so
 *     nothing needs clearing, but two calls whose kernels overlap on the GPU
 *     (different streams, or concurrent host threads) race on it.  Serialise
 *     them on one stream or with events.
 *   - a bounded-wait report goes to the device's usual status word when the
 *     device was set up with cute_b200_init, else to words owned by this entry
 *     point; cute_b200_synchronize and cute_b200_device_status read (and
 *     clear) either without allocating anything. */
cute_b200_status cute_b200_gemm_tn_static(const cute_b200_gemm_desc *desc, uint64_t dA, uint64_t dB, uint64_t dC,
                                          void *stream);

/* ---- SIMT sgemm ------------------------------------------------------------
 * C = alpha * (A * B^T) + beta * C, all f32 and column-major: a[i + l*m],
 * b[j + l*n], c[i + j*m].  fma.rn.f32 accumulation with l ascending and a
 * mul, mul, add epilogue, so the result is bit-identical to the reference
 * kernel's (examples/sgemm.rs:23-81).  m and n multiples of 128, k >= 0. */
cute_b200_status cute_b200_sgemm_nt(int32_t m, int32_t n, int32_t k, float alpha, float beta, uint64_t dA,
                                    uint64_t dB, uint64_t dC, void *stream);

/* ---- elementwise add -------------------------------------------------------
 * out[i] = x[i] + y[i] for i < n, IEEE binary32, no flush to zero; elements
 * at and past n are not touched.  Replaces elementwise_add::{naive, tiled}
 * (examples/elementwise_add.rs:23-80).  Pointers need 4-byte alignment; the
 * 128-bit path runs when all three share their offset within 16 bytes. */
cute_b200_status cute_b200_elementwise_add_f32(uint64_t dX, uint64_t dY, uint64_t dOut, uint64_t n, void *stream);

/* ---- launch by kernel name -------------------------------------------------
 * Counterpart of CudaContext::launch_on_device (src/cuda.rs:414-426): the
 * arguments in declaration order, one slot each, plus the launch shape.  The
 * checks of check_launch (src/sim/mod.rs:328-385) are applied with the same
 * messages: argument count, block size, grid/cluster divisibility, the block
 * size the kernel was built for, buffer dtype and length, scalar multiples.
 * Problem sizes follow from the grid and the buffer lengths exactly as the
 * reference kernels derive them.  Known names: tensorop_gemm,
 * tensorop_gemm_unswizzled, tensorop_gemm_bf16, tensorop_gemm_bf16_unswizzled
 * (a, b, c), runtime_gemm (a, b, c, n, k), sgemm_nt (a, b, c, alpha, beta),
 * elementwise_add_naive, elementwise_add_tiled (a, b, c). */
typedef struct {
    int32_t is_scalar; /* 0 = buffer, 1 = scalar */
    int32_t dtype;     /* cute_b200_dtype of the elements / the scalar */
    uint64_t value;    /* device pointer, or the scalar's bits in the low bytes (src/cuda.rs:332-349) */
    uint64_t len;      /* buffers: number of elements */
} cute_b200_arg;

typedef struct {
    uint32_t grid[3], block[3], cluster[3]; /* LaunchConfig, src/sim/mod.rs:41-61 */
} cute_b200_launch_config;

cute_b200_status cute_b200_launch(const char *kernel_name, const cute_b200_launch_config *cfg,
                                  const cute_b200_arg *args, int32_t num_args, void *stream);

/* Counterpart of CudaContext::launch (src/cuda.rs:443-473): buffer arguments
 * hold HOST pointers; every buffer is uploaded, the kernel runs, the call
 * waits for it, and every buffer is copied back in place.  `seconds`, if not
 * NULL, receives the kernel's device time (LaunchStats.kernel_seconds,
 * src/cuda.rs:65-69), measured with CUDA events. */
cute_b200_status cute_b200_launch_host(const char *kernel_name, const cute_b200_launch_config *cfg,
                                       const cute_b200_arg *args, int32_t num_args, double *seconds);

/* ---- device buffers (CudaContext::upload / download / DeviceBuffer drop,
 * src/cuda.rs:282-304, 491-502) ------------------------------------------- */
cute_b200_status cute_b200_upload(const void *host, uint64_t bytes, uint64_t *device_out);
cute_b200_status cute_b200_download(uint64_t device, void *host, uint64_t bytes);
cute_b200_status cute_b200_free(uint64_t device);
/* CudaContext::synchronize (src/cuda.rs:306-311); also folds a kernel's
 * bounded-wait report into the return value. */
cute_b200_status cute_b200_synchronize(void);

/* ---- row-sharded GEMM for several GPUs ------------------------------------
 * One process (or thread) per GPU.  Rank r of `world` owns the contiguous
 * row block [row_begin, row_begin + rows) of A and C; B is whole in every
 * GPU's own memory.  No data crosses between GPUs here: a caller that wants
 * C replicated all-gathers the row blocks afterwards (NCCL).  The reference
 * has no multi-GPU path; this extends its launcher. */
cute_b200_status cute_b200_shard_rows(int32_t m, int32_t world, int32_t rank, int32_t *row_begin, int32_t *rows);
/* desc->m is the GLOBAL row count; dA_shard points at this rank's rows of A,
 * dC_base at row 0 of a full-size C (c_is_full != 0) or at this rank's block. */
cute_b200_status cute_b200_gemm_tn_shard(const cute_b200_gemm_desc *desc, int32_t world, int32_t rank,
                                         uint64_t dA_shard, uint64_t dB, uint64_t dC_base, int32_t c_is_full,
                                         void *stream);

/* ---- peer memory for the replicated result --------------------------------
 * One process per GPU: to let a GPU write its rows of C straight into the
 * other GPUs' copies over NVLink, every process allocates its C with
 * cute_b200_alloc, exports it, and opens the others' handles (CUDA IPC; the
 * 64-byte handles travel over whatever channel the caller has, e.g. the
 * torch.distributed store).  cute_b200_copy_async is a device-to-device copy
 * on a stream (copy engines, no SM), local or to a peer mapping.
 * cute_b200_alloc makes every buffer above 2 MiB a whole number of 2 MiB
 * (see cute_b200_gemm_tn_multi for why).  No counterpart in the reference
 * (single GPU). */
cute_b200_status cute_b200_alloc(uint64_t bytes, uint64_t *device_out);
cute_b200_status cute_b200_ipc_export(uint64_t device, uint8_t handle_out[64]);
cute_b200_status cute_b200_ipc_open(const uint8_t handle[64], uint64_t *device_out);
cute_b200_status cute_b200_ipc_close(uint64_t device);
cute_b200_status cute_b200_copy_async(uint64_t dst, uint64_t src, uint64_t bytes, void *stream);

/* The GEMM with its result written to several copies of C at once: dC_list[0]
 * is normally this GPU's C, the others are peer mappings of the same rows in
 * other GPUs' C (cute_b200_ipc_open).  The epilogue stores every tile to the
 * first; a further warp of each CTA then copies the finished tile from there
 * (it is still in L2) to every other destination with TMA loads and bulk
 * tensor stores, while the tensor cores work on the next tiles: compute and
 * collective in one kernel, no NCCL call.  That form needs every C 16-byte
 * aligned with a row pitch that is a multiple of 16 bytes; otherwise the
 * epilogue warps store to all destinations from registers (slower over
 * NVLink).  alpha must be 1 and beta 0; no k split; 1 <= count <= 8; every
 * destination aligned like the first (same offset within 32 bytes).  The
 * caller makes the result visible to the peers the usual way (stream
 * synchronisation followed by a barrier among the processes).  Measured: a
 * destination exported by CUDA IPC should be an allocation whose size is a
 * whole number of 2 MiB (2 GiB + 256 bytes in one allocation made the stores
 * of eight GPUs into one another more than twice as slow as 2 GiB).  No
 * counterpart in the reference. */
cute_b200_status cute_b200_gemm_tn_multi(const cute_b200_gemm_desc *desc, uint64_t dA, uint64_t dB,
                                         const uint64_t *dC_list, int32_t count, void *stream);

/* The same with a completion signal in place of a barrier among the processes.
 * dSignal_list[i], i >= 1, is the address (as this process sees it, e.g. a
 * cute_b200_ipc_open mapping) of a 32-bit counter in the memory of the GPU
 * that owns dC_list[i]; entry 0 is ignored.  When every CTA of the launch has
 * finished - all stores to the first C and all stores to every other
 * destination complete - the last CTA adds 1 to each counter (release, system
 * scope).  The owner of a destination learns that its copy of these rows is
 * complete by waiting for its counters: cute_b200_wait_signal queues a
 * one-thread kernel on `stream` that polls the 32-bit counters dSignals[i]
 * for every bit i set in `mask` (acquire, system scope) until each has reached
 * `at_least` (compared as wrapping counts) or `timeout_ms` has passed; running
 * out is reported like every other bounded wait ({7, at_least, index of the
 * counter that was short, its value} in cute_b200_device_status,
 * CUTE_B200_ERR_DEVICE_TIMEOUT from cute_b200_synchronize), and the device
 * stays usable.  The intended use is one counter per sender in every
 * receiver's memory, each growing by one per step, so that a sender that runs
 * a step ahead cannot be mistaken for one that is a step behind.  Counters are
 * never reset by the library; the caller zeroes them once (cute_b200_alloc
 * does not).  k must be positive; one signalling launch at a time per device
 * (they share the device's count of finished CTAs).  No host synchronisation
 * and no collective call is needed on the step.  No counterpart in the
 * reference. */
cute_b200_status cute_b200_gemm_tn_multi_signal(const cute_b200_gemm_desc *desc, uint64_t dA, uint64_t dB,
                                                const uint64_t *dC_list, const uint64_t *dSignal_list, int32_t count,
                                                void *stream);
cute_b200_status cute_b200_wait_signal(uint64_t dSignals, uint32_t mask, uint32_t at_least, uint32_t timeout_ms,
                                       void *stream);

/* ---- one call for all the GPUs of a box -------------------------------------
 * The launcher next to CudaContext::launch (src/cuda.rs:443-473) for a GEMM too
 * large, or too urgent, for one GPU: ONE process drives `ngpus` devices, one
 * host thread and one set of streams each, with peer access enabled between
 * every pair.  GPU g of the communicator owns the row block
 * cute_b200_shard_rows(desc->m, ngpus, g) of A and C; B is whole in every
 * GPU's memory; no data crosses between GPUs while the blocks are computed.
 * Both calls return when every GPU has finished (like launch: buffers in, a
 * wait, buffers back), with the first failure of any GPU as the status and its
 * message in cute_b200_last_error ("GPU 3 (device 3): ...", worded like
 * src/cuda.rs:532-546).  One call at a time per communicator; the reference has
 * no multi-GPU path, this extends its launcher.
 *
 * cute_b200_comm_create: `ordinals` NULL means devices 0 .. ngpus-1; at most 8.
 * A device may be named more than once (its blocks are then computed one after
 * the other on that device; useful to run a partition meant for more GPUs than
 * are present).  cute_b200_comm_info: out = {ngpus, all devices distinct, peer
 * access between every pair, collective library loadable}.
 *
 * cute_b200_gemm_tn_sharded (device buffers, one pointer per GPU, each in that
 * GPU's memory): dA_shard[g] = GPU g's rows of A, dB[g] = all of B.  With
 * replicate_c == CUTE_B200_REPLICATE_NONE, dC[g] is GPU g's row block of C.
 * Otherwise dC[g] is a FULL (m, n) C on GPU g and every GPU ends up with all
 * of it:
 *   CUTE_B200_REPLICATE_FUSED       the GEMM kernel's pusher warp stores each
 *       finished tile into the peers' C over NVLink while the tensor cores go
 *       on (cute_b200_gemm_tn_multi); needs alpha 1, beta 0, peer access;
 *   CUTE_B200_REPLICATE_COLLECTIVE  GEMM into the own block, then ncclAllGather
 *       (ncclBroadcast per block when the blocks are uneven); NCCL is loaded
 *       with dlopen("libnccl.so.2") on first need, as the reference loads
 *       libcuda (src/cuda.rs:88-196);
 *   CUTE_B200_REPLICATE_COPIES      GEMM, then one device-to-device copy of the
 *       block per peer;
 *   CUTE_B200_REPLICATE_AUTO        FUSED when it applies and every C takes the
 *       TMA stores (16-byte aligned base and row pitch), else COLLECTIVE when
 *       NCCL is there, else COPIES.
 *
 * cute_b200_gemm_tn_sharded_host (host buffers, the convention of
 * CudaContext::launch): hA (m, k), hB (n, k) and hC (m, n) are whole matrices
 * in host memory (pinned memory makes the copies faster).  Every GPU uploads
 * its rows of A and only 1/ngpus of B's rows, and passes what it fetched of B
 * on to the other GPUs by device-to-device copies over NVLink.  The way back
 * to hC is the longest leg, so it starts early: from 8192 columns on, C is cut
 * into blocks of about 4096 columns and B goes up block by block; the first
 * block is multiplied panel by panel of A's rows as they arrive, the later
 * ones as soon as their rows of B are complete, and every finished block of C
 * goes back to hC while the following uploads and products run ahead.  hC is
 * read first only when beta != 0.  Staging memory is kept by the communicator.
 * `seconds`, if not NULL, receives the duration of the call. */
enum {
    CUTE_B200_REPLICATE_NONE = 0,
    CUTE_B200_REPLICATE_AUTO = 1,
    CUTE_B200_REPLICATE_FUSED = 2,
    CUTE_B200_REPLICATE_COLLECTIVE = 3,
    CUTE_B200_REPLICATE_COPIES = 4
};
cute_b200_status cute_b200_comm_create(int32_t ngpus, const int32_t *ordinals, void **comm_out);
cute_b200_status cute_b200_comm_destroy(void *comm);
cute_b200_status cute_b200_comm_info(void *comm, int32_t out[4]);
cute_b200_status cute_b200_gemm_tn_sharded(void *comm, const cute_b200_gemm_desc *desc, const uint64_t *dA_shard,
                                           const uint64_t *dB, const uint64_t *dC, int32_t replicate_c);
cute_b200_status cute_b200_gemm_tn_sharded_host(void *comm, const cute_b200_gemm_desc *desc, const void *hA, const void *hB,
                                                void *hC, double *seconds);

/* ---- bounded waits ----------------------------------------------------------
 * Every spin on an mbarrier inside the GEMM kernel has a time limit.  A CTA
 * that gives up records {code, role/stage, block index, parity} here and the
 * kernel drains and returns instead of hanging.  Reads and clears the word
 * of the current device (synchronises the device).  out[0] == 0: no report. */
cute_b200_status cute_b200_device_status(uint32_t out[4]);

/* ---- what the compiled GEMM kernel is built from ------------------------------
 * The constants of one tiling (cta_group 1 or 2, tile_n 128 or 256, tile_m 64,
 * 128 or 256, the operand and result types), produced by the very expressions
 * the kernel is compiled from: the tcgen05.mma instruction descriptor, the
 * shared-memory matrix descriptor of a 128-byte-swizzled tile at `smem_addr`,
 * the bytes and depth of the TMA ring, the accumulators' place in TMEM, the
 * arrival and transaction counts of the pipeline's mbarriers and the pusher's
 * chunk shape.  Host arithmetic only (works without a GPU).  It lets the
 * Sm100 atoms (the form in which src/atom would describe this kernel, cf.
 * src/atom/mma.rs:148-198, src/atom/copy.rs:46-90) and the protocol checker be
 * held against the kernel as it is built rather than against a copy of its
 * numbers.  No counterpart in the reference. */
typedef struct {
    uint32_t instruction_descriptor;
    uint32_t umma_m, umma_n, umma_k; /* shape of one tcgen05.mma over the CTA group */
    uint32_t block_k;                /* k per k block: one 128-byte swizzle row of 16-bit values */
    uint32_t cta_rows;               /* rows of C per CTA */
    uint32_t a_block_bytes, b_block_bytes; /* one k block of this CTA's rows of A / of B */
    uint32_t k_blocks_per_stage;     /* k blocks behind one pair of full/empty barriers */
    uint32_t stage_bytes, stages;
    uint32_t accumulator_halves;     /* 128-lane accumulators per CTA */
    uint32_t half_columns;           /* TMEM columns of one of them */
    uint32_t accumulator_buffers;    /* 2 = the epilogue overlaps the next tile's main loop */
    uint32_t tmem_columns;           /* allocated */
    uint32_t threads, epilogue_warps;
    uint32_t full_arrivals, empty_arrivals, tmem_full_arrivals, tmem_empty_arrivals;
    uint32_t full_expect_tx_bytes_per_k_block; /* announced on the (leader's) full barrier for every k block a stage holds */
    uint32_t push_chunk_bytes, push_chunk_rows, push_chunks_per_tile;
    uint32_t shared_memory_bytes;
    uint32_t descriptor_k_step;      /* added to a descriptor's address field per umma_k */
    uint64_t smem_descriptor;
} cute_b200_gemm_layout;

cute_b200_status cute_b200_gemm_layout_info(int32_t cta_group, int32_t tile_n, int32_t tile_m, int32_t ab_dtype,
                                            int32_t c_dtype, uint32_t smem_addr, cute_b200_gemm_layout *out);

/* Which tiling cute_b200_gemm_tn would run `desc` with on a GPU of `sm_count` SMs (0 = 148, a B200):
 * out = {cta_group, tile_n, tile_m, split_k}.  Fields of `desc` that are not zero are kept.  Host
 * arithmetic only (works without a GPU).  No counterpart in the reference, whose tiling is fixed
 * by the kernel's source (examples/tensorop_gemm.rs:36-39). */
cute_b200_status cute_b200_gemm_plan(const cute_b200_gemm_desc *desc, int32_t sm_count, int32_t out[4]);

/* Number of kernels this library has launched from the calling process. */
uint64_t cute_b200_launch_count(void);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* CUTE_B200_H */
