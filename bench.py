#!/usr/bin/env python
"""Benchmark of the cute-rs hot path on B200: bf16 GEMM TFLOP/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

N = 1  : runtime_gemm, bf16 in / bf16 out, 8192 x 8192 x 8192, normal(0, 0.02)
         inputs, alpha 1, beta 0 - one step is one GEMM launch.
N > 1  : (launched by torchrun, one rank per GPU) the row-sharded GEMM
         32768 x 32768 x 8192: rank r computes its contiguous block of rows of
         C from its rows of A and a full copy of B in its own memory; no
         collective on the data path (the optional all-gather of C is timed
         separately and reported under "replicated").

`value` is the whole-job TFLOP/s with operands resident in HBM, timed with
CUDA events on the launching stream (max over ranks).  `e2e` is the same
metric through the host-buffer C-ABI call with the host<->device copies inside
the timed region: cute_b200_gemm_tn_host on one GPU; on N > 1 the launcher for
all the GPUs of the box, cute_b200_gemm_tn_sharded_host, which is one process
driving every GPU - rank 0 makes that call while the other ranks wait on a
host-side barrier with their GPUs idle.  `roofline` compares the dominant
kernel with the measured cuBLAS bf16 throughput of the same kind of GPU;
`cpu_baseline` times the CPU oracle on the host cores.  `parity` entries
compare bands of rows of the results with the oracle (outside every timed
region) under the reference's bound for tensor-core results plus one bf16 unit
in the last place.  `--impl reference` times the reference's CPU arithmetic (the oracle:
the reference itself is Rust and cannot be built in this image) on a bounded
sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "bf16_gemm_tflops"
UNIT = "TFLOP/s"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# DRAM bytes (read + write) of one 8192^3 bf16->bf16 launch of gemm_tn_kernel as one ncu capture
# measured them (dram__bytes_read.sum 822.7 MB + dram__bytes_write.sum 120.9 MB): a constant taken
# from that capture, not re-measured by this program.
NCU_TRAFFIC_8192 = 943.6e6


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        p["_source"] = "measured"
        return p
    p = dict(FALLBACK_PEAKS)
    p["_source"] = "fallback"
    return p


def workload(n_gpus: int):
    if n_gpus == 1:
        return dict(name="runtime_gemm bf16 8192x8192x8192 (normal(0,0.02) seed 3, alpha=1, beta=0, bf16 C)",
                    m=8192, n=8192, k=8192, seed=3)
    return dict(name="row-sharded bf16 GEMM 32768x32768x8192 (normal(0,0.02) seed 4, bf16 C, B replicated)",
                m=32768, n=32768, k=8192, seed=4)


def gen_b(torch, w, device="cuda"):
    g = torch.Generator(device=device).manual_seed(w["seed"])
    return (torch.randn(w["n"], w["k"], device=device, generator=g) * 0.02).bfloat16()  # the same on every rank


def gen_a_rows(torch, w, rank, rows, device="cuda"):
    """Rank `rank`'s rows of A: a stream of its own, so that any rank can rebuild any other's rows."""
    g = torch.Generator(device=device).manual_seed(w["seed"] * 1000 + rank)
    return (torch.randn(rows, w["k"], device=device, generator=g) * 0.02).bfloat16()


class BandCheck:
    """Oracle results for a few bands of rows of C = A B^T (bf16 in, bf16 out), computed once
    and compared with any number of candidate results.  The bound is the reference's for
    tensor-core results (tests/gpu.rs:146-176: 2 k 2^-23 sum|a b| per element) plus one bf16
    unit in the last place for the final rounding.  The oracle is the checker only and runs
    outside every timed region."""

    def __init__(self, a_rows, b_bits, bands, k):
        import numpy as np
        import oracle
        self.np, self.oracle, self.bands, self.k = np, oracle, bands, k
        self.want, self.allowed = [], []
        for lo, hi in bands:
            acc = oracle.gemm_tn(a_rows, b_bits, oracle.BF16, rows=(lo, hi))[lo:hi]
            mag = oracle.gemm_tn_abs(a_rows, b_bits, oracle.BF16, rows=(lo, hi))[lo:hi]
            ulp = 2.0 ** (np.floor(np.log2(np.maximum(np.abs(acc.astype(np.float64)), 2.0 ** -126))) - 7)
            self.want.append(acc.astype(np.float64))
            self.allowed.append(2.0 * k * 2.0 ** -23 * mag.astype(np.float64) + ulp)

    def check(self, c_rows_bits, row_offset=0):
        """c_rows_bits: uint16 (rows, n) array holding (at least) the bands, whose row 0 is row `row_offset` of the block."""
        np, worst, rows = self.np, -1.0, 0
        for (lo, hi), want, allowed in zip(self.bands, self.want, self.allowed):
            got = self.oracle.bf16_bits_to_f32(c_rows_bits[lo - row_offset:hi - row_offset]).astype(np.float64)
            worst = max(worst, float((np.abs(got - want) - allowed).max()))
            rows += hi - lo
        return {"rows_checked": rows, "max_excess": worst, "ok": bool(worst <= 0.0)}


def band_bits(torch, c, bands):
    """The bands of a device (rows, n) bf16 tensor as one uint16 host array per band, stacked with their offsets kept."""
    import numpy as np
    lo0 = bands[0][0]
    hi1 = bands[-1][1]
    out = np.zeros((hi1 - lo0, c.shape[1]), np.uint16)
    for lo, hi in bands:
        out[lo - lo0:hi - lo0] = c[lo:hi].view(torch.int16).cpu().numpy().view(np.uint16)
    return out, lo0


def three_bands(rows, height=32):
    if rows <= 3 * height:
        return [(0, rows)]
    mid = (rows // 2) // 8 * 8
    return [(0, height), (mid, mid + height), (rows - height, rows)]


def to_bits(torch, t):
    import numpy as np
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while a region runs."""

    def __init__(self, index: int):
        self.samples, self.power, self.reasons, self.max_mhz, self.power_limit = [], [], set(), None, None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            try:
                self.power_limit = pynvml.nvmlDeviceGetEnforcedPowerLimit(self.h) / 1000.0
            except Exception:
                pass
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {"hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
                 "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                 "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                 "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
                 "hw_power_brake": getattr(nv, "nvmlClocksEventReasonHwPowerBrakeSlowdown", 0x80)}
        get = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    self.power.append(nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0)
                except Exception:
                    pass
                mask = get(self.h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.002)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread:
            self._thread.join()

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "samples": len(self.samples), "reasons": sorted(self.reasons),
                "power_w": max(self.power) if self.power else None, "power_limit_w": self.power_limit}


def run_reference(args):
    """The reference's CPU path (restated: the oracle) on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np
    import oracle
    oracle.use_all_cores()
    w = workload(args.gpus)
    rows = 1024 if args.gpus == 1 else 256  # bounded sample: a band of rows of the same GEMM
    rng = np.random.default_rng(w["seed"])
    a = oracle.f32_to_bf16_bits(rng.normal(0, 0.02, (rows, w["k"])).astype(np.float32))
    b = oracle.f32_to_bf16_bits(rng.normal(0, 0.02, (w["n"], w["k"])).astype(np.float32))
    flop = 2.0 * rows * w["n"] * w["k"]
    for _ in range(min(args.warmup, 2)):
        oracle.gemm_tn(a, b, oracle.BF16, oracle.BF16)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.gemm_tn(a, b, oracle.BF16, oracle.BF16)
    dt = (time.perf_counter() - t0) / args.steps
    value = flop / dt / 1e12
    sample = f"{rows} of {w['m']} rows of C per step (full n, k); the oracle's blocked sequential-k f32 GEMM incl. its bf16->f32 packing"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak" if args.gpus == 1 else "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": w["name"]},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": oracle.num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "reference = C restatement of Kernel::simulate's arithmetic (oracle/); the Rust crate cannot be built here",
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--skip-extras", action="store_true", help="skip cpu_baseline / e2e / secondary kernels (profiling runs)")
    ap.add_argument("--only", choices=["add", "sgemm", "multi", "gemm"],
                    help="run just this secondary kernel (for ncu captures) and exit; multi = the several-destination GEMM "
                         "with its copies of C on this one GPU; gemm = runtime_gemm bf16 -> bf16 of --shape")
    ap.add_argument("--shape", default="8192,128,8192", help="--only gemm: m,n,k")
    ap.add_argument("--tiling", default="0,0,0,0", help="--only gemm: cta_group,tile_n,tile_m,split_k (0 = the library chooses)")
    ap.add_argument("--log2n", type=int, default=28, help="--only add: log2 of the element count")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import torch.distributed as dist
    from cute_rs_b200 import _lib as lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback")
    torch.cuda.set_device(local_rank)
    lib.init(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    if args.only:
        if args.only == "add":
            res = bench_add(lib, torch, peaks(), 1 << args.log2n)
        elif args.only == "sgemm":
            res = bench_sgemm(lib, torch)
        elif args.only == "gemm":
            res = bench_gemm_shape(lib, torch, [int(x) for x in args.shape.split(",")], [int(x) for x in args.tiling.split(",")],
                                   max(args.steps, 1) if args.steps != 100 else 20, peaks())
        else:
            res = bench_multi(lib, torch)
        print(json.dumps(res))
        return

    w = workload(world)
    M, N, K = w["m"], w["n"], w["k"]
    row_begin, rows = lib.shard_rows(M, world, rank)
    B = gen_b(torch, w)
    A = gen_a_rows(torch, w, rank, rows)
    C = torch.empty(rows, N, device="cuda", dtype=torch.bfloat16)
    if world > 1:
        os.environ.setdefault("GLOO_SOCKET_IFNAME", "lo")  # one node: the loopback interface always exists
    host_group = dist.new_group(backend="gloo") if world > 1 else None  # barriers that leave the GPUs idle
    desc = lib.gemm_desc(M, N, K, lib.BF16, lib.BF16)
    stream = torch.cuda.current_stream().cuda_stream

    def step():
        lib.gemm_tn_shard(desc, world, rank, A.data_ptr(), B.data_ptr(), C.data_ptr(), False, stream)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = lib.launch_count()
    with ClockSampler(local_rank) as clocks:
        barrier()
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        barrier()
    launches = lib.launch_count() - launches0
    ms_total = e0.elapsed_time(e1)
    status = lib.device_status()
    if status[0] != 0:
        raise SystemExit(f"kernel reported a bounded-wait timeout: {status}")
    t = torch.tensor([ms_total], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / args.steps
    flop = 2.0 * M * N * K
    value = flop / (ms_step * 1e-3) / 1e12

    pk = peaks()
    region_s = ms_step * args.steps * 1e-3
    peak_kind = "bf16_tflops" if region_s < 1.0 else "bf16_tflops_sustained"
    per_gpu_tflops = value / world
    roofline = {"bound": "tensor", "achieved": per_gpu_tflops, "peak": pk[peak_kind], "unit": "TFLOP/s",
                "frac": per_gpu_tflops / pk[peak_kind], "traffic": NCU_TRAFFIC_8192 if world == 1 else None,
                "kernel": "gemm_tn_kernel<cta_group 2, BN 256, MH 2>: 512x256 pair tile, BK 64, 4-stage TMA ring", "peak_kind": f"{peak_kind} ({pk['_source']})",
                "frac_of_nominal_2250": per_gpu_tflops / 2250.0,
                "algorithmic_flop_per_launch": 2.0 * rows * N * K}

    out = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
           "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak" if world == 1 else "strong",
           "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
           "config": {"workload": w["name"], "rows_per_gpu": rows, "l2": "operands (A+B+C >= 384 MB per GPU) exceed the 126 MB L2",
                      "timing": "cuda events on the launching stream, max over ranks"},
           "roofline": roofline, "clocks": clocks.summary(), "gpu_launches": int(launches)}
    roofline["traffic_source"] = "one ncu capture of this kernel and shape, a constant of this program" if world == 1 else None

    # ---- parity of the timed step's result: bands of this rank's rows against the oracle ----
    if not args.skip_extras:
        b_bits = to_bits(torch, B)
        own = BandCheck(to_bits(torch, A), b_bits, three_bands(rows), K)
        got, off = band_bits(torch, C, own.bands)
        mine = own.check(got, off)
        if world > 1:
            gathered = [None] * world
            dist.all_gather_object(gathered, mine, group=host_group)
            out["parity"] = {"what": "the compute-only step: every rank checks three bands of its own rows of C against the oracle",
                             "rows_checked": sum(x["rows_checked"] for x in gathered),
                             "max_excess": max(x["max_excess"] for x in gathered), "ok": all(x["ok"] for x in gathered)}
        else:
            out["parity"] = dict(mine, what="three bands of rows of the timed step's C against the oracle")

    # ---- end to end through the host-buffer C-ABI call --------------------------------
    if not args.skip_extras and world == 1:
        hA = torch.empty(rows, K, dtype=torch.bfloat16).pin_memory()
        hB = torch.empty(N, K, dtype=torch.bfloat16).pin_memory()
        hC = torch.empty(rows, N, dtype=torch.bfloat16).pin_memory()
        hA.copy_(A)
        hB.copy_(B)
        sub = lib.gemm_desc(rows, N, K, lib.BF16, lib.BF16)
        e2e_steps = max(3, min(args.steps, 10))
        for _ in range(2):
            lib.gemm_tn_host(sub, hA.data_ptr(), hB.data_ptr(), hC.data_ptr())
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            lib.gemm_tn_host(sub, hA.data_ptr(), hB.data_ptr(), hC.data_ptr())  # synchronous: returns with C on the host
        checksum = float(hC[0, 0])  # the step's result is read on the host
        dt = time.perf_counter() - t0
        tt = torch.tensor([dt], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        dt = float(tt.item()) / e2e_steps
        out["e2e"] = {"value": flop / dt / 1e12, "unit": UNIT, "h2d_bytes_per_step": (rows * K + N * K) * 2,
                      "d2h_bytes_per_step": rows * N * 2, "ms_per_step": dt * 1e3, "steps": e2e_steps,
                      "api": "cute_b200_gemm_tn_host (pinned host buffers, synchronous)", "checksum": checksum}
        lib.release_workspace()
        del hA, hB, hC

    # ---- optional replicated C (exchange over NVLink), N > 1 only ---------------------------
    # Every variant leaves the whole C on every GPU.  They are timed interleaved, one step of each
    # in turn, so that drift of the clocks under the power cap falls on all of them alike; a step
    # is timed with CUDA events from its first launch to the point where the rank holds the peers'
    # rows too (the variants that push into peer memory end with a barrier, which is inside).
    if world > 1 and not args.skip_extras:
        from cute_rs_b200.sharded import PeerBuffer, RowShardedGemm, launch_replicated_fused, launch_replicated_p2p
        plan = RowShardedGemm(M, N, K, lib.BF16, lib.BF16, world, rank)
        full_nccl = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        peer_c = PeerBuffer(M * N * 2, world, rank)
        full = peer_c.tensor((M, N), torch.bfloat16)
        comm_stream = torch.cuda.Stream()
        copy_streams = [torch.cuda.Stream() for _ in range(world - 1)]
        reps = max(3, min(args.steps, 10))

        def gemm_then_gather():
            step()
            dist.all_gather_into_tensor(full_nccl, C)

        variants = {
            "compute_only": step,
            "gemm_then_all_gather": gemm_then_gather,
            "overlapped_panels": lambda: plan.launch_replicated(A.data_ptr(), B.data_ptr(), full_nccl, panels=8,
                                                                comm_stream=comm_stream),
            "peer_copies": lambda: launch_replicated_p2p(plan, A.data_ptr(), B.data_ptr(), peer_c, 2, panels=8,
                                                         copy_streams=copy_streams),
            "fused_pusher_warp": lambda: launch_replicated_fused(plan, A.data_ptr(), B.data_ptr(), peer_c, 2),
            "fused_pusher_warp_all_reduce_barrier": lambda: launch_replicated_fused(plan, A.data_ptr(), B.data_ptr(), peer_c, 2,
                                                                                    barrier="all_reduce"),
            "fused_pusher_warp_tile_m_128": lambda: launch_replicated_fused(plan, A.data_ptr(), B.data_ptr(), peer_c, 2, tile_m=128),
            "fused_register_stores": lambda: launch_replicated_fused(plan, A.data_ptr(), B.data_ptr(), peer_c, 2, tile_m=128,
                                                                     register_stores=True),
        }
        # The oracle's view of rows that a PEER computes and delivers into this rank's copy of C: the
        # next rank's rows of A are rebuilt here from its seed.
        peer = (rank + 1) % world
        peer_begin, peer_rows = plan.spans[peer]
        peer_check = BandCheck(to_bits(torch, gen_a_rows(torch, w, peer, peer_rows)), b_bits, three_bands(peer_rows), K)
        # correctness of each variant against the all-gather of the compute-only C
        step()
        ref_full = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        dist.all_gather_into_tensor(ref_full, C)
        equal, parity = {}, {}
        for name, fn in variants.items():
            if name == "compute_only":
                continue
            dst = full if name.startswith(("peer", "fused")) else full_nccl
            dst.zero_()
            barrier()
            fn()
            barrier()
            equal[name] = bool(torch.equal(dst, ref_full))
            got, off = band_bits(torch, dst[row_begin:row_begin + rows], own.bands)
            a_, b_ = own.check(got, off), None
            got, off = band_bits(torch, dst[peer_begin:peer_begin + peer_rows], peer_check.bands)
            b_ = peer_check.check(got, off)
            parity[name] = {"rows_checked": a_["rows_checked"] + b_["rows_checked"], "max_excess": max(a_["max_excess"], b_["max_excess"]),
                            "ok": a_["ok"] and b_["ok"]}
        del ref_full
        all_parity = [None] * world
        dist.all_gather_object(all_parity, parity, group=host_group)
        sums = torch.zeros(len(variants), device="cuda", dtype=torch.float64)
        gate = torch.zeros(1, device="cuda")
        for r in range(reps + 1):
            for i, fn in enumerate(variants.values()):
                barrier()
                # the ranks' hosts leave the barrier at slightly different times; a tiny all-reduce queued in
                # front of the step lets every rank's stream pass e0 at the same moment instead
                dist.all_reduce(gate)
                e0.record()
                fn()
                e1.record()
                torch.cuda.synchronize()
                if r > 0:  # the first round warms up
                    sums[i] += e0.elapsed_time(e1)
        sums /= reps
        dist.all_reduce(sums, op=dist.ReduceOp.MAX)
        how = {
            "compute_only": "row blocks of C stay on their GPUs (the headline number's step, timed the same way)",
            "gemm_then_all_gather": "one ncclAllGather of the bf16 row blocks of C after the GEMM",
            "overlapped_panels": "8 row panels; each is sent to the peers (NCCL send/recv) while the next is multiplied",
            "peer_copies": "8 row panels; each is pushed into every peer's C with device-to-device copies over NVLink "
                           "(CUDA IPC mappings, copy engines, no NCCL) while the next is multiplied; closing barrier",
            "fused_pusher_warp": "one GEMM launch that also writes every finished tile into the peers' C over NVLink peer "
                                 "mappings: a pusher warp per CTA copies the tile by TMA (load from its own C in L2, bulk "
                                 "tensor store to each peer) beside the next tiles' main loop; the last CTA then adds 1 to this "
                                 "rank's counter in every peer's memory and a one-thread kernel behind the GEMM waits (bounded) for "
                                 "the peers' counters: no host synchronisation, no collective call",
            "fused_pusher_warp_all_reduce_barrier": "the same kernel, closed by a one-element NCCL all-reduce queued behind it instead "
                                                    "of the counters",
            "fused_pusher_warp_tile_m_128": "the same with 128 rows of C per CTA (double-buffered accumulators)",
            "fused_register_stores": "one GEMM launch whose epilogue warps store every chunk to the peers' C from registers "
                                     "(32 bytes per lane), 128 rows of C per CTA; closing barrier",
        }
        rep = {"unit": UNIT, "timing": "%d interleaved steps of each variant, CUDA events from a device-side rendezvous of the ranks "
                                       "to the end of the step, max over ranks" % reps}
        # What bounds a step that leaves all of C on every GPU: the slower of this GPU's share of the flops at the
        # measured cuBLAS peak and the bytes it must send at the measured peer-copy rate (770 GB/s per direction).
        # The variants run back to back for about a second, so the GPU sits at its power cap: the sustained figure.
        t_flops = flop / world / (pk.get("bf16_tflops_sustained", pk["bf16_tflops"]) * 1e12) * 1e3
        t_link = (world - 1) * rows * N * 2 / 770e9 * 1e3
        rep["target"] = {"ms": max(t_flops, t_link), "flops_ms": t_flops, "nvlink_ms": t_link,
                         "bound": "tensor" if t_flops >= t_link else "nvlink",
                         "how": "max(2mnk / N / measured sustained bf16 peak, (N-1)/N * bytes of C / 770 GB/s measured peer copy)"}
        for i, name in enumerate(variants):
            ms_v = float(sums[i].item())
            rep[name] = {"value": flop / (ms_v * 1e-3) / 1e12, "ms_per_step": ms_v, "how": how[name]}
            if name in equal:
                rep[name]["equals_all_gather_result"] = equal[name]
                rep[name]["frac_of_target"] = rep["target"]["ms"] / ms_v
                per_rank = [x[name] for x in all_parity]
                rep[name]["parity"] = {"rows_checked": sum(x["rows_checked"] for x in per_rank),
                                       "max_excess": max(x["max_excess"] for x in per_rank), "ok": all(x["ok"] for x in per_rank)}
        rep["parity_what"] = ("every rank checks, against the oracle, three bands of its own rows and three bands of the rows the "
                              "next rank computed and delivered into this rank's copy of C")
        out["replicated"] = rep
        del full, full_nccl
        peer_c.close()

    # ---- N > 1: end to end and the one-call launcher, both through the C ABI from ONE process ------
    # cute_b200_comm_create / cute_b200_gemm_tn_sharded[_host] drive all the GPUs from a single process
    # (a host thread per GPU).  Rank 0 makes those calls; the other ranks have released their device
    # memory and wait on a host-side (gloo) barrier, so nothing of theirs runs on any GPU meanwhile.
    if world > 1 and not args.skip_extras:
        del A, B, C
        torch.cuda.empty_cache()
        torch.cuda.synchronize()
        dist.barrier(group=host_group)
        if rank == 0:
            try:
                out.update(bench_launcher(lib, torch, w, world, pk, max(3, min(args.steps, 10))))
            except Exception as exc:  # noqa: BLE001 - reported in the line, never hidden
                out["e2e"] = {"error": f"{type(exc).__name__}: {exc}"}
            torch.cuda.set_device(local_rank)
        dist.barrier(group=host_group)

    # ---- secondary kernels and the CPU baseline: rank 0 of a 1-GPU run only ----------------
    if world == 1 and not args.skip_extras:
        # The headline line must survive a failure of a side measurement: each one reports its own error.
        extras = {
            "elementwise_add": lambda: bench_add(lib, torch, pk),
            "sgemm": lambda: bench_sgemm(lib, torch),
            "cpu_baseline": lambda: cpu_baseline(A, B, M, N, K),
            "reference_gpu_kernel_restated": lambda: bench_ref_kernel(A, B, M, N, K, torch),
            "cublas_same_run": lambda: bench_cublas(A, B, args.steps, args.warmup, flop, step, torch, local_rank),
            "strong_scaling_anchor": lambda: bench_anchor(lib, torch, pk),
        }
        for name, fn in extras.items():
            try:
                out[name] = fn()
            except Exception as exc:  # noqa: BLE001 - reported in the line, never hidden
                out[name] = {"error": f"{type(exc).__name__}: {exc}"}

    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


def bench_launcher(lib, torch, w, world, pk, steps):
    """Rank 0 only, every other rank idle: the whole 32768 x 32768 x 8192 GEMM through the launcher
    that one process makes for all the GPUs.  `e2e`: whole matrices in pinned host memory in, C in
    host memory out, every step (cute_b200_gemm_tn_sharded_host: each GPU uploads its rows of A and
    its 1/N share of B, the shares travel on over NVLink, each GPU sends its rows of C back).
    `c_abi_launcher`: the same GEMM on device buffers through cute_b200_gemm_tn_sharded, compute only
    and with C replicated on every GPU (the fused form, and device-to-device copies for comparison),
    wall-clock per call since the call returns when every GPU is done."""
    import numpy as np
    M, N, K = w["m"], w["n"], w["k"]
    flop = 2.0 * M * N * K
    comm = lib.comm_create(world)
    res = {}
    try:
        info = lib.comm_info(comm)
        spans = [lib.shard_rows(M, world, g) for g in range(world)]
        hA = torch.empty(M, K, dtype=torch.bfloat16).pin_memory()
        hB = torch.empty(N, K, dtype=torch.bfloat16).pin_memory()
        hC = torch.empty(M, N, dtype=torch.bfloat16).pin_memory()
        torch.cuda.set_device(0)
        hB.copy_(gen_b(torch, w))
        for g, (lo, rows) in enumerate(spans):
            hA[lo:lo + rows].copy_(gen_a_rows(torch, w, g, rows))
        torch.cuda.empty_cache()
        desc = lib.gemm_desc(M, N, K, lib.BF16, lib.BF16)
        for _ in range(2):
            lib.gemm_tn_sharded_host(comm, desc, hA.data_ptr(), hB.data_ptr(), hC.data_ptr())
        t0 = time.perf_counter()
        for _ in range(steps):
            lib.gemm_tn_sharded_host(comm, desc, hA.data_ptr(), hB.data_ptr(), hC.data_ptr())  # returns with C on the host
        checksum = float(hC[0, 0])  # the step's result is read on the host
        dt = (time.perf_counter() - t0) / steps
        # parity: bands of rows in the first, a middle and the last GPU's block, against the oracle
        a_bits = hA.view(torch.int16).numpy().view(np.uint16)
        b_bits = hB.view(torch.int16).numpy().view(np.uint16)
        c_bits = hC.view(torch.int16).numpy().view(np.uint16)
        bands = []
        for g in sorted({0, world // 2, world - 1}):
            lo, rows = spans[g]
            bands += [(lo + 64, lo + 96), (lo + rows - 32, lo + rows)]
        chk = BandCheck(a_bits, b_bits, bands, K)
        par = chk.check(c_bits, 0)
        res["e2e"] = {"value": flop / dt / 1e12, "unit": UNIT, "h2d_bytes_per_step": (M * K + N * K) * 2, "d2h_bytes_per_step": M * N * 2,
                      "ms_per_step": dt * 1e3, "steps": steps,
                      "api": "cute_b200_gemm_tn_sharded_host (one process, a host thread per GPU; pinned host buffers; synchronous); "
                             "rank 0 calls it while the other ranks wait on a host-side barrier with their GPUs idle",
                      "h2d_bytes_per_gpu": (spans[0][1] * K + N * K // world) * 2, "d2h_bytes_per_gpu": spans[0][1] * N * 2,
                      "b_exchange": "each GPU uploads N/%d rows of B and passes them to the others by device-to-device copies over NVLink" % world,
                      "checksum": checksum, "parity": par}
        del hA, hB, hC, a_bits, b_bits, c_bits
        # device buffers: one tensor per GPU, made by this process on each device
        dA, dB, dC = [], [], []
        for g, (lo, rows) in enumerate(spans):
            torch.cuda.set_device(g)
            dA.append(gen_a_rows(torch, w, g, rows, device=f"cuda:{g}"))
            dB.append(gen_b(torch, w, device=f"cuda:{g}"))
            dC.append(torch.empty(M, N, dtype=torch.bfloat16, device=f"cuda:{g}"))
        torch.cuda.set_device(0)
        ptr = lambda ts: [t.data_ptr() for t in ts]
        blocks = [c[lo:lo + rows] for c, (lo, rows) in zip(dC, spans)]
        modes = {"compute_only": (lib.REPLICATE_NONE, ptr(blocks)), "replicated_fused": (lib.REPLICATE_FUSED, ptr(dC)),
                 "replicated_copies": (lib.REPLICATE_COPIES, ptr(dC))}
        launcher = {"unit": UNIT, "api": "cute_b200_gemm_tn_sharded (one process; returns when every GPU is done)",
                    "timing": "host clock around %d back-to-back calls, each of which waits for all GPUs" % steps,
                    "peer_access": info["peer_access"]}
        if not info["peer_access"]:
            modes.pop("replicated_fused")
        for name, (mode, cptrs) in modes.items():
            for _ in range(2):
                lib.gemm_tn_sharded(comm, desc, ptr(dA), ptr(dB), cptrs, mode)
            t0 = time.perf_counter()
            for _ in range(steps):
                lib.gemm_tn_sharded(comm, desc, ptr(dA), ptr(dB), cptrs, mode)
            ms = (time.perf_counter() - t0) / steps * 1e3
            launcher[name] = {"value": flop / (ms * 1e-3) / 1e12, "ms_per_step": ms}
            if mode != lib.REPLICATE_NONE:
                # GPU 0's copy of C must hold the rows the LAST GPU computed
                lo, rows = spans[world - 1]
                a_last = to_bits(torch, dA[world - 1])
                chk = BandCheck(a_last, to_bits(torch, dB[0]), three_bands(rows), K)
                got, off = band_bits(torch, dC[0][lo:lo + rows], chk.bands)
                launcher[name]["parity"] = chk.check(got, off)
                dC[0].zero_()
        res["c_abi_launcher"] = launcher
        del dA, dB, dC, blocks
    finally:
        lib.comm_destroy(comm)
    return res


def bench_anchor(lib, torch, pk):
    """The workload of the multi-GPU runs, 32768 x 32768 x 8192, on this one GPU (it fits: 3 GiB):
    the same-workload base for the strong-scaling curve of `bench.py --gpus 2/4/8`."""
    w = workload(2)
    M, N, K = w["m"], w["n"], w["k"]
    B = gen_b(torch, w)
    A = torch.cat([gen_a_rows(torch, w, r, M // 8) for r in range(8)])
    C = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    d = lib.gemm_desc(M, N, K, lib.BF16, lib.BF16)
    s = torch.cuda.current_stream().cuda_stream
    for _ in range(3):
        lib.gemm_tn(d, A.data_ptr(), B.data_ptr(), C.data_ptr(), s)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(10):
        lib.gemm_tn(d, A.data_ptr(), B.data_ptr(), C.data_ptr(), s)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / 10
    chk = BandCheck(to_bits(torch, A), to_bits(torch, B), three_bands(M), K)
    got, off = band_bits(torch, C, chk.bands)
    tf = 2.0 * M * N * K / ms / 1e9
    return {"workload": w["name"] + ", all rows on one GPU", "value": tf, "unit": UNIT, "ms_per_step": ms, "steps": 10,
            "frac_of_sustained_peak": tf / pk.get("bf16_tflops_sustained", pk["bf16_tflops"]), "parity": chk.check(got, off),
            "note": "N = 1 base of the strong-scaling curve; the N = 1 headline above is the 8192^3 configuration"}


def bench_add(lib, torch, pk, n=1 << 28):
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.rand(n, device="cuda", generator=g) * 2 - 1
    y = torch.rand(n, device="cuda", generator=g) * 2 - 1
    o = torch.empty(n, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    for _ in range(3):
        lib.elementwise_add_f32(x.data_ptr(), y.data_ptr(), o.data_ptr(), n, s)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(20):
        lib.elementwise_add_f32(x.data_ptr(), y.data_ptr(), o.data_ptr(), n, s)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / 20
    gbs = 12.0 * n / ms / 1e6
    return {"workload": f"elementwise_add f32 {n} elements, uniform[-1,1) seed 1 (3 x {4 * n / 2 ** 30:.2f} GiB, larger than L2)",
            "gbs": gbs, "ms": ms, "bound": "hbm", "peak": pk["hbm_gbs"], "frac": gbs / pk["hbm_gbs"],
            "peak_kind": f"hbm_gbs ({pk['_source']})", "frac_of_nominal_8000": gbs / 8000.0,
            "algorithmic_bytes_per_launch": 12 * n}


def bench_sgemm(lib, torch):
    n = 4096
    g = torch.Generator(device="cuda").manual_seed(2)
    a, b, c = (torch.rand(n * n, device="cuda", generator=g) * 2 - 1 for _ in range(3))
    s = torch.cuda.current_stream().cuda_stream
    for _ in range(3):
        lib.sgemm_nt(n, n, n, 1.5, 0.5, a.data_ptr(), b.data_ptr(), c.data_ptr(), s)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(10):
        lib.sgemm_nt(n, n, n, 1.5, 0.5, a.data_ptr(), b.data_ptr(), c.data_ptr(), s)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / 10
    return {"workload": "sgemm_nt f32 4096^3 column-major, alpha 1.5, beta 0.5", "tflops": 2.0 * n ** 3 / ms / 1e9, "ms": ms,
            "bound": "fp32 FFMA pipe", "peak_nominal": 148 * 128 * 2 * 1.965e9 / 1e12}


def bench_gemm_shape(lib, torch, shape, tiling, iters, pk):
    """One runtime_gemm shape (bf16 in, bf16 out, normal(0, 0.02) seed 3), timed with CUDA events, with
    torch.matmul on the same operands beside it and the two rooflines of the shape: the tensor pipe
    (2mnk at the measured bf16 rate) and HBM (the operands and the result once, at the measured copy rate)."""
    m, n, k = shape
    g = torch.Generator(device="cuda").manual_seed(3)
    A = (torch.randn(m, k, device="cuda", generator=g) * 0.02).bfloat16()
    B = (torch.randn(n, k, device="cuda", generator=g) * 0.02).bfloat16()
    C = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
    d = lib.gemm_desc(m, n, k, lib.BF16, lib.BF16, cta_group=tiling[0], tile_n=tiling[1], tile_m=tiling[2], split_k=tiling[3])
    s = torch.cuda.current_stream().cuda_stream
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    n0 = lib.launch_count()
    ms = timed(lambda: lib.gemm_tn(d, A.data_ptr(), B.data_ptr(), C.data_ptr(), s))
    launches = (lib.launch_count() - n0) // (iters + 3)
    Bt = B.t()
    ms_t = timed(lambda: torch.matmul(A, Bt))
    flop, byts = 2.0 * m * n * k, 2.0 * (m * k + n * k + m * n)
    t_tensor, t_hbm = flop / (pk["bf16_tflops"] * 1e12) * 1e3, byts / (pk["hbm_gbs"] * 1e9) * 1e3
    chk = BandCheck(to_bits(torch, A), to_bits(torch, B), three_bands(m), k)
    got, off = band_bits(torch, C, chk.bands)
    return {"workload": f"runtime_gemm bf16 {m}x{n}x{k} -> bf16, normal(0,0.02) seed 3", "ms": ms, "tflops": flop / ms / 1e9,
            "kernels_per_call": launches, "plan": dict(zip(("cta_group", "tile_n", "tile_m", "k_ranges"), lib.gemm_plan(d))),
            "torch_matmul_ms": ms_t, "ratio_to_torch": ms / ms_t,
            "bound": "hbm" if t_hbm > t_tensor else "tensor", "roofline_ms": max(t_tensor, t_hbm),
            "frac_of_roofline": max(t_tensor, t_hbm) / ms, "algorithmic_bytes": byts, "gbs": byts / ms / 1e6,
            "parity": chk.check(got, off), "status": list(lib.device_status())}


def bench_multi(lib, torch, copies=3):
    """The GEMM that also delivers C to further destinations (the pusher warp), with all copies in
    this GPU's own memory: what one rank of the replicated multi-GPU form runs, minus NVLink."""
    n = 8192
    g = torch.Generator(device="cuda").manual_seed(3)
    A = (torch.randn(n, n, device="cuda", generator=g) * 0.02).bfloat16()
    B = (torch.randn(n, n, device="cuda", generator=g) * 0.02).bfloat16()
    dests = [torch.empty(n, n, device="cuda", dtype=torch.bfloat16) for _ in range(copies)]
    ptrs = [t.data_ptr() for t in dests]
    d = lib.gemm_desc(n, n, n, lib.BF16, lib.BF16)
    s = torch.cuda.current_stream().cuda_stream
    out = {"workload": f"bf16 8192^3 -> bf16, C written to {copies} buffers of this GPU"}
    for label, fn in (("one_destination", lambda: lib.gemm_tn(d, A.data_ptr(), B.data_ptr(), ptrs[0], s)),
                      ("pusher_warp", lambda: lib.gemm_tn_multi(d, A.data_ptr(), B.data_ptr(), ptrs, s))):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / 10
        out[label] = {"ms": ms, "tflops": 2.0 * n ** 3 / ms / 1e9}
    out["copies_equal"] = all(bool(torch.equal(dests[0], t)) for t in dests[1:])
    return out


def bench_cublas(A, B, steps, warmup, flop, step, torch, gpu_index=0):
    """torch.matmul (cuBLAS) on the same operands, the same number of back-to-back launches, the
    same GPU and process: a comparator beside the headline number, not part of it.  Long runs of
    launches settle at the power cap, so the two are also timed in alternation (ten rounds of
    thirty launches each), with the SM clock sampled during each side's rounds: time x clock is the
    kernel's length in SM cycles, which separates what the power cap does to the clock from what
    the kernel does with its cycles."""
    Bt = B.t()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed(fn, n):
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    mm = lambda: torch.matmul(A, Bt)
    for _ in range(warmup):
        mm()
    torch.cuda.synchronize()
    ms = timed(mm, steps)
    ours, theirs, mhz_ours, mhz_theirs = [], [], [], []
    for _ in range(10):
        with ClockSampler(gpu_index) as c:
            ours.append(timed(step, 30))
        mhz_ours += c.samples
        with ClockSampler(gpu_index) as c:
            theirs.append(timed(mm, 30))
        mhz_theirs += c.samples
    mo, mt = statistics.median(ours), statistics.median(theirs)
    alt = {"this_library_ms": mo, "cublas_ms": mt, "ratio": mo / mt,
           "how": "medians of ten rounds of thirty launches each, the two in turn"}
    if mhz_ours and mhz_theirs:
        fo, ft = statistics.median(mhz_ours), statistics.median(mhz_theirs)
        alt.update({"this_library_sm_mhz": fo, "cublas_sm_mhz": ft, "this_library_kcycles": mo * fo, "cublas_kcycles": mt * ft,
                    "cycles_ratio": (mo * fo) / (mt * ft),
                    "cycles_how": "ms x median sampled SM MHz = thousands of SM cycles per launch (NVML clock samples of each side's rounds)"})
    return {"value": flop / (ms * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": ms, "steps": steps, "alternating": alt}


def bench_ref_kernel(A, B, M, N, K, torch):
    """The reference's tensorop_gemm kernel structure (mma.sync.m16n8k16, 3-stage
    cp.async ring, 128 x 128 x 32 tiles, f32 C), restated by hand in
    oracle/ref_kernel_sm80.cu because the reference's own PTX needs mlir-opt;
    compute_80 PTX JIT-compiled by the driver on this GPU.  A baseline beside the
    headline number, not part of it."""
    import oracle
    C = torch.empty(M, N, device="cuda", dtype=torch.float32)
    s = torch.cuda.current_stream().cuda_stream
    run = lambda: oracle.ref_tensorop_gemm(True, M, N, K, A.data_ptr(), B.data_ptr(), C.data_ptr(), s)
    for _ in range(2):
        run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(5):
        run()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / 5
    return {"workload": f"bf16 {M}x{N}x{K} -> f32, the reference kernel's structure restated", "tflops": 2.0 * M * N * K / ms / 1e9,
            "ms": ms, "kind": "restated (the reference's mlir-opt PTX cannot be built here)"}


def cpu_baseline(A, B, M, N, K):
    """The oracle timed on the host cores: one pass over the whole GEMM of the
    step (test infrastructure used as the reported CPU baseline only)."""
    import numpy as np
    import torch
    import oracle
    oracle.use_all_cores()
    rows = M
    a = A[:rows].view(torch.int16).cpu().numpy().view(np.uint16)
    b = B.view(torch.int16).cpu().numpy().view(np.uint16)
    oracle.gemm_tn(a[:64], b, oracle.BF16, oracle.BF16)  # build + page in
    t0 = time.perf_counter()
    oracle.gemm_tn(a, b, oracle.BF16, oracle.BF16)
    dt = time.perf_counter() - t0
    return {"value": 2.0 * rows * N * K / dt / 1e12, "unit": UNIT, "cores": oracle.num_threads(), "kind": "port",
            "sample": f"the whole {M}x{N}x{K} GEMM of one step, one pass, {dt:.2f} s on {oracle.num_threads()} threads"}


if __name__ == "__main__":
    main()
