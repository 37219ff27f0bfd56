"""Row-sharded GEMM over the GPUs of one box, one process per GPU.

The reference crate is single-GPU; this extends its launcher.  Rank r owns a
contiguous block of whole 128-row tiles of A and C (``cute_b200_shard_rows``),
B is replicated in every GPU's own memory, and the GEMM itself needs no
exchange.  Only a caller that wants C replicated pays for a collective: the
row blocks are all-gathered over NCCL (NVLink / NVSwitch).  The plumbing is
``torch.distributed``; the arithmetic is the C-ABI GEMM.
"""
from __future__ import annotations

from . import _lib


class RowShardedGemm:
    def __init__(self, m: int, n: int, k: int, ab_dtype: int, c_dtype: int, world: int, rank: int,
                 alpha: float = 1.0, beta: float = 0.0):
        self.m, self.n, self.k, self.world, self.rank = m, n, k, world, rank
        self.desc = _lib.gemm_desc(m, n, k, ab_dtype, c_dtype, alpha, beta)
        self.spans = [_lib.shard_rows(m, world, r) for r in range(world)]
        self.row_begin, self.rows = self.spans[rank]

    def even(self) -> bool:
        return len({rows for _, rows in self.spans}) == 1

    def launch(self, dA_shard: int, dB: int, dC: int, c_is_full: bool = False, stream: int = 0) -> None:
        """This rank's rows of C = A_shard * B^T.  `dC` is row 0 of a full C
        when `c_is_full`, else this rank's block."""
        _lib.gemm_tn_shard(self.desc, self.world, self.rank, dA_shard, dB, dC, c_is_full, stream)

    def all_gather(self, c_block, full, group=None) -> None:
        """Replicate C: `full` (m, n) receives every rank's block in row order."""
        import torch.distributed as dist
        if self.even():
            dist.all_gather_into_tensor(full, c_block, group=group)
            return
        for r, (begin, rows) in enumerate(self.spans):  # ragged split: one broadcast per block
            if rows == 0:
                continue
            view = full[begin:begin + rows]
            if r == self.rank:
                view.copy_(c_block)
            dist.broadcast(view, src=r, group=group)

    def panels(self, count: int = 8):
        """Row panels of this rank's block as (first row within the block, rows):
        whole 128-row tiles, at most `count` of them."""
        if self.rows == 0:
            return []
        tiles = (self.rows + 127) // 128
        count = max(1, min(count, tiles))
        per = ((tiles + count - 1) // count) * 128
        return [(r, min(per, self.rows - r)) for r in range(0, self.rows, per)]

    def launch_replicated(self, dA_shard: int, dB: int, full, panels: int = 8, comm_stream=None, group=None,
                          compute_panel=None) -> None:
        """C replicated on every GPU, with the exchange hidden behind the math.

        This rank's block is computed panel by panel straight into its rows of
        `full` (m, n); as soon as a panel is done it is sent to every peer and the
        peers' matching panels are received into their rows, on a second stream,
        while the next panel is being multiplied.  Needs an even split (every rank
        the same number of rows); a ragged split falls back to GEMM + all_gather.
        `compute_panel(first_row_in_block, rows)` replaces the GEMM launch (tests).
        """
        import torch
        import torch.distributed as dist
        k_bytes = self.k * 2
        c_elem = full.element_size()

        def gemm_panel(r0, rows):
            d = _lib.gemm_desc(rows, self.n, self.k, self.desc.ab_dtype, self.desc.c_dtype, self.desc.alpha,
                               self.desc.beta)
            stream = torch.cuda.current_stream().cuda_stream
            _lib.gemm_tn(d, dA_shard + r0 * k_bytes, dB,
                         full.data_ptr() + (self.row_begin + r0) * self.n * c_elem, stream)

        run = compute_panel or gemm_panel
        if not self.even() or self.world == 1:
            for r0, rows in self.panels(1):
                run(r0, rows)
            if self.world > 1:
                self.all_gather(full[self.row_begin:self.row_begin + self.rows].clone(), full, group=group)
            return
        on_gpu = full.is_cuda
        comm = comm_stream or (torch.cuda.Stream() if on_gpu else None)
        pending = []
        for r0, rows in self.panels(panels):
            run(r0, rows)
            ops = []
            for peer in range(self.world):
                if peer == self.rank:
                    continue
                mine = full[self.row_begin + r0:self.row_begin + r0 + rows]
                theirs = full[self.spans[peer][0] + r0:self.spans[peer][0] + r0 + rows]
                ops.append(dist.P2POp(dist.isend, mine, peer, group=group))
                ops.append(dist.P2POp(dist.irecv, theirs, peer, group=group))
            if on_gpu:
                done = torch.cuda.Event()
                done.record()
                with torch.cuda.stream(comm):
                    comm.wait_event(done)
                    pending += dist.batch_isend_irecv(ops)
            else:
                pending += dist.batch_isend_irecv(ops)
        for req in pending:
            req.wait()
        if on_gpu:
            torch.cuda.current_stream().wait_stream(comm)


class PeerBuffer:
    """A device buffer of the same size on every rank, each rank's copy mapped
    into every other rank's address space (CUDA IPC over NVLink).

    `ptrs[r]` is rank r's copy as seen from this process; `tensor(...)` views
    this rank's own copy as a torch tensor.  Collective: every rank of `group`
    must construct it at the same time.
    """

    FLAG_BYTES = 256  # counter r counts the launches of rank r that have landed here (launch_replicated_fused)
    GRANULE = 2 << 20

    def __init__(self, nbytes: int, world: int, rank: int, group=None):
        import torch
        import torch.distributed as dist
        self.nbytes, self.world, self.rank = nbytes, world, rank
        # The data is an allocation of its own, a whole number of 2 MiB, and the counters live in a second,
        # small allocation.  With the counters appended to the data (2 GiB + 256 bytes in one allocation)
        # every variant that writes peer memory through these mappings was slower than with the bare 2 GiB
        # buffer: on four GPUs the copy-engine pushes 4.7-4.9 ms against 4.1, the fused kernel 4.0 against
        # 3.4; on eight GPUs the fused kernel 7.3 ms against 3.3 for the same kernel on directly enabled peer
        # pointers.  (Presumably the odd-sized allocation is mapped into the peers with small pages.)
        self.local = _lib.alloc((max(nbytes, 1) + self.GRANULE - 1) // self.GRANULE * self.GRANULE)
        self.flags_local = _lib.alloc(self.GRANULE)
        self.steps = 0  # signalled steps so far (every rank counts alike)
        self._zero_flags()
        handles = [None] * world
        dist.all_gather_object(handles, (_lib.ipc_export(self.local), _lib.ipc_export(self.flags_local)), group=group)
        self.ptrs = [self.local if r == rank else _lib.ipc_open(handles[r][0]) for r in range(world)]
        self.flag_ptrs = [self.flags_local if r == rank else _lib.ipc_open(handles[r][1]) for r in range(world)]
        dist.barrier(group=group)

    def _zero_flags(self) -> None:
        import torch
        zeros = torch.zeros(self.FLAG_BYTES, dtype=torch.uint8, device="cuda")
        _lib.copy_async(self.flags_local, zeros.data_ptr(), self.FLAG_BYTES, torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()

    def reset_signals(self, group=None) -> None:
        """Zero every rank's completion counters and start counting steps again (after a step in
        which a rank did not send, which leaves its counters one short everywhere).  Collective."""
        import torch
        import torch.distributed as dist
        torch.cuda.synchronize()
        dist.barrier(group=group)
        self._zero_flags()
        self.steps = 0
        dist.barrier(group=group)

    def tensor(self, shape, dtype):
        import torch

        class _View:  # torch reads device memory it does not own through this protocol
            pass

        v = _View()
        typestr = {torch.bfloat16: "<u2", torch.float16: "<f2", torch.float32: "<f4"}[dtype]
        v.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (self.local, False), "version": 3}
        t = torch.as_tensor(v, device="cuda")
        return t.view(torch.bfloat16) if dtype == torch.bfloat16 else t

    def close(self, group=None) -> None:
        import torch
        import torch.distributed as dist
        torch.cuda.synchronize()
        dist.barrier(group=group)
        for r in range(self.world):
            if r != self.rank:
                _lib.ipc_close(self.ptrs[r])
                _lib.ipc_close(self.flag_ptrs[r])
        dist.barrier(group=group)
        _lib.free(self.local)
        _lib.free(self.flags_local)
        self.ptrs, self.flag_ptrs = [], []


def launch_replicated_p2p(plan: RowShardedGemm, dA_shard: int, dB: int, peer_c: PeerBuffer, c_elem: int, panels: int = 8,
                          copy_streams=None, group=None) -> None:
    """C replicated on every GPU by peer-to-peer copies hidden behind the math.

    `peer_c` holds the full (m, n) C of every rank.  This rank multiplies its row
    block panel by panel into its own copy; each finished panel is pushed into
    the same rows of every peer's copy with device-to-device copies, one stream
    per peer so that several copy engines and all NVLink ports work at once (no
    SM is taken from the GEMM, and no NCCL kernel has to find room beside the
    persistent GEMM CTAs), while the next panel is being multiplied.  Returns
    after all ranks' pushes have landed.
    """
    import torch
    import torch.distributed as dist
    if copy_streams is None:
        copy_streams = [torch.cuda.Stream() for _ in range(plan.world - 1)]
    compute = torch.cuda.current_stream()
    row_bytes = plan.n * c_elem
    for r0, rows in plan.panels(panels):
        d = _lib.gemm_desc(rows, plan.n, plan.k, plan.desc.ab_dtype, plan.desc.c_dtype, plan.desc.alpha, plan.desc.beta)
        off = (plan.row_begin + r0) * row_bytes
        _lib.gemm_tn(d, dA_shard + r0 * plan.k * 2, dB, peer_c.local + off, compute.cuda_stream)
        done = torch.cuda.Event()
        done.record(compute)
        for step in range(1, plan.world):  # rank r talks to r+1, r+2, ...: every link carries one copy at a time
            peer = (plan.rank + step) % plan.world
            stream = copy_streams[(step - 1) % len(copy_streams)]
            stream.wait_event(done)
            _lib.copy_async(peer_c.ptrs[peer] + off, peer_c.local + off, rows * row_bytes, stream.cuda_stream)
    for stream in copy_streams:
        stream.synchronize()
    compute.synchronize()
    dist.barrier(group=group)  # every rank's pushes into this GPU have landed


def launch_replicated_fused(plan: RowShardedGemm, dA_shard: int, dB: int, peer_c: PeerBuffer, c_elem: int, group=None,
                            tile_m: int = 0, register_stores: bool = False, barrier: str = "signal",
                            timeout_ms: int = 30000) -> None:
    """C replicated on every GPU by the GEMM kernel itself: one launch that
    stores every finished tile into this rank's rows of its own C and then
    copies it, from inside the kernel, into the same rows of every peer's C
    (peer mappings over NVLink): a pusher warp per CTA loads the tile back by TMA
    (it is still in L2) and issues one bulk tensor store per peer while the
    tensor cores work on the following tiles.  ``register_stores`` selects the
    fallback instead, 32-byte stores to every destination straight from the
    epilogue's registers, which NVLink carries far less well.  No collective
    library moves data.

    How a rank learns that all peers' stores into its C have completed
    (``barrier``): "signal" (default) - the last CTA of every rank's launch adds 1
    to its own counter in each peer's memory, and a one-thread kernel queued behind
    the GEMM waits, with a time limit, until the counters of all peers that have
    rows have reached this step's number; no host synchronisation beyond the wait
    for the stream and no collective call.  "all_reduce" - the earlier form, a
    one-element NCCL all-reduce queued behind the kernel.  The plan's epilogue
    must be the plain one (alpha 1, beta 0).  A rank without rows (more ranks
    than 128-row tiles) launches nothing, sends no count and only waits."""
    import torch
    import torch.distributed as dist
    off = plan.row_begin * plan.n * c_elem
    dests = [peer_c.local + off] + [peer_c.ptrs[(plan.rank + s) % plan.world] + off for s in range(1, plan.world)]
    if not (plan.desc.alpha == 1.0 and plan.desc.beta == 0.0):
        raise ValueError("launch_replicated_fused needs alpha = 1, beta = 0")
    stream = torch.cuda.current_stream()
    d = _lib.gemm_desc(max(plan.rows, 1), plan.n, plan.k, plan.desc.ab_dtype, plan.desc.c_dtype, tile_m=tile_m)
    if register_stores:
        d.tuning[0] |= 16
    if barrier == "signal" and plan.k > 0:
        order = [(plan.rank + s) % plan.world for s in range(plan.world)]
        flags = [peer_c.flag_ptrs[r] + 4 * plan.rank for r in order]  # this rank's counter at every peer
        if plan.rows > 0:
            _lib.gemm_tn_multi_signal(d, dA_shard, dB, dests, flags, stream.cuda_stream)
        peer_c.steps += 1
        senders = sum(1 << r for r, (_, rows) in enumerate(plan.spans) if rows > 0 and r != plan.rank)
        _lib.wait_signal(peer_c.flags_local, senders, peer_c.steps, timeout_ms, stream.cuda_stream)
        stream.synchronize()
        return
    if plan.rows > 0:
        _lib.gemm_tn_multi(d, dA_shard, dB, dests, stream.cuda_stream)
    # A one-element all-reduce queued behind the kernel is the barrier: it cannot finish on any rank
    # before every rank has joined it, which each does only after its own pushes have completed.
    # One wait for the stream then covers the kernel and the barrier.
    token = torch.zeros(1, device="cuda")
    dist.all_reduce(token, group=group)
    stream.synchronize()
