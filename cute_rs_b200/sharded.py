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
