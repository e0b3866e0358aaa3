"""N-column sharding of a quantized linear over the GPUs of one box.

Output column n of `x @ dequant(W)^T` depends only on row n of W and of its scales, and both
are stored row-major, so a shard is a contiguous row block of `w_packed` / `scales`: slicing is
zero-copy, nothing is repacked and no group straddles a shard.  Each rank (one process per GPU)
runs the single-GPU kernel on its rows with the full, replicated activation, and one all-gather
(NCCL over NVLink on GPUs) reassembles the output on every rank.  The reference has no
multi-GPU code at all; this layer is additive.

Gathered layout: rank g contributes y_g = [M, N/G]; the all-gather yields [G, M, N/G], which for
M = 1 already *is* the row-major [1, N].  For M > 1 `forward(..., layout="row_major")` transposes
it into [M, N]; `layout="gathered"` returns the [G, M, N/G] buffer untouched.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist


def shard_rows(n: int, world: int, rank: int) -> Tuple[int, int]:
    """Row range [r0, r1) of W owned by `rank`.  N must divide evenly so every rank gathers equal blocks."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} for world size {world}")
    if n % world:
        raise ValueError(f"N={n} is not divisible by the {world} ranks of the shard group")
    per = n // world
    return rank * per, (rank + 1) * per


class ShardedQuantLinear:
    """One quantized linear whose output columns are split across a process group.

    w, scales: either the FULL tensors (each rank keeps only its row block) or, with
    `already_local=True`, this rank's block.  `matmul` is the local operator; it defaults to
    locomp_b200.quantized_matmul and exists as a parameter so the host-side logic can be
    exercised without a GPU.
    """

    def __init__(self, w, scales, group_size: int = 32, bits: int = 4, group: Optional[dist.ProcessGroup] = None,
                 already_local: bool = False, n_total: Optional[int] = None, matmul: Optional[Callable] = None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.group_size, self.bits = group_size, bits
        if already_local:
            self.n_local = w.shape[0]
            self.n_total = n_total if n_total is not None else self.n_local * self.world
            if self.n_total != self.n_local * self.world:
                raise ValueError("local shards must all hold N / world rows")
            self.w, self.scales = w, scales
        else:
            self.n_total = w.shape[0]
            r0, r1 = shard_rows(self.n_total, self.world, self.rank)
            self.n_local = r1 - r0
            self.w, self.scales = w[r0:r1], scales[r0:r1]       # contiguous row blocks: views, no copy
        if matmul is None:
            from .ops import quantized_matmul
            matmul = quantized_matmul
        self._matmul = matmul
        self._gather_buf = None

    def local(self, x, **kw):
        """This rank's columns only: [M, N/G]."""
        return self._matmul(x, self.w, self.scales, self.group_size, bits=self.bits, **kw)

    def forward(self, x, layout: str = "row_major", **kw):
        """Full output on every rank.  x: [K] or [M, K], replicated on all ranks."""
        if layout not in ("row_major", "gathered"):
            raise ValueError("layout must be 'row_major' or 'gathered'")
        squeeze = x.dim() == 1
        y = self.local(x.unsqueeze(0) if squeeze else x, **kw)       # [M, N/G]
        m = y.shape[0]
        if self.world == 1:
            full = y.unsqueeze(0)
        else:
            buf = self._gather_buf
            if buf is None or buf.shape != (self.world, m, self.n_local) or buf.dtype != y.dtype or buf.device != y.device:
                buf = torch.empty((self.world, m, self.n_local), dtype=y.dtype, device=y.device)
                self._gather_buf = buf
            # concatenation form of the output (accepted by both NCCL and gloo)
            dist.all_gather_into_tensor(buf.view(self.world * m, self.n_local), y.contiguous(), group=self.group)
            full = buf
        if layout == "gathered":
            return full
        out = full.permute(1, 0, 2).reshape(m, self.n_total)           # a view when M == 1
        return out[0] if squeeze else out
