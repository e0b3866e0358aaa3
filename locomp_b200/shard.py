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


class PeerGather:
    """All-gather of equal slices over NVLink peer memory (see include/locomp_b200.h,
    lcq_allgather_push): every rank pushes its slice into every rank's region with one kernel.

    One instance owns one region on this rank plus mappings of the peers' regions.  Set-up
    (allocation, exchange of CUDA IPC handles through the process group, a barrier) happens in the
    constructor; `push(src)` is the hot call: one kernel launch, no allocation, no NCCL.
    """

    def __init__(self, bytes_per_rank: int, group: Optional[dist.ProcessGroup] = None):
        import ctypes
        from . import _lib
        self._lib, self._ct = _lib, ctypes
        L = _lib.lib()
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if bytes_per_rank <= 0 or bytes_per_rank % 16:
            raise ValueError("slices must be a positive multiple of 16 bytes")
        if self.world > 8:
            raise ValueError("PeerGather supports up to 8 ranks of one box")
        self.bytes_per_rank = bytes_per_rank
        self.device = torch.cuda.current_device()
        region_bytes = L.lcq_peer_region_bytes(bytes_per_rank, self.world)
        mine = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(64)
        _lib.check(L.lcq_peer_alloc(region_bytes, ctypes.byref(mine), handle))
        self._mine = mine.value
        handles = [None] * self.world
        dist.all_gather_object(handles, handle.raw, group=group)
        self._regions = (ctypes.c_void_p * self.world)()
        self._opened = []
        for r in range(self.world):
            if r == self.rank:
                self._regions[r] = self._mine
            else:
                p = ctypes.c_void_p()
                _lib.check(L.lcq_peer_open(handles[r], ctypes.byref(p)))
                self._regions[r] = p.value
                self._opened.append(p.value)
        self._state = torch.zeros(2, dtype=torch.int32, device=torch.device("cuda", self.device))
        torch.cuda.synchronize()
        dist.barrier(group=group)                   # every region is mapped everywhere before the first push

    def gathered(self, dtype: torch.dtype, shape) -> torch.Tensor:
        """Zero-copy torch view of this rank's gathered data area ([world, ...slice shape])."""
        class _Mem:
            pass
        m = _Mem()
        n = 1
        for d in shape:
            n *= d
        itemsize = torch.empty(0, dtype=dtype).element_size()
        if n * itemsize != self.world * self.bytes_per_rank:
            raise ValueError("shape does not match the region")
        m.__cuda_array_interface__ = {"shape": (self.world * self.bytes_per_rank,), "typestr": "|u1",
                                      "data": (self._mine + 256, False), "version": 3}
        self._keep = m
        return torch.as_tensor(m, device=torch.device("cuda", self.device)).view(dtype).view(*shape)

    def push(self, src: torch.Tensor, stream=None) -> None:
        """Enqueue the all-gather of `src` (this rank's slice, contiguous, bytes_per_rank bytes)."""
        if src.numel() * src.element_size() != self.bytes_per_rank or not src.is_contiguous():
            raise ValueError("src must be a contiguous tensor of bytes_per_rank bytes")
        sp = torch.cuda.current_stream().cuda_stream if stream is None else int(stream)
        self._lib.check(self._lib.lib().lcq_allgather_push(src.data_ptr(), self.bytes_per_rank, self._regions,
                                                           self.rank, self.world, self._state.data_ptr(), sp))

    def close(self) -> None:
        L = self._lib.lib()
        torch.cuda.synchronize()
        for p in self._opened:
            L.lcq_peer_close(p)
        self._opened = []
        if self._mine:
            L.lcq_peer_free(self._mine)
            self._mine = None


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
                 already_local: bool = False, n_total: Optional[int] = None, matmul: Optional[Callable] = None,
                 gather: str = "nccl"):
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
        if gather not in ("nccl", "nvlink"):
            raise ValueError("gather must be 'nccl' or 'nvlink'")
        self.gather = gather            # "nvlink": PeerGather (peer stores), two regions used alternately
        self._peer = {}                 # (m, dtype) -> [PeerGather, PeerGather], next index

    def prepare(self, m: int, dtype: torch.dtype) -> None:
        """Set up what `forward` needs for M = m outputs of `dtype`, so that the hot call allocates
        nothing and runs no collective of its own: with gather="nvlink" the two peer-memory regions
        (a cudaMalloc, an exchange of IPC handles through the process group and a barrier -- every
        rank must call prepare with the same arguments); with gather="nccl" the gathered buffer.
        Call it before capturing `forward` in a CUDA graph."""
        if self.world == 1:
            return
        if self.gather == "nvlink":
            key = (m, dtype)
            if key not in self._peer:
                nbytes = m * self.n_local * torch.empty(0, dtype=dtype).element_size()
                self._peer[key] = [[PeerGather(nbytes, self.group), PeerGather(nbytes, self.group)], 0]
        else:
            dev = self.w.device
            buf = self._gather_buf
            if buf is None or buf.shape != (self.world, m, self.n_local) or buf.dtype != dtype:
                self._gather_buf = torch.empty((self.world, m, self.n_local), dtype=dtype, device=dev)

    def close(self) -> None:
        """Release the peer-memory regions (every rank, after its last forward has completed).
        Destroy CUDA graphs that captured `forward` first, and call this -- and destroy those
        graphs -- before torch.distributed.destroy_process_group(): a graph that still holds
        captured NCCL work keeps the communicator busy and its destruction then blocks."""
        for pair, _ in self._peer.values():
            for pg in pair:
                pg.close()
        self._peer = {}
        self._gather_buf = None

    def local(self, x, **kw):
        """This rank's columns only: [M, N/G]."""
        return self._matmul(x, self.w, self.scales, self.group_size, bits=self.bits, **kw)

    def forward(self, x, layout: str = "row_major", **kw):
        """Full output on every rank.  x: [K] or [M, K], replicated on all ranks.

        Lifetime of the result: with layout="gathered" (and for M = 1, where the row-major form is
        a view of it) the returned tensor aliases the layer's gather buffer -- with gather="nccl"
        it is overwritten by the next forward, with gather="nvlink" by the forward after the next
        (two regions alternate; peers write into them).  Copy it if it must live longer.  For
        M > 1 layout="row_major" returns a fresh tensor."""
        if layout not in ("row_major", "gathered"):
            raise ValueError("layout must be 'row_major' or 'gathered'")
        squeeze = x.dim() == 1
        y = self.local(x.unsqueeze(0) if squeeze else x, **kw)       # [M, N/G]
        m = y.shape[0]
        if self.world == 1:
            full = y.unsqueeze(0)
        elif self.gather == "nvlink":
            key = (m, y.dtype)
            if key not in self._peer:
                self.prepare(m, y.dtype)          # first use: allocates and synchronises the ranks
            pair, nxt = self._peer[key]
            pg = pair[nxt]
            self._peer[key][1] = nxt ^ 1          # back-to-back calls alternate regions
            pg.push(y.contiguous())
            full = pg.gathered(y.dtype, (self.world, m, self.n_local))
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
