"""Quantized linear layers as a decode loop holds them: weights resident on the GPU, one call
per projection, nothing allocated per call.

`QuantLinear` replaces the `_matvec(W, x, out, N, K)` call sites of the reference's SmolLM2 loop
(examples/54_smollm2_inference.py:491-492, :503-574) with a quantized weight.  `fuse_rows`
concatenates projections that read the same activation (q|k|v, gate|up) into one weight: rows of
W are independent, so the fused output is the concatenation of the separate outputs, with one
launch and one read of x instead of several (the dense analogue is examples/42_fused_qkv.py:83-105).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from .ops import matmul_workspace_bytes, quantized_matmul
from .tensor import _TORCH_TO_KIND


class QuantLinear:
    """y = x @ dequant(W)^T with W int4 (uint8 [N, K/2]) or int8 ([N, K]) and per-group scales."""

    def __init__(self, w: torch.Tensor, scales: torch.Tensor, group_size: int = 32, bits: int = 4):
        if not (w.is_cuda and scales.is_cuda):
            raise ValueError("QuantLinear keeps its weights on a CUDA device")
        self.w, self.scales = w.contiguous(), scales.contiguous()
        self.group_size, self.bits = group_size, bits
        self.out_features = w.shape[0]
        self.in_features = w.shape[1] * (2 if bits == 4 else 1)

    def __call__(self, x: torch.Tensor, out: Optional[torch.Tensor] = None, **kw) -> torch.Tensor:
        return quantized_matmul(x, self.w, self.scales, self.group_size, bits=self.bits, out=out, **kw)

    @property
    def weight_bytes(self) -> int:
        return self.w.numel() * self.w.element_size() + self.scales.numel() * self.scales.element_size()


def fuse_rows(parts: Sequence[Tuple[torch.Tensor, torch.Tensor]], group_size: int = 32, bits: int = 4):
    """Stack the rows of several (w, scales) pairs that share K.  Returns (QuantLinear, splits)
    where splits[i] = (start, stop) of part i in the fused output."""
    if not parts:
        raise ValueError("nothing to fuse")
    k_bytes = parts[0][0].shape[1]
    for w, s in parts:
        if w.shape[1] != k_bytes or s.shape[1] != parts[0][1].shape[1]:
            raise ValueError("fused projections must share K and the group size")
    w = torch.cat([p[0] for p in parts], dim=0)
    s = torch.cat([p[1] for p in parts], dim=0)
    splits, r = [], 0
    for p in parts:
        splits.append((r, r + p[0].shape[0]))
        r += p[0].shape[0]
    return QuantLinear(w, s, group_size, bits), splits


class DecodeStack:
    """The quantized linears of one decode step of a Llama-style stack (SmolLM2 shapes by default),
    chained on fixed activation buffers: q|k|v, o, gate|up, down per layer, then the lm_head.
    Only the linears run -- attention, norms and activations between them are not part of this
    path -- so every linear reads a prepared activation buffer of its input width.
    `fused=True` uses one launch for q|k|v and one for gate|up (4 launches per layer instead of 7).
    `glue=True` (with fused) also runs what sits between the linears in the reference's layer
    (examples/54_smollm2_inference.py:494-554, :556-578) except attention itself: embedding lookup,
    input RMS norm, residual add + post-attention norm (one kernel), SiLU * up, residual add, final
    norm, and a greedy argmax of the logits on the device -- a real dependency chain on one hidden
    state, 8 launches per layer."""

    def __init__(self, layers: int = 30, hidden: int = 576, inter: int = 1536, q_heads: int = 9, kv_heads: int = 3,
                 head_dim: int = 64, vocab: int = 49152, fused: bool = False, device="cuda", seed: int = 0,
                 dtype=torch.float16, glue: bool = False):
        g = torch.Generator(device=device).manual_seed(seed)

        def make(n, k):
            w = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device=device, generator=g)
            s = (torch.randn(n, k // 32, device=device, generator=g).abs() * 0.02).to(torch.float16)
            return w, s
        qd, kvd = q_heads * head_dim, kv_heads * head_dim
        if glue and not fused:
            raise ValueError("glue=True runs the fused layer form")
        self.glue = glue
        self.ops = []                                  # with glue: the step as a list of zero-argument launches
        self.calls: List[Tuple[QuantLinear, torch.Tensor, torch.Tensor]] = []   # (linear, x, out)
        x_h = torch.randn(1, hidden, device=device, generator=g).to(dtype)
        x_i = torch.randn(1, inter, device=device, generator=g).to(dtype)
        x_q = torch.randn(1, qd, device=device, generator=g).to(dtype)

        def add(lin, x):
            self.calls.append((lin, x, torch.empty(1, lin.out_features, dtype=dtype, device=device)))
        if glue:
            from . import decode_ops as D
            self.table = (torch.randn(vocab, hidden, device=device, generator=g) * 0.02).to(dtype)
            self.token = torch.zeros(1, dtype=torch.int32, device=device)
            self.next_token = torch.zeros(1, dtype=torch.int32, device=device)
            self.hidden = torch.zeros(1, hidden, dtype=dtype, device=device)
            self.normed = torch.zeros(1, hidden, dtype=dtype, device=device)
            self.mlp = torch.zeros(1, inter, dtype=dtype, device=device)

            def lin_op(lin, x):
                out = torch.empty(1, lin.out_features, dtype=dtype, device=device)
                self.calls.append((lin, x, out))
                self.ops.append(lambda: lin(x, out=out, workspace_buf=self.workspace))
                return out
            self.ops.append(lambda: D.embed_lookup(self.token, self.table, self.hidden, 1, hidden))
            for _ in range(layers):
                q, k, v, o = make(qd, hidden), make(kvd, hidden), make(kvd, hidden), make(hidden, qd)
                gate, up, down = make(inter, hidden), make(inter, hidden), make(hidden, inter)
                w_in = (1 + 0.1 * torch.randn(hidden, device=device, generator=g)).to(dtype)
                w_post = (1 + 0.1 * torch.randn(hidden, device=device, generator=g)).to(dtype)
                self.ops.append(lambda w=w_in: D.rms_norm(self.hidden, w, 1e-5, out=self.normed))
                lin_op(fuse_rows([q, k, v])[0], self.normed)
                o_out = lin_op(QuantLinear(*o), x_q)            # attention is not part of this path: o reads a prepared buffer
                self.ops.append(lambda w=w_post, d=o_out: D.residual_rms_norm(self.hidden, d, w, 1e-5, out=self.normed))
                gu = lin_op(fuse_rows([gate, up])[0], self.normed)
                self.ops.append(lambda gu=gu: D.silu_mul(gu[:, :inter], gu[:, inter:], out=self.mlp))
                d_out = lin_op(QuantLinear(*down), self.mlp)
                self.ops.append(lambda d=d_out: D.add_inplace(self.hidden, d))
            w_fin = (1 + 0.1 * torch.randn(hidden, device=device, generator=g)).to(dtype)
            self.ops.append(lambda: D.rms_norm(self.hidden, w_fin, 1e-5, out=self.normed))
            self.logits = lin_op(QuantLinear(*make(vocab, hidden)), self.normed)
            self.ops.append(lambda: D.argmax(self.logits, out=self.next_token))
            layers = 0                                 # the plain construction below adds nothing more
        for _ in range(layers):
            q, k, v, o = make(qd, hidden), make(kvd, hidden), make(kvd, hidden), make(hidden, qd)
            gate, up, down = make(inter, hidden), make(inter, hidden), make(hidden, inter)
            if fused:
                add(fuse_rows([q, k, v])[0], x_h)
                add(QuantLinear(*o), x_q)
                add(fuse_rows([gate, up])[0], x_h)
                add(QuantLinear(*down), x_i)
            else:
                for p in (q, k, v):
                    add(QuantLinear(*p), x_h)
                add(QuantLinear(*o), x_q)
                add(QuantLinear(*gate), x_h)
                add(QuantLinear(*up), x_h)
                add(QuantLinear(*down), x_i)
        if not glue:
            add(QuantLinear(*make(vocab, hidden)), x_h)
        self.launches_per_step = len(self.ops) if glue else len(self.calls)
        self.weight_bytes = sum(c[0].weight_bytes for c in self.calls)
        # one scratch buffer for the whole stack (calls are stream-ordered), allocated up front so
        # that nothing is allocated while a CUDA graph is being captured
        kind = _TORCH_TO_KIND[dtype]
        need = max(matmul_workspace_bytes(1, c[0].out_features, c[0].in_features, 32, 4, kind, "f16", kind)
                   for c in self.calls)
        self.workspace = torch.zeros(max(need, 256), dtype=torch.uint8, device=device)
        self._graph = None

    def step(self):
        if self.glue:
            for op in self.ops:
                op()
            return
        for lin, x, out in self.calls:
            lin(x, out=out, workspace_buf=self.workspace)

    def capture(self):
        """Record the whole step in one CUDA graph (launch-bound otherwise)."""
        self.step()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        s = torch.cuda.Stream()
        with torch.cuda.graph(g, stream=s):
            self.step()
        self._graph = g
        return g

    def replay(self):
        self._graph.replay()
