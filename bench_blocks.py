"""Secondary measurements of bench.py: every benchmark configuration besides the headline sweep,
each as one small block of the JSON line (config 1 int8 matvec, config 3 decode stack, config 4
prefill GEMM, config 5 column-sharded 70B-class shapes, the dequantize operator, and the
resident-weights end-to-end figure).  All timings are CUDA events on the launching stream around
CUDA-graph replays of back-to-back launches over rotating weight buffers larger than L2.
"""
from __future__ import annotations

import hashlib
import os
import statistics

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
GROUP = 32
L2_ROTATE_BYTES = 450e6          # rotate over at least this many weight bytes (L2 is 126 MB)


def weight_bytes(k: int, n: int, bits: int = 4, scale_bytes: int = 2, group: int = GROUP) -> int:
    return n * k * bits // 8 + n * (k // group) * scale_bytes


def source_hash(*names: str) -> str:
    """Short hash of kernel sources: ties a recorded ncu traffic figure to the code it was taken from."""
    h = hashlib.sha256()
    for name in names:
        with open(os.path.join(ROOT, "locomp_b200", "csrc", name), "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:12]


class Ctx:
    """What every block needs: modules, device, stream, peaks, rank info."""

    def __init__(self, torch, lib, _lib, L, dev, peaks, rank=0, world=1, dist=None):
        self.torch, self.lib, self._lib, self.L, self.dev = torch, lib, _lib, L, dev
        self.peaks, self.rank, self.world, self.dist = peaks, rank, world, dist
        self.stream = torch.cuda.Stream(device=dev)
        self.launches = 0            # kernels of this library launched inside timed regions

    def check(self):
        self._lib.check(self.lib.lcq_check_device_status(None))

    def max_over_ranks(self, value: float) -> float:
        if self.dist is None:
            return value
        t = self.torch.tensor([value], device=self.dev, dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())


def graph_us(ctx: Ctx, launchers, min_launches: int = 200, replays: int = 3, per_launch_kernels: int = 1,
             sync_ranks: bool = False) -> float:
    """Average microseconds per launcher call: the launchers (one per rotating buffer set) are
    captured back to back in one CUDA graph, `reps` times over, and the graph is replayed `replays`
    times between two events on the launching stream; the median replay is reported."""
    torch = ctx.torch
    st = ctx.stream
    n = len(launchers)
    reps = max(1, -(-min_launches // n))
    torch.cuda.synchronize()                      # inputs were made on the default stream; `st` does not wait for it
    with torch.cuda.stream(st):
        for f in launchers:                       # eager warm-up: sets kernel attributes before capture
            f(st.cuda_stream)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=st):
        sp = torch.cuda.current_stream().cuda_stream
        for _ in range(reps):
            for f in launchers:
                f(sp)
    times = []
    with torch.cuda.stream(st):
        g.replay()                                # warm replay
        for _ in range(replays):
            if sync_ranks and ctx.dist is not None:
                torch.cuda.synchronize()
                ctx.dist.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(st)
            g.replay()
            b.record(st)
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b) * 1e3 / (reps * n))
    ctx.launches += replays * reps * n * per_launch_kernels
    del g
    return statistics.median(times)


class Problem:
    """One quantized-linear problem with `nbuf` rotating copies of its weights, bound to the C ABI."""

    def __init__(self, ctx: Ctx, k: int, n: int, m: int, x_kind: str = "f16", bits: int = 4, group: int = GROUP,
                 scale_kind: str = "f16", nbuf: int = 0, seed: int = 0, algo: int = 0):
        torch, _lib = ctx.torch, ctx._lib
        self.ctx, self.k, self.n, self.m, self.bits, self.group, self.algo = ctx, k, n, m, bits, group, algo
        tdt = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}
        code = {"f16": _lib.F16, "bf16": _lib.BF16, "f32": _lib.F32}
        self.xc, self.sc = code[x_kind], code[scale_kind]
        sb = 2 if scale_kind != "f32" else 4
        self.wbytes = weight_bytes(k, n, bits, sb, group)
        if nbuf <= 0:
            nbuf = max(2, min(64, int(L2_ROTATE_BYTES // self.wbytes) + 1))
        g = torch.Generator(device=ctx.dev).manual_seed(seed)
        self.w, self.s = [], []
        for _ in range(nbuf):
            if bits == 4:
                self.w.append(torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device=ctx.dev, generator=g))
                self.s.append((torch.randn(n, k // group, device=ctx.dev, generator=g).abs() * 0.02).to(tdt[scale_kind]))
            else:
                self.w.append(torch.randint(-127, 128, (n, k), dtype=torch.int8, device=ctx.dev, generator=g))
                self.s.append((torch.randn(n, k // group, device=ctx.dev, generator=g).abs() * 0.01).to(tdt[scale_kind]))
        self.x = torch.randn(m, k, device=ctx.dev, generator=g).to(tdt[x_kind])
        self.out = torch.empty(m, n, dtype=tdt[x_kind], device=ctx.dev)
        need = ctx.lib.lcq_matmul_workspace_bytes(bits, m, n, k, group, self.xc, self.sc, self.xc, algo)
        assert need != (1 << 64) - 1, "no kernel covers this problem"
        self.ws = torch.zeros(max(need, 256), dtype=torch.uint8, device=ctx.dev)
        self.fn = ctx.lib.lcq_matmul_int4 if bits == 4 else ctx.lib.lcq_matmul_int8
        self.selected = ctx.lib.lcq_matmul_select_algo(bits, m, n, k, group, self.xc, self.sc, self.xc) if algo == 0 else algo

    def launcher(self, i: int):
        w, s = self.w[i], self.s[i]
        args = (self.x.data_ptr(), w.data_ptr(), s.data_ptr(), self.out.data_ptr(), self.m, self.n, self.k, self.group,
                self.xc, self.sc, self.xc, self.algo, self.ws.data_ptr(), self.ws.numel())

        def f(sp):
            rc = self.fn(*args, sp)
            if rc != 0:
                raise RuntimeError(self.ctx.lib.lcq_last_error().decode())
        return f

    def launchers(self):
        return [self.launcher(i) for i in range(len(self.w))]

    def kernel_name(self) -> str:
        _lib = self.ctx._lib
        return {_lib.ALGO_SIMT: "gemv_simt_kernel", _lib.ALGO_GEMV_TC: "w4a16_gemv_kernel", _lib.ALGO_GEMM_TC: "w4a16_gemm_kernel",
                _lib.ALGO_GEMV_W8: "w8_gemv_kernel"}.get(self.selected, "?")


# ------------------------------------------------------------------------------------------ roofline of the dominant kernel
# dram__bytes_read.sum + dram__bytes_write.sum per launch, from the ncu captures summarised under
# profiles/, valid only for the kernel source they were taken from: {source hash: {(K, N, M): bytes}}
TRAFFIC_NCU = {
    "011311b5b0e9": {(2048, 49152, 1): 56_690_000, (2048, 49152, 16): 56_810_000, (2048, 8192, 1): 9_469_952},
}


def block_roofline(ctx: Ctx, k: int, n: int, m: int) -> dict:
    """HBM roofline of the decode kernel on one problem: algorithmic bytes (packed weights + scales)
    over the average duration of >= 200 back-to-back launches on rotating weight buffers."""
    pr = Problem(ctx, k, n, m, seed=77)
    us = graph_us(ctx, pr.launchers(), min_launches=200, replays=5)
    ctx.check()
    achieved = pr.wbytes / us / 1e3
    sha = source_hash("gemv_tc.cuh", "common.cuh")
    traffic = TRAFFIC_NCU.get(sha, {}).get((k, n, m))
    return {"bound": "hbm", "kernel": f"{pr.kernel_name()} M={m} K={k} N={n}", "achieved": achieved,
            "peak": ctx.peaks["hbm_gbs"], "peak_source": ctx.peaks["source"], "unit": "GB/s",
            "frac": achieved / ctx.peaks["hbm_gbs"], "avg_launch_us": us,
            "launches_timed": 5 * max(1, -(-200 // len(pr.w))) * len(pr.w), "timing": "CUDA graph of back-to-back launches, median of 5 replays",
            "algorithmic_bytes_per_launch": pr.wbytes, "traffic": traffic, "traffic_source_hash": sha}


# ------------------------------------------------------------------------------------------ config 1: int8 matvec, fp32
def block_cfg1(ctx: Ctx) -> dict:
    """M=1, K=576, N=1536, int8 weights, per-output-channel float32 scales, float32 x and out."""
    k, n = 576, 1536
    pr = Problem(ctx, k, n, 1, x_kind="f32", bits=8, group=k, scale_kind="f32", seed=1)
    us = graph_us(ctx, pr.launchers(), min_launches=400)
    ctx.check()
    algo_bytes = n * k + 4 * n + 4 * k + 4 * n
    gbs = algo_bytes / us / 1e3
    return {"workload": "cfg1: int8 GEMV M=1 K=576 N=1536, fp32 x/scales/out", "kernel": pr.kernel_name(),
            "us_per_call": us, "algorithmic_bytes": algo_bytes, "value": gbs, "unit": "GB/s",
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": ctx.peaks["hbm_gbs"], "frac": gbs / ctx.peaks["hbm_gbs"],
                         "note": "0.9 MB per call: launch latency, not bandwidth, bounds it"}}


# ------------------------------------------------------------------------------------------ dequantize operator
def block_dequant(ctx: Ctx) -> dict:
    """lcq_dequant_int4 on the largest prefill weight (4096 x 14336) -> float32: 4.56 B moved per weight."""
    torch, _lib = ctx.torch, ctx._lib
    n, k = 4096, 14336
    g = torch.Generator(device=ctx.dev).manual_seed(5)
    nbuf = 3
    ws = [torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device=ctx.dev, generator=g) for _ in range(nbuf)]
    ss = [(torch.randn(n, k // GROUP, device=ctx.dev, generator=g).abs() * 0.02).half() for _ in range(nbuf)]
    outs = [torch.empty(n, k, dtype=torch.float32, device=ctx.dev) for _ in range(nbuf)]

    def mk(i):
        def f(sp):
            rc = ctx.lib.lcq_dequant_int4(ws[i].data_ptr(), ss[i].data_ptr(), outs[i].data_ptr(), n, k, GROUP, _lib.F16, _lib.F32, sp)
            if rc != 0:
                raise RuntimeError(ctx.lib.lcq_last_error().decode())
        return f
    us = graph_us(ctx, [mk(i) for i in range(nbuf)], min_launches=30)
    moved = n * k // 2 + n * (k // GROUP) * 2 + 4 * n * k
    gbs = moved / us / 1e3
    return {"workload": "dequant_int4 4096x14336 -> f32", "kernel": "dequant_w4_words_kernel", "us_per_call": us,
            "algorithmic_bytes": moved, "value": gbs, "unit": "GB/s (read + written)",
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": ctx.peaks["hbm_gbs"], "frac": gbs / ctx.peaks["hbm_gbs"]}}


# ------------------------------------------------------------------------------------------ config 3: decode stack
def block_cfg3(ctx: Ctx, steps: int = 20) -> dict:
    """One decode step of the 30-layer SmolLM2-135M-shaped stack, quantized linears only (211 launches;
    121 with q|k|v and gate|up fused), and the same step with the norm / activation / residual kernels
    between the linears.  Four stacks rotate so a stack's 76 MB of weights is out of L2 when reused."""
    torch, L = ctx.torch, ctx.L
    out = {"workload": "cfg3: decode step of a 30-layer SmolLM2-135M-shaped stack, W4A16 g=32, M=1"}
    for name, fused, glue in (("us_per_token", False, False), ("us_per_token_fused_qkv_gateup", True, False),
                              ("us_per_token_fused_with_glue", True, True)):
        stacks = [L.DecodeStack(fused=fused, glue=glue, seed=100 + i) for i in range(4)]
        for stx in stacks:
            stx.capture()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for i in range(4):
            stacks[i].replay()
        a.record()
        for i in range(steps):
            stacks[i % 4].replay()
        b.record()
        torch.cuda.synchronize()
        out[name] = a.elapsed_time(b) / steps * 1e3
        out["launches_" + name] = stacks[0].launches_per_step
        ctx.launches += steps * stacks[0].launches_per_step
        if not fused:
            out["weight_bytes"] = stacks[0].weight_bytes
        del stacks
    ctx.check()
    out["weight_gbs"] = out["weight_bytes"] / out["us_per_token"] / 1e3
    out["roofline_lm_head"] = block_roofline(ctx, 576, 49152, 1)
    return out


# ------------------------------------------------------------------------------------------ config 4: prefill GEMM
CFG4_SHAPES = [(4096, 4096), (4096, 14336), (14336, 4096)]
CFG4_MS = [512, 2048, 8192]


def block_cfg4(ctx: Ctx) -> dict:
    """W4A16 g=32 prefill GEMM, bf16 activations and outputs, M in {512, 2048, 8192} x the
    Llama-3-8B-like shapes; TFLOP/s = 2*M*N*K / device time, including the bf16->fp16 pre-pass."""
    per_call, tot_flops, tot_us = {}, 0.0, 0.0
    top = None
    for (k, n) in CFG4_SHAPES:
        for m in CFG4_MS:
            pr = Problem(ctx, k, n, m, x_kind="bf16", nbuf=max(2, int(300e6 // weight_bytes(k, n)) + 1), seed=k + n + m)
            assert pr.selected == ctx._lib.ALGO_GEMM_TC
            flops = 2.0 * m * n * k
            us = graph_us(ctx, pr.launchers(), min_launches=max(8, int(4000 // max(1.0, flops / 1.0e9))), per_launch_kernels=2)
            per_call[f"M{m}_K{k}_N{n}"] = round(flops / us / 1e6, 1)
            tot_flops += flops
            tot_us += us
            if (k, n, m) == (4096, 14336, 8192):
                top = (flops / us / 1e6, us, flops)
            del pr
    ctx.check()
    peaks = ctx.peaks
    return {"workload": "cfg4: W4A16 g=32 prefill GEMM, bf16, M in {512,2048,8192} x (K,N) in {(4096,4096),(4096,14336),(14336,4096)}",
            "value": tot_flops / tot_us / 1e6, "unit": "TFLOP/s", "tflops_per_call": per_call,
            "roofline": {"bound": "tensor", "kernel": "w4a16_gemm_kernel (+ bf16->f16 pre-pass) M=8192 K=4096 N=14336",
                         "achieved": top[0], "peak": peaks["bf16_tflops"], "peak_sustained": peaks["bf16_tflops_sustained"],
                         "peak_source": peaks["source"] + " (burst)", "unit": "TFLOP/s", "frac": top[0] / peaks["bf16_tflops"],
                         "frac_of_sustained": top[0] / peaks["bf16_tflops_sustained"], "avg_launch_us": top[1],
                         "algorithmic_flops_per_launch": top[2], "traffic": None}}


# ------------------------------------------------------------------------------------------ config 5: column-sharded 70B-class shapes
CFG5_SHAPES = [(8192, 28672), (28672, 8192), (8192, 128256)]
CFG5_MS = [1, 16, 64]


def block_cfg5(ctx: Ctx, gather: str = "nccl") -> dict:
    """The 70B-class shapes split along N over the ranks (strong scaling): every rank runs the
    single-GPU kernel on N / world rows and the [M, N] output is reassembled by an all-gather.  Per
    (shape, M): device time of the compute alone and of compute + gather, each the max over ranks.
    Aggregate weight GB/s = all weight bytes of the nine calls / sum of their compute+gather times."""
    torch, dist, world, L = ctx.torch, ctx.dist, ctx.world, ctx.L
    rows, tot_bytes, tot_us_c, tot_us_g = {}, 0, 0.0, 0.0
    for (k, n) in CFG5_SHAPES:
        assert n % world == 0
        nl = n // world
        for m in CFG5_MS:
            nbuf = max(2, int(L2_ROTATE_BYTES // weight_bytes(k, nl)) + 1)
            pr = Problem(ctx, k, nl, m, nbuf=nbuf, seed=1000 * ctx.rank + k + n + m)
            kernels = -(-m // 16) if pr.selected == ctx._lib.ALGO_GEMV_TC else 1
            launchers = pr.launchers()
            us_c = ctx.max_over_ranks(graph_us(ctx, launchers, min_launches=40, per_launch_kernels=kernels, sync_ranks=True))
            us_g = us_c
            if world > 1:
                if gather == "nvlink":
                    pgs = [L.PeerGather(m * nl * 2), L.PeerGather(m * nl * 2)]   # two regions used alternately
                    cnt = [0]

                    def with_gather(f):
                        def h(sp):
                            f(sp)
                            pgs[cnt[0] & 1].push(pr.out, stream=sp)
                            cnt[0] += 1
                        return h
                else:
                    full = torch.empty(world, m, nl, dtype=pr.out.dtype, device=ctx.dev)

                    def with_gather(f):
                        def h(sp):
                            f(sp)
                            dist.all_gather_into_tensor(full.view(world * m, nl), pr.out)
                        return h
                glaunch = [with_gather(f) for f in launchers]
                if len(glaunch) % 2:
                    glaunch = glaunch[:-1] if len(glaunch) > 2 else glaunch + glaunch   # even count keeps the two regions alternating across replays
                us_g = ctx.max_over_ranks(graph_us(ctx, glaunch, min_launches=40, per_launch_kernels=kernels + 1, sync_ranks=True))
                if gather == "nvlink":
                    torch.cuda.synchronize()
                    dist.barrier()
                    for pg in pgs:
                        pg.close()
            rows[f"M{m}_K{k}_N{n}"] = {"compute_us": round(us_c, 2), "compute_plus_gather_us": round(us_g, 2),
                                      "weight_gbs_aggregate": round(weight_bytes(k, n) / us_g / 1e3, 1)}
            tot_bytes += weight_bytes(k, n)
            tot_us_c += us_c
            tot_us_g += us_g
            del pr
    ctx.check()
    return {"workload": f"cfg5: (K,N) in {CFG5_SHAPES} x M in {CFG5_MS}, W4A16 g=32 fp16, N split over {world} rank(s)",
            "scaling": "strong", "gather": None if world == 1 else ("NVLink peer-store kernel" if gather == "nvlink" else "NCCL all-gather"),
            "value": tot_bytes / tot_us_g / 1e3, "unit": "GB/s (aggregate weight bytes / compute+gather time)",
            "value_compute_only": tot_bytes / tot_us_c / 1e3, "per_call": rows}


# ------------------------------------------------------------------------------------------ end to end with resident weights
def block_e2e_resident(ctx: Ctx, shapes, ms, steps: int = 10) -> dict:
    """The way a decode loop calls the path: weights stay on the GPU in QuantLinear layers; per call x
    goes up from pinned host memory and y comes back.  Same sweep and metric as the headline."""
    torch, L = ctx.torch, ctx.L
    layers, xs, h2d, d2h, nbytes = [], [], 0, 0, 0
    g = torch.Generator(device=ctx.dev).manual_seed(9)
    for (k, n) in shapes:
        w = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device=ctx.dev, generator=g)
        s = (torch.randn(n, k // GROUP, device=ctx.dev, generator=g).abs() * 0.02).half()
        layers.append(L.QuantLinear(w, s))
        xs.append(torch.randn(16, k).half().pin_memory())
        for m in ms:
            h2d += m * k * 2
            d2h += m * n * 2
            nbytes += weight_bytes(k, n)
    outs = {(i, m): torch.empty(m, lay.out_features, dtype=torch.float16).pin_memory() for i, lay in enumerate(layers) for m in ms}

    def step():
        for i, lay in enumerate(layers):
            for m in ms:
                xd = xs[i][:m].to(ctx.dev, non_blocking=True)
                outs[(i, m)].copy_(lay(xd), non_blocking=True)
        torch.cuda.synchronize()
    step()
    import time
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = ctx.max_over_ranks(time.perf_counter() - t0)
    ctx.launches += steps * len(layers) * len(ms)
    return {"value": nbytes * ctx.world * steps / dt / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "steps": steps, "call": "locomp_b200.QuantLinear(x): weights resident on the GPU, x uploaded from pinned host memory "
                                    "and y copied back to pinned host memory every call"}
