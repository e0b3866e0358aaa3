#!/usr/bin/env python
"""Benchmark of the weight-quantized matmul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload cfg2|cfg4|cfg5]

Default workload (cfg2): the W4A16 g=32 decode sweep -- M in {1, 4, 16} over the SmolLM2-1.7B
projection shapes (K, N) in {(2048,2048), (2048,8192), (8192,2048), (2048,49152)}.  One step is
one pass over the 12 (shape, M) calls.  Metric: weight-HBM GB/s = (packed + scale bytes of all
calls) / device time.  Every call of a step reads its own weight buffer and steps rotate through
several sets of buffers, so no weight byte is re-read within ~700 MB of traffic (L2 is 126 MB).

With --gpus N > 1 (launched under torchrun, one rank per GPU) each rank holds an N-column shard
of every linear -- the shard has the cfg2 shape, so per-GPU work is fixed (weak scaling) and the
global linear is N times wider -- and the outputs are reassembled with an NCCL all-gather inside
the timed region.

The same JSON line carries one block per other configuration (bench_blocks.py): "cfg1" (int8
matvec), "cfg3" (decode stack, microseconds per token), "cfg4" (prefill GEMM TFLOP/s), "cfg5"
(70B-class shapes split along N over the ranks: compute-only and compute+gather), "dequant", and
"e2e_resident" (weights resident, x up / y down per call).

--impl reference times the reference's CPU path (the NumPy dequantise-then-BLAS matvec of
examples/38_quantized_matmul.py:215-232, restated in oracle/qmm_oracle.py) on the host cores.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CFG2_SHAPES = [(2048, 2048), (2048, 8192), (8192, 2048), (2048, 49152)]   # (K, N)
CFG2_MS = [1, 4, 16]
CFG4_SHAPES = [(4096, 4096), (4096, 14336), (14336, 4096)]
CFG4_MS = [512, 2048, 8192]
# cfg3: one decode step of a 30-layer SmolLM2-135M-shaped stack, quantized linears only: (K, N) per
# layer in call order q, k, v, o, gate, up, down, then the lm_head (examples/54_smollm2_inference.py:503-574)
CFG3_LAYER = [(576, 576), (576, 192), (576, 192), (576, 576), (576, 1536), (576, 1536), (1536, 576)]
CFG3_LM_HEAD = (576, 49152)
CFG5_SHAPES = [(8192, 28672), (28672, 8192), (8192, 128256)]
CFG5_MS = [1, 16, 64]
GROUP = 32


def weight_bytes(k: int, n: int) -> int:
    return n * k // 2 + n * (k // GROUP) * 2


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# --------------------------------------------------------------------------------------------
# clocks sampling during the timed region
# --------------------------------------------------------------------------------------------
_SAMPLER_CHILD = r"""
import sys, time, json
import pynvml
pynvml.nvmlInit()
h = pynvml.nvmlDeviceGetHandleByIndex(int(sys.argv[1]))
smax = pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)
print("ready", flush=True)
sys.stdin.readline()                      # "go"
import threading
stop = []
threading.Thread(target=lambda: (sys.stdin.readline(), stop.append(1)), daemon=True).start()
samples, mask = [], 0
while not stop:
    samples.append(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM))
    try:
        mask |= int(pynvml.nvmlDeviceGetCurrentClocksEventReasons(h))
    except Exception:
        mask |= int(pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(h))
    time.sleep(0.0005)
print(json.dumps({"samples": samples, "mask": mask, "smax": smax}), flush=True)
"""


class ClockSampler:
    """Samples SM clock and clock-event (throttle) reasons of one GPU through NVML about every
    millisecond between start() and stop().  It runs in a child process: the timed region is a
    few milliseconds of back-to-back launches during which a thread of this process would
    hardly get to run, and `nvidia-smi -lms` cannot sample faster than ~100 ms."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown"}

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self._err = None

    def prepare(self):
        """Start the child and let it set NVML up (slow): call before the timed region."""
        try:
            self.proc = subprocess.Popen([sys.executable, "-c", _SAMPLER_CHILD, str(self.gpu_index)],
                                         stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL,
                                         text=True)
            if self.proc.stdout.readline().strip() != "ready":
                raise RuntimeError("NVML sampler did not start")
        except Exception as e:
            self._err = repr(e)
            self.proc = None

    def start(self):
        if self.proc is not None:
            self.proc.stdin.write("go\n")
            self.proc.stdin.flush()

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": [self._err or "sampler not started"]}
        try:
            self.proc.stdin.write("stop\n")
            self.proc.stdin.flush()
            data = json.loads(self.proc.stdout.readline())
            self.proc.wait(timeout=5)
        except Exception as e:
            self.proc.kill()
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": [repr(e)]}
        samples = data["samples"]
        if not samples:
            return {"sm_mhz": None, "sm_max_mhz": data["smax"], "samples": 0, "reasons": ["no samples"]}
        reasons = sorted(name for bit, name in self.REASONS.items() if data["mask"] & bit)
        return {"sm_mhz": statistics.median(samples), "sm_min_mhz": min(samples), "sm_max_mhz": data["smax"],
                "samples": len(samples), "window": "warm-up steps + timed region", "reasons": reasons}


# --------------------------------------------------------------------------------------------
# reference arm: the reference's CPU path on the host cores
# --------------------------------------------------------------------------------------------
def run_reference(args, rank: int, world: int):
    if rank != 0:
        return
    from oracle import qmm_oracle as O
    rng = np.random.default_rng(0)
    cases = []
    for (k, n) in CFG2_SHAPES:
        wp, s = O.make_w4(rng, n, k, GROUP, np.float16)
        x = rng.standard_normal((16, k)).astype(np.float16)
        cases.append((k, n, wp, s, x))

    def sweep(sel):
        for (k, n, wp, s, x) in sel:
            for m in CFG2_MS:
                O.fast_matvec_int4(x[:m], wp, s, GROUP)

    # size the per-step sample from one full untimed sweep so the run ends within minutes
    t0 = time.perf_counter()
    sweep(cases)
    full = time.perf_counter() - t0
    total_steps = args.steps + args.warmup
    if full * total_steps <= 150.0:
        sel, sample = cases, "full cfg2 sweep (12 calls)"
    else:
        sel, sample = cases[:3], "cfg2 sweep without the (2048,49152) shape (9 calls)"
    nbytes = sum(weight_bytes(k, n) for (k, n, *_r) in sel) * len(CFG2_MS)
    for _ in range(args.warmup):
        sweep(sel)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        sweep(sel)
    dt = time.perf_counter() - t0
    value = nbytes * args.steps / dt / 1e9
    cores = os.cpu_count()
    line = {
        "impl": "reference", "metric": "w4a16_gemv_weight_hbm_gbs", "value": value, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "cfg2: W4A16 g=32 GEMV sweep, M in {1,4,16} x SmolLM2-1.7B shapes", "sample": sample},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": "port",
                         "sample": sample + "; NumPy dequantise-to-float32 + BLAS, as examples/38_quantized_matmul.py:215-232"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------
# our arm
# --------------------------------------------------------------------------------------------
class Call:
    """One (shape, M) quantized-linear call with device-resident operands, bound to the C ABI."""

    def __init__(self, lib, torch, k, n, m, dev, seed, x_dtype="f16"):
        from locomp_b200 import _lib
        g = torch.Generator(device=dev).manual_seed(seed)
        self.k, self.n, self.m = k, n, m
        self.w = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device=dev, generator=g)
        self.s = (torch.randn(n, k // GROUP, device=dev, generator=g).abs() * 0.02).to(torch.float16)
        xdt = torch.float16 if x_dtype == "f16" else torch.bfloat16
        self.x = torch.randn(m, k, device=dev, generator=g).to(xdt)
        self.out = torch.empty(m, n, dtype=xdt, device=dev)
        code = _lib.F16 if x_dtype == "f16" else _lib.BF16
        self.ws_bytes = lib.lcq_matmul_workspace_bytes(4, m, n, k, GROUP, code, _lib.F16, code, 0)
        assert self.ws_bytes != (1 << 64) - 1
        self.args = None
        self.lib = lib
        self.code = code

    def bind(self, ws):
        from locomp_b200 import _lib
        self.args = (self.x.data_ptr(), self.w.data_ptr(), self.s.data_ptr(), self.out.data_ptr(), self.m, self.n,
                     self.k, GROUP, self.code, _lib.F16, self.code, 0, ws.data_ptr(), ws.numel())

    def launch(self, stream_ptr):
        rc = self.lib.lcq_matmul_int4(*self.args, stream_ptr)
        if rc != 0:
            raise RuntimeError(f"lcq_matmul_int4 failed: {self.lib.lcq_last_error().decode()}")


def run_profile_shape(args):
    """A handful of launches of one (K, N, M) problem: the small case an `ncu` capture wants."""
    import torch
    from locomp_b200 import _lib
    lib = _lib.lib()
    k, n, m = (int(v) for v in args.profile_shape.lower().split("x"))
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    xdt = "bf16" if m > 16 else "f16"
    nbuf = max(2, min(8, int(300e6 // weight_bytes(k, n)) + 1))
    calls = [Call(lib, torch, k, n, m, dev, seed=i, x_dtype=xdt) for i in range(nbuf)]
    ws = torch.zeros(max(calls[0].ws_bytes, 256), dtype=torch.uint8, device=dev)
    for c in calls:
        c.bind(ws)
    sp = torch.cuda.current_stream().cuda_stream
    for i in range(args.warmup):
        calls[i % nbuf].launch(sp)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        calls[(args.warmup + i) % nbuf].launch(sp)
    e1.record()
    torch.cuda.synchronize()
    _lib.check(lib.lcq_check_device_status(None))
    us = e0.elapsed_time(e1) * 1e3 / args.steps
    print(json.dumps({"profile_shape": {"K": k, "N": n, "M": m}, "us_per_launch": us,
                      "weight_gbs": weight_bytes(k, n) / us / 1e3, "tflops": 2.0 * m * n * k / us / 1e6}), flush=True)


def run_profile_dequant(args):
    """A handful of launches of lcq_dequant_int4 on the 4096 x 14336 weight (-> float32): the small
    case an `ncu` capture of the dequantize kernel wants.  Three rotating buffer sets (800 MB)."""
    import torch
    from locomp_b200 import _lib
    lib = _lib.lib()
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    n, k = 4096, 14336
    g = torch.Generator(device=dev).manual_seed(5)
    ws = [torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device=dev, generator=g) for _ in range(3)]
    ss = [(torch.randn(n, k // GROUP, device=dev, generator=g).abs() * 0.02).half() for _ in range(3)]
    outs = [torch.empty(n, k, dtype=torch.float32, device=dev) for _ in range(3)]

    def launch(i):
        _lib.check(lib.lcq_dequant_int4(ws[i % 3].data_ptr(), ss[i % 3].data_ptr(), outs[i % 3].data_ptr(), n, k, GROUP,
                                        _lib.F16, _lib.F32, None))
    for i in range(args.warmup):
        launch(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        launch(args.warmup + i)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / args.steps
    moved = n * k // 2 + n * (k // GROUP) * 2 + 4 * n * k
    print(json.dumps({"profile_dequant": {"N": n, "K": k, "out": "f32"}, "us_per_launch": us, "gbs_moved": moved / us / 1e3}), flush=True)


def run_ours(args, rank: int, world: int, local_rank: int):
    import torch
    import locomp_b200 as L
    from locomp_b200 import _lib
    lib = _lib.lib()
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; there is no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import datetime
        import torch.distributed as dist_mod
        dist = dist_mod
        # Multi-GPU runs: no programmatic dependent launch next to NCCL kernels (it stays on with the
        # library's own all-gather kernel), and a short collective timeout so a stuck rank ends the run
        # instead of holding eight GPUs.
        if args.gather != "nvlink":
            os.environ["LCQ_NO_PDL"] = "1"
        os.environ.setdefault("TORCH_NCCL_ASYNC_ERROR_HANDLING", "1")
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=120))
    peaks = load_peaks()

    if args.workload == "cfg2":
        shapes, ms, xdt = CFG2_SHAPES, CFG2_MS, "f16"
    elif args.workload == "cfg3":
        shapes, ms, xdt = CFG3_LAYER * 30 + [CFG3_LM_HEAD], [1], "f16"
    elif args.workload == "cfg4":
        shapes, ms, xdt = CFG4_SHAPES, CFG4_MS, "bf16"
    else:
        shapes, ms, xdt = CFG5_SHAPES, CFG5_MS, "f16"

    # cfg5 is the strong-scaling form: the global N is split across ranks
    def local_n(n):
        if args.workload == "cfg5":
            assert n % world == 0
            return n // world
        return n

    per_set_bytes = sum(weight_bytes(k, local_n(n)) for (k, n) in shapes) * len(ms)
    nsets = max(2, min(8, int(np.ceil(640e6 / per_set_bytes))))
    sets = []
    for si in range(nsets):
        calls = []
        for ci, (k, n) in enumerate(shapes):
            for m in ms:
                calls.append(Call(lib, torch, k, local_n(n), m, dev, seed=1000 * si + 10 * ci + m + rank, x_dtype=xdt))
        sets.append(calls)
    ws = torch.zeros(max(max(c.ws_bytes for c in sets[0]), 256), dtype=torch.uint8, device=dev)
    for calls in sets:
        for c in calls:
            c.bind(ws)
    gathered = None
    peer = None
    if world > 1:
        gathered = [torch.empty(world, c.m, c.n, dtype=c.out.dtype, device=dev) for c in sets[0]]
        if args.gather == "nvlink":
            # one peer-memory region per call of a step; a region is pushed to again only one step later
            peer = [L.PeerGather(c.m * c.n * c.out.element_size()) for c in sets[0]]
    torch.cuda.synchronize()

    def gather_call(ci, c):
        if peer is not None:
            peer[ci].push(c.out, stream=torch.cuda.current_stream().cuda_stream)
        else:
            dist.all_gather_into_tensor(gathered[ci].view(world * c.m, c.n), c.out)

    stream = torch.cuda.Stream(device=dev)
    sp = stream.cuda_stream

    def step_eager(si):
        for ci, c in enumerate(sets[si]):
            c.launch(sp)
            if world > 1:
                gather_call(ci, c)

    # eager warm-up (also sets kernel attributes before any graph capture)
    with torch.cuda.stream(stream):
        for si in range(nsets):
            step_eager(si)
    torch.cuda.synchronize()
    _lib.check(lib.lcq_check_device_status(None))
    if peer is not None:
        # one-time check of the peer-memory all-gather against NCCL on the last warm-up outputs
        for ci, c in enumerate(sets[nsets - 1]):
            dist.all_gather_into_tensor(gathered[ci].view(world * c.m, c.n), c.out)
            got = peer[ci].gathered(c.out.dtype, (world, c.m, c.n))
            if not torch.equal(got, gathered[ci]):
                raise RuntimeError(f"peer all-gather mismatch on call {ci}")
        torch.cuda.synchronize()

    graphs = None
    graph_note = "eager"
    if not args.no_graph:
        try:
            graphs = []
            for si in range(nsets):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    cap = torch.cuda.current_stream().cuda_stream
                    for ci, c in enumerate(sets[si]):
                        c.launch(cap)
                        if world > 1:
                            gather_call(ci, c)
                graphs.append(g)
            torch.cuda.synchronize()
            graph_note = "cuda_graph"
        except Exception as e:      # e.g. a collective that cannot be captured: time the eager path instead
            graphs = None
            graph_note = f"eager (graph capture failed: {type(e).__name__})"
            torch.cuda.synchronize()

    def step(i):
        si = i % nsets
        if graphs is not None:
            graphs[si].replay()
        else:
            step_eager(si)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    with torch.cuda.stream(stream):
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.prepare()
            sampler.start()      # one NVML query takes milliseconds: sample from the warm-up on, through the timed region
        for i in range(args.warmup):
            step(i)
        # The timed region is exactly `steps` steps between a barrier + synchronize on both sides; it
        # is repeated until the repeats span about half a second, and the median repeat is reported.
        region_ms = []
        it = args.warmup
        budget_ms, spent_ms = 500.0, 0.0
        while True:
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for i in range(args.steps):
                step(it + i)
            e1.record(stream)
            barrier()
            it += args.steps
            reg = e0.elapsed_time(e1)
            if dist is not None:
                t = torch.tensor([reg], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                reg = float(t.item())
            region_ms.append(reg)
            spent_ms += reg
            if spent_ms >= budget_ms or len(region_ms) >= 200:
                break
        clocks = sampler.stop() if rank == 0 else None
    ms_total = statistics.median(region_ms)
    _lib.check(lib.lcq_check_device_status(None))

    total_bytes = per_set_bytes * world * args.steps
    flops = sum(2.0 * m * local_n(n) * k for (k, n) in shapes for m in ms) * world * args.steps
    if args.workload == "cfg4":
        metric, unit, value = "w4a16_prefill_gemm_tflops", "TFLOP/s", flops / (ms_total * 1e-3) / 1e12
    else:
        metric, unit, value = "w4a16_gemv_weight_hbm_gbs", "GB/s", total_bytes / (ms_total * 1e-3) / 1e9

    line = {
        "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_total / args.steps, "higher_is_better": True,
        "scaling": "strong" if args.workload == "cfg5" else "weak", "vs_baseline": None,
        "dtype": "f16" if xdt == "f16" else "bf16", "data": "synthetic",
        "config": {
            "workload": {"cfg2": "cfg2: W4A16 g=32 GEMV sweep, M in {1,4,16} x SmolLM2-1.7B shapes (K,N)",
                         "cfg3": "cfg3: decode step of a 30-layer SmolLM2-135M-shaped stack, 211 W4A16 g=32 linears at M=1",
                         "cfg4": "cfg4: W4A16 g=32 prefill GEMM, M in {512,2048,8192} x Llama-3-8B shapes",
                         "cfg5": "cfg5: column-sharded W4A16 g=32, 70B shapes, M in {1,16,64}"}[args.workload],
            "shapes_KN": shapes if len(shapes) <= 16 else "30 x " + str(CFG3_LAYER) + " + " + str(CFG3_LM_HEAD), "M": ms, "calls_per_step": len(shapes) * len(ms), "group_size": GROUP,
            "l2_hygiene": f"every call reads its own weights; {nsets} rotating sets of {per_set_bytes / 1e6:.0f} MB",
            "launch": graph_note,
            "sharding": None if world == 1 else (f"N-column shards + " + ("NVLink peer-store all-gather kernel" if peer is not None else "NCCL all-gather") + f", {world} ranks"),
        },
        "gpu_launches": args.steps * len(shapes) * len(ms) * len(region_ms),
        "timed_regions": {"count": len(region_ms), "steps_each": args.steps, "ms_median": ms_total, "ms_min": min(region_ms),
                          "ms_max": max(region_ms), "reported": "median"},
        "weight_bytes_per_step": per_set_bytes * world,
    }
    if args.workload == "cfg3":
        line["us_per_token"] = ms_total / args.steps * 1e3
    if rank == 0:
        line["clocks"] = clocks
    # ---------------------------------------------------------------- graphs hold NCCL work: drop them before anything else
    graphs = None
    import bench_blocks as B
    ctx = B.Ctx(torch, lib, _lib, L, dev, peaks, rank, world, dist)
    # ---------------------------------------------------------------- roofline of the dominant kernel
    if rank == 0 and args.workload in ("cfg2", "cfg3", "cfg5"):
        k, n = {"cfg2": (2048, 49152), "cfg3": (576, 49152), "cfg5": (8192, 128256 // world)}[args.workload]
        line["roofline"] = B.block_roofline(ctx, k, n, 1)
    if rank == 0 and args.workload == "cfg4":
        line["roofline"] = B.block_cfg4(ctx)["roofline"]
    # ---------------------------------------------------------------- end-to-end through the reference-facing call
    if args.workload == "cfg2":
        host_sets = []
        rng = np.random.default_rng(0)
        h2d = d2h = 0
        for (k, n) in shapes:
            wp = torch.from_numpy(rng.integers(0, 256, size=(n, k // 2), dtype=np.uint8)).pin_memory()
            s = torch.from_numpy((np.abs(rng.standard_normal((n, k // GROUP))) * 0.02).astype(np.float16)).pin_memory()
            x = torch.from_numpy(rng.standard_normal((16, k)).astype(np.float16)).pin_memory()
            host_sets.append((wp.numpy(), s.numpy(), x.numpy(), (wp, s, x)))
            for m in ms:
                h2d += wp.numel() + s.numel() * 2 + m * k * 2
                d2h += m * n * 2
        e2e_steps = max(3, min(args.steps, 10))

        def e2e_step():
            for (wp, s, x, _keep) in host_sets:
                for m in ms:
                    L.gpu_matvec_int4(x[:m], wp, s, GROUP)      # host arrays in, host array out
        e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        if dist is not None:
            t = torch.tensor([dt], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = float(t.item())
        line["e2e"] = {"value": per_set_bytes * world * e2e_steps / dt / 1e9, "unit": "GB/s",
                       "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                       "call": "locomp_b200.gpu_matvec_int4(x, w_packed, scales, 32) with pinned host arrays: "
                               "uploads x, weights and scales, runs the kernel, copies the result back -- every call"}
    # ---------------------------------------------------------------- CPU baseline on the host cores
    if rank == 0 and world == 1 and args.workload == "cfg2" and not args.no_cpu_baseline:
        from oracle import qmm_oracle as O
        rng = np.random.default_rng(0)
        k, n = 2048, 8192
        wp, s = O.make_w4(rng, n, k, GROUP, np.float16)
        x = rng.standard_normal((16, k)).astype(np.float16)
        reps = 0
        for _ in range(5):
            O.fast_matvec_int4(x[:1], wp, s, GROUP)
        t0 = time.perf_counter()
        while time.perf_counter() - t0 < 10.0 and reps < 15 * 3:
            for m in ms:
                O.fast_matvec_int4(x[:m], wp, s, GROUP)
            reps += 1
        dt = time.perf_counter() - t0
        line["cpu_baseline"] = {
            "value": weight_bytes(k, n) * len(ms) * reps / dt / 1e9, "unit": "GB/s", "cores": os.cpu_count(),
            "kind": "port",
            "sample": f"(K,N)=(2048,8192), M in {{1,4,16}}, {reps} passes; NumPy dequantise-to-float32 + BLAS "
                      "(oracle.fast_matvec_int4, restating examples/38_quantized_matmul.py:215-232)"}
    # ---------------------------------------------------------------- the other configurations, one block each
    if args.workload == "cfg2" and not args.no_extra:
        for calls in sets:                    # the headline's buffers are no longer needed
            calls.clear()
        torch.cuda.empty_cache()
        line["e2e_resident"] = B.block_e2e_resident(ctx, shapes, ms)
        line["cfg5"] = B.block_cfg5(ctx, gather=args.gather)        # every rank takes part
        if rank == 0 and world == 1:
            line["cfg1"] = B.block_cfg1(ctx)
            line["cfg3"] = B.block_cfg3(ctx)
            line["cfg4"] = B.block_cfg4(ctx)
            line["dequant"] = B.block_dequant(ctx)
        line["gpu_launches"] += ctx.launches
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        # Leave without tearing NCCL down: destroying a communicator that captured CUDA graphs still
        # reference blocks forever (seen at 2 and 8 ranks).  All ranks have printed / finished here.
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg2", choices=["cfg2", "cfg3", "cfg4", "cfg5"])
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--gather", default="nvlink", choices=["nccl", "nvlink"],
                    help="multi-GPU: reassemble outputs with NCCL or with the library's peer-store kernel")
    ap.add_argument("--watchdog", type=int, default=900, help="abort the process after this many seconds")
    ap.add_argument("--profile-shape", default=None, metavar="KxNxM",
                    help="run a few launches of one problem and exit (small case for ncu captures)")
    ap.add_argument("--profile-dequant", action="store_true", help="a few launches of the dequantize kernel, for ncu")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="headline only: skip the cfg1/cfg3/cfg4/cfg5/dequant blocks")
    args = ap.parse_args()
    if args.watchdog > 0:
        import threading

        def _give_up():
            sys.stderr.write(f"bench.py: watchdog expired after {args.watchdog} s, aborting\n")
            sys.stderr.flush()
            os._exit(3)
        t = threading.Timer(args.watchdog, _give_up)     # a thread: fires even while the main thread sits in a C call
        t.daemon = True
        t.start()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.profile_dequant:
        run_profile_dequant(args)
        return
    if args.profile_shape:
        run_profile_shape(args)
        return
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch multi-GPU runs with torch.distributed.run (one rank per GPU)")
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
