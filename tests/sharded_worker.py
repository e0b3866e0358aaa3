"""Worker of the multi-GPU sharding test: launched by tests/test_multi_gpu.py under
torch.distributed.run, one rank per GPU.  Every rank builds the same seeded full weight, keeps
its row block in a ShardedQuantLinear, runs forward() several times in a row with both gather
implementations and compares the gathered output with the NumPy oracle on the FULL weight."""
import datetime
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import locomp_b200 as L                      # noqa: E402
from locomp_b200 import _lib                 # noqa: E402
from oracle import qmm_oracle as O           # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=60))
    n, k = 128 * 3 * world + 32 * world, 2048          # rows per rank not a multiple of the 128-row tile
    rng = np.random.default_rng(0)                      # every rank draws the full seeded tensors
    wp, s = O.make_w4(rng, n, k, 32, np.float16)
    xs = [rng.standard_normal((16, k)).astype(np.float16) for _ in range(3)]
    wd, sd = torch.from_numpy(wp).to(dev), torch.from_numpy(s).to(dev)
    failures = []
    for gather in ("nccl", "nvlink"):
        layer = L.ShardedQuantLinear(wd, sd, 32, 4, gather=gather)
        assert layer.n_local == n // world
        for m in (1, 4, 16):
            layer.prepare(m, torch.float16)
            for layout in ("row_major", "gathered"):
                for call, xh in enumerate(xs):           # consecutive calls: the gather regions alternate
                    x = torch.from_numpy(np.ascontiguousarray(xh[:m])).to(dev)
                    y = layer.forward(x, layout=layout)
                    if layout == "gathered":
                        assert tuple(y.shape) == (world, m, n // world)
                        y = y.permute(1, 0, 2).reshape(m, n)
                    got = y.float().cpu().numpy()
                    ref = O.matmul_int4(xh[:m].astype(np.float32), wp, s, 32)
                    bad = np.abs(got - ref) > 1e-2 + 1e-2 * np.abs(ref)
                    if bad.any() or tuple(got.shape) != (m, n):
                        failures.append((gather, m, layout, call, int(bad.sum()), float(np.abs(got - ref).max())))
            if m == 1:                                    # the vector form: x [K] -> y [N]
                y1 = layer.forward(torch.from_numpy(xs[0][0]).to(dev))
                ref = O.matmul_int4(xs[0][0].astype(np.float32), wp, s, 32)
                if tuple(y1.shape) != (n,) or np.any(np.abs(y1.float().cpu().numpy() - ref) > 1e-2 + 1e-2 * np.abs(ref)):
                    failures.append((gather, "vector"))
        torch.cuda.synchronize()
        if _lib.lib().lcq_check_device_status(None) != 0:
            failures.append((gather, "device status", _lib.lib().lcq_last_error().decode()))
        layer.close()
    # ---- the same through the C-ABI sharding context (what a host without Python would call)
    import ctypes
    lib = _lib.lib()
    n_local = n // world
    ctx = ctypes.c_void_p()
    handles = ctypes.create_string_buffer(128)
    _lib.check(lib.lcq_shard_ctx_create(rank, world, 16 * n_local * 2, ctypes.byref(ctx), handles))
    gathered_handles = [None] * world
    dist.all_gather_object(gathered_handles, handles.raw)
    dist.barrier()                                           # every context exists before anyone connects
    _lib.check(lib.lcq_shard_ctx_connect(ctx, b"".join(gathered_handles)))
    dist.barrier()
    w_loc, s_loc = wd[rank * n_local:(rank + 1) * n_local], sd[rank * n_local:(rank + 1) * n_local]
    st = torch.cuda.current_stream().cuda_stream
    for m in (1, 16):
        for call, xh in enumerate(xs):
            x = torch.from_numpy(np.ascontiguousarray(xh[:m])).to(dev)
            out_ptr = ctypes.c_void_p()
            _lib.check(lib.lcq_sharded_matmul_int4(ctx, x.data_ptr(), w_loc.data_ptr(), s_loc.data_ptr(), ctypes.byref(out_ptr),
                                                   m, n, k, 32, _lib.F16, _lib.F16, _lib.F16, _lib.ALGO_AUTO, st))
            torch.cuda.synchronize()
            class _Mem:                                   # zero-copy view of the device pointer the library returned
                __cuda_array_interface__ = {"shape": (world * m * n_local,), "typestr": "<f2",
                                            "data": (out_ptr.value, False), "version": 3}
            host = torch.as_tensor(_Mem(), device=dev).cpu().numpy().reshape(world, m, n_local)
            got = host.transpose(1, 0, 2).reshape(m, n).astype(np.float32)
            ref = O.matmul_int4(xh[:m].astype(np.float32), wp, s, 32)
            if np.any(np.abs(got - ref) > 1e-2 + 1e-2 * np.abs(ref)):
                failures.append(("c-abi ctx", m, call, float(np.abs(got - ref).max())))
    if lib.lcq_check_device_status(None) != 0:
        failures.append(("c-abi ctx", "device status"))
    dist.barrier()
    _lib.check(lib.lcq_shard_ctx_destroy(ctx))
    ok = torch.tensor([0 if failures else 1], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    print(f"rank {rank}: {'SHARDED_OK' if not failures else 'SHARDED_FAIL ' + repr(failures[:6])}", flush=True)
    dist.barrier()
    torch.cuda.synchronize()
    dist.destroy_process_group()
    sys.exit(0 if int(ok.item()) == 1 else 1)


if __name__ == "__main__":
    main()
