"""Host-side logic of the N-column sharding layer on CPU: world_size-2 (and 4) gloo process
groups, with the NumPy oracle injected as the local operator (the CUDA operator itself is
covered by the gpu-marked tests).  Checks the row partition, the gathered layout and that the
reassembled output equals the unsharded oracle."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from locomp_b200.shard import ShardedQuantLinear, shard_rows
from oracle import qmm_oracle as O


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_matmul(x, w, scales, group_size, bits=4, **kw):
    xn = x.numpy().astype(np.float32)
    y = O.matmul_int4(xn, w.numpy(), scales.numpy(), group_size) if bits == 4 else \
        O.matmul_int8(xn, w.numpy(), scales.numpy(), group_size)
    return torch.from_numpy(np.asarray(y, dtype=np.float32))


def _worker(rank, world, port, n, k, m, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(0)                      # every rank draws the full seeded tensors
        wp, s = O.make_w4(rng, n, k, 32, np.float16)
        x = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32))
        layer = ShardedQuantLinear(torch.from_numpy(wp), torch.from_numpy(s), 32, 4, matmul=_oracle_matmul)
        r0, r1 = shard_rows(n, world, rank)
        assert layer.n_local == n // world and tuple(layer.w.shape) == (n // world, k // 2)
        assert layer.w.untyped_storage().nbytes() == wp.nbytes and layer.w.storage_offset() == r0 * (k // 2)   # a view of the full tensor's row block, not a copy
        full = layer.forward(x)
        ref = O.matmul_int4(x.numpy(), wp, s, 32).astype(np.float32)
        ok = bool(np.allclose(full.numpy(), ref, rtol=1e-6, atol=1e-6)) and tuple(full.shape) == (m, n)
        g = layer.forward(x, layout="gathered")
        ok = ok and tuple(g.shape) == (world, m, n // world)
        ok = ok and bool(np.allclose(g[rank].numpy(), ref[:, r0:r1], rtol=1e-6, atol=1e-6))
        y1 = layer.forward(x[0])                             # M = 1: gathered buffer is already row-major
        ok = ok and tuple(y1.shape) == (n,) and bool(np.allclose(y1.numpy(), ref[0], rtol=1e-6, atol=1e-6))
        q.put((rank, ok))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,n,k,m", [(2, 256, 128, 3), (4, 512, 64, 1)])
def test_sharded_linear_gloo(world, n, k, m):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n, k, m, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    results = dict(q.get(timeout=10) for _ in range(world))
    assert results == {r: True for r in range(world)}


def test_shard_rows():
    assert shard_rows(128256, 8, 3) == (3 * 16032, 4 * 16032)
    assert [shard_rows(8, 4, r) for r in range(4)] == [(0, 2), (2, 4), (4, 6), (6, 8)]
    with pytest.raises(ValueError):
        shard_rows(10, 4, 0)
    with pytest.raises(ValueError):
        shard_rows(8, 4, 4)


def test_single_process_is_identity():
    rng = np.random.default_rng(1)
    wp, s = O.make_w4(rng, 64, 64, 32, np.float16)
    x = torch.from_numpy(rng.standard_normal((2, 64)).astype(np.float32))
    layer = ShardedQuantLinear(torch.from_numpy(wp), torch.from_numpy(s), matmul=_oracle_matmul)
    assert layer.world == 1 and layer.n_local == 64
    np.testing.assert_allclose(layer.forward(x).numpy(), O.matmul_int4(x.numpy(), wp, s, 32), rtol=1e-6)
