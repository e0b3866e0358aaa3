"""Failure detection without faulting anything: a device-side wait is made to run out (it waits
for a flag that nothing sets), the kernel returns on its own, the host reads the error status,
and the context stays usable."""
import ctypes

import numpy as np
import pytest
import torch

import locomp_b200 as L
from locomp_b200 import _lib
from oracle import qmm_oracle as O

pytestmark = pytest.mark.gpu


def test_bounded_wait_runs_out_and_the_context_survives():
    lib = _lib.lib()
    assert lib.lcq_set_wait_limit_ns(5_000_000) == 0          # 5 ms instead of 2 s
    try:
        nbytes = 4096
        region_bytes = lib.lcq_peer_region_bytes(nbytes, 2)
        mine = torch.zeros(region_bytes, dtype=torch.uint8, device="cuda")
        absent_peer = torch.zeros(region_bytes, dtype=torch.uint8, device="cuda")   # a "rank 1" that never pushes
        regions = (ctypes.c_void_p * 2)(mine.data_ptr(), absent_peer.data_ptr())
        state = torch.zeros(2, dtype=torch.int32, device="cuda")
        src = torch.arange(nbytes, dtype=torch.int32, device="cuda").to(torch.uint8)
        assert lib.lcq_allgather_push(src.data_ptr(), nbytes, regions, 0, 2, state.data_ptr(), None) == 0
        assert lib.lcq_check_device_status(None) == _lib.ERR_TIMEOUT
        assert b"bounded wait" in lib.lcq_last_error()
        # this rank's slice is in slot 0 of its own region, and was pushed (as {word, sequence} pairs)
        # into the peer's staging area, before the wait gave up
        assert torch.equal(mine[256:256 + nbytes], src)
        assert int(absent_peer[256 + 2 * nbytes:].count_nonzero()) > 0 and int(absent_peer[256:256 + 2 * nbytes].count_nonzero()) == 0
        # the status word was cleared by the read, and the next kernel runs normally
        assert lib.lcq_check_device_status(None) == 0
        rng = np.random.default_rng(1)
        wp, s = O.make_w4(rng, 256, 512, 32, np.float16)
        x = rng.standard_normal((2, 512)).astype(np.float16)
        y = L.quantized_matmul(torch.from_numpy(x).cuda(), torch.from_numpy(wp).cuda(), torch.from_numpy(s).cuda(), 32)
        ref = O.matmul_int4(x.astype(np.float32), wp, s, 32)
        assert np.all(np.abs(y.float().cpu().numpy() - ref) <= 1e-2 + 1e-2 * np.abs(ref))
        assert lib.lcq_check_device_status(None) == 0
    finally:
        assert lib.lcq_set_wait_limit_ns(2_000_000_000) == 0


def test_wait_limit_must_be_positive():
    assert _lib.lib().lcq_set_wait_limit_ns(0) == _lib.ERR_BAD_ARG


def test_pair_form_unpacks_eight_ranks_on_one_gpu():
    """The receive side of the pair-form all-gather for world = 8, without any kernel waiting for
    another one: the staging area of rank 3's region is filled on the host with what the seven peers
    would have stored ({word, sequence number} pairs, buffer chosen by call parity), then rank 3's
    kernel runs alone -- it finds every pair on its first poll.  Two consecutive calls (sequence
    numbers 1 and 2, i.e. both staging buffers)."""
    lib = _lib.lib()
    world, rank, nbytes = 8, 3, 4096 + 16                      # 257 sixteen-byte pieces per slice
    n16, n32 = nbytes // 16, nbytes // 4
    region_bytes = lib.lcq_peer_region_bytes(nbytes, world)
    regs = [torch.zeros(region_bytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
    regions = (ctypes.c_void_p * world)(*[r.data_ptr() for r in regs])
    state = torch.zeros(2, dtype=torch.int32, device="cuda")
    rng = np.random.default_rng(8)
    for seq in (1, 2):
        slices = [rng.integers(0, 2 ** 32, n32, dtype=np.uint32) for _ in range(world)]
        staged = np.zeros(2 * world * n32 * 2, dtype=np.uint32)  # two buffers x world x (slice as pairs)
        buf = (seq & 1) * world
        for r in range(world):
            if r == rank:
                continue
            pairs = np.empty((n32, 2), dtype=np.uint32)
            pairs[:, 0] = slices[r]
            pairs[:, 1] = seq
            o = (buf + r) * n32 * 2
            staged[o:o + 2 * n32] = pairs.reshape(-1)
        mine = regs[rank]
        stage_off = 256 + world * nbytes
        mine[stage_off:stage_off + staged.nbytes] = torch.from_numpy(staged.view(np.uint8)).cuda()
        src = torch.from_numpy(slices[rank].view(np.uint8).copy()).cuda()
        torch.cuda.synchronize()
        assert lib.lcq_allgather_push(src.data_ptr(), nbytes, regions, rank, world, state.data_ptr(), None) == 0
        assert lib.lcq_check_device_status(None) == 0, lib.lcq_last_error()
        got = mine[256:256 + world * nbytes].cpu().numpy().view(np.uint32).reshape(world, n32)
        for r in range(world):
            assert np.array_equal(got[r], slices[r]), (seq, r)
        assert int(state[0].item()) == seq
        # and what this rank sent sits, as pairs, in every peer's staging area
        peer = regs[0][stage_off:stage_off + staged.nbytes].cpu().numpy().view(np.uint32)
        o = (buf + rank) * n32 * 2
        sent = peer[o:o + 2 * n32].reshape(n32, 2)
        assert np.array_equal(sent[:, 0], slices[rank]) and np.all(sent[:, 1] == seq)
