"""Peer-memory all-reduce (bw_peer_allreduce_f16).

On one GPU the ranks are emulated the allowed way: all "ranks'" buffers are local and the flags a
kernel would wait for are written beforehand, so that no launch ever waits for another launch.
With two or more GPUs the real thing runs as one process per GPU (NCCL only for the set-up and as
the comparison)."""
import ctypes
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from bitween_b200 import synth
from bitween_b200.kernels import _lib

pytestmark = pytest.mark.gpu
DEV = "cuda"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_rank_order_sum_with_preset_flags(world):
    L = _lib.lib()
    count = 64 * 1024
    parts = [torch.from_numpy(synth.normal(50 + r, (count,), 1.0)).to(DEV).half() for r in range(world)]
    flag_words = L.bw_peer_flag_bytes() // 4
    for rank in range(world):
        flags = [torch.zeros(flag_words, dtype=torch.int32, device=DEV) for _ in range(world)]
        flags[rank].fill_(1)                      # every peer has "signalled" call 1 in every block's slot
        state = torch.zeros(L.bw_peer_state_bytes(), dtype=torch.uint8, device=DEV)
        out = torch.empty(count, dtype=torch.float16, device=DEV)
        bufs = (ctypes.c_void_p * world)(*[p.data_ptr() for p in parts])
        fl = (ctypes.c_void_p * world)(*[f.data_ptr() for f in flags])
        rc = L.bw_peer_allreduce_f16(bufs, fl, rank, world, out.data_ptr(), count, state.data_ptr(), _lib.stream_ptr(out.device))
        assert rc == 0
        torch.cuda.synchronize()
        want = parts[0].float()
        for r in range(1, world):
            want = want + parts[r].float()
        assert torch.equal(out, want.half())
        # the kernel told every peer, in every block's slot, and advanced its call counter
        for r in range(world):
            if r != rank:
                got = flags[r].view(2, -1, 8)[:, :, rank].cpu().numpy()      # [phase][block]
                assert np.all(got[0] == 1) and np.all(got[1] == 0)          # the one-shot form has one barrier
        assert state.view(torch.int32).cpu().tolist() == [1, 0]
    assert L.bw_device_status() == 0
    # argument rules
    z = None
    assert L.bw_peer_allreduce_f16(bufs, fl, 0, 9, out.data_ptr(), 64, state.data_ptr(), z) == 3
    assert L.bw_peer_allreduce_f16(bufs, fl, 0, world, out.data_ptr(), 12, state.data_ptr(), z) == 3


@pytest.mark.parametrize("world", [2, 4, 8])
def test_two_shot_form_with_preset_flags(world):
    """Two passes over the emulated ranks: the first leaves every rank's reduced slice in its result
    buffer (nothing to collect yet), the second -- same inputs, flags preset for call 2 -- collects them."""
    L = _lib.lib()
    count = 8 * 1000 * world + 8 * 3                    # slices of unequal length at the end
    parts = [torch.from_numpy(synth.normal(70 + r, (count,), 1.0)).to(DEV).half() for r in range(world)]
    per = ((count // 8 + world - 1) // world) * 8
    res = [torch.zeros(per, dtype=torch.float16, device=DEV) for _ in range(world)]
    flag_words = L.bw_peer_flag_bytes() // 4
    states = [torch.zeros(L.bw_peer_state_bytes(), dtype=torch.uint8, device=DEV) for _ in range(world)]
    want = parts[0].float()
    for r in range(1, world):
        want = want + parts[r].float()
    want = want.half()
    bufs = (ctypes.c_void_p * world)(*[p.data_ptr() for p in parts])
    resp = (ctypes.c_void_p * world)(*[t.data_ptr() for t in res])
    for call in (1, 2):
        for rank in range(world):
            flags = [torch.zeros(flag_words, dtype=torch.int32, device=DEV) for _ in range(world)]
            flags[rank].fill_(call)
            fl = (ctypes.c_void_p * world)(*[f.data_ptr() for f in flags])
            out = torch.zeros(count, dtype=torch.float16, device=DEV)
            rc = L.bw_peer_allreduce2_f16(bufs, resp, fl, rank, world, out.data_ptr(), count, states[rank].data_ptr(),
                                          _lib.stream_ptr(out.device))
            assert rc == 0
            torch.cuda.synchronize()
            lo = rank * per
            assert torch.equal(out[lo:lo + per], want[lo:lo + per])        # the rank's own slice is always right
            if call == 2:
                assert torch.equal(out, want)
    assert L.bw_device_status() == 0


def test_two_processes_over_peer_memory():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, PYTHONPATH=ROOT, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29533",
                        os.path.join(ROOT, "tests", "peer_allreduce_ranks.py")],
                       env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "peer all-reduce ok" in r.stdout
