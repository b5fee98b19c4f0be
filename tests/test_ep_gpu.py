"""Expert parallelism on the GPU: the device-side steps (dispatch, experts on received rows, combine) through the
C ABI. On one GPU the ranks are emulated in one process (one handle per expert range, exchange by slicing); with
two or more GPUs a real two-process NCCL run is checked against the single-handle layer."""
import os
import subprocess
import sys

import numpy as np
import pytest

from tests import util
from tests.test_moe_gpu import device_x, make
from zerocool_b200 import synth

pytestmark = pytest.mark.gpu
SEED = 5
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("world,has_shared,hidden", [(2, 0, 4096), (4, 1, 2048)])
def test_emulated_ranks_equal_the_single_handle_layer(world, has_shared, hidden):
    import torch
    from zerocool_b200.ep import emulate
    base = dict(hidden=hidden, experts=64, top_k=10, has_shared=has_shared, max_tokens=16)
    full = make(util.cfg2(**base))
    full.synth_fill_layer(0, SEED)
    per = 64 // world
    parts = []
    for r in range(world):
        h = make(util.cfg2(first_expert=r * per, local_experts=per, **base))
        h.synth_fill_layer(0, SEED)
        parts.append(h)
    xs = [device_x(full, synth.activations(full.cfg, SEED + r, 0, 11 + r)) for r in range(world)]
    outs = emulate(parts, 64, 0, xs)
    for r in range(world):
        want = full.moe(0, xs[r]).float().cpu().numpy()
        got = outs[r].float().cpu().numpy()
        assert parts[r].status() == 0
        assert util.rel_max_error(got, want) < 1e-5, r


def ep_handles(world, has_shared, hidden, max_tokens=16):
    base = dict(hidden=hidden, experts=64, top_k=10, has_shared=has_shared, max_tokens=max_tokens)
    full = make(util.cfg2(**base))
    full.synth_fill_layer(0, SEED)
    per = 64 // world
    parts = []
    for r in range(world):
        h = make(util.cfg2(first_expert=r * per, local_experts=per, **base))
        h.synth_fill_layer(0, SEED)
        parts.append(h)
    return full, parts


@pytest.mark.parametrize("world,has_shared,hidden", [(2, 0, 4096), (4, 1, 2048)])
def test_peer_transport_with_emulated_ranks_equals_the_single_handle_layer(world, has_shared, hidden):
    """Rows, tags, results and flags through the windows (here all on one device, attached by address); two layers
    calls in a row so that the second runs on the first one's leftovers and a later epoch."""
    from zerocool_b200.ep import attach_local, emulate_peer
    full, parts = ep_handles(world, has_shared, hidden)
    attach_local(parts)
    for call in range(2):
        xs = [device_x(full, synth.activations(full.cfg, SEED + 10 * call + r, 0, 16 - 3 * r - call)) for r in range(world)]
        outs = emulate_peer(parts, 0, xs)
        for r in range(world):
            want = full.moe(0, xs[r]).float().cpu().numpy()
            got = outs[r].float().cpu().numpy()
            assert parts[r].status() == 0
            assert util.rel_max_error(got, want) < 1e-5, (call, r)


def test_peer_wait_runs_out_with_a_status_bit_and_the_handle_stays_usable():
    """A wait for a flag that nothing sets: the owner gives up after its (here 30 ms) limit, raises the time-out bit
    and finishes on what it has; the context stays usable and the same exchange then completes normally."""
    from zerocool_b200.ep import attach_local
    from zerocool_b200.moe import STATUS_TIMEOUT
    full, parts = ep_handles(2, 0, 2048)
    attach_local(parts)
    for h in parts:
        h.set_option("ep_wait_ms", 30)
    xs = [device_x(full, synth.activations(full.cfg, SEED + r, 0, 9)) for r in range(2)]
    parts[0].ep_send(0, xs[0])
    parts[0].ep_process(0)                      # rank 1 has not sent: its flag never arrives
    assert parts[0].status() & STATUS_TIMEOUT   # read (and cleared) after the stream has drained
    parts[1].ep_send(0, xs[1])
    parts[0].ep_process(0)                      # the same epoch again, now complete
    parts[1].ep_process(0)
    for r in range(2):
        got = parts[r].ep_finish(0, xs[r]).float().cpu().numpy()
        want = full.moe(0, xs[r]).float().cpu().numpy()
        assert parts[r].status() == 0
        assert util.rel_max_error(got, want) < 1e-5, r


def test_two_process_nccl_run():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29611", os.path.join(ROOT, "tests", "ep_nccl_check.py")]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "ep ok" in r.stdout
