"""The allocation-free router entry point (zc_router_logits_noalloc) against the handle-based one.

It is for callers that cannot call cudaMalloc and therefore cannot create a handle: a plugin running while the
host engine's allocator owns all of HBM, code running while another thread captures a CUDA graph, or a loop that
must not take the allocator lock. Its scratch is a fixed array inside the library. This file is collected last
on purpose, so that a run that stops at the first failure has already run every other test."""
import ctypes

import numpy as np
import pytest

from oracle import oracle
from tests import util
from zerocool_b200 import synth
from zerocool_b200.records import BF16, F32

pytestmark = pytest.mark.gpu


def test_noalloc_router_matches_the_handle_router_on_two_calls():
    import torch
    from zerocool_b200.moe import Moe, ZC_EINVAL
    cfg = util.cfg2(max_tokens=64)
    m = Moe(cfg, 0)
    w = synth.router(cfg, 4321, 0)
    m.load_layer(0, router_w=w, shared_gate_w=synth.shared_gate(cfg, 4321, 0))
    w_dev = torch.from_numpy(w).cuda()
    lib = m.lib
    stream = torch.cuda.current_stream().cuda_stream
    # two calls in a row, with different batch sizes, so the second runs on the first one's leftovers
    for call, tokens in enumerate((64, 5)):
        x = synth.activations(cfg, 4321 + call, 0, tokens)
        x_dev = torch.from_numpy(x).to(device="cuda", dtype=torch.bfloat16)
        want = m.router(0, x_dev)
        got = torch.full((tokens, cfg.experts), float("nan"), dtype=torch.float32, device="cuda")
        rc = lib.zc_router_logits_noalloc(x_dev.data_ptr(), BF16, w_dev.data_ptr(), F32, tokens, cfg.hidden, cfg.experts,
                                          got.data_ptr(), stream)
        assert rc == 0, lib.zc_last_error()
        torch.cuda.synchronize()
        # same kernel, same pinned accumulation order: bit-exact, the tolerance of the router tests
        assert torch.equal(got.view(torch.int32), want.view(torch.int32)), (call, tokens)
    # sizes beyond the built-in scratch are rejected with a clear message, nothing is launched
    big = torch.zeros((65, cfg.hidden), dtype=torch.bfloat16, device="cuda")
    out = torch.zeros((65, cfg.experts), dtype=torch.float32, device="cuda")
    rc = lib.zc_router_logits_noalloc(big.data_ptr(), BF16, w_dev.data_ptr(), F32, 65, cfg.hidden, cfg.experts, out.data_ptr(), stream)
    assert rc == ZC_EINVAL and b"tokens must be 1..64" in lib.zc_last_error()
    rc = lib.zc_router_logits_noalloc(big.data_ptr(), BF16, w_dev.data_ptr(), F32, 8, cfg.hidden, 1024, out.data_ptr(), stream)
    assert rc == ZC_EINVAL and b"at most 512" in lib.zc_last_error()


@pytest.mark.parametrize("act,router_dtype,hidden,experts", [(F32, F32, 2560, 64), (BF16, BF16, 3072, 512), (F32, BF16, 2048, 64), (BF16, F32, 2560, 512)])
def test_noalloc_router_at_its_documented_limits_against_the_cpu_checker(act, router_dtype, hidden, experts):
    """Both activation and router dtypes, the largest hidden size the entry point takes (3072) and the reference's own
    (2560), few and many experts: bit-exact against the CPU checker's pinned accumulation order, on two calls in a row
    (a full batch, then a short one that runs on the first call's leftovers in the shared scratch)."""
    import torch
    from zerocool_b200.moe import load_library
    lib = load_library()
    cfg = util.cfg2(hidden=hidden, experts=experts, act_dtype=act, router_dtype=router_dtype, max_tokens=64)
    w = synth.router(cfg, 99, 0)
    w_dev = torch.from_numpy(w.view(np.int16) if router_dtype == BF16 else w).cuda()
    stream = torch.cuda.current_stream().cuda_stream
    for call, tokens in enumerate((64, 9)):
        x = synth.activations(cfg, 99 + call, 0, tokens)
        x_dev = torch.from_numpy(x).to(device="cuda", dtype=torch.bfloat16 if act == BF16 else torch.float32)
        got = torch.full((tokens, experts), float("nan"), dtype=torch.float32, device="cuda")
        rc = lib.zc_router_logits_noalloc(x_dev.data_ptr(), act, w_dev.data_ptr(), router_dtype, tokens, hidden, experts, got.data_ptr(), stream)
        assert rc == 0, lib.zc_last_error()
        torch.cuda.synchronize()
        want = oracle.router_logits(x, w, router_dtype)
        assert np.array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32)), (call, tokens)
