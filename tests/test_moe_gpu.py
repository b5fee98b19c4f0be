"""GPU parity tests: every result of the CUDA path, obtained through the C ABI, against the CPU checker
(oracle/) on identical seeded inputs. Expert ids and permutation indices are compared bit for bit; layer
outputs with max-abs error <= 2e-3 x output RMS (the tolerance the benchmark specification states)."""
import os

import numpy as np
import pytest

from oracle import oracle
from tests import util
from tests.test_oracle_golden import exceptional_logits
from zerocool_b200 import synth
from zerocool_b200.records import ARITH_FP32, ARITH_REFERENCE, BF16, F16, F32, MoeConfig

pytestmark = pytest.mark.gpu

TOL = 2e-3     # max-abs error / output RMS
SEED = 1234


@pytest.fixture(scope="module")
def torch():
    import torch
    return torch


def make(cfg):
    from zerocool_b200.moe import Moe
    return Moe(cfg, 0)


def device_x(m, x):
    import torch
    return torch.from_numpy(np.ascontiguousarray(x)).to(device=m.device, dtype=m.act_torch)


def oracle_layer(cfg, seed, layer, x, ids_hint, **kw):
    records = util.selected_records(cfg, seed, layer, ids_hint)
    shared = synth.record(cfg, seed, layer, synth.SHARED_EXPERT) if cfg.has_shared else None
    gate = synth.shared_gate(cfg, seed, layer) if cfg.has_shared else None
    return oracle.moe_layer(cfg.as_dict(), records, synth.router(cfg, seed, layer), x, shared_record=shared,
                            shared_gate_w=gate, **kw)


def test_device_generator_matches_numpy_definition(torch):
    cfg = util.cfg2(experts=32, top_k=4, max_tokens=4)
    m = make(cfg)
    m.synth_fill_layer(0, SEED)
    torch.cuda.synchronize()
    for e in (0, 17, 31):
        got = m.read_layer_tensor(0, "records", cfg.record_bytes, e * cfg.record_stride)
        assert np.array_equal(got, synth.record(cfg, SEED, 0, e)[:cfg.record_bytes]), e
    got = m.read_layer_tensor(0, "shared_record", cfg.record_bytes)
    assert np.array_equal(got, synth.record(cfg, SEED, 0, synth.SHARED_EXPERT)[:cfg.record_bytes])
    got = m.read_layer_tensor(0, "router_w", cfg.experts * cfg.hidden * 4).view(np.float32)
    assert np.array_equal(got, synth.router(cfg, SEED, 0).reshape(-1))
    got = m.read_layer_tensor(0, "shared_gate_w", cfg.hidden * 4).view(np.float32)
    assert np.array_equal(got, synth.shared_gate(cfg, SEED, 0).reshape(-1))
    q8 = util.cfg2(experts=32, top_k=4, max_tokens=4, down_bits=8, q8_signed=1, meta_dtype=BF16, router_dtype=BF16)
    m8 = make(q8)
    m8.synth_fill_layer(0, SEED)
    got = m8.read_layer_tensor(0, "records", q8.record_bytes, 5 * q8.record_stride)
    assert np.array_equal(got, synth.record(q8, SEED, 0, 5)[:q8.record_bytes])
    got = m8.read_layer_tensor(0, "router_w", q8.experts * q8.hidden * 2).view(np.uint16)
    assert np.array_equal(got, synth.router(q8, SEED, 0).reshape(-1))


@pytest.mark.parametrize("act,router_dtype,tokens", [(BF16, F32, 1), (BF16, F32, 19), (F32, F32, 5), (F32, BF16, 11), (BF16, F32, 64)])
def test_router_logits_are_bit_exact(torch, act, router_dtype, tokens):
    cfg = util.cfg2(act_dtype=act, router_dtype=router_dtype, max_tokens=64)
    m = make(cfg)
    w = synth.router(cfg, SEED, 0)
    m.load_layer(0, router_w=w, shared_gate_w=synth.shared_gate(cfg, SEED, 0))
    x = synth.activations(cfg, SEED, 0, tokens)
    got = m.router(0, device_x(m, x)).cpu().numpy()
    want = oracle.router_logits(x, w, router_dtype)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_router_reproduces_mlx_bit_patterns(torch):
    """The reference's own router test (tests/test_qwen.cpp:798-826) through the CUDA kernel."""
    import json
    g = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_known_answers.json")))["router_mlx"]
    T, K, N = g["T"], g["K"], g["N"]
    cfg = util.cfg0(experts=N, act_dtype=F32, router_dtype=BF16, has_shared=0, max_tokens=T)
    n, k = np.meshgrid(np.arange(N, dtype=np.int64), np.arange(K, dtype=np.int64), indexing="ij")
    w = np.ldexp(((n * 17 + k * 23) % 251 - 125).astype(np.float32), -(k % 20 + 4).astype(np.int32)).astype(np.float32)
    wbits = (w.view(np.uint32) >> 16).astype(np.uint16)
    t, k2 = np.meshgrid(np.arange(T, dtype=np.int64), np.arange(K, dtype=np.int64), indexing="ij")
    x = (((k2 * 13 + t * 31) % 251 - 125).astype(np.float32) / np.float32(128)).astype(np.float32)
    m = make(cfg)
    m.load_layer(0, router_w=wbits)
    full = m.router(0, device_x(m, x)).cpu().numpy()
    assert [int(v) for v in full.reshape(-1)[g["indices"]].view(np.uint32)] == g["bits"]
    for offset, count in ((0, 1), (1, 7), (8, 3)):          # chunk invariance
        part = m.router(0, device_x(m, x[offset:offset + count])).cpu().numpy()
        assert np.array_equal(part, full[offset:offset + count])


def test_route_ties_exceptional_scores_and_chunks(torch):
    """tests/test_qwen.cpp:755-797 through the CUDA kernel; ids bit-exact against the CPU rule and the checker."""
    values = exceptional_logits()
    T = values.shape[0]
    cfg = util.cfg2(max_tokens=T, has_shared=0)
    m = make(cfg)
    logits = torch.from_numpy(values).cuda()
    ids, weights = m.route(logits)
    ids, weights = ids.cpu().numpy(), weights.cpu().numpy()
    want_ids, want_w = oracle.route(values, 10)
    assert np.array_equal(ids, want_ids)
    both_nan = np.isnan(weights) & np.isnan(want_w)
    assert np.array_equal(np.isnan(weights), np.isnan(want_w))
    assert np.allclose(weights[~both_nan], want_w[~both_nan], rtol=2e-6, atol=1e-9)
    for offset, count in ((0, 1), (1, 7), (8, 31), (39, 97), (136, 1)):
        a, b = m.route(logits[offset:offset + count].contiguous())
        assert np.array_equal(a.cpu().numpy(), ids[offset:offset + count])
        assert np.array_equal(b.cpu().numpy().view(np.uint32), weights[offset:offset + count].view(np.uint32))
    assert m.status() & 1          # tokens with fewer than ten selectable scores were flagged
    with pytest.raises(ValueError):
        m.route(logits, tokens=T - 1)
    with pytest.raises(ValueError):
        m.route(logits[:0], tokens=0)


@pytest.mark.parametrize("tokens,experts,k", [(1, 64, 8), (37, 64, 8), (64, 512, 10), (513, 512, 10), (2048, 512, 10)])
def test_permute_is_bit_exact(torch, tokens, experts, k):
    cfg = util.cfg2(experts=experts, top_k=k, max_tokens=tokens, has_shared=0)
    m = make(cfg)
    rng = np.random.default_rng(tokens)
    # distinct experts per token, skewed towards low ids
    ids = np.stack([rng.choice(experts, size=k, replace=False, p=None) for _ in range(tokens)]).astype(np.int32)
    if tokens > 8:
        ids[3] = np.arange(k)             # a token whose slots are already sorted
        ids[5] = np.arange(k)[::-1]
    offsets, perm = m.permute(torch.from_numpy(ids).cuda())
    want_off, want_perm = oracle.permute(ids, experts)
    assert np.array_equal(offsets.cpu().numpy(), want_off)
    assert np.array_equal(perm.cpu().numpy(), want_perm)
    assert m.status() == 0
    bad = ids.copy()
    bad[0, 0] = -1
    offsets, perm = m.permute(torch.from_numpy(bad).cuda())
    assert m.status() & 1
    assert int(offsets.cpu().numpy()[-1]) == tokens * k - 1


def check_layer(torch, cfg, tokens, seed=SEED, tol=TOL, layer=0, fold=None, exact_h=None):
    m = make(cfg)
    if fold is not None:
        m.set_option("fold_q4", fold)
    if exact_h is not None:
        m.set_option("exact_h", exact_h)
    m.synth_fill_layer(layer, seed)
    x = synth.activations(cfg, seed, layer, tokens)
    out = m.moe(layer, device_x(m, x))
    routing = m.last_routing(tokens)
    assert m.status() == 0
    out = out.float().cpu().numpy()
    want = oracle_layer(cfg, seed, layer, x, routing["ids"], want_intermediates=True)
    assert np.array_equal(routing["logits"].view(np.uint32), want["logits"].view(np.uint32))
    assert np.array_equal(routing["ids"], want["ids"])
    want_off, want_perm = oracle.permute(want["ids"], cfg.experts)
    assert np.array_equal(routing["offsets"], want_off)
    assert np.array_equal(routing["perm"], want_perm)
    assert np.allclose(routing["weights"], want["weights"], rtol=2e-6, atol=1e-9)
    err = util.rel_max_error(out, want["out"])
    assert err <= tol, err
    return out, want, m


def test_config1_single_token_fp32(torch):
    """benchmark configuration 1: hidden 2048, 64 experts top-8, ffn 512, one fp32 token, no shared expert."""
    check_layer(torch, util.cfg1(), 1)


@pytest.mark.parametrize("tokens", [1, 4, 16, 64])
def test_config2_decode_batches(torch, tokens):
    """benchmark configuration 2 (one layer of it): 512 experts top-10 + shared, bf16 activations, token batches 1/4/16/64."""
    check_layer(torch, util.cfg2(), tokens)


@pytest.mark.parametrize("tokens", [1, 16])
def test_config2_exact_q4_extraction(torch, tokens):
    """The kernel variant that removes the 1024 offset of the Q4 codes in FP16 before the tensor-core product."""
    out_exact, want, _ = check_layer(torch, util.cfg2(), tokens, fold=0)
    out_fold, _, _ = check_layer(torch, util.cfg2(), tokens, fold=1)
    assert util.rel_max_error(out_fold, out_exact) < 1e-3      # FP32 tensor-core accumulation of the folded offset


def test_config2_ragged_batch_and_bf16_output(torch):
    """A batch that is not a multiple of the 8-row MMA pass, with the output rounded to bf16: the error bound
    then allows one bf16 rounding of the output on top of the tolerance."""
    cfg = util.cfg2(out_dtype=BF16, max_tokens=32)
    m = make(cfg)
    m.synth_fill_layer(0, SEED)
    x = synth.activations(cfg, SEED, 0, 13)
    out = m.moe(0, device_x(m, x)).float().cpu().numpy()
    ids = m.last_routing(13)["ids"]
    want = oracle_layer(cfg, SEED, 0, x, ids)
    rms = np.sqrt(np.mean(want["out"].astype(np.float64) ** 2))
    bound = TOL * rms + np.abs(want["out"]) * 2.0 ** -8
    assert np.all(np.abs(out - want["out"]) <= bound)


def test_config5_hidden_4096(torch):
    """benchmark configuration 5 geometry on one GPU with a reduced expert count: hidden 4096, top-10, no shared expert."""
    check_layer(torch, util.cfg2(hidden=4096, experts=64, has_shared=0, max_tokens=16), 9)


def test_config4_mixed_q4_q8(torch):
    """benchmark configuration 4 geometry: gate/up Q4, down Q8 with signed int8 codes, a ragged 21-token batch."""
    check_layer(torch, util.cfg2(experts=64, has_shared=0, down_bits=8, q8_signed=1, max_tokens=32), 21)


def test_q8_everywhere_unsigned(torch):
    """The reference's own Q8 form (unsigned byte codes, qwen.metal:112-125) on all three projections + shared expert."""
    check_layer(torch, util.cfg2(experts=32, top_k=4, gate_bits=8, up_bits=8, down_bits=8, q8_signed=0, max_tokens=8), 3)


def test_reference_arithmetic_at_native_shape(torch):
    """Reference arithmetic (every BF16 boundary) at hidden 2560 / ffn 640 / top-10 + shared / BF16 metadata.
    Against the checker in the same mode the result may differ by BF16 rounding flips of intermediates, so the
    tolerance is the reference's own for its CPU oracle (scripts/qwen/reference_numpy.py:259-263):
    relative L2 < 0.01, cosine > 0.99995, expert ids exact."""
    cfg = util.cfg0()
    m = make(cfg)
    m.synth_fill_layer(0, SEED)
    T = 6
    x = synth.activations(cfg, SEED, 0, T)
    out = m.moe(0, device_x(m, x)).float().cpu().numpy()
    routing = m.last_routing(T)
    want = oracle_layer(cfg, SEED, 0, x, routing["ids"], want_intermediates=True)
    assert np.array_equal(routing["ids"], want["ids"])
    assert np.array_equal(routing["logits"].view(np.uint32), want["logits"].view(np.uint32))
    a, b = out.astype(np.float64).reshape(-1), want["out"].astype(np.float64).reshape(-1)
    rel = np.linalg.norm(a - b) / np.linalg.norm(b)
    cos = a @ b / (np.linalg.norm(a) * np.linalg.norm(b))
    assert rel < 0.01 and cos > 0.99995, (rel, cos)
    assert rel < 2e-3, rel
    assert np.array_equal(out, oracle.bf(out))             # every output is a bf16 value


def test_reference_numpy_golden_fixture(torch):
    """The committed outputs of scripts/qwen/reference_numpy.py::moe (tests/golden/numpy_moe_config0.npz)."""
    from tests.golden.make_golden import CONFIG0, CONFIG0_SEED, CONFIG0_TOKENS
    cfg = MoeConfig(**dict(CONFIG0, max_tokens=8))
    gold = np.load(os.path.join(os.path.dirname(__file__), "golden", "numpy_moe_config0.npz"))
    m = make(cfg)
    m.synth_fill_layer(0, CONFIG0_SEED)
    x = synth.activations(cfg, CONFIG0_SEED, 0, CONFIG0_TOKENS)
    out = m.moe(0, device_x(m, x)).float().cpu().numpy()
    ids = m.last_routing(CONFIG0_TOKENS)["ids"]
    assert np.array_equal(ids, gold["ids"])
    a, b = out.astype(np.float64).reshape(-1), gold["out"].astype(np.float64).reshape(-1)
    rel = np.linalg.norm(a - b) / np.linalg.norm(b)
    cos = a @ b / (np.linalg.norm(a) * np.linalg.norm(b))
    assert rel < 0.01 and cos > 0.99995, (rel, cos)


def test_outputs_land_only_in_their_slots(torch):
    """Guard regions around the output stay untouched (tests/test_qwen.cpp:1087-1099, 1517-1525 use sentinels)."""
    cfg = util.cfg2(experts=64, max_tokens=16)
    m = make(cfg)
    m.synth_fill_layer(0, SEED)
    T = 5
    x = device_x(m, synth.activations(cfg, SEED, 0, T))
    big = torch.full(((T + 2) * cfg.hidden,), -17.0, dtype=torch.float32, device="cuda")
    out = big[cfg.hidden:(T + 1) * cfg.hidden].view(T, cfg.hidden)
    m.moe(0, x, out=out)
    torch.cuda.synchronize()
    assert bool((big[:cfg.hidden] == -17).all()) and bool((big[(T + 1) * cfg.hidden:] == -17).all())
    assert bool((out != -17).all())


def test_argument_validation(torch):
    cfg = util.cfg2(experts=64, max_tokens=8)
    m = make(cfg)
    x = torch.zeros((4, cfg.hidden), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        m.moe(0, torch.zeros((9, cfg.hidden), dtype=torch.bfloat16, device="cuda"))     # above max_tokens
    with pytest.raises(IndexError):
        m.moe(1, x)                                                                      # layer outside the model
    with pytest.raises(ValueError):
        m.moe(0, x, out=x.view(torch.float32)[:, :cfg.hidden // 2].reshape(-1)[:4 * cfg.hidden // 2])  # aliasing
    from zerocool_b200.moe import Moe
    with pytest.raises(ValueError):
        Moe(util.cfg2(experts=48), 0)                                                    # not a multiple of 32
    with pytest.raises(IndexError):
        m.load_layer(0, records=np.zeros((2, cfg.record_stride), np.uint8), first_expert=63)


def test_invalid_router_output_is_reported(torch):
    """A token whose scores are all -inf selects nothing: ids -1, status flagged, like model.cpp:459."""
    cfg = util.cfg2(experts=64, max_tokens=4, router_dtype=F32)
    m = make(cfg)
    m.synth_fill_layer(0, SEED)
    router = np.full((64, cfg.hidden), np.inf, np.float32)          # x . inf = +-inf or NaN for every expert
    router[:, 1::2] = -np.inf
    m.load_layer(0, router_w=router)
    x = device_x(m, synth.activations(cfg, SEED, 0, 2))
    m.moe(0, x)
    with pytest.raises(RuntimeError, match="invalid router output"):
        m.check_status()


def test_stack_host_and_device_paths_agree(torch):
    """Three chained layers: the graph-replayed stack equals layer-by-layer calls with the same glue, stays finite,
    and the host-buffer entry points return the same bytes as the device ones."""
    cfg = util.cfg2(experts=64, layers=3, out_dtype=BF16, max_tokens=8)
    m = make(cfg)
    for l in range(3):
        m.synth_fill_layer(l, SEED)
    T = 4
    x_np = synth.activations(cfg, SEED, 0, T)
    x = device_x(m, x_np)
    first = m.stack(x).clone()
    second = m.stack(x).clone()          # graph replay
    assert torch.equal(first, second) and bool(torch.isfinite(first.float()).all())
    cur = x
    for l in range(3):
        o = m.moe(l, cur)
        if l < 2:
            f = o.float()
            d = f - f.mean(-1, keepdim=True)
            cur = (d * (1.0 / torch.sqrt((d * d).mean(-1, keepdim=True)))).to(torch.bfloat16)
    err = util.rel_max_error(first.float().cpu().numpy(), o.float().cpu().numpy())
    assert err < 0.05, err                # glue differs only in summation order; bf16 flips allowed
    x_host = torch.from_numpy(x_np).to(torch.bfloat16).pin_memory()
    out_host = torch.empty((T, cfg.hidden), dtype=torch.bfloat16).pin_memory()
    m.moe_host(0, x_host, out_host)
    assert torch.equal(out_host, m.moe(0, x).cpu())
    m.stack_host(x_host, out_host)
    assert torch.equal(out_host, first.cpu())
    assert m.launches > 0


@pytest.mark.parametrize("tokens", [3, 40])
def test_dependent_launch_does_not_change_results(torch, tokens):
    """The stack with programmatic dependent launch (kernels overlapping their predecessor's tail) returns the same
    bytes as with plainly serialised launches, eagerly and as a replayed graph."""
    cfg = util.cfg2(experts=64, layers=4, out_dtype=BF16, max_tokens=64)
    m = make(cfg)
    for l in range(cfg.layers):
        m.synth_fill_layer(l, SEED)
    x = device_x(m, synth.activations(cfg, SEED, 0, tokens))
    m.set_option("pdl", 0)
    plain = m.stack(x).clone()
    m.set_option("pdl", 1)
    overlapped = [m.stack(x).clone() for _ in range(3)]          # capture, then two replays
    eager = m.stack_eager(x).clone()
    assert all(torch.equal(plain, o) for o in overlapped) and torch.equal(plain, eager)
    assert m.status() == 0
    with pytest.raises(ValueError):
        m.set_option("no such option", 1)


def test_decode_token_order_invariance_at_full_shape(torch):
    """Config 2 at full size, 64 tokens: a token's output does not depend on where it sits in the batch."""
    cfg = util.cfg2(max_tokens=64)
    m = make(cfg)
    m.synth_fill_layer(0, SEED)
    x = synth.activations(cfg, SEED, 0, 64)
    out = m.decode(0, device_x(m, x)).clone()
    order = np.random.default_rng(4).permutation(64)
    out_p = m.decode(0, device_x(m, np.ascontiguousarray(x[order])))
    assert torch.equal(out_p, out[torch.from_numpy(order).to(out.device)])


@pytest.mark.parametrize("tokens", [4, 64])
def test_exact_intermediate_option(torch, tokens):
    """With "exact_h" nothing below FP32 is rounded between gate/up and down: the error drops from the FP16 rounding
    of the SwiGLU rows (~1e-3 x RMS) to the tensor cores' accumulation error."""
    out_exact, want, _ = check_layer(torch, util.cfg2(), tokens, exact_h=1, tol=5e-4)
    out_fast, _, _ = check_layer(torch, util.cfg2(), tokens, exact_h=0)
    assert util.rel_max_error(out_fast, out_exact) <= TOL
