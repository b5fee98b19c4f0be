"""GPU parity at the full sizes of the benchmark configurations and on the inputs that stress the error margin:
free biases, scaled activations, the mixed 4/8-bit ragged batch, 8192-token prefill, all 512 experts at hidden 4096,
a chained stack against the CPU checker chained with the same glue, the reference's known-answer vectors fed to the
device kernels, and the host-side contract (alignment, cancellation, graph cache, value-range status)."""
import json
import os

import numpy as np
import pytest

from oracle import oracle
from tests import util
from tests.test_moe_gpu import TOL, device_x, make, oracle_layer
from zerocool_b200 import synth
from zerocool_b200.records import ARITH_REFERENCE, BF16, F32, MoeConfig

pytestmark = pytest.mark.gpu
SEED = 4242
KNOWN = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_known_answers.json")))


def glue(out):
    """The stack's inter-layer stand-in on the CPU: bf16((out - mean) / std) per token."""
    o = out.astype(np.float32)
    d = o - o.mean(axis=-1, keepdims=True, dtype=np.float32)
    scale = (1.0 / np.sqrt(np.mean(d * d, axis=-1, keepdims=True, dtype=np.float32))).astype(np.float32)
    return oracle.bf(d * scale)


def load_asymmetric(cfg, seed=SEED, spread=0.03):
    rng = np.random.default_rng(11)
    records = [util.asymmetric_record(cfg, seed, 0, e, rng, spread) for e in range(cfg.experts)]
    shared = util.asymmetric_record(cfg, seed, 0, synth.SHARED_EXPERT, rng, spread) if cfg.has_shared else None
    m = make(cfg)
    m.load_layer(0, records=np.stack(records), router_w=synth.router(cfg, seed, 0), shared_record=shared,
                 shared_gate_w=synth.shared_gate(cfg, seed, 0) if cfg.has_shared else None)
    return m, records, shared


@pytest.mark.parametrize("tokens", [3, 64])
def test_decode_family_with_free_biases(tokens):
    """bias != -8 scale: the bias term b * sum(x) no longer cancels against the codes' offset, so a rounding of an
    activation to FP16 shows in the result unless it enters through the whole weight s q + b."""
    cfg = util.cfg2(experts=32, top_k=4, max_tokens=64)
    m, records, shared = load_asymmetric(cfg)
    x = synth.activations(cfg, SEED, 0, tokens)
    out = m.decode(0, device_x(m, x)).float().cpu().numpy()
    assert m.status() == 0
    want = oracle.moe_layer(cfg.as_dict(), records, synth.router(cfg, SEED, 0), x, shared_record=shared, shared_gate_w=synth.shared_gate(cfg, SEED, 0))
    assert np.array_equal(m.last_routing(tokens)["ids"], want["ids"])
    err = util.rel_max_error(out, want["out"])
    print("decode family, free biases, max-abs error / RMS:", err)
    assert err <= TOL, err


@pytest.mark.parametrize("family", ["decode", "prefill"])
@pytest.mark.parametrize("scale", [8.0, 0.125])
def test_scaled_activations_keep_the_margin(family, scale):
    """Activations eight times larger and eight times smaller than N(0, 1) (exact scalings of the BF16 inputs): the
    relative error must not depend on the input scale (no operand may drift towards FP16's limits)."""
    cfg = util.cfg2(experts=64, max_tokens=256)
    m = make(cfg)
    m.synth_fill_layer(0, SEED)
    tokens = 200 if family == "prefill" else 24
    x = synth.activations(cfg, SEED, 0, tokens) * np.float32(scale)
    out = getattr(m, family)(0, device_x(m, x)).float().cpu().numpy()
    assert m.status() == 0
    want = oracle_layer(cfg, SEED, 0, x, m.last_routing(tokens)["ids"])
    assert np.array_equal(m.last_routing(tokens)["ids"], want["ids"])
    err = util.rel_max_error(out, want["out"])
    print(family, "x scaled by", scale, "max-abs error / RMS:", err)
    assert err <= TOL, err


def test_values_beyond_fp16_raise_the_range_bit():
    """x scaled by 64 drives the SwiGLU rows past FP16's largest value: the status word says so instead of the
    infinities passing silently; the next call on normal inputs is clean again."""
    from zerocool_b200.moe import STATUS_RANGE
    cfg = util.cfg2(experts=64, max_tokens=256)
    m = make(cfg)
    m.synth_fill_layer(0, SEED)
    for family, tokens in (("decode", 16), ("prefill", 200)):
        x = synth.activations(cfg, SEED, 0, tokens)
        getattr(m, family)(0, device_x(m, x * np.float32(64.0)))
        assert m.status() & STATUS_RANGE, family
        getattr(m, family)(0, device_x(m, x))
        assert m.status() == 0, family


def test_config4_mixed_bits_ragged_batch_at_full_size():
    """benchmark configuration 4, one layer at full size: 512 experts top-10 + shared, gate/up Q4 and down Q8 (int8),
    32 requests of seeded lengths 1..512 flattened to one ragged batch. The first 64 tokens and the last 16 tokens of
    the longest request against the CPU checker; permuting the whole batch permutes the outputs bit for bit; both
    kernel families agree."""
    import torch
    lengths = np.random.default_rng(20261125).integers(1, 513, size=32)
    tokens = int(lengths.sum())
    cfg = util.cfg2(down_bits=8, q8_signed=1, max_tokens=tokens)
    m = make(cfg)
    m.synth_fill_layer(0, SEED)
    x = synth.activations(cfg, SEED, 0, tokens)
    before = m.launches
    out = m.moe(0, device_x(m, x)).clone()
    assert m.launches - before == 13                      # the tensor-core family took the batch: router, route, 3 x permute, 2 x few-row experts, 5 x grouped GEMM, combine
    routing = m.last_routing(tokens)
    ids = routing["ids"].copy()
    assert m.status() == 0
    offsets, perm = oracle.permute(ids, cfg.experts)
    assert np.array_equal(routing["offsets"], offsets) and np.array_equal(routing["perm"], perm)
    longest = int(np.argmax(lengths))
    end = int(lengths[:longest + 1].sum())
    for lo, hi in ((0, 64), (end - 16, end)):
        want = oracle_layer(cfg, SEED, 0, x[lo:hi], ids[lo:hi])
        assert np.array_equal(want["ids"], ids[lo:hi])
        err = util.rel_max_error(out[lo:hi].float().cpu().numpy(), want["out"])
        print("configuration 4, tokens", lo, hi, "max-abs error / RMS:", err)
        assert err <= TOL, err
    order = np.random.default_rng(8).permutation(tokens)
    out_p = m.moe(0, device_x(m, np.ascontiguousarray(x[order])))
    assert np.array_equal(m.last_routing(tokens)["ids"], ids[order])
    assert torch.equal(out_p, out[torch.from_numpy(order).to(out.device)])
    dec = m.decode(0, device_x(m, x[:96])).float().cpu().numpy()
    assert util.rel_max_error(dec, out[:96].float().cpu().numpy()) <= TOL
    assert m.status() == 0


def test_prefill_q8_everywhere_and_free_biases():
    """8-bit codes on all three projections through the tensor-core family (u8, the reference's Q8 form), with
    free biases: against the CPU checker."""
    cfg = util.cfg2(experts=32, top_k=4, gate_bits=8, up_bits=8, down_bits=8, q8_signed=0, max_tokens=256)
    m, records, shared = load_asymmetric(cfg, spread=0.3)
    x = synth.activations(cfg, SEED, 0, 150)
    out = m.prefill(0, device_x(m, x)).float().cpu().numpy()
    assert m.status() == 0
    want = oracle.moe_layer(cfg.as_dict(), records, synth.router(cfg, SEED, 0), x, shared_record=shared, shared_gate_w=synth.shared_gate(cfg, SEED, 0))
    assert np.array_equal(m.last_routing(150)["ids"], want["ids"])
    err = util.rel_max_error(out, want["out"])
    print("prefill family, Q8 everywhere, max-abs error / RMS:", err)
    assert err <= TOL, err


def test_config3_prefill_at_8192_tokens():
    """benchmark configuration 3 at its long length: 8192 tokens, Zipf(1.1) router bias, 512 experts top-10 + shared.
    Token-order invariance on the whole batch (bit for bit), the permutation against the checker, the first and the
    last 16 tokens against the CPU checker."""
    import torch
    tokens = 8192
    cfg = util.cfg2(max_tokens=tokens)
    m = make(cfg)
    m.synth_fill_layer(0, SEED)
    bias = synth.zipf_router_bias(cfg, SEED, 0)
    m.set_router_bias(0, bias)
    x = synth.activations(cfg, SEED, 0, tokens)
    out = m.prefill(0, device_x(m, x)).clone()
    routing = m.last_routing(tokens)
    ids = routing["ids"].copy()
    assert m.status() == 0
    offsets, perm = oracle.permute(ids, cfg.experts)
    assert np.array_equal(routing["offsets"], offsets) and np.array_equal(routing["perm"], perm)
    order = np.random.default_rng(3).permutation(tokens)
    out_p = m.prefill(0, device_x(m, np.ascontiguousarray(x[order])))
    assert m.status() == 0
    assert np.array_equal(m.last_routing(tokens)["ids"], ids[order])
    assert torch.equal(out_p, out[torch.from_numpy(order).to(out.device)])
    for lo, hi in ((0, 16), (tokens - 16, tokens)):
        want = oracle_layer(cfg, SEED, 0, x[lo:hi], ids[lo:hi], router_bias=bias)
        assert np.array_equal(want["ids"], ids[lo:hi])
        err = util.rel_max_error(out[lo:hi].float().cpu().numpy(), want["out"])
        print("configuration 3 at 8192, tokens", lo, hi, "max-abs error / RMS:", err)
        assert err <= TOL, err


def test_config5_all_512_experts_on_one_handle():
    """benchmark configuration 5's layer with every expert resident (hidden 4096, 512 experts top-10, no shared expert),
    its 256-token batch: routing bit-exact on all tokens, the first 24 outputs against the CPU checker."""
    cfg = util.cfg2(hidden=4096, has_shared=0, max_tokens=256)
    m = make(cfg)
    m.synth_fill_layer(0, SEED)
    tokens = 256
    x = synth.activations(cfg, SEED, 0, tokens)
    out = m.moe(0, device_x(m, x)).float().cpu().numpy()
    routing = m.last_routing(tokens)
    assert m.status() == 0
    logits = oracle.router_logits(x, synth.router(cfg, SEED, 0), cfg.router_dtype)
    assert np.array_equal(routing["logits"].view(np.uint32), logits.view(np.uint32))
    ids, _ = oracle.route(logits, cfg.top_k)
    assert np.array_equal(routing["ids"], ids)
    offsets, perm = oracle.permute(ids, cfg.experts)
    assert np.array_equal(routing["offsets"], offsets) and np.array_equal(routing["perm"], perm)
    want = oracle_layer(cfg, SEED, 0, x[:24], ids[:24])
    err = util.rel_max_error(out[:24], want["out"])
    print("configuration 5 layer, 512 experts, max-abs error / RMS:", err)
    assert err <= TOL, err


def test_four_layer_stack_against_the_chained_cpu_checker():
    """Teacher forcing: layer l of the device gets the CPU chain's input of layer l; ids must be bit-exact and the
    output within tolerance at every layer. Free running: the device's own two-layer chain (graph-replayed stack, glue
    in the combine kernel) against the CPU chain after two layers."""
    layers, tokens = 4, 12
    cfg = util.cfg2(experts=64, layers=layers, max_tokens=16)
    m = make(cfg)
    for layer in range(layers):
        m.synth_fill_layer(layer, SEED)
    x = synth.activations(cfg, SEED, 0, tokens)
    cpu_inputs, cpu_outputs = [], []
    for layer in range(layers):
        cpu_inputs.append(x)
        logits = oracle.router_logits(x, synth.router(cfg, SEED, layer), cfg.router_dtype)
        ids, _ = oracle.route(logits, cfg.top_k)
        want = oracle_layer(cfg, SEED, layer, x, ids)
        cpu_outputs.append(want)
        x = glue(want["out"])
    for layer in range(layers):
        got = m.moe(layer, device_x(m, cpu_inputs[layer])).float().cpu().numpy()
        assert m.status() == 0
        assert np.array_equal(m.last_routing(tokens)["ids"], cpu_outputs[layer]["ids"]), layer
        err = util.rel_max_error(got, cpu_outputs[layer]["out"])
        print("teacher-forced layer", layer, "max-abs error / RMS:", err)
        assert err <= TOL, (layer, err)
    two = MoeConfig(**{**cfg.__dict__, "layers": 2})
    m2 = make(two)
    for layer in range(2):
        m2.synth_fill_layer(layer, SEED)
    free = m2.stack(device_x(m2, cpu_inputs[0])).float().cpu().numpy()
    assert m2.status() == 0
    # Layer 1 sees layer 0's error through the BF16 rounding of the glue: an input that moves by 1e-3 crosses a BF16
    # boundary (2^-7 apart near 1) in a few per cent of its coordinates, which moves a logit by ~1e-3 and can swap two
    # neighbouring experts of a token. Tokens that routed exactly as the CPU chain did are compared; they must be the
    # majority, and the selected sets may differ in at most one expert for the others.
    ids = m2.last_routing(tokens)["ids"]
    same = np.all(ids == cpu_outputs[1]["ids"], axis=1)
    for t in np.nonzero(~same)[0]:
        assert len(set(ids[t]) ^ set(cpu_outputs[1]["ids"][t])) <= 2, t
    assert same.sum() * 2 > tokens, same
    a, b = free[same].astype(np.float64), cpu_outputs[1]["out"][same].astype(np.float64)
    rel_l2 = float(np.linalg.norm(a - b) / np.linalg.norm(b))
    err = util.rel_max_error(free[same], cpu_outputs[1]["out"][same])
    print("free-running two-layer chain:", int(same.sum()), "of", tokens, "tokens routed identically; relative L2", rel_l2, "max-abs error / RMS:", err)
    assert rel_l2 <= 5e-3 and err <= 3e-2, (rel_l2, err)


def test_moe_sum_midpoint_vector_through_the_combine_kernel():
    """The reference's own known answer for the reduction order (tests/test_qwen.cpp:827-842): (p0 + p8) + (p1 + p9)
    first decides a BF16 midpoint; expected 0.01190185546875. Fed to combine_kernel in reference arithmetic."""
    import torch
    g = KNOWN["moe_sum_midpoint"]
    H = 128
    cfg = util.cfg2(hidden=H, ffn=128, experts=32, top_k=10, has_shared=1, arith=ARITH_REFERENCE, act_dtype=F32, out_dtype=F32, max_tokens=4)
    m = make(cfg)
    eo = np.zeros((1, 10, H), np.float32)
    eo[0, :, 0] = np.array(g["values"], np.float32)
    w = np.array(g["weight_bits"], np.uint32).view(np.float32)[None].copy()
    shared = np.zeros((1, H), np.float32)
    shared[0, 0] = g["shared"]
    gate = np.array([g["gate"]], np.float32)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()          # noqa: E731
    out = m.combine(dev(eo), dev(w), dev(np.zeros((1, 10), np.int32)), dev(shared), dev(np.concatenate([gate, np.zeros(3, np.float32)]))).cpu().numpy()
    assert out[0, 0] == np.float32(g["expected"])
    assert np.all(out[0, 1:] == 0)
    want = oracle.combine(cfg.as_dict(), eo, w, shared, gate)
    assert np.array_equal(out, want)


def test_activation_tables_on_the_device():
    """The 64-point SiLU / sigmoid tables and the -6.84375 boundary the reference holds (tests/test_qwen.cpp:876-897),
    through the device's sigmoid_bf."""
    import torch
    g = KNOWN["activations"]
    m = make(util.cfg2(experts=32, top_k=4, max_tokens=4))
    x = torch.tensor(g["x"] + [KNOWN["sigmoid_boundary"]["x"], -KNOWN["sigmoid_boundary"]["x"]], dtype=torch.float32, device="cuda")
    sg, si = m.activation_bf16(x)
    sg, si = sg.cpu().numpy(), si.cpu().numpy()
    assert np.array_equal(sg[:64], np.array(g["sigmoid"], np.float32))
    assert np.array_equal(si[:64], np.array(g["silu"], np.float32))
    assert si[64] == np.float32(KNOWN["sigmoid_boundary"]["silu"]) and si[65] == np.float32(-KNOWN["sigmoid_boundary"]["x"])


def test_misaligned_and_aliased_buffers_are_argument_errors():
    """Every entry point that takes a caller buffer refuses a pointer off the 16-byte grid before anything is launched."""
    import torch
    from zerocool_b200.moe import ZC_EINVAL, _ptr
    cfg = util.cfg2(experts=64, max_tokens=8)
    m = make(cfg)
    m.synth_fill_layer(0, SEED)
    lib, h, s = m.lib, m._h, torch.cuda.current_stream().cuda_stream
    T = 4
    x = torch.zeros((T * cfg.hidden + 8,), dtype=torch.bfloat16, device="cuda")
    f = torch.zeros((T * cfg.experts + 8,), dtype=torch.float32, device="cuda")
    i32 = torch.zeros((T * cfg.top_k + 8,), dtype=torch.int32, device="cuda")
    out = torch.zeros((T * cfg.hidden + 8,), dtype=torch.float32, device="cuda")
    before = m.launches
    assert lib.zc_moe_router(h, 0, _ptr(x) + 2, T, _ptr(f), s) == ZC_EINVAL
    assert lib.zc_moe_router(h, 0, _ptr(x), T, _ptr(f) + 4, s) == ZC_EINVAL
    assert lib.zc_moe_route(h, _ptr(f) + 4, T, _ptr(i32), _ptr(f), s) == ZC_EINVAL
    assert lib.zc_moe_permute(h, _ptr(i32) + 4, T, _ptr(i32), _ptr(i32), s) == ZC_EINVAL
    assert lib.zc_moe_forward(h, 0, _ptr(x) + 2, T, _ptr(out), s) == ZC_EINVAL
    assert lib.zc_moe_forward(h, 0, _ptr(x), T, _ptr(out) + 4, s) == ZC_EINVAL
    assert lib.zc_moe_ep_dispatch(h, 0, _ptr(x) + 2, T, _ptr(out), _ptr(i32), s) == ZC_EINVAL
    w = torch.zeros((cfg.experts * cfg.hidden + 8,), dtype=torch.float32, device="cuda")
    assert lib.zc_router_logits_noalloc(_ptr(x) + 2, BF16, _ptr(w), F32, T, cfg.hidden, cfg.experts, _ptr(f), s) == ZC_EINVAL
    assert lib.zc_router_logits_noalloc(_ptr(x), BF16, _ptr(w) + 4, F32, T, cfg.hidden, cfg.experts, _ptr(f), s) == ZC_EINVAL
    assert lib.zc_router_logits_noalloc(_ptr(x), BF16, _ptr(w), F32, T, cfg.hidden, cfg.experts, _ptr(w), s) == ZC_EINVAL      # logits over router_w
    assert m.launches == before
    torch.cuda.synchronize()
    assert m.status() == 0


def test_cancel_flag_stops_the_stack():
    """The reference's cancel flag: set before a call -> "generation cancelled" and nothing is issued; cleared -> the
    stack runs and returns the same bytes as before."""
    import torch
    from zerocool_b200.moe import Cancelled
    cfg = util.cfg2(experts=64, layers=3, out_dtype=BF16, max_tokens=8)
    m = make(cfg)
    for layer in range(3):
        m.synth_fill_layer(layer, SEED)
    x = device_x(m, synth.activations(cfg, SEED, 0, 5))
    want = m.stack(x).clone()
    flag = np.zeros(1, np.int32)
    m.set_cancel(flag)
    flag[0] = 1
    before = m.launches
    for call in (lambda: m.stack(x), lambda: m.stack_eager(x), lambda: m.moe(0, x)):
        with pytest.raises(Cancelled):
            call()
    assert m.launches == before
    flag[0] = 0
    assert torch.equal(m.stack(x), want)
    m.set_cancel(None)


def test_graph_cache_follows_bias_changes_and_stays_bounded():
    """A captured stack must not outlive what it captured: removing a router bias drops the captures (the replay
    equals the eager run again), and more distinct (x, out) pairs than the cache holds still give right answers."""
    import torch
    cfg = util.cfg2(experts=64, layers=2, out_dtype=BF16, max_tokens=8)
    m = make(cfg)
    for layer in range(2):
        m.synth_fill_layer(layer, SEED)
    x = device_x(m, synth.activations(cfg, SEED, 0, 6))
    plain = m.stack(x).clone()
    m.set_router_bias(0, synth.zipf_router_bias(cfg, SEED, 0))
    biased = m.stack(x).clone()
    assert not torch.equal(plain, biased)
    m.set_router_bias(0, None)
    assert torch.equal(m.stack(x), plain) and torch.equal(m.stack_eager(x), plain)
    keep = []
    for i in range(12):                                   # more captures than the cache holds
        xi, oi = x.clone(), torch.empty_like(plain)
        keep.append((xi, oi))
        m.stack(xi, oi)
        assert torch.equal(oi, plain), i
    for xi, oi in keep[:3]:                               # evicted entries are captured again
        oi.zero_()
        m.stack(xi, oi)
        assert torch.equal(oi, plain)
    assert m.status() == 0


def test_replay_of_a_traced_run_reproduces_it_bit_for_bit(tmp_path):
    """Route trace -> replay: the ids of a three-layer run are written as a route trace, read back, and forced into
    the layers (router for the scores, no top-k search): same bytes out. A foreign selection is honoured too."""
    import torch
    from zerocool_b200.route_trace import RouteTrace, read_route_trace
    cfg = util.cfg2(experts=64, layers=3, max_tokens=16)
    m = make(cfg)
    for layer in range(cfg.layers):
        m.synth_fill_layer(layer, SEED)
    tokens = 7
    xs = [device_x(m, synth.activations(cfg, SEED, layer, tokens)) for layer in range(cfg.layers)]
    path = tmp_path / "routes.jsonl"
    outs = []
    with RouteTrace(path, {"test": "replay"}, cfg.layers, cfg.top_k) as trace:
        trace.request_begin("r0", [], tokens)
        trace.begin(1, 0, tokens, phase="prefill")
        for layer in range(cfg.layers):
            outs.append(m.moe(layer, xs[layer]).clone())
            trace.routes(layer, 0, tokens, m.last_routing(tokens)["ids"])
        trace.commit(tokens)
        trace.request_end([], "stop")
        trace.finish()
    (recorded,) = read_route_trace(path, cfg.layers, cfg.top_k, cfg.experts)
    for layer in range(cfg.layers):
        ids = torch.from_numpy(recorded["routes"][layer]).cuda()
        again = m.moe_routed(layer, xs[layer], ids)
        assert torch.equal(again, outs[layer]), layer
        assert np.array_equal(m.last_routing(tokens)["ids"], recorded["routes"][layer])
    assert m.status() == 0
    foreign = torch.from_numpy(np.stack([np.arange(t, t + cfg.top_k) % cfg.experts for t in range(tokens)]).astype(np.int32)).cuda()
    other = m.moe_routed(0, xs[0], foreign)
    routing = m.last_routing(tokens)
    assert m.status() == 0 and bool(torch.isfinite(other).all()) and not torch.equal(other, outs[0])
    assert np.allclose(routing["weights"].sum(-1), 1.0, atol=1e-5) and np.array_equal(routing["ids"], foreign.cpu().numpy())
    logits = oracle.router_logits(synth.activations(cfg, SEED, 0, tokens), synth.router(cfg, SEED, 0), cfg.router_dtype)
    picked = np.take_along_axis(logits, foreign.cpu().numpy().astype(np.int64), axis=1).astype(np.float64)
    want_w = np.exp(picked - picked[:, :1])
    assert np.allclose(routing["weights"], want_w / want_w.sum(-1, keepdims=True), rtol=1e-5)
    bad = foreign.clone()
    bad[0, 0] = cfg.experts + 3
    m.moe_routed(0, xs[0], bad)
    assert m.status() & 1


def test_hyper_connection_mix_and_fused_residual_update():
    """The steps either side of the layer. hc_mix on the device against the reference oracle's fixture, bit for bit; the
    combine with hc_add as its epilogue against combine followed by the CPU hc_add - in reference arithmetic (BF16
    boundaries) and in FP32 arithmetic, where the fused and the two-step results must be equal to the last bit."""
    import torch
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "hyper_connection.npz"))
    T, H = g["out"].shape
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a, np.float32)).cuda()          # noqa: E731
    for arith in (ARITH_REFERENCE, 0):
        cfg = util.cfg0(arith=arith, act_dtype=F32, max_tokens=4)
        m = make(cfg)
        m.synth_fill_layer(0, SEED)
        x = m.hc_mix(dev(g["normed"]), dev(g["gate"]))
        assert np.array_equal(x.cpu().numpy(), g["mixed"])
        streams, inject = dev(g["streams"]), dev(g["injection"])
        fused = m.moe_hc(0, x, streams, inject).cpu().numpy().reshape(T, 4, H)
        plain = m.moe(0, x).cpu().numpy()
        assert m.status() == 0
        want = oracle.hc_add(g["streams"].reshape(T, 4, H), plain, g["injection"], ref=arith == ARITH_REFERENCE)
        assert np.array_equal(fused, want), arith
    # against the CPU checker end to end (reference arithmetic): layer on the mixed input, then hc_add
    cfg = util.cfg0(act_dtype=F32, max_tokens=4)
    layer = oracle_layer(cfg, SEED, 0, g["mixed"], m.last_routing(T)["ids"])
    want = oracle.hc_add(g["streams"].reshape(T, 4, H), layer["out"], g["injection"]).reshape(-1).astype(np.float64)
    mref = make(cfg)
    mref.synth_fill_layer(0, SEED)
    got = mref.moe_hc(0, dev(g["mixed"]), streams, inject).cpu().numpy().reshape(-1).astype(np.float64)
    assert np.linalg.norm(got - want) / np.linalg.norm(want) < 2e-3


@pytest.mark.parametrize("family,tokens", [("decode", 9), ("prefill", 200)])
def test_mixed_artifact_routed_q4_shared_q8_in_one_handle(family, tokens):
    """The reference's mixed artifact (src/engine/metal.mm:1103-1123): routed experts Q4, the layer's shared expert Q8
    with unsigned codes, one handle (shared_*_bits). Both kernel families against the CPU checker."""
    cfg = util.cfg2(experts=64, shared_gate_bits=8, shared_up_bits=8, shared_down_bits=8, q8_signed=0, max_tokens=256)
    assert cfg.shared_cfg().record_bytes > cfg.record_bytes
    m = make(cfg)
    m.synth_fill_layer(0, SEED)
    got = m.read_layer_tensor(0, "shared_record", cfg.shared_cfg().record_bytes)
    assert np.array_equal(got, synth.record(cfg, SEED, 0, synth.SHARED_EXPERT)[:cfg.shared_cfg().record_bytes])      # generator twins agree on the Q8 layout
    shared = util.asymmetric_record(cfg.shared_cfg(), SEED, 0, synth.SHARED_EXPERT, np.random.default_rng(3), spread=0.3)    # centred u8 weights
    m.load_layer(0, shared_record=shared)
    x = synth.activations(cfg, SEED, 0, tokens)
    out = getattr(m, family)(0, device_x(m, x)).float().cpu().numpy()
    ids = m.last_routing(tokens)["ids"]
    assert m.status() == 0
    want = oracle.moe_layer(cfg.as_dict(), util.selected_records(cfg, SEED, 0, ids), synth.router(cfg, SEED, 0), x,
                            shared_record=shared, shared_gate_w=synth.shared_gate(cfg, SEED, 0))
    assert np.array_equal(ids, want["ids"])
    err = util.rel_max_error(out, want["out"])
    print("mixed artifact,", family, "max-abs error / RMS:", err)
    assert err <= TOL, err


def test_few_row_experts_take_the_streaming_kernels_in_a_long_batch():
    """In a long batch, experts with at most `prefill_small_rows` rows run on the streaming kernels and the grouped GEMM
    takes the others. Every setting of the threshold (none, some, all experts small) must agree with the CPU checker, and
    with each other within the tolerance."""
    cfg = util.cfg2(experts=128, max_tokens=512)
    router = synth.router(cfg, SEED, 0).copy()
    router *= (1.0 + 40.0 / (1.0 + np.arange(cfg.experts, dtype=np.float32)))[:, None]       # skewed: a few hot experts, many with a handful of rows
    m = make(cfg)
    m.synth_fill_layer(0, SEED)
    m.load_layer(0, router_w=router)
    tokens = 400
    x = synth.activations(cfg, SEED, 0, tokens)
    outs = {}
    for small in (0, 16, 64):
        m.set_option("prefill_small_rows", small)
        outs[small] = m.prefill(0, device_x(m, x)).float().cpu().numpy()
        assert m.status() == 0
    routing = m.last_routing(tokens)
    counts = np.diff(routing["offsets"])
    assert (counts > 64).sum() >= 2 and ((counts > 0) & (counts <= 16)).sum() >= 8      # both kinds of expert are present
    want = oracle.moe_layer(cfg.as_dict(), util.selected_records(cfg, SEED, 0, routing["ids"][:48]), router, x[:48],
                            shared_record=synth.record(cfg, SEED, 0, synth.SHARED_EXPERT), shared_gate_w=synth.shared_gate(cfg, SEED, 0))
    assert np.array_equal(want["ids"], routing["ids"][:48])
    for small, out in outs.items():
        err = util.rel_max_error(out[:48], want["out"])
        print("few-row threshold", small, "max-abs error / RMS:", err)
        assert err <= TOL, (small, err)
    with pytest.raises(ValueError):
        m.set_option("prefill_small_rows", 65)


@pytest.mark.parametrize("tokens", [5, 40])
def test_metadata_blocks_give_the_same_bits(tokens):
    """hidden 4096 (config 5's geometry): scales and biases fetched eight groups at a time (default) or per ring stage
    (option meta_blocks = 0) feed the same arithmetic: identical bits, and within tolerance of the CPU checker."""
    import torch
    cfg = util.cfg2(hidden=4096, experts=32, top_k=4, max_tokens=64)
    m = make(cfg)
    m.synth_fill_layer(0, SEED)
    x = synth.activations(cfg, SEED, 0, tokens)
    blocks = m.decode(0, device_x(m, x)).clone()
    m.set_option("meta_blocks", 0)
    stages = m.decode(0, device_x(m, x)).clone()
    assert m.status() == 0
    assert torch.equal(blocks, stages)
    routing = m.last_routing(tokens)
    records = util.selected_records(cfg, SEED, 0, routing["ids"])
    want = oracle.moe_layer(cfg.as_dict(), records, synth.router(cfg, SEED, 0), x,
                            shared_record=synth.record(cfg, SEED, 0, synth.SHARED_EXPERT), shared_gate_w=synth.shared_gate(cfg, SEED, 0))
    assert np.array_equal(routing["ids"], want["ids"])
    assert util.rel_max_error(blocks.float().cpu().numpy(), want["out"]) <= TOL


def test_tuning_switches_do_not_change_a_bit():
    """Every switch that only moves work around (copy sizes of the metadata, CTAs per few-row expert, router tile
    buffering, prefetch form, dependent launches) must leave a long batch and a short batch bit-identical."""
    import torch
    cfg = util.cfg2(max_tokens=1280)
    m = make(cfg)
    m.synth_fill_layer(0, SEED)
    m.set_router_bias(0, synth.zipf_router_bias(cfg, SEED, 0))
    long_x = device_x(m, synth.activations(cfg, SEED, 0, 1200))          # whole-K router tiles, hybrid dispatch, many-CTA permutation
    short_x = device_x(m, synth.activations(cfg, SEED, 1, 24))
    base_long, base_short = m.moe(0, long_x).clone(), m.moe(0, short_x).clone()
    ids_long = m.last_routing(24)["ids"].copy()
    for name, value, restore in (("meta_blocks", 0, 1), ("meta_blocks", 2, 1), ("meta_blocks", 3, 1), ("few_tiles_gate_up", 2, 1),
                                 ("few_tiles_down", 4, 2), ("router_db", 0, 1), ("pdl", 0, 1)):
        m.set_option(name, value)
        assert torch.equal(m.moe(0, long_x), base_long), (name, value)
        assert torch.equal(m.moe(0, short_x), base_short), (name, value)
        assert np.array_equal(m.last_routing(24)["ids"], ids_long)
        m.set_option(name, restore)
    assert m.status() == 0
    # fold_q4 is not in that list: removing the 1024 offset in FP16 before the product instead of from the FP32 group sum
    # changes the rounding of the group sums (both forms are inside the tolerance, the folded one is the default)
    m.set_option("fold_q4", 0)
    unfolded = m.moe(0, short_x)
    assert util.rel_max_error(unfolded.float().cpu().numpy(), base_short.float().cpu().numpy()) <= TOL
