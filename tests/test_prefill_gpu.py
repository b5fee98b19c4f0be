"""GPU parity tests of the prefill family (tcgen05 grouped GEMM) through the C ABI: ids and permutation
bit-exact, outputs within 2e-3 x RMS of the CPU checker, on even, skewed and ragged expert loads."""
import numpy as np
import pytest

from oracle import oracle
from tests import util
from tests.test_moe_gpu import TOL, device_x, make, oracle_layer
from zerocool_b200 import synth
from zerocool_b200.records import BF16, F32

pytestmark = pytest.mark.gpu
SEED = 77


def run_prefill(cfg, tokens, router=None):
    import torch
    m = make(cfg)
    m.synth_fill_layer(0, SEED)
    if router is not None:
        m.load_layer(0, router_w=router)
    x = synth.activations(cfg, SEED, 0, tokens)
    out = m.prefill(0, device_x(m, x)).float().cpu().numpy()
    routing = m.last_routing(tokens)
    assert m.status() == 0                                    # no invalid route, no device-side timeout
    return m, x, out, routing


def check_against_oracle(cfg, x, out, routing, router=None):
    records = util.selected_records(cfg, SEED, 0, routing["ids"])
    want = oracle.moe_layer(cfg.as_dict(), records, synth.router(cfg, SEED, 0) if router is None else router, x,
                            shared_record=synth.record(cfg, SEED, 0, synth.SHARED_EXPERT) if cfg.has_shared else None,
                            shared_gate_w=synth.shared_gate(cfg, SEED, 0) if cfg.has_shared else None)
    assert np.array_equal(routing["ids"], want["ids"])
    offsets, perm = oracle.permute(want["ids"], cfg.experts)
    assert np.array_equal(routing["offsets"], offsets) and np.array_equal(routing["perm"], perm)
    err = util.rel_max_error(out, want["out"])
    print("prefill max-abs error / RMS:", err)
    assert err <= TOL, err
    return err


def test_prefill_matches_oracle_small_experts():
    """64 experts, 300 tokens: ~47 rows per expert, one token tile each, plus the shared expert's three tiles."""
    cfg = util.cfg2(experts=64, max_tokens=512)
    m, x, out, routing = run_prefill(cfg, 300)
    check_against_oracle(cfg, x, out, routing)


def test_prefill_equals_decode_family_on_skewed_loads():
    """Router rows scaled by a Zipf-like factor: a few experts receive hundreds of rows (several 64-token
    tiles), many receive a handful or none. The prefill family must agree with the decode family."""
    cfg = util.cfg2(experts=128, max_tokens=1024)
    router = synth.router(cfg, SEED, 0).copy()
    router *= (1.0 + 60.0 / (1.0 + np.arange(cfg.experts, dtype=np.float32)))[:, None]
    tokens = 700
    m, x, out, routing = run_prefill(cfg, tokens, router=router)
    counts = np.diff(routing["offsets"])
    assert counts.max() > 256 and (counts < 16).sum() > 4           # genuinely skewed and ragged
    dec = m.decode(0, device_x(m, x)).float().cpu().numpy()
    assert m.status() == 0
    print("loads max", counts.max(), "below 16:", int((counts < 16).sum()), "prefill vs decode:", util.rel_max_error(out, dec))
    assert util.rel_max_error(out, dec) <= TOL
    # spot-check the first 24 tokens against the CPU checker
    sub = oracle.moe_layer(cfg.as_dict(), util.selected_records(cfg, SEED, 0, routing["ids"][:24]), router, x[:24],
                           shared_record=synth.record(cfg, SEED, 0, synth.SHARED_EXPERT), shared_gate_w=synth.shared_gate(cfg, SEED, 0))
    assert np.array_equal(sub["ids"], routing["ids"][:24])
    assert util.rel_max_error(out[:24], sub["out"]) <= TOL


def test_prefill_with_asymmetric_biases():
    """bias != -8 scale: the second term of the affine form, (8 s + b) * sum(x), is then not zero and runs through
    the correction stages of the kernel (metadata tile times the activations' group sums)."""
    from zerocool_b200.records import build_record, float_to_meta
    cfg = util.cfg2(experts=32, top_k=4, max_tokens=512)
    rng = np.random.default_rng(5)

    def skewed(expert):
        parts = []
        for p in range(3):
            codes, sbits, bbits = synth.projection_parts(cfg, SEED, 0, expert, p)
            s = sbits.view(np.float16).astype(np.float32)
            b = -8.0 * s + rng.uniform(-0.03, 0.03, size=s.shape).astype(np.float32)
            parts.append((codes, sbits, float_to_meta(b, cfg.meta_dtype).reshape(bbits.shape)))
        return build_record(cfg, parts)

    records = [skewed(e) for e in range(cfg.experts)]
    shared = skewed(synth.SHARED_EXPERT)
    m = make(cfg)
    m.load_layer(0, records=np.stack(records), router_w=synth.router(cfg, SEED, 0), shared_record=shared, shared_gate_w=synth.shared_gate(cfg, SEED, 0))
    x = synth.activations(cfg, SEED, 0, 200)
    out = m.prefill(0, device_x(m, x)).float().cpu().numpy()
    assert m.status() == 0
    want = oracle.moe_layer(cfg.as_dict(), records, synth.router(cfg, SEED, 0), x, shared_record=shared, shared_gate_w=synth.shared_gate(cfg, SEED, 0))
    assert np.array_equal(m.last_routing(200)["ids"], want["ids"])
    err = util.rel_max_error(out, want["out"])
    print("asymmetric biases, prefill max-abs error / RMS:", err)
    assert err <= TOL, err
    dec = m.decode(0, device_x(m, x)).float().cpu().numpy()
    assert util.rel_max_error(dec, want["out"]) <= TOL


def test_prefill_config5_shape():
    """hidden 4096 (config 5's geometry), no shared expert, a token count that is not a multiple of 16."""
    cfg = util.cfg2(hidden=4096, experts=32, top_k=4, has_shared=0, max_tokens=512)
    m, x, out, routing = run_prefill(cfg, 261)
    check_against_oracle(cfg, x, out, routing)


def test_forward_picks_the_family_by_token_count():
    cfg = util.cfg2(experts=64, max_tokens=512)
    import torch
    m = make(cfg)
    m.synth_fill_layer(0, SEED)
    x = device_x(m, synth.activations(cfg, SEED, 0, 320))
    before = m.launches
    a = m.moe(0, x)
    used = m.launches - before
    b = m.prefill(0, x)
    assert torch.equal(a, b) and used == 10             # router, route, gate/up + down for few-row experts, tiles, activations + sums, gate/up, sums, down, combine
    small = device_x(m, synth.activations(cfg, SEED, 0, 8))
    before = m.launches
    m.moe(0, small)
    assert m.launches - before == 5
    with pytest.raises(ValueError):
        make(util.cfg2(experts=64, max_tokens=16)).prefill(0, small)


def test_full_shape_token_order_invariance():
    """benchmark configuration 3 at full size (512 experts, top-10 + shared, 2048 tokens, Zipf router bias): permuting the
    tokens of the batch permutes the outputs bit for bit, for both kernel families' routing and for the grouped GEMM
    (a token's result must not depend on its position in a tile or on its neighbours), and the first tokens agree
    with the CPU checker."""
    import torch
    cfg = util.cfg2(max_tokens=2048)
    m = make(cfg)
    m.synth_fill_layer(0, SEED)
    bias = synth.zipf_router_bias(cfg, SEED, 0)
    m.set_router_bias(0, bias)
    tokens = 2048
    x = synth.activations(cfg, SEED, 0, tokens)
    out = m.prefill(0, device_x(m, x)).clone()
    ids = m.last_routing(tokens)["ids"].copy()
    order = np.random.default_rng(3).permutation(tokens)
    out_p = m.prefill(0, device_x(m, np.ascontiguousarray(x[order])))
    assert m.status() == 0
    assert np.array_equal(m.last_routing(tokens)["ids"], ids[order])
    assert torch.equal(out_p, out[torch.from_numpy(order).to(out.device)])
    counts = np.bincount(ids.reshape(-1), minlength=cfg.experts)
    assert counts.max() > 512 and (counts == 0).sum() > 100          # the skew of the configuration
    check = 16
    want = oracle.moe_layer(cfg.as_dict(), util.selected_records(cfg, SEED, 0, ids[:check]), synth.router(cfg, SEED, 0), x[:check],
                            shared_record=synth.record(cfg, SEED, 0, synth.SHARED_EXPERT), shared_gate_w=synth.shared_gate(cfg, SEED, 0),
                            router_bias=bias)
    assert np.array_equal(want["ids"], ids[:check])
    assert util.rel_max_error(out[:check].float().cpu().numpy(), want["out"]) <= TOL


@pytest.mark.parametrize("bits", [(4, 4, 4), (4, 4, 8)])
def test_prefill_at_the_native_geometry(bits):
    """hidden 2560 / ffn 640 (the reference's own layer shape): 40 groups per gate/up row and 10 per down row, so the
    metadata tile and the group sums are padded to a multiple of eight groups, the down rows' metadata is read value by
    value (20-byte rows) and the last 128-byte code line of a down row is half full. BF16 metadata and router."""
    cfg = util.cfg0(arith=oracle.ARITH_FP32, act_dtype=BF16, experts=32, top_k=10,
                    gate_bits=bits[0], up_bits=bits[1], down_bits=bits[2], max_tokens=512)
    m, x, out, routing = run_prefill(cfg, 333)
    err = check_against_oracle(cfg, x, out, routing)
    dec = m.decode(0, device_x(m, x)).float().cpu().numpy()
    assert m.status() == 0
    assert util.rel_max_error(out, dec) <= TOL
    print("native geometry", bits, "error", err)


def test_bounded_waits_give_up_and_leave_the_context_usable():
    """The give-up path of the tensor-core kernels on its own: both kinds of bounded wait face a barrier that nothing
    arrives on, run out (about 2 ms), raise the time-out bit, the CTA returns its tensor memory, and the next layer on
    the same handle runs and matches the checker - no fault, no hang, no lost context."""
    from zerocool_b200.moe import STATUS_TIMEOUT
    cfg = util.cfg2(experts=32, top_k=4, max_tokens=256)
    m, x, out, routing = run_prefill(cfg, 150)
    waited, polled, abort_flag, _ = m.wait_selftest(polls=2000)
    assert waited == 0 and polled == 0 and abort_flag == 1
    assert m.status() & STATUS_TIMEOUT                      # read and cleared
    again = m.prefill(0, device_x(m, x)).float().cpu().numpy()
    assert m.status() == 0
    assert np.array_equal(again, out)
    check_against_oracle(cfg, x, again, routing)


def test_bf16_scale_below_fp16_range_raises_the_range_bit():
    """BF16 metadata reaches far below FP16: a scale of 2e-6 would lose bits (FP16 subnormal) as the factor of the
    two-term weights, so the tensor-core family reports it in the status word instead of rounding it silently."""
    from zerocool_b200.moe import STATUS_RANGE
    from zerocool_b200.records import build_record, float_to_meta
    cfg = util.cfg2(experts=32, top_k=4, max_tokens=256, meta_dtype=BF16)
    tiny = None
    records = []
    for e in range(cfg.experts):
        parts = []
        for p in range(3):
            codes, sbits, bbits = synth.projection_parts(cfg, SEED, 0, e, p)
            if p == 0:
                sbits = sbits.copy()
                sbits.reshape(-1)[5] = float_to_meta(np.array([2e-6], np.float32), BF16)[0]
                tiny = sbits
            parts.append((codes, sbits, bbits))
        records.append(build_record(cfg, parts))
    m = make(cfg)
    m.load_layer(0, records=np.stack(records), router_w=synth.router(cfg, SEED, 0), shared_record=synth.record(cfg, SEED, 0, synth.SHARED_EXPERT),
                 shared_gate_w=synth.shared_gate(cfg, SEED, 0))
    x = synth.activations(cfg, SEED, 0, 200)
    m.prefill(0, device_x(m, x))
    assert m.status() & STATUS_RANGE
    assert tiny is not None
