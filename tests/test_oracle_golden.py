"""Pins the CPU checker (oracle/) to the reference: every known-answer vector that the reference's own
unit tests hold for the MoE path (tests/test_qwen.cpp, line ranges in each test), the Q8 packing case of
scripts/qwen/test_shared_expert_reference.py:62-68, and the committed outputs of the reference's numpy
oracle (scripts/qwen/reference_numpy.py::moe) — see tests/golden/make_golden.py."""
import json
import os

import numpy as np
import pytest

from oracle import oracle
from zerocool_b200 import synth
from zerocool_b200.records import ARITH_REFERENCE, BF16, F32, MoeConfig, bf16_bits, bf16_to_float

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
KNOWN = json.load(open(os.path.join(GOLDEN, "reference_known_answers.json")))


def round_bf16(v):
    return bf16_to_float(bf16_bits(np.asarray(v, np.float32)))


REFERENCE_ROOT = os.environ.get("ZC_REFERENCE_ROOT", "")


def test_router_matches_mlx_bit_patterns():
    """tests/test_qwen.cpp:798-826 — synthetic W/x formulas (:801-806), 16 captured fp32 bit patterns, chunk invariance."""
    g = KNOWN["router_mlx"]
    T, K, N = g["T"], g["K"], g["N"]
    n, k = np.meshgrid(np.arange(N, dtype=np.int64), np.arange(K, dtype=np.int64), indexing="ij")
    w = np.ldexp(((n * 17 + k * 23) % 251 - 125).astype(np.float32), -(k % 20 + 4).astype(np.int32)).astype(np.float32)
    wbits = (w.view(np.uint32) >> 16).astype(np.uint16)          # truncation, as the test stores it
    t, k2 = np.meshgrid(np.arange(T, dtype=np.int64), np.arange(K, dtype=np.int64), indexing="ij")
    x = (((k2 * 13 + t * 31) % 251 - 125).astype(np.float32) / np.float32(128)).astype(np.float32)
    full = oracle.router_logits(x, wbits, BF16)
    got = full.reshape(-1)[g["indices"]].view(np.uint32)
    assert [int(v) for v in got] == g["bits"]
    for offset, count in ((0, 1), (1, 7), (8, 3)):
        part = oracle.router_logits(x[offset:offset + count], wbits, BF16)
        assert np.array_equal(part, full[offset:offset + count])
    exact = x.astype(np.float64) @ bf16_to_float(wbits).astype(np.float64).T
    assert np.abs(exact - full).max() < 0.00005


def test_q4_matmul_against_double_precision():
    """tests/test_qwen.cpp:634-660 — nibble order 0x76543210, scale 2^-4 / bias -0.25 as BF16 bits."""
    K, N, T = 128, 7, 3
    words = (np.uint32(0x76543210) + (np.arange(N * K // 8, dtype=np.uint32) % 8) * np.uint32(0x11111111)).astype(np.uint32)
    s = np.full(N * K // 64, 0x3D80, np.uint16)
    b = np.full(N * K // 64, 0xBE80, np.uint16)
    x = ((np.arange(T * K) % 11 - 5) / 16).astype(np.float32).reshape(T, K)
    got = oracle.affine(4, words, s, b, N, K, x)
    nib = ((words.reshape(N, K // 8)[:, :, None] >> (4 * np.arange(8, dtype=np.uint32))) & 15).reshape(N, K).astype(np.float64)
    expect = round_bf16((x.astype(np.float64) @ (nib / 16.0 - 0.25).T).astype(np.float32))
    assert np.allclose(got, expect, rtol=1e-4, atol=0)
    # fused gate/up with the same matrix on both sides: round_bf16(round_bf16(v*sig(v))*v), exactly
    for v in got.reshape(-1):
        y = round_bf16(1 / round_bf16(1 + round_bf16(np.exp(np.float32(abs(v))))))
        gate = y if v < 0 else round_bf16(1 - y)
        assert oracle.lib().zco_bf(oracle.lib().zco_bf(float(v) * float(gate)) * float(v)) == pytest.approx(float(round_bf16(round_bf16(v * gate) * v)), abs=0)


def test_q8_byte_codes_signed_metadata_and_tails():
    """tests/test_qwen.cpp:661-696 — unsigned byte codes, +/- scales and biases, result == round_bf16(float(double dot))."""
    for K, N, G in ((320, 7, 64), (640, 8, 32), (2560, 8, 64)):
        T = 3
        w = ((np.arange(K * N, dtype=np.int64) * 17 + 251) % 256).astype(np.uint8)
        i = np.arange(K * N // G)
        s = np.where(i % 2 == 1, 0xBB80, 0x3B80).astype(np.uint16)
        b = np.where(i % 3 != 0, 0xBF00, 0x3E80).astype(np.uint16)
        x = ((np.arange(T * K) % 9 - 4) / 16).astype(np.float32).reshape(T, K)
        got = oracle.affine(8, w, s, b, N, K, x, group=G)
        decoded = (w.reshape(N, K).astype(np.float32) * np.repeat(bf16_to_float(s).reshape(N, -1), G, 1)
                   + np.repeat(bf16_to_float(b).reshape(N, -1), G, 1)).astype(np.float32)
        expect = round_bf16((x.astype(np.float64) @ decoded.astype(np.float64).T).astype(np.float32))
        assert np.array_equal(got, expect)


def test_q8_little_endian_group_boundaries():
    """scripts/qwen/test_shared_expert_reference.py:62-68 — packed uint32 words decode byte 0 first; groups of 64."""
    codes = np.array(([0, 1, 127, 255] * 16) + ([255, 128, 2, 0] * 16), dtype=np.uint8).reshape(1, 128)
    packed = codes.copy().view("<u4")
    s = bf16_bits(np.array([0.5, -2.0], np.float32))
    b = bf16_bits(np.array([-4.0, 1.0], np.float32))
    eye = np.eye(128, dtype=np.float32)
    got = oracle.affine(8, packed, s, b, 1, 128, eye, round_out=False).reshape(-1)
    expect = np.concatenate((codes[0, :64] * 0.5 - 4, codes[0, 64:].astype(np.float64) * -2 + 1))
    assert np.array_equal(got, expect.astype(np.float32))


def test_route_selects_ten_and_normalises():
    """tests/test_qwen.cpp:744-754."""
    values = (np.arange(512) % 41).astype(np.float32) - 100
    ids, weights = oracle.route(values[None], 10)
    order = np.argsort(-values, kind="stable")[:10]
    assert np.array_equal(ids[0], order)
    assert abs(float(weights.sum()) - 1) < 1e-6


def exceptional_logits(T=137, E=512, seed=123):
    """The score matrix of tests/test_qwen.cpp:757-773 (mt19937(123); ties, signed zeros, infinities, NaN)."""
    rs = np.random.RandomState(seed)
    raw = rs.randint(0, 2 ** 32, size=2 * T * E, dtype=np.uint64).astype(np.int64).reshape(T, E, 2)
    v = np.ldexp((raw[..., 0] % 2001 - 1000).astype(np.float32), -(raw[..., 1] % 12).astype(np.int32)).astype(np.float32)
    e = np.arange(E)
    for t in range(T):
        c = t % 10
        if c == 0: v[t] = e
        elif c == 1: v[t] = -e.astype(np.float32)
        elif c == 2: v[t] = e % 13
        elif c == 3: v[t] = np.where(e % 2 == 1, 0.0, -0.0)
        elif c == 4: v[t] = np.where(e < 9, e, -np.inf)
        elif c == 5: v[t] = np.where(e % 41 == 0, np.nan, v[t])
        elif c == 6: v[t] = np.where(e % 33 == 0, np.inf, v[t])
        elif c == 7: v[t] = -np.inf
        elif c == 8: v[t] = np.nan
    return v.astype(np.float32)


def test_route_ties_exceptional_scores_and_chunks():
    """tests/test_qwen.cpp:755-797 — CPU rule :776-780: stable descending sort of the values > -inf, padded with -1."""
    values = exceptional_logits()
    T = values.shape[0]
    ids, weights = oracle.route(values, 10)
    for t in range(T):
        with np.errstate(invalid="ignore"):
            cand = [e for e in range(512) if values[t, e] > -np.inf]
        cand.sort(key=lambda e: -values[t, e])            # Python's sort is stable
        cand = (cand + [-1] * 10)[:10]
        assert list(ids[t]) == cand, t
    for offset, count in ((0, 1), (1, 7), (8, 31), (39, 97), (136, 1)):
        a, b = oracle.route(values[offset:offset + count], 10)
        assert np.array_equal(a, ids[offset:offset + count])
        assert np.array_equal(b.view(np.uint32), weights[offset:offset + count].view(np.uint32))
    finite = [t for t in range(T) if t % 10 in (0, 1, 2, 3, 9)]
    assert np.allclose(weights[finite].sum(-1), 1, atol=1e-6)


def test_moe_sum_midpoint_known_answer():
    """tests/test_qwen.cpp:827-842 — the (p0+p8)+(p1+p9) order decides a BF16 midpoint."""
    g = KNOWN["moe_sum_midpoint"]
    H = 4
    cfg = dict(hidden=H, ffn=64, experts=16, top_k=10, has_shared=1, arith=ARITH_REFERENCE)
    eo = np.zeros((1, 10, H), np.float32)
    eo[0, :, 0] = np.array(g["values"], np.float32)
    w = np.array(g["weight_bits"], np.uint32).view(np.float32)[None]
    shared = np.zeros((1, H), np.float32)
    shared[0, 0] = g["shared"]
    out = oracle.combine(cfg, eo, w, shared, np.array([g["gate"]], np.float32))
    assert out[0, 0] == np.float32(g["expected"])
    assert np.all(out[0, 1:] == 0)


def test_affine_bias_uses_bf16_input_sum_rounding():
    """tests/test_qwen.cpp:863-874 — each BF16 ((1 + 1/512) - 1) rounds to zero, so the row is exactly 0."""
    codes = np.zeros(16, np.uint32)
    one = np.full(2, 0x3F80, np.uint16)
    x = np.zeros(128, np.float32)
    x[0::4], x[1::4], x[2::4] = 1, 1.0 / 512, -1
    assert oracle.affine(4, codes, one, one, 1, 128, x[None])[0, 0] == 0
    # the fp32 mode keeps the mathematically exact value 1/16
    assert oracle.affine(4, codes, one, one, 1, 128, x[None], ref=False, round_out=False)[0, 0] == np.float32(1 / 16)


def test_bf16_activation_tables():
    """tests/test_qwen.cpp:876-888 (64-point SiLU / sigmoid tables captured from MLX 0.31.1) and :890-897."""
    g = KNOWN["activations"]
    lib = oracle.lib()
    for x, sg, si in zip(g["x"], g["sigmoid"], g["silu"]):
        assert np.float32(lib.zco_bf(lib.zco_sigmoid_bf(x))) == np.float32(sg)
        assert np.float32(lib.zco_silu_bf(x)) == np.float32(si)
    b = KNOWN["sigmoid_boundary"]
    assert np.float32(lib.zco_silu_bf(b["x"])) == np.float32(b["silu"])
    assert np.float32(lib.zco_silu_bf(-b["x"])) == np.float32(-b["x"])


def config0():
    from tests.golden.make_golden import CONFIG0, CONFIG0_SEED, CONFIG0_TOKENS
    return MoeConfig(**CONFIG0), CONFIG0_SEED, CONFIG0_TOKENS


def test_reference_numpy_moe_anchor():
    """Reference-arithmetic mode against scripts/qwen/reference_numpy.py::moe (:169-181) at the native shape.
    Tolerances are the reference's own for this oracle (reference_numpy.py:259-263, 281-282): expert ids equal,
    relative L2 < 0.01, cosine > 0.99995."""
    cfg, seed, T = config0()
    gold = np.load(os.path.join(GOLDEN, "numpy_moe_config0.npz"))
    records = [synth.record(cfg, seed, 0, e) for e in range(cfg.experts)]
    x = synth.activations(cfg, seed, 0, T)
    res = oracle.moe_layer(cfg.as_dict(), records, synth.router(cfg, seed, 0), x,
                           shared_record=synth.record(cfg, seed, 0, synth.SHARED_EXPERT),
                           shared_gate_w=synth.shared_gate(cfg, seed, 0), want_intermediates=True)
    assert np.array_equal(res["ids"], gold["ids"])
    assert np.abs(res["logits"] - gold["logits"]).max() < 5e-5
    a, b = res["out"].astype(np.float64).reshape(-1), gold["out"].astype(np.float64).reshape(-1)
    rel = np.linalg.norm(a - b) / np.linalg.norm(b)
    cos = a @ b / (np.linalg.norm(a) * np.linalg.norm(b))
    assert rel < 0.01 and cos > 0.99995, (rel, cos)
    # much tighter in practice: at most a few BF16 ulps on a few coordinates
    assert rel < 2e-3, rel


@pytest.mark.skipif(not os.path.isdir(os.path.join(REFERENCE_ROOT, "scripts", "qwen")), reason="ZC_REFERENCE_ROOT does not name a reference tree")
def test_committed_numpy_fixture_is_reproducible():
    """Where ZC_REFERENCE_ROOT names the reference tree, regenerating the fixture gives the committed bytes."""
    from pathlib import Path
    from tests.golden import make_golden
    fresh = make_golden.numpy_moe(Path(REFERENCE_ROOT))
    gold = np.load(os.path.join(GOLDEN, "numpy_moe_config0.npz"))
    for k in ("out", "ids", "logits"):
        assert np.array_equal(fresh[k], gold[k])


def test_hyper_connection_steps_match_the_reference_numpy_oracle():
    """hc_mix and hc_add (kernels/metal/qwen.metal:582-595) against the reference CPU oracle's hyper() and its residual
    update (scripts/qwen/reference_numpy.py:99-106, :237), fixture tests/golden/hyper_connection.npz: bit for bit."""
    g = np.load(os.path.join(GOLDEN, "hyper_connection.npz"))
    T, H = g["out"].shape
    assert np.array_equal(oracle.hc_mix(g["normed"].reshape(T, 4, H), g["gate"].reshape(T, 4, H)), g["mixed"])
    assert np.array_equal(oracle.hc_add(g["streams"].reshape(T, 4, H), g["out"], g["injection"]).reshape(T, 4 * H), g["updated"])
    if os.path.isdir(os.path.join(REFERENCE_ROOT, "scripts", "qwen")):
        from pathlib import Path
        from tests.golden import make_golden
        fresh = make_golden.hyper_connection(Path(REFERENCE_ROOT))
        assert all(np.array_equal(fresh[k], g[k]) for k in g.files)


def test_permute_is_a_stable_counting_sort():
    """src/engine/model.cpp:449-461, 473-474 and src/engine/pipeline.cpp:18-23."""
    rng = np.random.default_rng(5)
    ids = rng.integers(0, 64, size=(37, 8), dtype=np.int32)
    offsets, perm = oracle.permute(ids, 64)
    flat = ids.reshape(-1)
    positions = [[] for _ in range(64)]
    for p, e in enumerate(flat):
        positions[e].append(p)
    assert list(perm) == [p for e in range(64) for p in positions[e]]
    assert list(offsets) == list(np.concatenate(([0], np.cumsum([len(p) for p in positions]))))
    bad = ids.copy()
    bad[3, 2] = -1
    with pytest.raises(ValueError):
        oracle.permute(bad, 64)
