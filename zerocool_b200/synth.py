"""Seeded synthetic tensors with the benchmark's shapes and value distributions.

The real checkpoint is not available, so every input is a pure function of
``(seed, layer, expert, tensor kind, element index)`` through a counter-based hash. The same function
is implemented three times — here in numpy (the definition), in the CUDA generator that fills HBM
directly for the 40 GB+ stacks (``zc_synth_*`` in csrc/synth.cu), and nowhere else — so the CPU
checker can rebuild exactly the records a GPU run used without moving them over PCIe.

Distributions: Q4 codes uniform 0..15; Q8 codes uniform -127..127 (signed) or 0..255; scales
U(0.004, 0.02) rounded to the metadata dtype; bias = -8 * scale; router weights and the shared-gate
vector ~N(0, 0.02) and activations ~N(0, 1), both as a sum of eight 16-bit uniforms (Irwin-Hall,
|z| <= 4.9) so that no transcendental function enters the generator.
"""
import numpy as np

from .records import BF16, F16, F32, MoeConfig, float_to_meta

_GOLD = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)

KIND_CODES, KIND_SCALES, KIND_ROUTER, KIND_SHARED_GATE, KIND_ACT = 0, 1, 2, 3, 4
SHARED_EXPERT = 0xFFFFFF      # expert index used for the layer's shared expert
NORMAL_STD = 65536.0 * (8.0 / 12.0) ** 0.5   # std of a sum of eight 16-bit uniforms


def _splitmix(z):
    with np.errstate(over="ignore"):
        z = (z + _GOLD).astype(np.uint64)
        z = ((z ^ (z >> np.uint64(30))) * _M1).astype(np.uint64)
        z = ((z ^ (z >> np.uint64(27))) * _M2).astype(np.uint64)
        return z ^ (z >> np.uint64(31))


def stream_id(layer, expert, projection, kind):
    return (int(layer) << 32) | (int(expert) << 8) | (int(projection) << 4) | int(kind)


def stream_key(seed, stream):
    s = _splitmix(np.array([stream], np.uint64))
    return _splitmix(np.array([seed], np.uint64) ^ s)[0]


def rand32(key, index):
    """index: uint64 array -> uint32 array."""
    with np.errstate(over="ignore"):
        z = (np.uint64(key) + np.asarray(index, np.uint64) * _GOLD).astype(np.uint64)
    return (_splitmix(z) >> np.uint64(32)).astype(np.uint32)


def normal_scale(sigma):
    return np.float32(sigma / NORMAL_STD)


def approx_normal(key, n, sigma, first=0):
    """n values ~N(0, sigma): (sum of eight 16-bit uniforms - 8*32767.5) * sigma/std, one fp32 multiply."""
    idx = (np.arange(n, dtype=np.uint64) + np.uint64(first)) * np.uint64(4)
    total = np.zeros(n, np.int64)
    for j in range(4):
        r = rand32(key, idx + np.uint64(j)).astype(np.int64)
        total += (r & 0xFFFF) + (r >> 16)
    return (total - 262140).astype(np.float32) * normal_scale(sigma)


def uniform_scale(key, n):
    """U(0.004, 0.02) in fp32 with one multiply chain and one add, each individually rounded."""
    u = (rand32(key, np.arange(n, dtype=np.uint64)) >> np.uint32(8)).astype(np.float32)
    frac = u * np.float32(1.0 / 16777216.0)
    return np.float32(0.004) + np.float32(0.016) * frac


def projection_parts(cfg: MoeConfig, seed, layer, expert, projection):
    lay = cfg.projection_layout(projection)
    n, k = lay["N"], lay["K"]
    ck = stream_key(seed, stream_id(layer, expert, projection, KIND_CODES))
    if lay["bits"] == 4:
        words = rand32(ck, np.arange(n * k // 8, dtype=np.uint64))
        codes = words.view(np.uint8).reshape(n, k // 2)
    else:
        r = rand32(ck, np.arange(n * k, dtype=np.uint64))
        if cfg.q8_signed:
            codes = ((r % np.uint32(255)).astype(np.int32) - 127).astype(np.int8).view(np.uint8).reshape(n, k)
        else:
            codes = (r & np.uint32(255)).astype(np.uint8).reshape(n, k)
    sk = stream_key(seed, stream_id(layer, expert, projection, KIND_SCALES))
    scale = uniform_scale(sk, n * (k // cfg.group))
    sbits = float_to_meta(scale, cfg.meta_dtype)
    if cfg.meta_dtype == F16:
        srounded = sbits.view(np.float16).astype(np.float32)
    else:
        srounded = (sbits.astype(np.uint32) << 16).view(np.float32)
    bbits = float_to_meta(np.float32(-8.0) * srounded, cfg.meta_dtype)
    return codes, sbits.reshape(n, -1), bbits.reshape(n, -1)


def record(cfg: MoeConfig, seed, layer, expert):
    """One expert record (uint8 [record_stride]); ``expert=SHARED_EXPERT`` gives the shared expert, in the layout of
    ``cfg.shared_cfg()`` (its own bit widths)."""
    from .records import build_record
    if expert == SHARED_EXPERT:
        cfg = cfg.shared_cfg()
    return build_record(cfg, [projection_parts(cfg, seed, layer, expert, p) for p in range(3)])


def _plain(cfg, values):
    if cfg.router_dtype == F32:
        return values.astype(np.float32)
    return float_to_meta(values, BF16)


def router(cfg: MoeConfig, seed, layer):
    """Router weight [E, H] in the configured router dtype (fp32 array or bf16 bit patterns)."""
    key = stream_key(seed, stream_id(layer, 0, 0, KIND_ROUTER))
    return _plain(cfg, approx_normal(key, cfg.experts * cfg.hidden, 0.02)).reshape(cfg.experts, cfg.hidden)


def shared_gate(cfg: MoeConfig, seed, layer):
    key = stream_key(seed, stream_id(layer, 0, 0, KIND_SHARED_GATE))
    return _plain(cfg, approx_normal(key, cfg.hidden, 0.02)).reshape(1, cfg.hidden)


def activations(cfg: MoeConfig, seed, layer, tokens, first_token=0):
    """x [T, H] ~N(0,1) as fp32 values; rounded to bf16 when the activation dtype is bf16 (or when
    the reference arithmetic is selected, whose fp32 buffers hold bf16 values)."""
    key = stream_key(seed, stream_id(layer, 0, 0, KIND_ACT))
    x = approx_normal(key, tokens * cfg.hidden, 1.0, first=first_token * cfg.hidden).reshape(tokens, cfg.hidden)
    if cfg.act_dtype == BF16 or cfg.arith == 1:
        bits = float_to_meta(x, BF16)
        x = (bits.astype(np.uint32) << 16).view(np.float32)
    return x


def zipf_router_bias(cfg: MoeConfig, seed, layer, s=1.1):
    """Per-expert additive logit bias b_e = -s * ln(rank_e) with ranks 1..E in a seeded random order: expert
    loads then follow a Zipf(s)-like law on top of the input-dependent logits (skewed-load configuration)."""
    key = stream_key(seed, stream_id(layer, 0, 0, 5))
    order = np.argsort(rand32(key, np.arange(cfg.experts, dtype=np.uint64)), kind="stable")
    rank = np.empty(cfg.experts, np.int64)
    rank[order] = np.arange(1, cfg.experts + 1)
    return (-s * np.log(rank.astype(np.float64))).astype(np.float32)
