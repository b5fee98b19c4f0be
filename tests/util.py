"""Shared helpers of the test-suite: the benchmark's configurations at test sizes, and input builders."""
import numpy as np

from zerocool_b200 import synth
from zerocool_b200.records import ARITH_FP32, ARITH_REFERENCE, BF16, F16, F32, MoeConfig


def cfg1(**kw):
    """benchmark configuration 1: one layer, hidden 2048, 64 experts top-8, ffn 512, Q4 g64 fp16 metadata, fp32 activations."""
    base = dict(hidden=2048, ffn=512, experts=64, top_k=8, layers=1, meta_dtype=F16, act_dtype=F32, out_dtype=F32,
                router_dtype=F32, has_shared=0, arith=ARITH_FP32, max_tokens=8)
    base.update(kw)
    return MoeConfig(**base)


def cfg2(**kw):
    """benchmark configuration 2 geometry: hidden 2048, 512 experts top-10 + shared, ffn 512, bf16 activations."""
    base = dict(hidden=2048, ffn=512, experts=512, top_k=10, layers=1, meta_dtype=F16, act_dtype=BF16, out_dtype=F32,
                router_dtype=F32, has_shared=1, arith=ARITH_FP32, max_tokens=64)
    base.update(kw)
    return MoeConfig(**base)


def cfg0(**kw):
    """The reference's native shape (hidden 2560, ffn 640, top-10 + shared, BF16 metadata, reference arithmetic)."""
    base = dict(hidden=2560, ffn=640, experts=32, top_k=10, layers=1, meta_dtype=BF16, act_dtype=F32, out_dtype=F32,
                router_dtype=BF16, has_shared=1, arith=ARITH_REFERENCE, max_tokens=16)
    base.update(kw)
    return MoeConfig(**base)


class LazyRecords:
    """Sequence of E records regenerated on demand from the seed (only the selected experts are ever built)."""

    def __init__(self, cfg, seed, layer):
        self.cfg, self.seed, self.layer, self.cache = cfg, seed, layer, {}

    def __getitem__(self, e):
        if e not in self.cache:
            self.cache[e] = synth.record(self.cfg, self.seed, self.layer, e)
        return self.cache[e]


def selected_records(cfg, seed, layer, ids):
    """List of E entries: a record for every expert in ids, None elsewhere."""
    lazy = LazyRecords(cfg, seed, layer)
    wanted = set(int(e) for e in np.unique(ids) if e >= 0)
    return [lazy[e] if e in wanted else None for e in range(cfg.experts)]


def rel_max_error(got, want):
    """max |got - want| / rms(want): the parity metric of the benchmark specification."""
    want = np.asarray(want, np.float64)
    got = np.asarray(got, np.float64)
    return float(np.abs(got - want).max() / np.sqrt(np.mean(want * want)))


def asymmetric_record(cfg, seed, layer, expert, rng, spread=0.03):
    """A record with the generator's codes and scales but free biases: bias = -(mean code) * scale + U(-spread, spread),
    so the weights stay roughly centred while the affine form's bias term no longer cancels against the codes."""
    from zerocool_b200.records import build_record, float_to_meta, meta_to_float
    parts = []
    for p in range(3):
        codes, sbits, bbits = synth.projection_parts(cfg, seed, layer, expert, p)
        s = meta_to_float(sbits, cfg.meta_dtype)
        offset = -8.0 if cfg.bits(p) == 4 else (0.0 if cfg.q8_signed else -127.5)
        b = offset * s + rng.uniform(-spread, spread, size=s.shape).astype(np.float32)
        parts.append((codes, sbits, float_to_meta(b, cfg.meta_dtype).reshape(bbits.shape)))
    return build_record(cfg, parts)
