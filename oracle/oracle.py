"""ctypes binding of the CPU checker (TEST INFRASTRUCTURE, not part of the shipped library).

Only tests, the smoke check and the CPU-baseline leg of the benchmark may import this module.
The arithmetic lives in ``zc_oracle.cpp``; this file only marshals numpy arrays.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libzc_oracle.so")

BF16, F32, F16 = 0, 1, 2
ARITH_FP32, ARITH_REFERENCE = 0, 1


class Desc(ctypes.Structure):
    """Same field order as ``zc_moe_desc`` in include/zc_moe.h."""
    _fields_ = [
        ("hidden", ctypes.c_uint32), ("ffn", ctypes.c_uint32), ("experts", ctypes.c_uint32),
        ("top_k", ctypes.c_uint32), ("layers", ctypes.c_uint32), ("group", ctypes.c_uint32),
        ("max_tokens", ctypes.c_uint32), ("first_expert", ctypes.c_uint32),
        ("local_experts", ctypes.c_uint32), ("reserved0", ctypes.c_uint32),
        ("gate_bits", ctypes.c_uint8), ("up_bits", ctypes.c_uint8), ("down_bits", ctypes.c_uint8),
        ("q8_signed", ctypes.c_uint8), ("meta_dtype", ctypes.c_uint8), ("act_dtype", ctypes.c_uint8),
        ("out_dtype", ctypes.c_uint8), ("router_dtype", ctypes.c_uint8), ("has_shared", ctypes.c_uint8),
        ("arith", ctypes.c_uint8),
        ("shared_gate_bits", ctypes.c_uint8), ("shared_up_bits", ctypes.c_uint8), ("shared_down_bits", ctypes.c_uint8), ("reserved", ctypes.c_uint8 * 3),
        ("record_bytes", ctypes.c_uint64), ("record_stride", ctypes.c_uint64),
    ]


def build(force=False):
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(os.path.join(_HERE, "zc_oracle.cpp")):
        subprocess.run(["make", "-C", _HERE, "-B", "libzc_oracle.so"], check=True, capture_output=True)
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.zco_bf.restype = ctypes.c_float
        _lib.zco_bf.argtypes = [ctypes.c_float]
        _lib.zco_sigmoid_bf.restype = ctypes.c_float
        _lib.zco_sigmoid_bf.argtypes = [ctypes.c_float]
        _lib.zco_silu_bf.restype = ctypes.c_float
        _lib.zco_silu_bf.argtypes = [ctypes.c_float]
        _lib.zco_threads.restype = ctypes.c_int
        _lib.zco_permute.restype = ctypes.c_int
        _lib.zco_moe_layer.restype = ctypes.c_int
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def threads():
    return lib().zco_threads()


def set_threads(n):
    lib().zco_set_threads(ctypes.c_int(int(n)))


def make_desc(cfg):
    """cfg: dict with the zc_moe_desc field names (missing fields default to 0 / group 64)."""
    d = Desc()
    for name, _ in Desc._fields_:
        if name == "reserved":
            continue
        setattr(d, name, int(cfg.get(name, 64 if name == "group" else 0)))
    return d


def router_logits(x, w, w_dtype):
    x = _f32(x)
    T, H = x.shape
    w = np.ascontiguousarray(w)
    E = w.shape[0]
    out = np.empty((T, E), np.float32)
    lib().zco_router_logits(_p(x), _p(w), ctypes.c_int(w_dtype), ctypes.c_uint32(T), ctypes.c_uint32(H), ctypes.c_uint32(E), _p(out))
    return out


def route(logits, K):
    logits = _f32(logits)
    T, E = logits.shape
    ids = np.empty((T, K), np.int32)
    weights = np.empty((T, K), np.float32)
    lib().zco_route(_p(logits), ctypes.c_uint32(T), ctypes.c_uint32(E), ctypes.c_uint32(K), _p(ids), _p(weights))
    return ids, weights


def permute(ids, E):
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    T, K = ids.shape
    offsets = np.empty(E + 1, np.int32)
    perm = np.empty(T * K, np.int32)
    rc = lib().zco_permute(_p(ids), ctypes.c_uint32(T), ctypes.c_uint32(K), ctypes.c_uint32(E), _p(offsets), _p(perm))
    if rc:
        raise ValueError("invalid router output")
    return offsets, perm


def affine(bits, codes, scales, biases, N, K, x, *, group=64, meta_dtype=BF16, ref=True, signed=False, round_out=True):
    """Metal::linear for an affine matrix: x [T,K] fp32 -> [T,N]."""
    x = _f32(x).reshape(-1, K)
    T = x.shape[0]
    codes = np.ascontiguousarray(codes)
    scales = np.ascontiguousarray(scales)
    biases = np.ascontiguousarray(biases)
    out = np.empty((T, N), np.float32)
    lib().zco_affine(ctypes.c_uint32(bits), ctypes.c_int(int(signed)), ctypes.c_int(meta_dtype), ctypes.c_int(int(ref)),
                     _p(codes), _p(scales), _p(biases), ctypes.c_uint32(N), ctypes.c_uint32(K), ctypes.c_uint32(group),
                     _p(x), ctypes.c_uint32(T), _p(out), ctypes.c_int(int(round_out)))
    return out


def expert(cfg, record, x):
    """One expert record applied to rows x [n,H]: returns (h [n,F], y [n,H])."""
    d = make_desc(cfg)
    x = _f32(x).reshape(-1, d.hidden)
    n = x.shape[0]
    record = np.ascontiguousarray(record, dtype=np.uint8)
    h = np.empty((n, d.ffn), np.float32)
    y = np.empty((n, d.hidden), np.float32)
    lib().zco_expert(ctypes.byref(d), _p(record), _p(x), ctypes.c_uint32(n), _p(h), _p(y))
    return h, y


def combine(cfg, expert_out, weights, shared=None, gate=None):
    d = make_desc(cfg)
    expert_out = _f32(expert_out)
    weights = _f32(weights)
    T = weights.shape[0]
    out = np.empty((T, d.hidden), np.float32)
    shared = None if shared is None else _f32(shared)
    gate = None if gate is None else _f32(gate)
    lib().zco_combine(ctypes.byref(d), _p(expert_out), _p(weights), _p(shared), _p(gate), ctypes.c_uint32(T), _p(out))
    return out


def set_router_bias(bias):
    """fp32 [E] array added to the logits of every later router call, or None. Returns the array to keep alive."""
    keep = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    lib().zco_set_router_bias(_p(keep))
    return keep


def moe_layer(cfg, records, router_w, x, shared_record=None, shared_gate_w=None, want_intermediates=False, router_bias=None):
    """Whole layer. ``records``: sequence of E uint8 arrays (or None for experts known to be unselected),
    or one [E, stride] uint8 array. x: fp32 [T,H]. Returns dict(out, ids, weights[, logits, expert_out, shared, gate])."""
    if cfg.get("has_shared") and any(cfg.get(k) for k in ("shared_gate_bits", "shared_up_bits", "shared_down_bits")):
        return _moe_layer_mixed(cfg, records, router_w, x, shared_record, shared_gate_w, want_intermediates, router_bias)
    d = make_desc(cfg)
    x = _f32(x).reshape(-1, d.hidden)
    T = x.shape[0]
    E, K, H = d.experts, d.top_k, d.hidden
    keep = []
    ptrs = (ctypes.c_void_p * E)()
    for e in range(E):
        r = records[e]
        if r is None:
            ptrs[e] = None
        else:
            r = np.ascontiguousarray(r, dtype=np.uint8)
            keep.append(r)
            ptrs[e] = r.ctypes.data
    router_w = np.ascontiguousarray(router_w)
    out = np.empty((T, H), np.float32)
    ids = np.empty((T, K), np.int32)
    weights = np.empty((T, K), np.float32)
    logits = np.empty((T, E), np.float32) if want_intermediates else None
    eo = np.empty((T, K, H), np.float32) if want_intermediates else None
    so = np.empty((T, H), np.float32) if want_intermediates and d.has_shared else None
    go = np.empty((T,), np.float32) if want_intermediates and d.has_shared else None
    if d.has_shared:
        shared_record = np.ascontiguousarray(shared_record, dtype=np.uint8)
        shared_gate_w = np.ascontiguousarray(shared_gate_w)
    keep_bias = set_router_bias(router_bias)
    rc = lib().zco_moe_layer(ctypes.byref(d), ptrs, _p(router_w), _p(shared_record) if d.has_shared else None,
                             _p(shared_gate_w) if d.has_shared else None, _p(x), ctypes.c_uint32(T), _p(out), _p(ids),
                             _p(weights), _p(logits), _p(eo), _p(so), _p(go))
    set_router_bias(None)
    del keep_bias
    if rc == -1:
        raise ValueError("invalid router output")
    if rc == -2:
        raise KeyError("a selected expert has no record")
    res = dict(out=out, ids=ids, weights=weights)
    if want_intermediates:
        res.update(logits=logits, expert_out=eo, shared=so, gate=go)
    return res


def bf(x):
    """Vectorised bf16 rounding (same bit arithmetic as the C helper)."""
    x = np.asarray(x, dtype=np.float32)
    u = x.view(np.uint32)
    r = ((u + np.uint32(0x7FFF) + ((u >> 16) & 1)) & np.uint32(0xFFFF0000)).view(np.float32)
    return np.where(np.isnan(x), np.float32(np.nan), r)


def hc_mix(normed, mix):
    """hc_mix (kernels/metal/qwen.metal:582-588): normed, mix fp32 [T, 4, H] -> [T, H];
    sum = bf(sum + bf(n * w)) over the four streams from zero, then bf(sum / 4)."""
    normed, mix = _f32(normed), _f32(mix)
    total = np.zeros(normed[:, 0].shape, np.float32)
    for h in range(normed.shape[1]):
        total = bf(total + bf(normed[:, h] * mix[:, h]))
    return bf(total / np.float32(4))


def hc_add(hyper, x, inject, ref=True):
    """hc_add (kernels/metal/qwen.metal:589-595): hyper fp32 [T, 4, H], x fp32 [T, H], inject fp32 [T, 4] ->
    bf(hyper + bf(x * inject)); ref=False drops both roundings (plain fp32)."""
    hyper, x, inject = _f32(hyper), _f32(x), _f32(inject)
    p = x[:, None, :] * inject[:, :, None]
    return bf(hyper + bf(p)) if ref else (hyper + p).astype(np.float32)


def _moe_layer_mixed(cfg, records, router_w, x, shared_record, shared_gate_w, want_intermediates, router_bias):
    """A layer whose shared expert's record has its own bit widths (the reference's mixed artifact, src/engine/metal.mm:1103-1123):
    the routed part as a layer without shared expert, the shared expert through `expert` with the shared bit widths, the
    gate scalar as router row E (src/engine/model.cpp:482-485), then the fixed-order combine."""
    routed_cfg = dict(cfg, has_shared=0, shared_gate_bits=0, shared_up_bits=0, shared_down_bits=0)
    res = moe_layer(routed_cfg, records, router_w, x, want_intermediates=True, router_bias=router_bias)
    shared_cfg = dict(routed_cfg, gate_bits=cfg.get("shared_gate_bits") or cfg["gate_bits"], up_bits=cfg.get("shared_up_bits") or cfg["up_bits"],
                      down_bits=cfg.get("shared_down_bits") or cfg["down_bits"])
    x = _f32(x).reshape(-1, cfg["hidden"])
    shared = expert(shared_cfg, shared_record, x)[1]
    gate = router_logits(x, np.ascontiguousarray(shared_gate_w), cfg.get("router_dtype", F32))[:, 0]
    if cfg.get("arith", 0) == ARITH_REFERENCE:
        gate = bf(gate)
    out = combine(dict(cfg, has_shared=1), res["expert_out"], res["weights"], shared, gate)
    full = dict(out=out, ids=res["ids"], weights=res["weights"])
    if want_intermediates:
        full.update(logits=res["logits"], expert_out=res["expert_out"], shared=shared, gate=gate)
    return full
