"""CPU-side checks: record geometry against the reference's constants, the synthetic generator, and that the
C-ABI library loads and exports every symbol include/zc_moe.h declares (no compute without a GPU)."""
import ctypes
import os
import re

import numpy as np
import pytest

from zerocool_b200 import build as zbuild
from zerocool_b200 import moe as zmoe
from zerocool_b200 import synth
from zerocool_b200.records import BF16, F16, MoeConfig, dequantise, pack_q4, unpack_q4
from tests import util

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_record_geometry_matches_reference_constants():
    """include/engine/storage.hpp:32-33 (2,764,800 B payload, 2,768,896 B stride) and expert_linear's offsets
    (src/engine/metal.mm:1124-1129: projection p at p*921600, scales +819200, biases +870400)."""
    cfg = MoeConfig(hidden=2560, ffn=640, experts=512, top_k=10, meta_dtype=BF16)
    assert cfg.record_bytes == 2764800 and cfg.record_stride == 2768896
    for p in range(3):
        lay = cfg.projection_layout(p)
        assert lay["codes"] == p * 921600 and lay["scales"] == p * 921600 + 819200 and lay["biases"] == p * 921600 + 870400
    assert util.cfg2().record_bytes == 1769472                    # 108 x 16 KiB
    assert MoeConfig(hidden=4096, ffn=512, experts=512, top_k=10).record_bytes == 3538944
    assert MoeConfig(hidden=2048, ffn=512, experts=512, top_k=10, down_bits=8).record_bytes == 2293760


def test_q4_packing_is_little_endian_nibbles():
    """Nibble k%8 of word k/8, k ascending from the least significant nibble (kernels/metal/qwen.metal:53)."""
    codes = (np.arange(64, dtype=np.uint8) % 16).reshape(2, 32)
    packed = pack_q4(codes)
    words = packed.view("<u4")
    for k in range(32):
        assert (int(words[0, k // 8]) >> (4 * (k % 8))) & 15 == codes[0, k]
    assert np.array_equal(unpack_q4(packed, 32), codes)


def test_synthetic_distributions():
    cfg = util.cfg1()
    rec = synth.record(cfg, 7, 0, 3)
    assert np.array_equal(rec, synth.record(cfg, 7, 0, 3))
    assert not np.array_equal(rec, synth.record(cfg, 8, 0, 3))
    lay = cfg.projection_layout(0)
    codes = unpack_q4(rec[lay["codes"]:lay["codes"] + lay["code_bytes"]].reshape(lay["N"], -1), lay["K"])
    assert codes.min() == 0 and codes.max() == 15 and abs(codes.mean() - 7.5) < 0.02
    s = rec[lay["scales"]:lay["scales"] + lay["meta_bytes"]].view(np.float16).astype(np.float32)
    b = rec[lay["biases"]:lay["biases"] + lay["meta_bytes"]].view(np.float16).astype(np.float32)
    assert s.min() >= 0.004 - 1e-5 and s.max() <= 0.02 + 1e-5
    assert np.array_equal(b, -8 * s)
    w = dequantise(cfg, rec, 0)
    assert abs(w.mean() + 0.5 * 0.012) < 1e-3          # E[s (q - 8)] with q uniform 0..15
    r = synth.router(cfg, 7, 0)
    assert r.shape == (64, 2048) and abs(r.std() - 0.02) < 5e-4
    x = synth.activations(cfg, 7, 0, 4)
    assert abs(x.std() - 1) < 0.02
    q8 = MoeConfig(hidden=256, ffn=128, experts=32, top_k=2, down_bits=8, q8_signed=1)
    rec8 = synth.record(q8, 1, 0, 0)
    lay8 = q8.projection_layout(2)
    c8 = rec8[lay8["codes"]:lay8["codes"] + lay8["code_bytes"]].view(np.int8)
    assert c8.min() == -127 and c8.max() == 127


def declared_functions():
    text = open(os.path.join(ROOT, "include", "zc_moe.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(zc_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_loads_and_exports_every_declared_symbol():
    path = zbuild.build()
    lib = ctypes.CDLL(path)
    names = declared_functions()
    assert len(names) >= 18
    for name in names:
        assert hasattr(lib, name), name
    assert sorted(zmoe.EXPORTS) == names


def test_descriptor_finalize_and_loud_failure_without_a_device():
    lib = zmoe.load_library()
    cfg = util.cfg2()
    d = zmoe.make_desc(cfg)
    d.record_bytes = d.record_stride = 0
    assert lib.zc_moe_desc_finalize(ctypes.byref(d)) == 0
    assert d.record_bytes == cfg.record_bytes and d.record_stride == cfg.record_stride and d.local_experts == 512
    bad = zmoe.make_desc(cfg)
    bad.group = 32
    h = ctypes.c_void_p()
    assert lib.zc_moe_create(ctypes.byref(bad), 0, ctypes.byref(h)) == zmoe.ZC_EINVAL
    assert b"group" in lib.zc_last_error()
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if not has_gpu:
        ok = zmoe.make_desc(cfg)
        rc = lib.zc_moe_create(ctypes.byref(ok), 0, ctypes.byref(h))
        assert rc == zmoe.ZC_EEXEC and not h.value
        assert b"no CUDA device" in lib.zc_last_error()
