"""Expert-record geometry and the layer configuration shared by the host code.

The prepared expert record keeps the reference's byte layout (``expert_linear`` in
src/engine/metal.mm:1124-1129, writer scripts/qwen/prepare_storage.py:140-160, constants
include/engine/storage.hpp:32-33): three projections gate, up, down, each stored as
``[codes | scales | biases]``; codes are row-major ``[N, K*bits/8]`` bytes (Q4: little-endian uint32
words holding 8 nibbles, k ascending from the least significant nibble; Q8: one byte per weight);
scales and biases are ``[N, K/group]`` 16-bit floats. gate/up have N = ffn, K = hidden; down has
N = hidden, K = ffn. Records are laid out at a stride rounded up to 16 KiB.

The reference fixes hidden 2560 / ffn 640 / Q4 / BF16 metadata at compile time; here the same layout
is parametric and additionally admits 8-bit codes per projection and FP16 metadata.
"""
from dataclasses import dataclass, asdict

import numpy as np

BF16, F32, F16 = 0, 1, 2          # same numbering as Resident::dtype, src/engine/metal.mm:1100-1102
ARITH_FP32, ARITH_REFERENCE = 0, 1
RECORD_ALIGN = 16384               # prepare_storage.py ALIGN


@dataclass
class MoeConfig:
    hidden: int
    ffn: int
    experts: int
    top_k: int
    layers: int = 1
    group: int = 64
    max_tokens: int = 64
    first_expert: int = 0
    local_experts: int = 0          # 0 = all experts are local
    gate_bits: int = 4
    up_bits: int = 4
    down_bits: int = 4
    q8_signed: int = 0
    meta_dtype: int = F16
    act_dtype: int = BF16
    out_dtype: int = F32
    router_dtype: int = F32
    has_shared: int = 0
    arith: int = ARITH_FP32
    shared_gate_bits: int = 0       # the shared expert's record: 4 or 8 per projection, 0 = as the routed experts
    shared_up_bits: int = 0
    shared_down_bits: int = 0

    def bits(self, projection):
        return (self.gate_bits, self.up_bits, self.down_bits)[projection]

    def shape(self, projection):
        """(N, K) of a projection: gate/up [ffn, hidden], down [hidden, ffn]."""
        return (self.hidden, self.ffn) if projection == 2 else (self.ffn, self.hidden)

    def projection_bytes(self, projection):
        n, k = self.shape(projection)
        return n * k * self.bits(projection) // 8 + 2 * n * (k // self.group) * 2

    def projection_layout(self, projection):
        """Byte offsets inside a record: dict(codes, scales, biases, code_bytes, meta_bytes, N, K, bits)."""
        offset = sum(self.projection_bytes(p) for p in range(projection))
        n, k = self.shape(projection)
        code_bytes = n * k * self.bits(projection) // 8
        meta_bytes = n * (k // self.group) * 2
        return dict(codes=offset, scales=offset + code_bytes, biases=offset + code_bytes + meta_bytes,
                    code_bytes=code_bytes, meta_bytes=meta_bytes, N=n, K=k, bits=self.bits(projection))

    @property
    def record_bytes(self):
        return sum(self.projection_bytes(p) for p in range(3))

    @property
    def record_stride(self):
        return (self.record_bytes + RECORD_ALIGN - 1) // RECORD_ALIGN * RECORD_ALIGN

    def shared_cfg(self):
        """The configuration that describes the shared expert's record (the reference's mixed artifact keeps routed experts
        Q4 and the shared expert Q8, src/engine/metal.mm:1103-1123): same geometry, the shared bit widths."""
        from dataclasses import replace
        return replace(self, gate_bits=self.shared_gate_bits or self.gate_bits, up_bits=self.shared_up_bits or self.up_bits,
                       down_bits=self.shared_down_bits or self.down_bits, shared_gate_bits=0, shared_up_bits=0, shared_down_bits=0)

    @property
    def n_local(self):
        return self.local_experts or self.experts

    def as_dict(self):
        d = asdict(self)
        d["record_bytes"] = self.record_bytes
        d["record_stride"] = self.record_stride
        return d

    def validate(self):
        if self.hidden % 128 or self.ffn % 128:
            raise ValueError("hidden and ffn must be multiples of 128")
        if self.group != 64:
            raise ValueError("only group 64 is supported")
        for p in range(3):
            if self.bits(p) not in (4, 8):
                raise ValueError("projection bits must be 4 or 8")
        if any(b not in (0, 4, 8) for b in (self.shared_gate_bits, self.shared_up_bits, self.shared_down_bits)):
            raise ValueError("shared projection bits must be 0, 4 or 8")
        if not 0 < self.top_k <= min(self.experts, 128):
            raise ValueError("top_k must be in 1..min(experts,128)")


def pack_q4(codes):
    """codes uint8 [N, K] with values 0..15 -> little-endian uint32 words [N, K/8] as bytes [N, K/2]."""
    codes = np.asarray(codes, dtype=np.uint8)
    n, k = codes.shape
    lo, hi = codes[:, 0::2].astype(np.uint8), codes[:, 1::2].astype(np.uint8)
    return (lo | (hi << 4)).astype(np.uint8).reshape(n, k // 2)


def unpack_q4(packed, k):
    packed = np.asarray(packed, dtype=np.uint8)
    out = np.empty((packed.shape[0], k), np.uint8)
    out[:, 0::2] = packed & 15
    out[:, 1::2] = packed >> 4
    return out


def float_to_meta(values, dtype):
    """fp32 array -> uint16 bit patterns of bf16 (round to nearest even) or fp16."""
    values = np.asarray(values, dtype=np.float32)
    if dtype == F16:
        return values.astype(np.float16).view(np.uint16)
    u = values.view(np.uint32)
    return (((u + np.uint32(0x7FFF) + ((u >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)


def meta_to_float(bits, dtype):
    bits = np.asarray(bits, dtype=np.uint16)
    if dtype == F16:
        return bits.view(np.float16).astype(np.float32)
    return (bits.astype(np.uint32) << 16).view(np.float32)


def bf16_bits(values):
    return float_to_meta(values, BF16)


def bf16_to_float(bits):
    return meta_to_float(bits, BF16)


def build_record(cfg, parts):
    """parts: 3 tuples (code_bytes uint8 [N, K*bits/8], scale_bits uint16 [N,K/g], bias_bits uint16 [N,K/g])."""
    record = np.zeros(cfg.record_stride, np.uint8)
    for p, (codes, scales, biases) in enumerate(parts):
        lay = cfg.projection_layout(p)
        record[lay["codes"]:lay["codes"] + lay["code_bytes"]] = np.ascontiguousarray(codes, dtype=np.uint8).reshape(-1)
        record[lay["scales"]:lay["scales"] + lay["meta_bytes"]] = np.ascontiguousarray(scales, dtype=np.uint16).reshape(-1).view(np.uint8)
        record[lay["biases"]:lay["biases"] + lay["meta_bytes"]] = np.ascontiguousarray(biases, dtype=np.uint16).reshape(-1).view(np.uint8)
    return record


def dequantise(cfg, record, projection):
    """Mathematical fp64 matrix [N, K] of one projection (for independent checks)."""
    lay = cfg.projection_layout(projection)
    n, k = lay["N"], lay["K"]
    raw = record[lay["codes"]:lay["codes"] + lay["code_bytes"]].reshape(n, -1)
    if lay["bits"] == 4:
        q = unpack_q4(raw, k).astype(np.float64)
    elif cfg.q8_signed:
        q = raw.view(np.int8).astype(np.float64)
    else:
        q = raw.astype(np.float64)
    s = meta_to_float(record[lay["scales"]:lay["scales"] + lay["meta_bytes"]].view(np.uint16), cfg.meta_dtype).reshape(n, -1)
    b = meta_to_float(record[lay["biases"]:lay["biases"] + lay["meta_bytes"]].view(np.uint16), cfg.meta_dtype).reshape(n, -1)
    return q * np.repeat(s.astype(np.float64), cfg.group, 1) + np.repeat(b.astype(np.float64), cfg.group, 1)
