#!/usr/bin/env python3
"""Regenerates the committed fixtures in this directory from the reference project.

Run where the reference tree is available:

    python tests/golden/make_golden.py /path/to/reference

It writes
  reference_known_answers.json  constants copied out of the reference's own unit tests
                                (tests/test_qwen.cpp): router bit patterns, activation tables,
                                the expert-reduction midpoint case.
  numpy_moe_config0.npz         outputs of the reference's CPU oracle scripts/qwen/reference_numpy.py
                                (function ``moe``, imported unmodified) on a seeded synthetic layer at
                                the reference's native shape (hidden 2560, ffn 640, top-10, BF16
                                metadata, shared expert), E = 32 experts, T = 5 tokens.
  hyper_connection.npz          the reference CPU oracle's hyper-connection arithmetic either side of the MoE layer
                                (``hyper``, reference_numpy.py:99-106, called unmodified through a stand-in weights
                                object, and the residual update of its layer loop, :237) on seeded inputs, T = 2.
The inputs of the second fixture are regenerated from the seed by zerocool_b200.synth, so only the
outputs are stored.
"""
import importlib.util
import json
import os
import re
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

from zerocool_b200 import synth  # noqa: E402
from zerocool_b200.records import ARITH_REFERENCE, BF16, F32, MoeConfig  # noqa: E402

CONFIG0 = dict(hidden=2560, ffn=640, experts=32, top_k=10, layers=1, meta_dtype=BF16, act_dtype=F32,
               out_dtype=F32, router_dtype=BF16, has_shared=1, arith=ARITH_REFERENCE)
CONFIG0_SEED, CONFIG0_TOKENS = 20260914, 5


def floats(text):
    return [float(v.rstrip("f")) for v in re.findall(r"-?\d+\.?\d*(?:e-?\d+)?f", text)]


def known_answers(reference):
    src = (reference / "tests" / "test_qwen.cpp").read_text()
    out = {}
    block = src[src.index("FP32 router matches MLX accumulation"):]
    idx = re.search(r"indices\{([^}]*)\}", block).group(1)
    exp = re.search(r"expected\{([^}]*)\}", block).group(1)
    out["router_mlx"] = dict(T=11, K=2560, N=512, indices=[int(v) for v in idx.split(",")],
                             bits=[int(v, 16) for v in re.findall(r"0x[0-9a-f]+", exp)])
    block = src[src.index("BF16 activations match MLX 0.31.1 captured GPU values"):]
    out["activations"] = dict(
        x=floats(re.search(r"vector<float> x\{([^}]*)\}", block).group(1)),
        sigmoid=floats(re.search(r"vector<float> sigmoid\{([^}]*)\}", block).group(1)),
        silu=floats(re.search(r"vector<float> silu\{([^}]*)\}", block).group(1)))
    block = src[src.index("expert reduction preserves the reference BF16 midpoint decision"):]
    out["moe_sum_midpoint"] = dict(
        gate=-1.4765625, shared=0.0157470703125, expected=0.01190185546875,
        values=floats(re.search(r"values\{([^}]*)\}", block).group(1)),
        weight_bits=[int(v, 16) for v in re.findall(r"0x[0-9a-f]+", re.search(r"bits\{([^}]*)\}", block).group(1))])
    out["sigmoid_boundary"] = dict(x=-6.84375, silu=-0.00726318359375)
    return out


def write_safetensors(path, tensors):
    header, blobs, cursor = {}, [], 0
    for name, (dtype, array) in tensors.items():
        raw = np.ascontiguousarray(array).tobytes()
        header[name] = dict(dtype=dtype, shape=list(array.shape), data_offsets=[cursor, cursor + len(raw)])
        blobs.append(raw)
        cursor += len(raw)
    text = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(len(text).to_bytes(8, "little"))
        f.write(text)
        for raw in blobs:
            f.write(raw)


def config0_tensors(cfg, seed):
    """The synthetic layer as the checkpoint tensors reference_numpy.Weights reads."""
    base = "language_model.model.layers.0.mlp."
    tensors = {base + "gate.weight": ("BF16", synth.router(cfg, seed, 0)),
               base + "shared_expert_gate.weight": ("BF16", synth.shared_gate(cfg, seed, 0))}
    for p, name in enumerate(("gate_proj", "up_proj", "down_proj")):
        stacks = [[], [], []]
        for e in range(cfg.experts):
            for i, part in enumerate(synth.projection_parts(cfg, seed, 0, e, p)):
                stacks[i].append(part)
        n, k = cfg.shape(p)
        tensors[base + f"switch_mlp.{name}.weight"] = ("U32", np.stack(stacks[0]).view(np.uint32).reshape(cfg.experts, n, k // 8))
        tensors[base + f"switch_mlp.{name}.scales"] = ("BF16", np.stack(stacks[1]))
        tensors[base + f"switch_mlp.{name}.biases"] = ("BF16", np.stack(stacks[2]))
        codes, scales, biases = synth.projection_parts(cfg, seed, 0, synth.SHARED_EXPERT, p)
        tensors[base + f"shared_expert.{name}.weight"] = ("U32", codes.view(np.uint32).reshape(n, k // 8))
        tensors[base + f"shared_expert.{name}.scales"] = ("BF16", scales)
        tensors[base + f"shared_expert.{name}.biases"] = ("BF16", biases)
    return tensors


def numpy_moe(reference):
    spec = importlib.util.spec_from_file_location("reference_numpy", reference / "scripts" / "qwen" / "reference_numpy.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    cfg = MoeConfig(**CONFIG0)
    with tempfile.TemporaryDirectory() as tmp:
        tensors = config0_tensors(cfg, CONFIG0_SEED)
        write_safetensors(os.path.join(tmp, "model.safetensors"), tensors)
        Path(tmp, "model.safetensors.index.json").write_text(json.dumps(dict(weight_map={k: "model.safetensors" for k in tensors})))
        weights = module.Weights(Path(tmp))
        x = synth.activations(cfg, CONFIG0_SEED, 0, CONFIG0_TOKENS)
        out, idx = module.moe(weights, "model.layers.0.mlp", x)
        logits = weights.linear("model.layers.0.mlp.gate", x, floating=True)
    return dict(out=out.astype(np.float32), ids=idx.astype(np.int32), logits=logits.astype(np.float32))


def load_reference_numpy(reference):
    spec = importlib.util.spec_from_file_location("reference_numpy", reference / "scripts" / "qwen" / "reference_numpy.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def hyper_connection(reference):
    """``hyper`` of the reference oracle with a stand-in weights object: unit norm weight, and seeded arrays in place of
    the three small projections (their products are not part of the MoE path). Stored: the normalised streams, the
    mixing gate (both recomputed with the module's own norm / sigmoid / bf), ``hyper``'s two outputs, and the residual
    update bf(h + bf(out x injection)) of the layer loop evaluated with the module's bf."""
    module = load_reference_numpy(reference)
    rng = np.random.default_rng(20261125)
    T, H = 2, 2560
    streams = module.bf(rng.standard_normal((T, 4 * H)).astype(np.float32))
    pre_gate = module.bf(rng.standard_normal((T, 4 * H)).astype(np.float32) * 2)
    pre_inject = module.bf(rng.standard_normal((T, 4)).astype(np.float32) * 3)
    low = module.bf(rng.standard_normal((T, 64)).astype(np.float32))

    class Weights:
        def get(self, name):
            return np.ones(4 * H, np.float32)

        def linear(self, name, x, floating=False):
            return {"input_mix_weight_down": low, "input_mix_weight_up": pre_gate, "block_inject_weight": pre_inject}[name.rsplit(".", 1)[-1]]

    w = Weights()
    mixed, injection = module.hyper(w, "h", streams)
    normed = module.norm(w, "h.hc_norm", streams, True)
    gate = module.bf(module.sigmoid(pre_gate))
    out = module.bf(rng.standard_normal((T, H)).astype(np.float32))
    updated = module.bf(streams + module.bf(out[:, None, :] * injection[:, :, None]).reshape(T, 4 * H))
    return dict(streams=streams, normed=normed.astype(np.float32), gate=gate.astype(np.float32), mixed=mixed.astype(np.float32),
                injection=injection.astype(np.float32), out=out, updated=updated.astype(np.float32))


def main():
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("ZC_REFERENCE_ROOT")
    if not root:
        sys.exit("usage: make_golden.py <reference tree>   (or set ZC_REFERENCE_ROOT)")
    reference = Path(root)
    (HERE / "reference_known_answers.json").write_text(json.dumps(known_answers(reference), indent=1))
    np.savez_compressed(HERE / "numpy_moe_config0.npz", **numpy_moe(reference))
    np.savez_compressed(HERE / "hyper_connection.npz", **hyper_connection(reference))
    print("wrote", HERE / "reference_known_answers.json", HERE / "numpy_moe_config0.npz", "and", HERE / "hyper_connection.npz")


if __name__ == "__main__":
    main()
