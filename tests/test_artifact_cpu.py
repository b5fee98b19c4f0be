"""Prepared-record directories (zc-affine-records-v1): writer, manifest checks and the streaming reader, on CPU.
Mirrors the reference's checks in PreparedArtifact (src/engine/storage.cpp:316-378) and its tiny-geometry
writer test (tests/test_checkpoint_io.cpp:158-190)."""
import json
import os

import numpy as np
import pytest

from zerocool_b200 import artifact, synth
from zerocool_b200.records import BF16, F16, F32, MoeConfig

SEED = 11


def tiny(**kw):
    base = dict(hidden=128, ffn=128, experts=8, top_k=2, layers=2, meta_dtype=F16, act_dtype=BF16, out_dtype=F32, router_dtype=F32)
    base.update(kw)
    return MoeConfig(**base)


def write(tmp_path, cfg):
    return artifact.write_artifact(str(tmp_path), cfg, lambda layer: (synth.record(cfg, SEED, layer, e) for e in range(cfg.experts)))


def test_layout_matches_the_reference_constants():
    """At the reference's native geometry the nine pieces have its offsets and lengths (metal.mm:1124-1129)."""
    cfg = MoeConfig(hidden=2560, ffn=640, experts=512, top_k=10, meta_dtype=BF16)
    lay = artifact.expert_layout(cfg)
    assert [e["offset"] for e in lay] == [0, 819200, 870400, 921600, 1740800, 1792000, 1843200, 2662400, 2713600]
    assert [e["length"] for e in lay] == [819200, 51200, 51200] * 3
    assert lay[0]["shape"] == [640, 320] and lay[6]["shape"] == [2560, 80] and lay[1]["dtype"] == "BF16"
    assert cfg.record_bytes == 2764800 and cfg.record_stride == 2768896


def test_round_trip_in_runs(tmp_path):
    cfg = tiny()
    manifest = write(tmp_path, cfg)
    assert manifest["format"] == "zc-affine-records-v1" and len(manifest["expert_layout"]) == 9 and len(manifest["experts"]) == 2
    prepared = artifact.PreparedExperts(str(tmp_path), cfg)
    for layer in range(cfg.layers):
        seen = []
        for first, block in prepared.runs(layer, run_experts=3):
            assert block.shape[1] == cfg.record_stride
            for i in range(block.shape[0]):
                assert np.array_equal(block[i], synth.record(cfg, SEED, layer, first + i))
                seen.append(first + i)
        assert seen == list(range(cfg.experts))
    # a sub-range, as an expert-parallel rank would read it
    sub = [(first, block.shape[0]) for first, block in prepared.runs(1, first_expert=4, count=4, run_experts=3)]
    assert sub == [(4, 3), (7, 1)]
    with pytest.raises(IndexError):
        list(prepared.runs(0, first_expert=6, count=4))


def test_changed_file_is_detected(tmp_path):
    cfg = tiny()
    write(tmp_path, cfg)
    path = os.path.join(str(tmp_path), artifact.layer_file(1))
    with open(path, "r+b") as f:
        f.seek(cfg.record_stride * 3 + 17)
        byte = f.read(1)
        f.seek(cfg.record_stride * 3 + 17)
        f.write(bytes([byte[0] ^ 0x40]))
    prepared = artifact.PreparedExperts(str(tmp_path), cfg)
    list(prepared.runs(0))                                    # layer 0 is intact
    with pytest.raises(RuntimeError, match="changed since verification"):
        list(prepared.runs(1))


def test_manifest_checks(tmp_path):
    cfg = tiny()
    write(tmp_path, cfg)
    with pytest.raises(RuntimeError, match="unsupported prepared expert projection"):
        artifact.PreparedExperts(str(tmp_path), tiny(ffn=256))            # another geometry
    with pytest.raises(RuntimeError, match="unsupported prepared expert projection"):
        artifact.PreparedExperts(str(tmp_path), tiny(meta_dtype=BF16))    # another metadata dtype
    mpath = os.path.join(str(tmp_path), "manifest.json")
    good = json.load(open(mpath))
    for mutate, message in (
        (lambda m: m.update(format="zc-affine-records-v0"), "incompatible"),
        (lambda m: m["experts"][0].update(stride=cfg.record_stride * 2), "unsupported prepared expert range"),
        (lambda m: m["experts"][1].update(file=m["experts"][0]["file"]), "duplicate"),
        (lambda m: m["files"][0].update(path="../x.bin"), "invalid prepared filename"),
        (lambda m: m["experts"].pop(), "incomplete"),
    ):
        bad = json.loads(json.dumps(good))
        mutate(bad)
        json.dump(bad, open(mpath, "w"))
        with pytest.raises(RuntimeError, match=message):
            artifact.PreparedExperts(str(tmp_path), cfg)
    json.dump(good, open(mpath, "w"))
    os.truncate(os.path.join(str(tmp_path), artifact.layer_file(0)), cfg.record_stride * 7)
    with pytest.raises(RuntimeError, match="invalid prepared expert length"):
        artifact.PreparedExperts(str(tmp_path), cfg)


def test_repack_of_stacked_checkpoint_tensors_is_lossless(tmp_path):
    """The nine stacked tensors of a checkpoint layer (switch_mlp.<proj>.<piece>[expert]) become the records byte for
    byte (scripts/qwen/prepare_storage.py:133-152), for 4- and 8-bit projections; wrong shapes are refused."""
    cfg = tiny(down_bits=8)
    stacks = {name: [] for name in artifact.PIECES}
    for e in range(cfg.experts):
        for p, proj in enumerate(("gate_proj", "up_proj", "down_proj")):
            codes, scales, biases = synth.projection_parts(cfg, SEED, 1, e, p)
            lay = cfg.projection_layout(p)
            stacks[proj + ".weight"].append(np.ascontiguousarray(codes, dtype=np.uint8).reshape(lay["N"], -1).view(np.uint32))
            stacks[proj + ".scales"].append(scales)
            stacks[proj + ".biases"].append(biases)
    tensors = {name: np.stack(v) for name, v in stacks.items()}
    records = list(artifact.repack_switch_mlp(cfg, tensors))
    assert len(records) == cfg.experts
    for e, record in enumerate(records):
        assert np.array_equal(record, synth.record(cfg, SEED, 1, e))
    artifact.write_artifact(str(tmp_path), tiny(down_bits=8, layers=1), lambda layer: artifact.repack_switch_mlp(cfg, tensors))
    prepared = artifact.PreparedExperts(str(tmp_path), tiny(down_bits=8, layers=1))
    got = np.concatenate([block.copy() for _, block in prepared.runs(0, run_experts=3)])      # the staging buffer is reused between runs
    assert np.array_equal(got, np.stack(records))
    bad = dict(tensors)
    bad["up_proj.scales"] = tensors["up_proj.scales"][:, :, :-1]
    with pytest.raises(ValueError):
        list(artifact.repack_switch_mlp(cfg, bad))
    with pytest.raises(ValueError):
        list(artifact.repack_switch_mlp(cfg, {k: v for k, v in tensors.items() if k != "down_proj.biases"}))
