"""Prepared expert records on disk: reading a ``zc-affine-records-v1`` directory into HBM.

The reference writes one ``experts-LL.bin`` per layer (scripts/qwen/prepare_storage.py:140-160: for every expert
the nine pieces gate/up/down x weight/scales/biases back to back, padded to a 16 KiB stride) and a ``manifest.json``
whose ``expert_layout`` (nine entries: name, offset, length, shape, dtype, bits, group_size), ``experts`` (per layer:
layer, file, count, offset, length, stride, alignment) and ``files`` (path, size, sha256) describe them. Its reader
(src/engine/storage.cpp:316-378) checks those entries against compile-time constants and then serves single
records to the SSD cache. Here the same manifest drives a loader with a parametric geometry: the entries are checked
against a ``MoeConfig``, the file is streamed through a reusable pinned host buffer in runs of whole records, each run
is handed to ``zc_moe_load_layer`` (one host-to-device copy per run), and the SHA-256 of the stream is compared with
the manifest's on the way. 8-bit projections and FP16 metadata (``dtype: "F16"``) are admitted next to the
reference's Q4 / BF16.

``write_artifact`` produces such a directory from records in memory (tests, synthetic checkpoints);
``repack_switch_mlp`` turns a checkpoint layer's nine stacked tensors into those records, the lossless repack of
prepare_storage.py:133-152 for a parametric geometry.
"""
import hashlib
import json
import os

import numpy as np

from .records import BF16, F16, RECORD_ALIGN, MoeConfig

FORMAT = "zc-affine-records-v1"
PIECES = ("gate_proj.weight", "gate_proj.scales", "gate_proj.biases",
          "up_proj.weight", "up_proj.scales", "up_proj.biases",
          "down_proj.weight", "down_proj.scales", "down_proj.biases")


def expert_layout(cfg: MoeConfig):
    """The nine manifest entries of one record for this geometry (storage.cpp:352-362)."""
    meta = "F16" if cfg.meta_dtype == F16 else "BF16"
    out = []
    for p in range(3):
        lay = cfg.projection_layout(p)
        n, k, bits = lay["N"], lay["K"], lay["bits"]
        out.append(dict(name=PIECES[3 * p], offset=lay["codes"], length=lay["code_bytes"], shape=[n, k * bits // 32],
                        dtype="U32", bits=bits, group_size=cfg.group))
        out.append(dict(name=PIECES[3 * p + 1], offset=lay["scales"], length=lay["meta_bytes"], shape=[n, k // cfg.group],
                        dtype=meta, bits=bits, group_size=cfg.group))
        out.append(dict(name=PIECES[3 * p + 2], offset=lay["biases"], length=lay["meta_bytes"], shape=[n, k // cfg.group],
                        dtype=meta, bits=bits, group_size=cfg.group))
    return out


def repack_switch_mlp(cfg: MoeConfig, tensors):
    """The records of one layer from the checkpoint's stacked expert tensors.

    tensors maps the nine piece names (``gate_proj.weight`` ... ``down_proj.biases``, the suffix of the checkpoint's
    ``...mlp.switch_mlp.<piece>`` keys) to arrays whose first axis is the expert: weights ``[E, N, K*bits/32]`` uint32
    (or the same bytes as uint8), scales and biases ``[E, N, K/group]`` as 16-bit patterns in the metadata dtype. Yields
    cfg.experts records of record_stride bytes: for every expert its nine slices back to back in that order, padded to
    the stride - bytes are moved, never re-encoded. Shapes and sizes are checked against the geometry first (the
    reference's writer refuses a checkpoint whose pieces do not add up to the record length, prepare_storage.py:143-144)."""
    layout = expert_layout(cfg)
    pieces = []
    for entry in layout:
        if entry["name"] not in tensors:
            raise ValueError(f"missing tensor {entry['name']}")
        t = np.ascontiguousarray(tensors[entry["name"]])
        if t.shape[0] != cfg.experts:
            raise ValueError(f"{entry['name']}: {t.shape[0]} experts, geometry has {cfg.experts}")
        width = 4 if entry["dtype"] == "U32" else 2
        if t.dtype.itemsize not in (1, width) or t.dtype.kind not in "ui":
            raise ValueError(f"{entry['name']}: expected {entry['dtype']} bit patterns (or bytes), got {t.dtype}")
        per_expert = t.reshape(cfg.experts, -1).view(np.uint8)
        if per_expert.shape[1] != entry["length"]:
            raise ValueError(f"{entry['name']}: {per_expert.shape[1]} bytes per expert, layout has {entry['length']} (shape {entry['shape']})")
        pieces.append((entry["offset"], per_expert))
    if sum(p.shape[1] for _, p in pieces) != cfg.record_bytes:
        raise ValueError("unsupported expert format: the pieces do not add up to the record length")
    for e in range(cfg.experts):
        record = np.zeros(cfg.record_stride, np.uint8)
        for offset, per_expert in pieces:
            record[offset:offset + per_expert.shape[1]] = per_expert[e]
        yield record


def layer_file(layer):
    return f"experts-{layer:02d}.bin"


def write_artifact(directory, cfg: MoeConfig, records_of_layer):
    """records_of_layer(layer) -> iterable of cfg.experts uint8 arrays of record_stride (or record_bytes) bytes."""
    os.makedirs(directory, exist_ok=True)
    files, experts = [], []
    for layer in range(cfg.layers):
        name = layer_file(layer)
        digest, size = hashlib.sha256(), 0
        with open(os.path.join(directory, name), "wb") as f:
            count = 0
            for record in records_of_layer(layer):
                record = np.ascontiguousarray(record, dtype=np.uint8).reshape(-1)
                if record.size not in (cfg.record_bytes, cfg.record_stride):
                    raise ValueError("record has neither the payload nor the stride length")
                block = np.zeros(cfg.record_stride, np.uint8)
                block[:cfg.record_bytes] = record[:cfg.record_bytes]
                data = block.tobytes()
                f.write(data)
                digest.update(data)
                size += len(data)
                count += 1
            if count != cfg.experts:
                raise ValueError(f"layer {layer}: {count} records for {cfg.experts} experts")
        files.append(dict(path=name, size=size, sha256=digest.hexdigest()))
        experts.append(dict(layer=layer, file=name, count=cfg.experts, offset=0, length=cfg.record_bytes,
                            stride=cfg.record_stride, alignment=RECORD_ALIGN))
    manifest = dict(schema=1, format=FORMAT, recipe="synthetic", expert_layout=expert_layout(cfg), experts=experts, files=files,
                    prepared_bytes=sum(f["size"] for f in files))
    with open(os.path.join(directory, "manifest.json"), "w") as f:
        json.dump(manifest, f, indent=1)
    return manifest


class PreparedExperts:
    """A verified view of the expert records of a prepared directory."""

    def __init__(self, directory, cfg: MoeConfig):
        self.directory, self.cfg = directory, cfg
        with open(os.path.join(directory, "manifest.json")) as f:
            self.manifest = m = json.load(f)
        if m.get("schema") != 1 or m.get("format") != FORMAT:
            raise RuntimeError("unverified or incompatible prepared artifact")
        want = expert_layout(cfg)
        got = m.get("expert_layout", [])
        if len(got) != 9:
            raise RuntimeError("incomplete prepared layout")
        for w, g in zip(want, got):
            for key in ("name", "offset", "length", "dtype", "bits", "group_size"):
                if g.get(key) != w[key]:
                    raise RuntimeError(f"unsupported prepared expert projection: {w['name']} {key} {g.get(key)!r}, expected {w[key]!r}")
            if list(g.get("shape", [])) != w["shape"]:
                raise RuntimeError(f"unsupported prepared expert projection: {w['name']} shape")
        self.files = {}
        for entry in m.get("files", []):
            name = entry["path"]
            if not name or os.path.basename(name) != name or name in (".", "..") or name in self.files:
                raise RuntimeError("invalid prepared filename")
            self.files[name] = entry
        self.layers = {}
        used = set()
        for e in m.get("experts", []):
            layer = e["layer"]
            if (e["count"] != cfg.experts or e["offset"] != 0 or e["length"] != cfg.record_bytes or e["stride"] != cfg.record_stride
                    or e["alignment"] != RECORD_ALIGN):
                raise RuntimeError("unsupported prepared expert range")
            name = e["file"]
            if name in used or name not in self.files:
                raise RuntimeError("duplicate or unlisted prepared file range")
            used.add(name)
            path = os.path.join(directory, name)
            if not os.path.exists(path):
                raise RuntimeError("missing prepared file")
            if os.path.getsize(path) != cfg.record_stride * cfg.experts or self.files[name]["size"] != os.path.getsize(path):
                raise RuntimeError("invalid prepared expert length")
            self.layers[layer] = name
        if sorted(self.layers) != list(range(cfg.layers)):
            raise RuntimeError("incomplete prepared layout")

    def runs(self, layer, first_expert=0, count=None, run_experts=64, buffer=None):
        """Yields (first expert of the run, uint8 array [n, record_stride]) over experts [first_expert, first_expert + count),
        reading the file sequentially into ``buffer`` (a reusable uint8 array of run_experts * stride bytes; numpy memory
        or the numpy view of a pinned torch tensor). The whole-file SHA-256 is checked when the range covers the file."""
        cfg = self.cfg
        count = cfg.experts - first_expert if count is None else count
        if first_expert < 0 or count < 0 or first_expert + count > cfg.experts:
            raise IndexError("prepared expert range")
        stride = cfg.record_stride
        if buffer is None:
            buffer = np.empty(run_experts * stride, np.uint8)
        run_experts = buffer.size // stride
        if run_experts < 1:
            raise ValueError("the staging buffer holds less than one record")
        whole = first_expert == 0 and count == cfg.experts
        digest = hashlib.sha256() if whole else None
        name = self.layers[layer]
        with open(os.path.join(self.directory, name), "rb", buffering=0) as f:
            f.seek(first_expert * stride)
            at = first_expert
            while at < first_expert + count:
                n = min(run_experts, first_expert + count - at)
                view = memoryview(buffer)[: n * stride]
                got = f.readinto(view)
                if got != n * stride:
                    raise RuntimeError("short read of a prepared file")
                if digest is not None:
                    digest.update(view)
                yield at, buffer[: n * stride].reshape(n, stride)
                at += n
        if digest is not None and digest.hexdigest() != self.files[name]["sha256"]:
            raise RuntimeError(f"prepared file changed since verification: {name}")

    def load_layer(self, moe, layer, run_experts=64, pinned=True):
        """Streams the records of this handle's expert range of one layer into HBM. Returns the bytes copied."""
        cfg = self.cfg
        first, count = cfg.first_expert, cfg.n_local
        buffer = None
        if pinned:
            import torch
            keep = torch.empty(run_experts * cfg.record_stride, dtype=torch.uint8).pin_memory()
            buffer = keep.numpy()
        copied = 0
        for at, block in self.runs(layer, first, count, run_experts, buffer):
            moe.load_layer(layer, records=block, first_expert=at)      # a synchronous copy: the staging buffer is free again
            copied += block.size
        return copied
