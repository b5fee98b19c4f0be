"""Loading a prepared-record directory into HBM through the streaming loader gives the same resident bytes and the
same layer output as handing the records over directly."""
import numpy as np
import pytest

from tests import util
from tests.test_moe_gpu import device_x, make
from zerocool_b200 import artifact, synth

pytestmark = pytest.mark.gpu
SEED = 23


def test_loader_fills_hbm_like_a_direct_load(tmp_path):
    import torch
    cfg = util.cfg2(experts=32, top_k=4, max_tokens=16)
    artifact.write_artifact(str(tmp_path), cfg, lambda layer: (synth.record(cfg, SEED, layer, e) for e in range(cfg.experts)))
    prepared = artifact.PreparedExperts(str(tmp_path), cfg)
    a, b = make(cfg), make(cfg)
    copied = prepared.load_layer(a, 0, run_experts=5)
    assert copied == cfg.experts * cfg.record_stride
    b.load_layer(0, records=np.stack([synth.record(cfg, SEED, 0, e) for e in range(cfg.experts)]))
    for m in (a, b):
        m.load_layer(0, router_w=synth.router(cfg, SEED, 0), shared_record=synth.record(cfg, SEED, 0, synth.SHARED_EXPERT),
                     shared_gate_w=synth.shared_gate(cfg, SEED, 0))
    for e in (0, 13, 31):
        got = a.read_layer_tensor(0, "records", cfg.record_bytes, offset=e * cfg.record_stride)
        assert np.array_equal(np.frombuffer(got, np.uint8), synth.record(cfg, SEED, 0, e)[:cfg.record_bytes])
    x = synth.activations(cfg, SEED, 0, 9)
    assert torch.equal(a.moe(0, device_x(a, x)), b.moe(0, device_x(b, x)))
