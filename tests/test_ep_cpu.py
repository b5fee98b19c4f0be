"""Host-side logic of expert parallelism (zerocool_b200/ep.py) on two CPU ranks over gloo: the split sizes, the
all-to-all exchange and the return path, with the checker standing in for the device steps. The result of the
two ranks together must equal the single-process layer on the same tokens."""
import os

import numpy as np
import torch
import torch.multiprocessing as mp

from oracle import oracle
from zerocool_b200 import synth
from zerocool_b200.records import F16, F32, MoeConfig

SEED, WORLD, T_LOCAL = 31, 2, 5
CFG = dict(hidden=256, ffn=128, experts=64, top_k=4, layers=1, meta_dtype=F16, act_dtype=F32, out_dtype=F32, router_dtype=F32, has_shared=1)


def tokens(rank):
    return synth.activations(MoeConfig(**CFG), SEED + rank, 0, T_LOCAL)


def worker(rank, world, port, results):
    import torch.distributed as dist
    from tests.ep_backend import OracleBackend
    from zerocool_b200.ep import ExpertParallel
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = MoeConfig(**CFG)
    per = cfg.experts // world
    ep = ExpertParallel(OracleBackend(cfg, SEED, rank * per, per), cfg.experts, rank, world, dist)
    out = ep.moe(0, torch.from_numpy(tokens(rank)))
    results[rank] = (out.numpy(), ep.last_plan)
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_exchange_matches_single_process():
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(worker, args=(WORLD, 29577, results), nprocs=WORLD, join=True)
    cfg = MoeConfig(**CFG)
    records = [synth.record(cfg, SEED, 0, e) for e in range(cfg.experts)]
    sent = received = 0
    for rank in range(WORLD):
        x = tokens(rank)
        want = oracle.moe_layer(cfg.as_dict(), records, synth.router(cfg, SEED, 0), x,
                                shared_record=synth.record(cfg, SEED, 0, synth.SHARED_EXPERT), shared_gate_w=synth.shared_gate(cfg, SEED, 0))
        got, plan = results[rank]
        assert np.array_equal(got, want["out"]), rank
        assert plan["rows_sent"] == T_LOCAL * cfg.top_k
        sent += plan["rows_sent"]
        received += plan["rows_received"]
    assert sent == received


def test_emulated_ranks_match_single_process():
    """The in-process emulation used on one GPU follows the same plan."""
    from tests.ep_backend import OracleBackend
    from zerocool_b200.ep import emulate
    cfg = MoeConfig(**CFG)
    per = cfg.experts // 4
    backends = [OracleBackend(cfg, SEED, r * per, per) for r in range(4)]
    xs = [torch.from_numpy(synth.activations(cfg, SEED + r, 0, 3)) for r in range(4)]
    outs = emulate(backends, cfg.experts, 0, xs)
    records = [synth.record(cfg, SEED, 0, e) for e in range(cfg.experts)]
    for r in range(4):
        want = oracle.moe_layer(cfg.as_dict(), records, synth.router(cfg, SEED, 0), xs[r].numpy(),
                                shared_record=synth.record(cfg, SEED, 0, synth.SHARED_EXPERT), shared_gate_w=synth.shared_gate(cfg, SEED, 0))
        assert np.array_equal(outs[r].numpy(), want["out"])
