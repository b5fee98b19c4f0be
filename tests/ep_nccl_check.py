"""Two (or more) ranks, one GPU each: the expert-parallel layer against the single-handle layer, over both
transports (NCCL all-to-all with host-read splits; peer stores into mapped windows), plus a three-layer
expert-parallel stack replayed from a graph against the single-handle stack.
Launched by tests/test_ep_gpu.py through torch.distributed.run; prints "ep ok" on rank 0."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from tests import util  # noqa: E402
from zerocool_b200 import synth  # noqa: E402
from zerocool_b200.ep import ExpertParallel, PeerExpertParallel  # noqa: E402
from zerocool_b200.moe import Moe  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    layers = 3
    base = dict(hidden=4096, experts=64, top_k=10, has_shared=0, max_tokens=32, layers=layers)
    per = 64 // world
    full = Moe(util.cfg2(**base), local)
    part = Moe(util.cfg2(first_expert=rank * per, local_experts=per, **base), local)
    for layer in range(layers):
        full.synth_fill_layer(layer, 9)
        part.synth_fill_layer(layer, 9)
    x = torch.from_numpy(synth.activations(full.cfg, 9 + rank, 0, 32 - rank)).to(device="cuda", dtype=torch.bfloat16)
    ep = ExpertParallel(part, 64, rank, world, dist)
    got = ep.moe(0, x).float().cpu().numpy()
    want = full.moe(0, x).float().cpu().numpy()
    errs = {"nccl": util.rel_max_error(got, want)}
    peer = PeerExpertParallel(part, dist)
    for call in range(2):                              # the second call runs a later epoch on the first one's leftovers
        errs[f"peer{call}"] = util.rel_max_error(peer.moe(0, x).float().cpu().numpy(), want)
    want_stack = full.stack(x).float().cpu().numpy()
    for call in range(2):                              # capture, then replay
        errs[f"stack{call}"] = util.rel_max_error(peer.stack(x).float().cpu().numpy(), want_stack)
    worst = max(errs.values())
    ok = torch.tensor([1 if worst < 1e-5 and part.status() == 0 else 0], device="cuda")
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("ep ok" if int(ok.item()) else f"ep mismatch: {errs}", ep.last_plan)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if int(ok.item()) else 1)


if __name__ == "__main__":
    main()
