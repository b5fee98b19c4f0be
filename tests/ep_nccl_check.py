"""Two (or more) ranks, one GPU each: the expert-parallel layer over NCCL against the single-handle layer.
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
from zerocool_b200.ep import ExpertParallel  # noqa: E402
from zerocool_b200.moe import Moe  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    base = dict(hidden=4096, experts=64, top_k=10, has_shared=0, max_tokens=32)
    per = 64 // world
    full = Moe(util.cfg2(**base), local)
    part = Moe(util.cfg2(first_expert=rank * per, local_experts=per, **base), local)
    full.synth_fill_layer(0, 9)
    part.synth_fill_layer(0, 9)
    x = torch.from_numpy(synth.activations(full.cfg, 9 + rank, 0, 32)).to(device="cuda", dtype=torch.bfloat16)
    ep = ExpertParallel(part, 64, rank, world, dist)
    got = ep.moe(0, x).float().cpu().numpy()
    want = full.moe(0, x).float().cpu().numpy()
    err = util.rel_max_error(got, want)
    ok = torch.tensor([1 if err < 1e-5 and part.status() == 0 else 0], device="cuda")
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("ep ok" if int(ok.item()) else f"ep mismatch: {err}", ep.last_plan)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if int(ok.item()) else 1)


if __name__ == "__main__":
    main()
