"""Expert-parallel MoE layer over the ranks of one node.

The reference engine is single-GPU; this is new design for the expert-parallel configuration: rank r holds the
records of experts [r*E/N, (r+1)*E/N) of every layer, the router / shared expert / shared gate are replicated,
and tokens start data parallel. Per layer each rank runs

    dispatch (local)  ->  all-to-all of token rows + expert ids  ->  experts (local)
                      ->  all-to-all of the results back          ->  combine (local)

Two transports:

* `ExpertParallel`: the exchange is `torch.distributed.all_to_all_single` (NCCL over NVLink on GPUs; gloo in the
  CPU tests). The three local steps come from a backend: a `zerocool_b200.moe.Moe` handle on a GPU, or any object
  with the same `ep_dispatch / ep_experts / ep_combine` methods. The split sizes are read on the host, so every
  layer costs two host synchronisations.
* `PeerExpertParallel`: rows, results and flags travel as peer stores issued by the library's own kernels into
  windows the ranks map from each other (`zc_moe_ep_layer`, `zc_moe_ep_stack`); the process group is used once,
  to exchange the window handles. Nothing is read on the host per layer and a whole stack replays from a graph.

Results do not depend on arrival order: every contribution is stored at its router slot and reduced in fixed
slot order by the combine step.
"""
import numpy as np


def owner_bounds(offsets, experts, world):
    """Positions in the expert-sorted row list where each rank's expert range starts: int64 [world + 1]."""
    if experts % world:
        raise ValueError("experts must divide evenly over the ranks")
    per = experts // world
    return np.asarray([int(offsets[r * per]) for r in range(world + 1)], dtype=np.int64)


class ExpertParallel:
    """One rank's view. `backend` provides the local steps; `dist` is torch.distributed (already initialised)."""

    def __init__(self, backend, experts, rank, world, dist=None, group=None):
        self.backend, self.experts, self.rank, self.world = backend, experts, rank, world
        self.dist, self.group = dist, group
        self.last_plan = None

    def _exchange(self, tensor, send_counts, recv_counts):
        import torch
        out = torch.empty((int(sum(recv_counts)),) + tuple(tensor.shape[1:]), dtype=tensor.dtype, device=tensor.device)
        self.dist.all_to_all_single(out, tensor[:int(sum(send_counts))].contiguous(), output_split_sizes=[int(c) for c in recv_counts],
                                    input_split_sizes=[int(c) for c in send_counts], group=self.group)
        return out

    def moe(self, layer, x, out=None):
        """x: this rank's tokens [T_local, H] -> out [T_local, H]."""
        import torch
        rows, row_experts, offsets = self.backend.ep_dispatch(layer, x)
        bounds = owner_bounds(offsets, self.experts, self.world)
        send = np.diff(bounds)
        counts = torch.as_tensor(send, dtype=torch.int64, device=rows.device)
        recv_t = torch.empty_like(counts)
        self.dist.all_to_all_single(recv_t, counts, group=self.group)
        recv = recv_t.cpu().numpy()
        x_recv = self._exchange(rows, send, recv)
        e_recv = self._exchange(row_experts, send, recv)
        y_recv = self.backend.ep_experts(layer, x_recv, e_recv)
        y_back = self._exchange(y_recv, recv, send)
        total = x.shape[0] * (rows.shape[0] // max(x.shape[0], 1))
        if y_back.shape[0] < total:                       # slots dropped by an invalid route: pad to the full slot count
            pad = torch.zeros((total - y_back.shape[0], y_back.shape[1]), dtype=y_back.dtype, device=y_back.device)
            y_back = torch.cat([y_back, pad])
        self.last_plan = dict(send=send, recv=recv, rows_sent=int(send.sum()), rows_received=int(recv.sum()))
        return self.backend.ep_combine(layer, x, y_back, out)


class PeerExpertParallel:
    """One rank's view of the peer-store transport. `moe` is a `zerocool_b200.moe.Moe` holding this rank's expert
    range; `dist` is torch.distributed (initialised), used only to exchange the window handles."""

    def __init__(self, moe, dist, group=None):
        self.handle = moe
        moe.ep_attach_group(dist, group)

    def moe(self, layer, x, out=None):
        """x: this rank's tokens [T_local, H] -> out [T_local, H]; stream-ordered, no host synchronisation."""
        return self.handle.ep_layer(layer, x, out)

    def stack(self, x, out=None, eager=False):
        """All layers chained through act((out - mean) / std), replayed from one CUDA graph."""
        return self.handle.ep_stack(x, out, eager=eager)


def emulate_peer(handles, layer, xs):
    """The peer-store transport with every rank in this process on one device: all sends, then all owners, then
    all finishes, in stream order - no kernel ever has to wait for a later launch. handles[r] must already be
    attached to each other (attach_local)."""
    for h, x in zip(handles, xs):
        h.ep_send(layer, x)
    for h in handles:
        h.ep_process(layer)
    return [h.ep_finish(layer, x) for h, x in zip(handles, xs)]


def attach_local(handles):
    """Attaches handles that live in one process on one device to each other by window address."""
    windows = [h.ep_export()[1] for h in handles]
    for r, h in enumerate(handles):
        h.ep_attach(r, len(handles), pointers=windows)


def emulate(backends, experts, layer, xs):
    """All ranks in one process (one GPU, or the CPU checker): the same plan with the exchange done by slicing.
    backends[r] holds rank r's expert range, xs[r] its tokens. Returns the list of outputs."""
    import torch
    world = len(backends)
    disp = [b.ep_dispatch(layer, x) for b, x in zip(backends, xs)]
    bounds = [owner_bounds(d[2], experts, world) for d in disp]
    outs = []
    y_parts = [[None] * world for _ in range(world)]      # y_parts[src][dst]
    for dst in range(world):
        pieces = [disp[src][0][bounds[src][dst]:bounds[src][dst + 1]] for src in range(world)]
        ids = [disp[src][1][bounds[src][dst]:bounds[src][dst + 1]] for src in range(world)]
        y = backends[dst].ep_experts(layer, torch.cat(pieces), torch.cat(ids))
        at = 0
        for src in range(world):
            n = pieces[src].shape[0]
            y_parts[src][dst] = y[at:at + n]
            at += n
    for src in range(world):
        y_back = torch.cat(y_parts[src])
        total = disp[src][0].shape[0]
        if y_back.shape[0] < total:
            y_back = torch.cat([y_back, torch.zeros((total - y_back.shape[0], y_back.shape[1]), dtype=y_back.dtype, device=y_back.device)])
        outs.append(backends[src].ep_combine(layer, xs[src], y_back))
    return outs
