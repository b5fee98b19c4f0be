"""A CPU stand-in for the three local steps of expert parallelism, built on the checker (test infrastructure).
It lets the host-side exchange logic of zerocool_b200/ep.py run on CPU ranks (gloo) without a GPU."""
import numpy as np
import torch

from oracle import oracle
from zerocool_b200 import synth


class OracleBackend:
    def __init__(self, cfg, seed, first_expert, local_experts):
        self.cfg, self.seed = cfg, seed
        self.first, self.local = first_expert, local_experts
        self.keep = {}

    def record(self, layer, e):
        assert self.first <= e < self.first + self.local, "row sent to a rank that does not hold its expert"
        return synth.record(self.cfg, self.seed, layer, e)

    def ep_dispatch(self, layer, x):
        cfg = self.cfg
        xf = x.numpy().astype(np.float32)
        logits = oracle.router_logits(xf, synth.router(cfg, self.seed, layer), cfg.router_dtype)
        ids, weights = oracle.route(logits, cfg.top_k)
        offsets, perm = oracle.permute(ids, cfg.experts)
        self.keep[layer] = (ids, weights, perm)
        rows = torch.from_numpy(xf[perm // cfg.top_k])
        return rows, torch.from_numpy(ids.reshape(-1)[perm].astype(np.int32)), offsets

    def ep_experts(self, layer, rows, row_experts):
        cfg = self.cfg
        y = np.zeros((rows.shape[0], cfg.hidden), np.float32)
        for i, e in enumerate(row_experts.numpy()):
            y[i] = oracle.expert(cfg.as_dict(), self.record(layer, int(e)), rows[i].numpy())[1][0]
        return torch.from_numpy(y)

    def ep_combine(self, layer, x, y_sorted, out=None):
        cfg = self.cfg
        ids, weights, perm = self.keep[layer]
        xf = x.numpy().astype(np.float32)
        T = xf.shape[0]
        eo = np.zeros((T * cfg.top_k, cfg.hidden), np.float32)
        eo[perm] = y_sorted.numpy()[:len(perm)]
        shared = gate = None
        if cfg.has_shared:
            shared = oracle.expert(cfg.as_dict(), synth.record(cfg, self.seed, layer, synth.SHARED_EXPERT), xf)[1]
            gate = oracle.router_logits(xf, synth.shared_gate(cfg, self.seed, layer), cfg.router_dtype)[:, 0]
        return torch.from_numpy(oracle.combine(cfg.as_dict(), eo.reshape(T, cfg.top_k, cfg.hidden), weights, shared, gate))
