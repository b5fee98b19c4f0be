#!/usr/bin/env python3
"""Benchmark of the MoE-layer hot path: decode MoE stack at the Qwen3-Next-like shape.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload decode|prefill|mixed|ep]

A step is one pass of the 48-layer MoE stack (hidden 2048, 512 routed experts top-10 + 1 shared expert,
ffn 512, affine-Q4 group 64 with fp16 scale/bias, bf16 activations) over one batch of tokens, the layers
chained on one stream through x_{l+1} = bf16((out_l - mean) / std) per token. All 48 layers' records (43.5 GB) are
resident in HBM, so every step streams its weights from DRAM (inputs far larger than the 126 MB L2).
Inputs are seeded synthetic tensors with the shapes and value distributions of the benchmark
specification; the real checkpoint is not available.

Rank 0 prints ONE JSON line. `value` is whole-job tokens/s of the decode stack (benchmark configuration 2) with
inputs resident in HBM; `e2e` is the same metric through the host-buffer entry point (pinned host activations
copied in and out inside the timed region); `roofline` reports the dominant kernel against the measured HBM
bandwidth; `cpu_baseline` is the CPU restatement of the reference's arithmetic (oracle/) timed on this machine's
host cores on a bounded sample. The same line carries the other configurations of the specification as
sub-records: `prefill` (configuration 3: 2048 and 8192 tokens, Zipf-skewed loads, tensor roofline), `mixed`
(configuration 4: gate/up Q4 + down Q8, ragged batch of 32 requests) and `ep` (configuration 5: hidden 4096,
256-token batch; expert-parallel over the N ranks when N >= 2, one GPU holding all 87 GB when N = 1).
With --impl reference the CPU code is the thing timed.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from zerocool_b200 import synth  # noqa: E402
from zerocool_b200.records import BF16, F16, F32, MoeConfig  # noqa: E402

METRIC = "MoE-layer tokens/s at Qwen3-Next shape (decode, 48-layer MoE stack)"
SEED = 20261125
BATCHES = (1, 4, 16, 64)
EXTRA_OPTIONS = []    # (name, value) pairs from --opt, applied to the long-batch handle (tuning sweeps)
SMALL_ROWS = 16       # long batches: experts with at most this many rows take the streaming kernels (option prefill_small_rows)
TOL = 2e-3            # max-abs error / output RMS, fp32 accumulation (the tolerance of the benchmark specification)


def config(layers, max_tokens, **kw):
    base = dict(hidden=2048, ffn=512, experts=512, top_k=10, layers=layers, meta_dtype=F16, act_dtype=BF16,
                out_dtype=BF16, router_dtype=F32, has_shared=1, max_tokens=max_tokens)
    base.update(kw)
    return MoeConfig(**base)


def config5(layers, max_tokens, rank=0, world=1):
    per = 512 // world
    return MoeConfig(hidden=4096, ffn=512, experts=512, top_k=10, layers=layers, meta_dtype=F16, act_dtype=BF16, out_dtype=BF16,
                     router_dtype=F32, has_shared=0, max_tokens=max_tokens, first_expert=rank * per if world > 1 else 0,
                     local_experts=per if world > 1 else 0)


def mixed_lengths():
    """Configuration 4: 32 requests with seeded lengths U{1..512}, flattened to one ragged token batch."""
    return np.random.default_rng(SEED).integers(1, 513, size=32)


def workload(cfg, tokens, n_gpus, kind="decode"):
    shape = (f"{cfg.layers} layers, hidden {cfg.hidden}, {cfg.experts} routed experts top-{cfg.top_k}" + (" + 1 shared" if cfg.has_shared else "") +
             f", ffn {cfg.ffn}")
    glue = "layers chained through bf16((out-mean)/std)"
    replicas = f"dp{n_gpus}: independent replicas, tokens sharded, no data-path collective"
    if kind == "prefill":
        return {"workload": f"benchmark configuration 3: prefill grouped GEMM, {shape}, affine-Q4 g64 fp16 scale/bias, bf16 activations, fp32 router with an "
                            f"additive Zipf(s=1.1) per-expert logit bias, sequence of {tokens} tokens per GPU, {glue}",
                "tokens_per_gpu": tokens, "layers": cfg.layers, "parallelism": replicas,
                "l2": "no flush needed: every layer streams its active records (43.5 GB resident) through a 126 MB L2",
                "accumulate": "f32", "weights": "q4_g64: exact integer codes on tcgen05.mma (FP16 operands, FP32 TMEM accumulators), scale and bias applied in FP32"}
    if kind == "mixed":
        return {"workload": f"benchmark configuration 4: mixed 4/8-bit continuous batching, {shape}, gate/up affine-Q4 g64 and down affine-Q8 g64 (int8), "
                            f"fp16 scale/bias, ragged batch of 32 requests with seeded lengths 1..512 = {tokens} tokens, {glue}",
                "tokens_per_gpu": tokens, "layers": cfg.layers, "parallelism": replicas,
                "l2": "no flush needed: every layer streams its active records (56 GB resident) through a 126 MB L2",
                "accumulate": "f32", "weights": "gate/up q4_g64, down q8_g64"}
    return {"workload": f"benchmark configuration 2: decode MoE stack, {shape}, affine-Q4 g64 fp16 scale/bias, bf16 activations, fp32 router, "
                        f"batch of {tokens} tokens per GPU, {glue}",
            "tokens_per_gpu": tokens, "layers": cfg.layers, "parallelism": replicas,
            "l2": "no flush needed: each step streams the selected records of 48 different layers (GBs per step, 43.5 GB resident) through a 126 MB L2",
            "accumulate": "f32", "weights": "q4_g64"}


def _peaks_file():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    return json.load(open(path)) if os.path.exists(path) else None


def peaks():
    p = _peaks_file()
    if p:
        return float(p["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


def tensor_peak():
    p = _peaks_file()
    if p:
        return float(p["bf16_tflops"]), float(p["bf16_tflops_sustained"]), "measured (MEASURED_PEAKS.json bf16_tflops burst / sustained)"
    return 1590.0, 1400.0, "fallback (1.59 PFLOP/s burst, earlier measurement on this pool)"


def ncu_traffic():
    """DRAM bytes per launch of the dominant kernel from the committed ncu summary, if there is one."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    return json.load(open(path)) if os.path.exists(path) else {}


class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        rows = [r.strip().split(",") for r in open(self.file.name) if r.strip()]
        os.unlink(self.file.name)
        sm, smax, power, reasons = [], [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in rows:
            try:
                sm.append(float(r[0])); smax.append(float(r[1])); power.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(names, r[3:7]):
                if v.strip().lower() == "active":
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(smax)), "power_w_max": float(max(power)),
                "samples": len(sm), "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------------------------------------
# CPU checker legs (parity gates and the CPU baseline): the only users of oracle/ in this file
# ---------------------------------------------------------------------------------------------------------
def rms_glue(out):
    """The inter-layer stand-in of the chained stack, on the CPU: bf16((out - mean) / std) per token."""
    from oracle import oracle
    o = out.astype(np.float32)
    d = o - o.mean(axis=-1, keepdims=True, dtype=np.float32)
    scale = (1.0 / np.sqrt(np.mean(d * d, axis=-1, keepdims=True, dtype=np.float32))).astype(np.float32)
    return oracle.bf(d * scale)


def cpu_layer(cfg, layer, x, cache, bias=None):
    """One layer on the CPU checker; records of the selected experts are regenerated from the seed (cached)."""
    from oracle import oracle
    router = cache.setdefault(("router", layer), synth.router(cfg, SEED, layer))
    keep = oracle.set_router_bias(bias)
    logits = oracle.router_logits(x, router, cfg.router_dtype)
    oracle.set_router_bias(None)
    del keep
    ids, _ = oracle.route(logits, cfg.top_k)
    records = [None] * cfg.experts
    for e in np.unique(ids):
        if e >= 0:
            records[e] = cache.setdefault(("record", layer, int(e)), synth.record(cfg, SEED, layer, int(e)))
    shared = gate = None
    if cfg.has_shared:
        shared = cache.setdefault(("shared", layer), synth.record(cfg, SEED, layer, synth.SHARED_EXPERT))
        gate = cache.setdefault(("gate", layer), synth.shared_gate(cfg, SEED, layer))
    t0 = time.perf_counter()
    res = oracle.moe_layer(cfg.as_dict(), records, router, x, shared_record=shared, shared_gate_w=gate, router_bias=bias)
    return res, time.perf_counter() - t0


def cpu_sample(cfg, tokens, sample_layers, cache):
    """Chained CPU run over the first `sample_layers` layers; returns seconds of arithmetic (generation excluded)."""
    from oracle import oracle
    x = synth.activations(cfg, SEED, 0, tokens)
    total = 0.0
    for layer in range(sample_layers):
        res, dt = cpu_layer(cfg, layer, x, cache)
        total += dt
        x = rms_glue(oracle.bf(res["out"]))
    return total


def parity_gate(torch, cfg, tokens, x_np, bias=None, out_bf16=None, checked=64, routing=None, runner=None):
    """Layer 0 against the CPU checker, outside every timed region. The device result comes from a one-layer handle of
    the same geometry and weights whose output dtype is FP32, so that the stated tolerance (max-abs error <= 2e-3 x
    output RMS) is applied as it stands; the error of the benchmark handle's BF16 output is reported beside it.
    `runner(x_dev) -> (out fp32 numpy, routing dict)` replaces the one-layer handle (expert-parallel runs)."""
    from oracle import oracle
    from zerocool_b200.moe import Moe
    checked = min(tokens, checked)
    if runner is None:
        c32 = MoeConfig(**{**cfg.__dict__, "layers": 1, "out_dtype": F32, "max_tokens": tokens})
        m32 = Moe(c32, torch.cuda.current_device())
        m32.synth_fill_layer(0, SEED)
        if bias is not None:
            m32.set_router_bias(0, bias)
        x_dev = torch.from_numpy(x_np).to(device="cuda", dtype=torch.bfloat16)
        got = m32.moe(0, x_dev).float().cpu().numpy()
        routing = m32.last_routing(tokens)
        status = m32.status()
        m32.close()
    else:
        got, routing, status = runner()
    want, _ = cpu_layer(cfg, 0, x_np[:checked], {}, bias)
    ids_all = routing["ids"]
    offsets, perm = oracle.permute(want["ids"] if checked == tokens else ids_all, cfg.experts)    # long batches: from the device's own (checked) ids
    rms = float(np.sqrt(np.mean(want["out"].astype(np.float64) ** 2)))
    err = float(np.abs(got[:checked] - want["out"]).max() / rms)
    parity = {
        "layer": 0, "tokens": tokens, "tokens_checked_against_cpu": checked,
        "ids_bit_exact": bool(np.array_equal(ids_all[:checked], want["ids"])),
        "perm_bit_exact": bool(np.array_equal(routing["perm"], perm) and np.array_equal(routing["offsets"], offsets)),
        "max_abs_err_over_rms": err, "within_tolerance": bool(err <= TOL), "device_status": int(status),
        "tolerance": "max-abs error <= 2e-3 x output RMS on an FP32-output handle of the same geometry and weights",
    }
    if out_bf16 is not None:
        parity["max_abs_err_over_rms_bf16_output"] = float(np.abs(out_bf16[:checked] - want["out"]).max() / rms)
    if not (parity["ids_bit_exact"] and parity["perm_bit_exact"] and parity["within_tolerance"] and status == 0):
        raise RuntimeError(f"parity gate failed: {parity}")
    return parity


def run_reference(args):
    """The reference arm: the CPU implementation of the path (the port under oracle/ - the reference's native
    code is Apple Metal and cannot be built here), all host threads, on a bounded sample of the same workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle
    oracle.build()
    oracle.set_threads(len(os.sched_getaffinity(0)))      # a multi-rank launcher exports OMP_NUM_THREADS=1: use every host core anyway
    cfg = config(48, args.tokens)
    sample_layers = args.cpu_layers
    cache = {}
    cpu_sample(cfg, args.tokens, sample_layers, cache)        # builds the record cache, untimed
    for _ in range(max(args.warmup - 1, 0)):
        cpu_sample(cfg, args.tokens, sample_layers, cache)
    times = [cpu_sample(cfg, args.tokens, sample_layers, cache) for _ in range(args.steps)]
    per_step = float(np.mean(times)) * cfg.layers / sample_layers
    value = args.tokens / per_step
    cores = oracle.threads()
    sample = f"layers 0..{sample_layers - 1} of {cfg.layers} chained, {args.tokens} tokens, scaled by {cfg.layers}/{sample_layers}"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": workload(cfg, args.tokens, args.gpus),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------------
# Device-side measurement helpers
# ---------------------------------------------------------------------------------------------------------
def time_steps(torch, fn, steps, dist):
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        fn()
    stop.record()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    ms = start.elapsed_time(stop)
    if dist is not None:
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms / steps


def layer_bytes(cfg, active, tokens):
    """Algorithmic bytes of one layer: (U + S) records + the router matrix + activations in and out."""
    return (active + cfg.has_shared) * cfg.record_bytes + cfg.experts * cfg.hidden * 4 + tokens * cfg.hidden * 2 * 2


def kernel_profile(m, run, steps):
    """Per-kernel device times over `steps` eager passes (event pairs around every launch)."""
    run()
    m._torch.cuda.synchronize()
    m.profile_begin()
    for _ in range(steps):
        run()
    prof = m.profile_end()
    total = sum(v[0] for v in prof.values()) or 1.0
    return {k: {"launches": n, "avg_us": 1e3 * t / max(n, 1), "share": t / total} for k, (t, n) in prof.items() if n}


def fill(m, cfg, biased=False):
    biases = {}
    for layer in range(cfg.layers):
        m.synth_fill_layer(layer, SEED)
        if biased:
            biases[layer] = synth.zipf_router_bias(cfg, SEED, layer)
            m.set_router_bias(layer, biases[layer])
    m._torch.cuda.synchronize()
    return biases


def make_inputs(torch, cfg, tokens, rank):
    x = synth.activations(cfg, SEED + rank, 0, tokens)
    host = torch.from_numpy(x).to(torch.bfloat16).pin_memory()
    return x, host, host.cuda()


def measure_long_batch(torch, m, cfg, tokens, steps, warmup, kind, biases, skip_parity):
    """Configurations 3 and 4 on one GPU: the chained stack over one long batch (the tensor-core family)."""
    hbm_peak, peak_source = peaks()
    burst, sustained, tsource = tensor_peak()
    x_np, _, x_dev = make_inputs(torch, cfg, tokens, 0)
    out_dev = torch.empty((tokens, cfg.hidden), dtype=torch.bfloat16, device="cuda")
    m.set_option("prefill_small_rows", SMALL_ROWS)
    for name, value in EXTRA_OPTIONS:
        m.set_option(name, value)
    parity = None
    if not skip_parity:
        got16 = m.moe(0, x_dev).float().cpu().numpy()
        parity = parity_gate(torch, cfg, tokens, x_np, biases.get(0), out_bf16=got16)
    for _ in range(warmup):
        m.stack(x_dev, out_dev)
    before = m.launches
    ms = time_steps(torch, lambda: m.stack(x_dev, out_dev), steps, None)
    launches = m.launches - before
    active = m.active_counts()
    if not bool(torch.isfinite(out_dev.float()).all()):
        raise RuntimeError("the chained stack produced non-finite values")
    kernels = kernel_profile(m, lambda: m.stack_eager(x_dev, out_dev), min(steps, 3))
    rows = tokens * (cfg.top_k + cfg.has_shared)
    # Rows per kernel family: experts with at most SMALL_ROWS rows run on the streaming kernels, the grouped GEMM takes the
    # rest and the shared expert (counted on the last layer's routing, which the handle still holds).
    counts = np.diff(m.last_routing(tokens)["offsets"])
    rows_small = int(counts[counts <= SMALL_ROWS].sum())
    rows_big = int(counts[counts > SMALL_ROWS].sum()) + tokens * cfg.has_shared
    per_row = {"gate_up": 2.0 * 2 * cfg.ffn * cfg.hidden, "down": 2.0 * cfg.hidden * cfg.ffn}
    flops = {"prefill_gate_up": rows_big * per_row["gate_up"], "prefill_down": rows_big * per_row["down"],
             "gate_up": rows_small * per_row["gate_up"], "down": rows_small * per_row["down"]}
    expert_kernels = [k for k in kernels if k in flops]
    dominant = max(expert_kernels, key=lambda k: kernels[k]["share"])
    tf = flops[dominant] / (kernels[dominant]["avg_us"] * 1e-6) / 1e12
    step_flops = cfg.layers * 6.0 * rows * cfg.hidden * cfg.ffn
    step_bytes = float(sum(layer_bytes(cfg, int(a), tokens) for a in active))
    return {
        "config": workload(cfg, tokens, 1, kind), "tokens": tokens, "steps": steps, "warmup": warmup, "ms_per_step": ms,
        "tokens_per_s": tokens / (ms * 1e-3), "gpu_launches": int(launches), "mean_active_experts": float(np.mean(active)),
        "family": {k: ("tcgen05 grouped GEMM" if k.startswith("prefill") else f"mma.sync streaming kernels (experts with at most {SMALL_ROWS} rows)") for k in expert_kernels},
        "rows_last_layer": {"tensor_core_family": rows_big, "streaming_family": rows_small},
        "roofline": {"bound": "tensor", "kernel": dominant, "achieved": tf, "peak": burst, "unit": "TFLOP/s", "frac": tf / burst,
                     "frac_of_sustained": tf / sustained, "peak_source": tsource, "algorithmic_flops_per_launch": flops[dominant],
                     "avg_launch_us": kernels[dominant]["avg_us"],
                     "traffic": ncu_traffic().get(dominant) if (kind == "prefill" and tokens == 2048) else None,      # the capture was taken at 2048 tokens
                     "definition": "2 x rows this kernel family processed (last layer's routing) x output columns x K of this launch (useful flops; "
                                   "padded token columns, the second FP16 term of the exact weights and the bias-correction stages are not counted)"},
        "roofline_step": {"tensor_tflops": step_flops / (ms * 1e-3) / 1e12, "frac_of_tensor_peak": step_flops / (ms * 1e-3) / 1e12 / burst,
                          "hbm_gbs": step_bytes / (ms * 1e-3) / 1e9, "frac_of_hbm_peak": step_bytes / (ms * 1e-3) / 1e9 / hbm_peak,
                          "algorithmic_flops_per_step": step_flops, "algorithmic_bytes_per_step": step_bytes, "peak_source": peak_source},
        "kernels": kernels, "parity": parity,
    }


def measure_ep(torch, dist, rank, world, local, layers, total_tokens, steps, warmup, skip_parity):
    """Configuration 5: hidden 4096, 512 experts top-10 (512/N per GPU), ffn 512, Q4 g64, one 256-token decode batch.
    N >= 2: expert parallel, rows and results exchanged by peer stores over NVLink (falls back to the NCCL all-to-all
    with host-read split sizes if the windows cannot be mapped). N = 1: one GPU holds all 87 GB (the comparison point)."""
    from zerocool_b200.moe import Moe
    hbm_peak, peak_source = peaks()
    t_local = total_tokens // world
    cfg = config5(layers, t_local, rank, world)
    m = Moe(cfg, local)
    for name, value in EXTRA_OPTIONS:
        m.set_option(name, value)
    fill(m, cfg)
    x_np, _, x_dev = make_inputs(torch, cfg, t_local, rank)
    out_dev = torch.empty((t_local, cfg.hidden), dtype=torch.bfloat16, device="cuda")
    transport, run, run_eager, layer0 = "none (one GPU holds every expert)", None, None, None
    if world > 1:
        from zerocool_b200.ep import ExpertParallel, PeerExpertParallel
        try:
            peer = PeerExpertParallel(m, dist)
            attached = 1
        except (RuntimeError, ValueError) as exc:
            attached, why = 0, str(exc)
        flag = torch.tensor([attached], device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()):
            transport = "peer stores into mapped windows (NVLink), flags with bounded waits, no host value per layer; 48 layers replayed from one CUDA graph"
            run = lambda: m.ep_stack(x_dev, out_dev)                       # noqa: E731
            run_eager = lambda: m.ep_stack(x_dev, out_dev, eager=True)     # noqa: E731
            layer0 = lambda: m.ep_layer(0, x_dev)                          # noqa: E731
        else:
            transport = "NCCL all_to_all_single with split sizes read on the host (two host synchronisations per layer)" + (f"; peer windows unavailable: {why}" if not attached else "")
            ep = ExpertParallel(m, cfg.experts, rank, world, dist)

            def run():
                x = x_dev
                for layer in range(cfg.layers):
                    out = ep.moe(layer, x)
                    if layer + 1 < cfg.layers:
                        f = out.float()
                        d = f - f.mean(-1, keepdim=True)
                        x = (d * torch.rsqrt((d * d).mean(-1, keepdim=True))).to(torch.bfloat16)
                out_dev.copy_(out)
            run_eager = None
            layer0 = lambda: ep.moe(0, x_dev)                              # noqa: E731
    else:
        run = lambda: m.stack(x_dev, out_dev)                              # noqa: E731
        run_eager = lambda: m.stack_eager(x_dev, out_dev)                  # noqa: E731
        layer0 = lambda: m.moe(0, x_dev)                                   # noqa: E731

    # ---- parity: layer 0 of this rank's tokens against the CPU checker (rank 0 checks; every rank runs the layer) ----
    parity = None
    if not skip_parity:
        got16 = layer0().float().cpu().numpy()
        routing = m.last_routing(t_local)
        status = m.status()
        if rank == 0:
            from oracle import oracle
            checked = min(t_local, 16)
            want, _ = cpu_layer(cfg, 0, x_np[:checked], {})
            rms = float(np.sqrt(np.mean(want["out"].astype(np.float64) ** 2)))
            err = np.abs(got16[:checked] - want["out"])
            offsets, perm = oracle.permute(routing["ids"], cfg.experts)
            parity = {"layer": 0, "tokens_checked_against_cpu": checked,
                      "ids_bit_exact": bool(np.array_equal(routing["ids"][:checked], want["ids"])),
                      "perm_bit_exact": bool(np.array_equal(routing["perm"], perm) and np.array_equal(routing["offsets"], offsets)),
                      "max_abs_err_over_rms_bf16_output": float(err.max() / rms),
                      "within_tolerance": bool(np.all(err <= TOL * rms + np.abs(want["out"]) * 2.0 ** -8)), "device_status": int(status),
                      "tolerance": "2e-3 x RMS + one bf16 rounding of this handle's bf16 output (the FP32-output bound is applied by the tests)"}
            if not (parity["ids_bit_exact"] and parity["perm_bit_exact"] and parity["within_tolerance"] and status == 0):
                raise RuntimeError(f"expert-parallel parity gate failed: {parity}")

    if dist is not None:
        dist.barrier()            # rank 0 spent seconds in the CPU checker: a device-side wait for its rows must not start before it is back
    for _ in range(warmup):
        run()
    before = m.launches
    ms = time_steps(torch, run, steps, dist)
    launches = m.launches - before
    status = m.status()
    finite = bool(torch.isfinite(out_dev.float()).all())
    if not finite or status:
        raise RuntimeError(f"expert-parallel stack: finite={finite}, device status {status}")
    active = (m.ep_active_counts() if world > 1 else m.active_counts()).astype(np.float64)
    ids_last = m.last_routing(t_local)["ids"]
    per = cfg.experts // world
    remote_rows = int(np.sum((ids_last // per) != rank)) if world > 1 else 0
    if dist is not None:
        dist.barrier()
    kernels = kernel_profile(m, run_eager, min(steps, 3)) if run_eager is not None else {}
    my_bytes = float(sum(a * cfg.record_bytes + cfg.experts * cfg.hidden * 4 + t_local * cfg.hidden * 4 for a in active))
    stats = torch.tensor([my_bytes, float(active.mean()), float(remote_rows)], dtype=torch.float64, device="cuda")
    if dist is not None:
        dist.all_reduce(stats)
    m.close()
    if rank != 0:
        return None
    total_bytes, active_sum, remote_sum = (float(v) for v in stats.tolist())
    row_bytes = cfg.hidden * 2
    ep_kinds = {k: v for k, v in kernels.items() if k == "ep"}
    return {
        "config": {"workload": f"benchmark configuration 5: expert-parallel full stack, {cfg.layers} layers, hidden 4096, 512 experts top-10 ({per} per GPU), "
                               f"ffn 512, affine-Q4 g64, {total_tokens}-token decode batch ({t_local} per GPU), layers chained through bf16((out-mean)/std)",
                   "parallelism": f"ep{world}" if world > 1 else "one GPU, all 512 experts resident (87 GB)", "tokens_total": total_tokens,
                   "layers": cfg.layers, "transport": transport,
                   "l2": "no flush needed: each rank streams its selected records of 48 layers (GBs per step)"},
        "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms, "tokens_per_s": total_tokens / (ms * 1e-3), "scaling": "strong",
        "gpu_launches_rank0": int(launches),
        "roofline_step": {"bound": "hbm", "achieved": total_bytes / (ms * 1e-3) / 1e9 / world, "peak": hbm_peak, "unit": "GB/s per GPU",
                          "frac": total_bytes / (ms * 1e-3) / 1e9 / world / hbm_peak, "peak_source": peak_source,
                          "mean_active_experts_all_ranks": active_sum,
                          "definition": "per rank: experts of its range that received rows x record bytes + its router matrix + its activations in/out, summed "
                                        "over ranks and layers, divided by the step time and by N"},
        "nvlink": {"remote_rows_per_layer_all_ranks": remote_sum, "bytes_per_layer_all_ranks": remote_sum * (row_bytes + cfg.hidden * 4 + 8),
                   "definition": "rows whose expert lives on another rank (last layer's routing): bf16 row + 8-byte tag out, fp32 result row back"},
        "kernels_rank0": kernels, "exchange_share_rank0": sum(v["share"] for v in ep_kinds.values()) if kernels else None,
        "exchange_note": "kind 'ep' = send, receive + sort of the received rows (includes the wait for the slowest sender) and return; the wait for "
                         "the owners' results is inside the combine kernel; event-timed eager launches on rank 0" if kernels else None,
        "parity": parity,
    }


def route_trace_run(torch, local, args):
    """--record-routes: one pass of the chained decode stack, layer by layer, writing every layer's selections as a route
    trace. --replay-routes: the recorded selections forced into the layers (the router still scores, the top-k search is
    skipped), timed per pass with CUDA events; the counterpart of the reference's dependency replay
    (src/engine/bench.cpp:43-104), with the whole layer - router scores, shared expert, combine - inside the timed region."""
    import hashlib
    from zerocool_b200.moe import Moe
    from zerocool_b200.route_trace import RouteTrace, read_route_trace
    cfg = config(args.layers, max(args.tokens, 64))

    def glue(out):
        f = out.float()
        d = f - f.mean(-1, keepdim=True)
        return (d * torch.rsqrt((d * d).mean(-1, keepdim=True))).to(torch.bfloat16)

    if args.record_routes:
        m = Moe(cfg, local)
        fill(m, cfg)
        _, _, x = make_inputs(torch, cfg, args.tokens, 0)
        with RouteTrace(args.record_routes, {"generator": "bench.py", "seed": SEED, "layers": cfg.layers, "experts": cfg.experts, "top_k": cfg.top_k},
                        cfg.layers, cfg.top_k) as trace:
            trace.request_begin("synthetic", [], args.tokens)
            trace.begin(1, 0, args.tokens, phase="decode")
            for layer in range(cfg.layers):
                out = m.moe(layer, x)
                trace.routes(layer, 0, args.tokens, m.last_routing(args.tokens)["ids"])
                x = glue(out)
            trace.commit(args.tokens)
            trace.request_end([], "stop")
            trace.finish()
        return {"recorded": args.record_routes, "tokens": args.tokens, "layers": cfg.layers, "output_sha256": hashlib.sha256(out.cpu().view(torch.int16).numpy().tobytes()).hexdigest()}
    passes = read_route_trace(args.replay_routes, cfg.layers, cfg.top_k, cfg.experts)
    cfg = config(args.layers, max(64, max(p["tokens"] for p in passes)))
    m = Moe(cfg, local)
    fill(m, cfg)
    hbm_peak, peak_source = peaks()
    runs = []
    for index, recorded in enumerate(passes):
        tokens = recorded["tokens"]
        ids = [torch.from_numpy(r).cuda() for r in recorded["routes"]]
        _, _, x0 = make_inputs(torch, cfg, tokens, 0)

        def one_pass():
            x = x0
            for layer in range(cfg.layers):
                out = m.moe_routed(layer, x, ids[layer])
                x = glue(out)
            return out

        for _ in range(args.warmup):
            out = one_pass()
        ms = time_steps(torch, one_pass, args.steps, None)
        active = [len(np.unique(r)) for r in recorded["routes"]]
        step_bytes = float(sum(layer_bytes(cfg, a, tokens) for a in active))
        runs.append({"recorded_pass": index, "tokens": tokens, "offset": recorded["offset"], "phase": recorded["phase"], "ms_per_pass": ms,
                     "tokens_per_s": tokens / (ms * 1e-3), "mean_active_experts": float(np.mean(active)),
                     "hbm_gbs": step_bytes / (ms * 1e-3) / 1e9, "frac_of_hbm_peak": step_bytes / (ms * 1e-3) / 1e9 / hbm_peak,
                     "device_status": m.status(), "output_sha256": hashlib.sha256(out.cpu().view(torch.int16).numpy().tobytes()).hexdigest()})
    return {"kind": "route_replay", "route_source": args.replay_routes, "steps": args.steps, "warmup": args.warmup, "peak_source": peak_source, "runs": runs,
            "note": "launch by launch with the inter-layer glue in PyTorch (no graph): a harness for recorded routing distributions, not the headline path"}


def run_ours(args):
    import torch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as d
        import datetime
        # a rank that fails inside a sub-record must not leave the others waiting for ten minutes
        d.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=240))
        dist = d
    from zerocool_b200.moe import Moe
    hbm_peak, peak_source = peaks()

    if args.record_routes or args.replay_routes:
        if world > 1:
            raise RuntimeError("route traces are recorded and replayed on one GPU")
        print(json.dumps(route_trace_run(torch, local, args)), flush=True)
        return

    if args.workload == "ep":
        ep = measure_ep(torch, dist, rank, world, local, args.layers, args.tokens, args.steps, args.warmup, args.skip_parity)
        if rank == 0:
            line = {"metric": METRIC, "value": ep["tokens_per_s"], "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                    "ms_per_step": ep["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                    "config": ep["config"], "gpu_launches": ep["gpu_launches_rank0"], "ep": ep, "e2e": None, "cpu_baseline": None}
            print(json.dumps(line), flush=True)
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()
        return

    if args.workload in ("prefill", "mixed"):
        if world > 1:
            raise RuntimeError("--workload prefill / mixed run on one GPU")
        if args.workload == "mixed":
            tokens = int(mixed_lengths().sum())
            cfg = config(args.layers, tokens, down_bits=8, q8_signed=1)
        else:
            tokens = args.tokens
            cfg = config(args.layers, tokens)
        m = Moe(cfg, local)
        biases = fill(m, cfg, biased=args.workload == "prefill")
        sampler = ClockSampler(local)
        rec = measure_long_batch(torch, m, cfg, tokens, args.steps, args.warmup, args.workload, biases, args.skip_parity)
        clocks = sampler.stop()
        line = {"metric": METRIC, "value": rec["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": rec["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": rec["config"], "gpu_launches": rec["gpu_launches"], "clocks": clocks, "roofline": rec["roofline"],
                "roofline_step": rec["roofline_step"], "kernels": rec["kernels"], "parity": rec["parity"], "e2e": None, "cpu_baseline": None}
        print(json.dumps(line), flush=True)
        return

    # ---- default: benchmark configuration 2 (the headline) + the other configurations as sub-records -------------
    extras = world == 1 and not args.skip_extras
    cfg = config(args.layers, max(BATCHES + (args.tokens,) + ((8192,) if extras else ())))
    m = Moe(cfg, local)
    for name, value in EXTRA_OPTIONS:
        m.set_option(name, value)
    fill(m, cfg)

    def inputs(tokens):
        return make_inputs(torch, cfg, tokens, rank)

    # ---- parity gate, outside every timed region: layer 0 against the CPU checker -------------------
    parity = None
    if rank == 0 and not args.skip_parity:
        x_np, _, x_dev = inputs(args.tokens)
        got16 = m.moe(0, x_dev).float().cpu().numpy()
        parity = parity_gate(torch, cfg, args.tokens, x_np, out_bf16=got16)

    # ---- timed region: K graph replays of the chained stack, inputs resident in HBM ------------------
    def measure(tokens, steps, warmup):
        _, host, x_dev = inputs(tokens)
        out_dev = torch.empty((tokens, cfg.hidden), dtype=torch.bfloat16, device="cuda")
        for _ in range(warmup):
            m.stack(x_dev, out_dev)
        before = m.launches
        ms = time_steps(torch, lambda: m.stack(x_dev, out_dev), steps, dist)
        launches = m.launches - before
        active = m.active_counts()
        finite = bool(torch.isfinite(out_dev.float()).all())
        return ms, launches, active, finite, host, x_dev, out_dev

    sampler = ClockSampler(local) if rank == 0 else None
    ms, launches, active, finite, host, x_dev, out_dev = measure(args.tokens, args.steps, args.warmup)
    clocks = sampler.stop() if sampler else None
    if not finite:
        raise RuntimeError("the chained stack produced non-finite values")
    tokens_total = args.tokens * world
    value = tokens_total / (ms * 1e-3)
    step_bytes = float(sum(layer_bytes(cfg, int(a), args.tokens) for a in active))

    # ---- end to end through the host-buffer entry point: pinned host x in, host out back, every step ----
    out_host = torch.empty((args.tokens, cfg.hidden), dtype=torch.bfloat16).pin_memory()
    for _ in range(args.warmup):
        m.stack_host(host, out_host)
    e2e_ms = time_steps(torch, lambda: m.stack_host(host, out_host), args.steps, dist)
    e2e = {"value": tokens_total / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
           "h2d_bytes_per_step": host.numel() * 2, "d2h_bytes_per_step": out_host.numel() * 2,
           "call": "zc_moe_stack_host (pinned host buffers; copies and the wait inside the timed region)"}

    # ---- the same boundary called layer by layer, the way a per-layer binding of Model::moe would call it -----------
    def per_layer_blocking():
        for layer in range(cfg.layers):
            m.moe_host(layer, host, out_host)
            m.status()

    def per_layer_async():
        for layer in range(cfg.layers):
            m.moe_host_async(layer, host, out_host)
        m.status()

    e2e_per_layer = {}
    for name, fn in (("blocking", per_layer_blocking), ("async", per_layer_async)):
        for _ in range(3):
            fn()
        t = time_steps(torch, fn, max(args.steps // 2, 5), dist)
        e2e_per_layer[name] = {"ms_per_step": t, "tokens_per_s": tokens_total / (t * 1e-3)}
    e2e_per_layer["definition"] = ("48 x zc_moe_forward_host (+ zc_moe_status) with pinned host activations in and out of every layer, no inter-layer glue: "
                                   "'blocking' waits after every layer (96 host round trips per step); 'async' = zc_moe_forward_host_async with one wait at the end")
    e2e_per_layer["h2d_bytes_per_step"] = host.numel() * 2 * cfg.layers
    e2e_per_layer["d2h_bytes_per_step"] = out_host.numel() * 2 * cfg.layers

    # ---- per-kernel device times over the same K steps (eager launches bracketed by CUDA events) --------
    kernels = kernel_profile(m, lambda: m.stack_eager(x_dev, out_dev), args.steps)
    dominant = max(kernels, key=lambda k: kernels[k]["share"])
    active_eager = m.active_counts()
    mean_items = float(np.mean(active_eager)) + cfg.has_shared
    proj = {"gate_up": cfg.projection_bytes(0) + cfg.projection_bytes(1), "down": cfg.projection_bytes(2)}
    act_bytes = {"gate_up": args.tokens * cfg.hidden * 2, "down": args.tokens * cfg.hidden * 2}
    kernel_rooflines = {}
    for k in proj:
        if k in kernels:
            alg = mean_items * proj[k] + act_bytes[k]
            gbs = alg / (kernels[k]["avg_us"] * 1e-6) / 1e9
            kernel_rooflines[k] = {"achieved": gbs, "frac": gbs / hbm_peak, "algorithmic_bytes_per_launch": alg, "avg_launch_us": kernels[k]["avg_us"]}
    alg = mean_items * proj[dominant] + act_bytes[dominant] if dominant in proj else step_bytes / cfg.layers
    achieved = alg / (kernels[dominant]["avg_us"] * 1e-6) / 1e9
    roofline = {"bound": "hbm", "kernel": dominant, "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                "traffic": ncu_traffic().get(dominant), "peak_source": peak_source, "algorithmic_bytes_per_launch": alg,
                "avg_launch_us": kernels[dominant]["avg_us"], "other_kernels": {k: v for k, v in kernel_rooflines.items() if k != dominant},
                "definition": "(distinct routed experts of the layer + shared) x projection bytes of this kernel + activation bytes, averaged over the layers"}
    step_achieved = step_bytes / (ms * 1e-3) / 1e9
    roofline_step = {"bound": "hbm", "achieved": step_achieved, "peak": hbm_peak, "unit": "GB/s", "frac": step_achieved / hbm_peak,
                     "algorithmic_bytes_per_step": step_bytes,
                     "definition": "sum over layers of (U + S) x record bytes + router matrix + activations in/out, over the whole step time"}

    # ---- the other decode batch sizes of the configuration (same stack, fewer steps) -------------------
    batches = {}
    if not args.skip_batches:
        for t in BATCHES:
            if t == args.tokens:
                bms, act = ms, active
            else:
                bms, _, act, _, _, _, _ = measure(t, max(args.steps // 2, 5), 3)
            b = float(sum(layer_bytes(cfg, int(a), t) for a in act))
            batches[str(t)] = {"tokens_per_s": t * world / (bms * 1e-3), "ms_per_step": bms, "hbm_gbs": b / (bms * 1e-3) / 1e9,
                               "frac_of_hbm_peak": b / (bms * 1e-3) / 1e9 / hbm_peak, "mean_active_experts": float(np.mean(act))}

    # ---- CPU baseline on this machine's host cores, bounded sample ------------------------------------
    cpu = None
    if rank == 0 and world == 1 and not args.skip_cpu:
        from oracle import oracle
        cache = {}
        cpu_sample(cfg, args.tokens, args.cpu_layers, cache)
        seconds = cpu_sample(cfg, args.tokens, args.cpu_layers, cache)
        per_step = seconds * cfg.layers / args.cpu_layers
        cpu = {"value": args.tokens / per_step, "unit": "tokens/s", "cores": oracle.threads(), "kind": "port",
               "sample": f"layers 0..{args.cpu_layers - 1} of {cfg.layers} chained, {args.tokens} tokens, scaled by {cfg.layers}/{args.cpu_layers}; "
                         f"{seconds:.1f} s of CPU arithmetic"}

    # ---- the other configurations of the specification, as sub-records of the same line ---------------------------
    prefill = mixed = ep = None
    if extras:
        prefill = {}
        biases = {}
        for layer in range(cfg.layers):
            biases[layer] = synth.zipf_router_bias(cfg, SEED, layer)
            m.set_router_bias(layer, biases[layer])
        for t in (2048, 8192):
            prefill[str(t)] = measure_long_batch(torch, m, cfg, t, 3, 3, "prefill", biases, args.skip_parity)
    m.close()
    del m
    if extras:
        tokens4 = int(mixed_lengths().sum())
        cfg4 = config(args.layers, tokens4, down_bits=8, q8_signed=1)
        m4 = Moe(cfg4, local)
        fill(m4, cfg4)
        mixed = measure_long_batch(torch, m4, cfg4, tokens4, 3, 3, "mixed", {}, args.skip_parity)
        mixed["request_lengths"] = [int(v) for v in mixed_lengths()]
        m4.close()
        del m4
    if not args.skip_ep:
        try:
            ep = measure_ep(torch, dist, rank, world, local, args.layers, 256, 10 if world > 1 else 5, 3, args.skip_parity)
        except Exception as exc:      # the headline measured above is still reported; the failure is part of the line
            ep = {"error": f"{type(exc).__name__}: {exc}"[:400]}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload(cfg, args.tokens, world), "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks,
            "roofline": roofline, "roofline_step": roofline_step, "kernels": kernels, "cpu_baseline": cpu, "batches": batches,
            "parity": parity, "mean_active_experts": float(np.mean(active)), "e2e_per_layer": e2e_per_layer,
            "prefill": prefill, "mixed": mixed, "ep": ep,
        }
        if world > 1:
            line["config"]["parallelism"] = (f"value / e2e: dp{world}, independent replicas of configuration 2, tokens sharded, no data-path collective; "
                                             f"the `ep` record of this line is configuration 5 expert-parallel over the same {world} GPUs")
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill", "mixed", "ep"],
                    help="decode: benchmark configuration 2 (the headline) with configurations 3, 4 and 5 as sub-records; "
                         "prefill / mixed / ep: configuration 3 / 4 / 5 alone")
    ap.add_argument("--tokens", type=int, default=0, help="tokens per GPU: decode 1/4/16/64 (default 64), prefill 2048/8192 (default 2048); ep: total (256)")
    ap.add_argument("--layers", type=int, default=48)
    ap.add_argument("--cpu-layers", type=int, default=8, help="layers of the stack the CPU baseline runs (scaled to 48)")
    ap.add_argument("--skip-cpu", action="store_true")
    ap.add_argument("--skip-parity", action="store_true")
    ap.add_argument("--skip-batches", action="store_true")
    ap.add_argument("--skip-extras", action="store_true", help="leave out the prefill and mixed sub-records (one-GPU runs)")
    ap.add_argument("--skip-ep", action="store_true", help="leave out the configuration-5 sub-record")
    ap.add_argument("--opt", action="append", default=[], metavar="NAME=VALUE", help="library option for the long-batch handle (zc_moe_set_option), repeatable")
    ap.add_argument("--small-rows", type=int, default=SMALL_ROWS, help="long batches: experts with at most this many rows take the streaming kernels (0: none)")
    ap.add_argument("--record-routes", default="", help="write the expert selections of one decode pass as a route trace (JSON lines) and exit")
    ap.add_argument("--replay-routes", default="", help="time the decode stack with the expert selections of a recorded route trace forced into every layer")
    args = ap.parse_args()
    globals()["SMALL_ROWS"] = args.small_rows
    for item in args.opt:
        name, _, value = item.partition("=")
        EXTRA_OPTIONS.append((name, int(value)))
    if args.warmup < 3:
        args.warmup = 3
    if not args.tokens:
        args.tokens = {"prefill": 2048, "ep": 256}.get(args.workload, 64)
    if args.impl == "reference":
        args.cpu_layers = min(args.cpu_layers, 2)
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
