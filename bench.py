"""Benchmark of the fused optimizer step over quantised states.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl b200|reference]

Prints ONE JSON line.  A "step" is one optimizer step over the whole synthetic
parameter set of the workload.  Metric: Gparams/s (parameters updated per second,
whole job).  `value` is measured with gradients already resident in HBM; `e2e`
goes through the same public API with the gradients in pinned host memory, the
host->device copy and a device->host read of the step's update norms inside the
timed region.  `roofline` describes the dominant kernel against the measured HBM
copy bandwidth; `cpu_baseline` is the CPU restatement of the reference's step
timed on this machine's host cores on a bounded sample.

`--impl reference` times the reference's own CPU path alone, with all host threads: the unmodified
reference package (its pure-PyTorch step, use_cuda_kernel=False) when an offline install of it is
present under baseline/_ref, else the C restatement under oracle/.

With N > 1 ranks the step is sharded ZeRO-1 style over the flat parameter space; the parameters
that travel are a bf16 compute copy written by the update kernels, the fp32 masters stay sharded.
"""
import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "adafactor-8bit_b200"))

import numpy as np  # noqa: E402


# ---------------------------------------------------------------------------
# workloads: parameter shapes of the named models, synthetic gradients
# ---------------------------------------------------------------------------
def llama_shapes(layers, hidden, mlp, kv_dim, vocab):
    shapes = [("embed", (vocab, hidden))]
    for _ in range(layers):
        shapes += [("q", (hidden, hidden)), ("k", (kv_dim, hidden)), ("v", (kv_dim, hidden)),
                   ("o", (hidden, hidden)), ("gate", (mlp, hidden)), ("up", (mlp, hidden)),
                   ("down", (hidden, mlp)), ("norm1", (hidden,)), ("norm2", (hidden,))]
    shapes += [("final_norm", (hidden,)), ("lm_head", (vocab, hidden))]
    return shapes


_ADAMW = dict(beta1=0.9, beta2=0.999, beta2_decay=None, beta3=None, factored=False,
              relative_step=False, scale_parameter=False, scale_weight_decay=False,
              d=0.0, eps=(1e-8, 1e-3))

WORKLOADS = {
    # AdamW UF8/AL8 (V block 2048) + Fira limiter on the TinyLlama-1.1B parameter set,
    # fp32 parameters, bf16 heavy-tailed gradients
    "tinyllama_adamw_fira": dict(
        shapes=lambda: llama_shapes(22, 2048, 5632, 256, 32000), grad="bf16", bytes_per_param=14,
        hp=dict(_ADAMW, lr=1e-3, weight_decay=0.01, block_size=2048, m_block_size=256,
                m_quant_type="uf8", v_quant_type="al8", enable_fira_for_adafactor=True, fira_margin=0.01)),
    # the same without the limiter: a single fused pass
    "tinyllama_adamw": dict(
        shapes=lambda: llama_shapes(22, 2048, 5632, 256, 32000), grad="bf16", bytes_per_param=14,
        hp=dict(_ADAMW, lr=1e-3, weight_decay=0.01, block_size=2048, m_block_size=256,
                m_quant_type="uf8", v_quant_type="al8")),
    # factored Adafactor, constructor defaults (relative step, parameter scaling, clip d=1),
    # AL8 second moment in blocks of 256, no momentum: TinyLlama-1.1B
    "tinyllama_adafactor": dict(
        shapes=lambda: llama_shapes(22, 2048, 5632, 256, 32000), grad="bf16", bytes_per_param=10,
        hp=dict(block_size=256)),
    # CAME: UF8 momentum, AL16 second moment and confidence (block 2048): Llama-2-7B shapes
    "llama2_7b_came": dict(
        shapes=lambda: llama_shapes(32, 4096, 11008, 4096, 32000), grad="bf16", bytes_per_param=12,
        hp=dict(beta1=0.9, beta2=0.999, beta2_decay=None, beta3=0.9999, factored=True, relative_step=False,
                scale_parameter=False, scale_weight_decay=False, d=1.0, eps_came=1e-16, lr=1e-4,
                m_quant_type="uf8", v_quant_type="al16", c_quant_type="al16", block_size=2048)),
    # one Llama-2-7B layer with CAME (202 M parameters): the small case for profiler captures
    "llama2_layer_came": dict(
        shapes=lambda: llama_shapes(1, 4096, 11008, 4096, 32000)[1:-2], grad="bf16", bytes_per_param=12,
        hp=dict(beta1=0.9, beta2=0.999, beta2_decay=None, beta3=0.9999, factored=True, relative_step=False,
                scale_parameter=False, scale_weight_decay=False, d=1.0, eps_came=1e-16, lr=1e-4,
                m_quant_type="uf8", v_quant_type="al16", c_quant_type="al16", block_size=2048)),
    # APOLLO rank 256 on the attention / MLP matrices, AdamW-style fallback elsewhere: Llama-3-8B shapes
    "llama3_8b_apollo": dict(
        shapes=lambda: llama_shapes(32, 4096, 14336, 1024, 128256), grad="bf16", bytes_per_param=10,
        apollo_targets=("q", "k", "v", "o", "gate", "up", "down"),
        hp=dict(_ADAMW, eps=(1e-6, 1e-3), lr=1e-3, weight_decay=0.01, block_size=2048, m_block_size=256,
                m_quant_type="uf8", v_quant_type="al8", apollo_rank=256, apollo_update_proj_gap=200,
                apollo_eps=1e-6, apollo_cache_proj=True, enable_fira_for_apollo=True)),
    # the same optimizer on one Llama-3-8B layer (small case for tests and profiler captures)
    "llama3_layer_apollo": dict(
        shapes=lambda: llama_shapes(1, 4096, 14336, 1024, 128256)[1:-2], grad="bf16", bytes_per_param=10,
        apollo_targets=("q", "k", "v", "o", "gate", "up", "down"),
        hp=dict(_ADAMW, eps=(1e-6, 1e-3), lr=1e-3, weight_decay=0.01, block_size=2048, m_block_size=256,
                m_quant_type="uf8", v_quant_type="al8", apollo_rank=256, apollo_update_proj_gap=200,
                apollo_eps=1e-6, apollo_cache_proj=True, enable_fira_for_apollo=True)),
    # one TinyLlama decoder layer (44 M parameters): the small case used for profiler captures
    "tinyllama_layer_adamw": dict(
        shapes=lambda: llama_shapes(1, 2048, 5632, 256, 32000)[1:-2], grad="bf16", bytes_per_param=14,
        hp=dict(_ADAMW, lr=1e-3, weight_decay=0.01, block_size=2048, m_block_size=256,
                m_quant_type="uf8", v_quant_type="al8")),
    # four TinyLlama decoder layers with the limiter (176 M parameters, 1.4 GB on the device):
    # the small case for profiler captures of the two-pass configuration
    "tinyllama_4layers_adamw_fira": dict(
        shapes=lambda: llama_shapes(4, 2048, 5632, 256, 32000)[1:-2], grad="bf16", bytes_per_param=14,
        hp=dict(_ADAMW, lr=1e-3, weight_decay=0.01, block_size=2048, m_block_size=256,
                m_quant_type="uf8", v_quant_type="al8", enable_fira_for_adafactor=True, fira_margin=0.01)),
    # the headline optimizer on bf16 parameters (10 B/param), rounded to nearest or stochastically
    "tinyllama_adamw_fira_bf16p": dict(
        shapes=lambda: llama_shapes(22, 2048, 5632, 256, 32000), grad="bf16", param="bf16", bytes_per_param=10,
        hp=dict(_ADAMW, lr=1e-3, weight_decay=0.01, block_size=2048, m_block_size=256,
                m_quant_type="uf8", v_quant_type="al8", enable_fira_for_adafactor=True, fira_margin=0.01)),
    "tinyllama_adamw_fira_bf16p_sr": dict(
        shapes=lambda: llama_shapes(22, 2048, 5632, 256, 32000), grad="bf16", param="bf16", bytes_per_param=10,
        hp=dict(_ADAMW, lr=1e-3, weight_decay=0.01, block_size=2048, m_block_size=256,
                m_quant_type="uf8", v_quant_type="al8", enable_fira_for_adafactor=True, fira_margin=0.01,
                stochastic_round_writeback=True)),
    # the headline optimizer with lag_norm=True: the limiter uses the previous step's norm, one pass
    "tinyllama_adamw_fira_lag": dict(
        shapes=lambda: llama_shapes(22, 2048, 5632, 256, 32000), grad="bf16", bytes_per_param=14,
        hp=dict(_ADAMW, lr=1e-3, weight_decay=0.01, block_size=2048, m_block_size=256,
                m_quant_type="uf8", v_quant_type="al8", enable_fira_for_adafactor=True, fira_margin=0.01, lag_norm=True)),
    # small cases (four layers) of the bf16-parameter and lag_norm variants for profiler captures
    "tinyllama_4layers_adamw_fira_bf16p_sr": dict(
        shapes=lambda: llama_shapes(4, 2048, 5632, 256, 32000)[1:-2], grad="bf16", param="bf16", bytes_per_param=10,
        hp=dict(_ADAMW, lr=1e-3, weight_decay=0.01, block_size=2048, m_block_size=256,
                m_quant_type="uf8", v_quant_type="al8", enable_fira_for_adafactor=True, fira_margin=0.01,
                stochastic_round_writeback=True)),
    "tinyllama_4layers_adamw_fira_bf16p": dict(
        shapes=lambda: llama_shapes(4, 2048, 5632, 256, 32000)[1:-2], grad="bf16", param="bf16", bytes_per_param=10,
        hp=dict(_ADAMW, lr=1e-3, weight_decay=0.01, block_size=2048, m_block_size=256,
                m_quant_type="uf8", v_quant_type="al8", enable_fira_for_adafactor=True, fira_margin=0.01)),
    "tinyllama_4layers_adamw_fira_lag": dict(
        shapes=lambda: llama_shapes(4, 2048, 5632, 256, 32000)[1:-2], grad="bf16", bytes_per_param=14,
        hp=dict(_ADAMW, lr=1e-3, weight_decay=0.01, block_size=2048, m_block_size=256,
                m_quant_type="uf8", v_quant_type="al8", enable_fira_for_adafactor=True, fira_margin=0.01, lag_norm=True)),
    # four TinyLlama decoder layers with factored Adafactor (constructor defaults): small case for profiler captures
    "tinyllama_4layers_adafactor": dict(
        shapes=lambda: llama_shapes(4, 2048, 5632, 256, 32000)[1:-2], grad="bf16", bytes_per_param=10,
        hp=dict(block_size=256)),
    # one 4096x4096 fp32 parameter with fp32 gradients
    "single_4096_adamw": dict(
        shapes=lambda: [("w", (4096, 4096))], grad="f32", bytes_per_param=16,
        hp=dict(_ADAMW, lr=1e-3, weight_decay=0.01, block_size=2048, m_block_size=256,
                m_quant_type="uf8", v_quant_type="al8")),
}
DEFAULT_WORKLOAD = "tinyllama_adamw_fira"

# dram__bytes_read.sum + dram__bytes_write.sum per parameter from the committed profiler summaries,
# (kernel, gradient dtype) -> (bytes per parameter, summary file).  A constant taken from a capture of
# the same kernel on a small case, not a measurement of this run.
NCU_TRAFFIC_BPP = {
    ("fullrank_fast_apply", "bf16"): (13.72, "profiles/fullrank_fast_apply_tinyllama_4layers.txt"),
    ("fullrank_stat", "bf16"): (4.12, "profiles/fullrank_stat_tinyllama_4layers.txt"),
    # the factored write pass: without momentum (Adafactor, 10 B/param) and with a UF8 momentum (CAME, 12 B/param)
    ("factored_apply", "bf16", 10): (9.68, "profiles/factored_update_nomomentum_tinyllama_4layers.txt"),
    ("factored_apply", "bf16", 12): (11.82, "profiles/factored_kernels_llama2_layer_came.txt"),
}


def make_groups(wl, named_params):
    """Parameter groups of a workload: APOLLO workloads route the target matrices to the
    low-rank path and everything else to the AdamW-style fallback (what the reference's
    build_param_groups(preset="apollo") produces); the others use one group."""
    targets = wl.get("apollo_targets")
    if not targets:
        return [dict(params=[p for _, p in named_params])]
    main = [p for n, p in named_params if n in targets]
    rest = [p for n, p in named_params if n not in targets]
    groups = [dict(params=main)]
    if rest:
        groups.append(dict(params=rest, apollo_rank=0))
    return groups


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# ---------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.samples = []
        self.stop = threading.Event()
        self.thread = None

    def _run(self):
        while not self.stop.is_set():
            try:
                out = subprocess.run(
                    ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-i", str(self.index)],
                    capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.samples.append([x.strip() for x in out.split(",")])
            except Exception:
                pass
            self.stop.wait(0.1)

    def __enter__(self):
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()
        return self

    def __exit__(self, *a):
        self.stop.set()
        self.thread.join(timeout=6)

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for s in self.samples:
            try:
                sm.append(float(s[0])); mx.append(float(s[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons),
                "samples": len(sm)}


# ---------------------------------------------------------------------------
# CPU implementation of the reference step (the oracle), bounded sample
# ---------------------------------------------------------------------------
def cpu_reference_run(workload, steps, warmup, sample_limit=24_000_000):
    """Time the CPU restatement of the reference's step on a bounded sample of
    the workload: its largest tensors are cut to at most `sample_limit`
    parameters in total (whole rows), all host threads."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    import af8_oracle as o
    import cases
    # all host threads this process may use (a multi-process launcher sets OMP_NUM_THREADS=1 for its ranks)
    try:
        o.set_num_threads(len(os.sched_getaffinity(0)))
    except AttributeError:
        o.set_num_threads(os.cpu_count() or 1)
    wl = WORKLOADS[workload]
    hp = o.hyper(**wl["hp"], param_dtype=wl.get("param", "f32"))
    sample, sample_names, total = sample_of(workload, sample_limit)
    spec = dict(dist="rowscale", std=1e-3, zero_frac=0.005, dtype="bf16" if wl["grad"] == "bf16" else "f32")
    params = [cases.make_param(s, 100 + i, dtype=wl.get("param", "f32")) for i, s in enumerate(sample)]
    targets = wl.get("apollo_targets")
    hps = [hp if (not targets or nm in targets) else dict(hp, apollo_rank=0) for nm in sample_names]
    states = [o.init_state(s, h) for s, h in zip(sample, hps)]
    for k, st in enumerate(states):
        if "apollo_seed" in st:
            st["apollo_seed"] = k + 1
        if hp["stochastic_round_writeback"] and hp["param_dtype"] != "f32":
            st["sr_seed"] = k + 1
    grads = [cases.make_grad(s, 200 + i, 1, spec) for i, s in enumerate(sample)]

    def one(p, g, st, h):
        if h["apollo_rank"] > 0 and p.ndim == 2:
            o.apollo_step(p, g, st, h)
        elif p.ndim == 2 and h["factored"]:
            o.factored_step(p, g, st, h)
        else:
            o.fullrank_step(p.reshape(-1), g.reshape(-1), st, h)

    times = []
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        for p, g, st, h in zip(params, grads, states, hps):
            one(p, g, st, h)
        dt = time.perf_counter() - t0
        if it >= warmup:
            times.append(dt)
    sec = float(np.mean(times))
    return dict(value=total / sec / 1e9, unit="Gparams/s", cores=o.num_threads(), kind="port",
                sample=f"{len(sample)} tensors of the workload ({total} parameters: one per distinct shape, "
                       f"largest cut to fit), {steps} timed steps after {warmup} warm-up, OpenMP over all host threads",
                ms_per_step=sec * 1e3, sample_params=total)


def reference_package_dir():
    path = os.path.join(ROOT, "baseline", "_ref")
    return path if os.path.exists(os.path.join(path, "adafactor8bit", "optimizer.py")) else None


def sample_of(workload, sample_limit=24_000_000):
    """The bounded sample both CPU legs step: one tensor of each distinct shape of the workload, in
    order, the one that would pass the limit cut to whole rows."""
    wl = WORKLOADS[workload]
    if wl.get("apollo_targets"):
        sample_limit = min(sample_limit, 6_000_000)      # the CPU projection costs 2*rank flops per parameter
    seen, sample, names, total = set(), [], [], 0
    for name, shp in wl["shapes"]():
        if shp in seen:
            continue
        seen.add(shp)
        n = int(np.prod(shp))
        if total + n > sample_limit and len(shp) == 2:
            rows = max(1, (sample_limit - total) // shp[1])
            shp = (min(rows, shp[0]), shp[1])
            n = int(np.prod(shp))
        if n == 0 or total + n > sample_limit * 1.05:
            continue
        sample.append(shp)
        names.append(name)
        total += n
    return sample, names, total


def reference_package_run(workload, steps, warmup):
    """Time the UNMODIFIED reference package (baseline/_ref, its pure-PyTorch CPU path through its own
    optimizer class) on the bounded sample, all host threads.  Must run in a process that has not
    imported this repository's package of the same name."""
    import torch
    sys.path[:] = [p for p in sys.path if not p.endswith("adafactor-8bit_b200")]
    sys.path.insert(0, reference_package_dir())
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    import adafactor8bit as ref
    assert os.path.realpath(ref.__file__).startswith(os.path.realpath(reference_package_dir()))
    import cases
    try:
        torch.set_num_threads(len(os.sched_getaffinity(0)))
    except AttributeError:
        torch.set_num_threads(os.cpu_count() or 1)
    wl = WORKLOADS[workload]
    sample, names, total = sample_of(workload)
    spec = dict(dist="rowscale", std=1e-3, zero_frac=0.005, dtype="bf16" if wl["grad"] == "bf16" else "f32")
    pdt = torch.bfloat16 if wl.get("param") == "bf16" else torch.float32
    params = []
    for i, s in enumerate(sample):
        p = torch.nn.Parameter(torch.from_numpy(cases.make_param(s, 100 + i, dtype=wl.get("param", "f32"))).to(pdt))
        p.grad_dtype = None                               # a bf16 gradient on an fp32 parameter
        params.append(p)
    grads = []
    for i, s in enumerate(sample):
        g = cases.make_grad(s, 200 + i, 1, spec)
        grads.append(torch.from_numpy(g.view(np.int16).copy()).view(torch.bfloat16).reshape(s) if g.dtype == np.uint16
                     else torch.from_numpy(g))
    targets = wl.get("apollo_targets")
    if targets:
        groups = [dict(params=[p for p, n in zip(params, names) if n in targets])]
        rest = [p for p, n in zip(params, names) if n not in targets]
        if rest:
            groups.append(dict(params=rest, apollo_rank=0))
        groups = [g for g in groups if g["params"]]
    else:
        groups = [dict(params=params)]
    opt = ref.Adafactor8Bit(groups, use_cuda_kernel=False, **wl["hp"])
    times = []
    for it in range(warmup + steps):
        for p, g in zip(params, grads):
            p.grad = g
        t0 = time.perf_counter()
        opt.step()
        dt = time.perf_counter() - t0
        if it >= warmup:
            times.append(dt)
    sec = float(np.mean(times))
    return dict(value=total / sec / 1e9, unit="Gparams/s", cores=torch.get_num_threads(), kind="reference",
                sample=f"the unmodified reference package, pure-PyTorch CPU path (use_cuda_kernel=False), on {len(sample)} tensors "
                       f"of the workload ({total} parameters: one per distinct shape, largest cut to fit), {steps} timed steps "
                       f"after {warmup} warm-up, {torch.get_num_threads()} torch threads",
                ms_per_step=sec * 1e3, sample_params=total)


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    wl = WORKLOADS[args.workload]
    port = cpu_reference_run(args.workload, max(1, min(args.steps, 50)), max(1, min(args.warmup, 5)))
    if reference_package_dir() is not None:
        steps = max(1, min(args.steps, 8))       # about 1 s per step on the sample
        warm = max(1, min(args.warmup, 2))
        r = reference_package_run(args.workload, steps, warm)
    else:
        steps, warm, r = max(1, min(args.steps, 50)), max(1, min(args.warmup, 5)), port
    cpu = {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")}
    cpu["port_value"] = port["value"]              # the C + OpenMP restatement (oracle/) on the same sample
    cpu["port_cores"] = port["cores"]
    line = {
        "impl": "reference", "metric": "optimizer_step_throughput", "value": r["value"], "unit": "Gparams/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warm, "ms_per_step": r["ms_per_step"],
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "grad_dtype": wl["grad"], "sample_params": r["sample_params"]},
        "cpu_baseline": cpu,
        "e2e": {"value": r["value"], "unit": "Gparams/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------
def make_grad_set(torch, shapes, dtype, seed, device):
    """Heavy-tailed synthetic gradients: N(0, 1e-3) * exp(N(0,1)) per row, 0.5 % exact zeros."""
    gen = torch.Generator(device=device).manual_seed(seed)
    out = []
    for _, shp in shapes:
        g = torch.randn(shp, generator=gen, device=device) * 1e-3
        rows = torch.randn(shp[:-1] + (1,) if len(shp) > 1 else (1,), generator=gen, device=device)
        g = g * torch.exp(rows)
        g = torch.where(torch.rand(shp, generator=gen, device=device) < 0.005, torch.zeros_like(g), g)
        out.append(g.to(dtype).contiguous())
    return out


def run_gpu_arm(args):
    import torch
    import torch.distributed as dist
    from adafactor8bit import Adafactor8Bit, ShardedAdafactor8Bit, _engine

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    wl = WORKLOADS[args.workload]
    shapes = wl["shapes"]()
    gdtype = torch.bfloat16 if wl["grad"] == "bf16" else torch.float32
    pdtype = torch.bfloat16 if wl.get("param") == "bf16" else torch.float32
    gen = torch.Generator(device=device).manual_seed(1234)
    named = []
    for name, shp in shapes:
        p = torch.nn.Parameter((torch.randn(shp, generator=gen, device=device) * 0.02).to(pdtype))
        p.grad_dtype = None
        named.append((name, p))
    params = [p for _, p in named]
    n_params = sum(p.numel() for p in params)
    groups = make_groups(wl, named)
    copy_dtype = None
    if world > 1:
        # ZeRO-1 over the flat parameter space: each rank updates its cells, then the in-place
        # all-gather of the parameters (strong scaling: the job is fixed).  fp32 parameters travel as
        # a bf16 compute copy written by the update kernels; the fp32 masters stay with their owner.
        copy_dtype = torch.bfloat16 if (pdtype == torch.float32 and not args.fp32_gather) else None
        opt = ShardedAdafactor8Bit(groups, compute_dtype=copy_dtype, **wl["hp"])
        # the sharded optimizer numbers the tensors group by group: follow its order from here on
        shape_of = {id(p): entry for (_, p), entry in zip(named, shapes)}
        params = list(opt.all_params)
        shapes = [shape_of[id(p)] for p in params]
        owned = sorted({i for (i, lo, hi, k, pc) in opt._local})      # tensors of which this rank updates a piece
    else:
        opt = Adafactor8Bit(groups, **wl["hp"])
        owned = list(range(len(params)))
    inner = opt.inner if world > 1 else opt
    # synthetic gradients only for the tensors this rank updates
    n_sets = 3
    own_shapes = [shapes[i] for i in owned]
    grad_sets = [make_grad_set(torch, own_shapes, gdtype, 77 + s_, device) for s_ in range(n_sets)]

    def set_grads(k):
        for i, g in zip(owned, grad_sets[k % n_sets]):
            params[i].grad = g

    gathered_bytes = 0
    if world > 1:
        gathered_bytes = opt.flat.numel() * opt.flat.element_size() * (world - 1) // world    # received per rank and step

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- warm-up ----
    for k in range(args.warmup):
        set_grads(k)
        opt.step()
    barrier()

    # ---- timed region: inputs resident in HBM ----
    _engine.LAUNCH_LOG = []
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        barrier()
        ev0.record()
        for k in range(args.steps):
            set_grads(k)
            opt.step()           # N > 1: local update with the parameter all-gather pipelined behind it
        ev1.record()
        barrier()
    ms = ev0.elapsed_time(ev1) / args.steps
    log = _engine.LAUNCH_LOG
    _engine.LAUNCH_LOG = None
    gather_ms = update_ms = 0.0
    if world > 1:
        # the two phases on their own, outside the timed region: update without communication,
        # and the all-gather of unchanged parameters
        for phase in ("update", "gather"):
            barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for k in range(3):
                if phase == "update":
                    set_grads(k)
                    opt.local_step()
                else:
                    opt.gather()
            b.record()
            barrier()
            if phase == "update":
                update_ms = a.elapsed_time(b) / 3
            else:
                gather_ms = a.elapsed_time(b) / 3
        # the all-gather of the same layout in fp32 (what a run without the compute copy moves), for comparison
        gather32_ms = 0.0
        if copy_dtype is not None:
            free_b, _ = torch.cuda.mem_get_info()
            if opt.flat.numel() * 4 < free_b // 2:
                tmp = torch.empty(opt.flat.numel(), dtype=torch.float32, device=device)
                unit = world * opt.cell
                barrier()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                for rep in range(4):
                    if rep == 1:
                        a.record()
                    for k in range(opt.parts):
                        u = tmp[k * unit:(k + 1) * unit]
                        dist.all_gather_into_tensor(u, u[opt.rank * opt.cell:(opt.rank + 1) * opt.cell])
                b.record()
                barrier()
                gather32_ms = a.elapsed_time(b) / 3
                del tmp
        t = torch.tensor([ms, gather_ms, update_ms, gather32_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, gather_ms, update_ms, gather32_ms = (float(x) for x in t.tolist())
    value = n_params / (ms * 1e-3) / 1e9

    # ---- per-kernel durations inside the timed region (events on the launch stream) ----
    per_kernel = {}
    for name, units, e0, e1 in log:
        d = per_kernel.setdefault(name, [0.0, 0, 0])
        d[0] += e0.elapsed_time(e1); d[1] += 1; d[2] += units
    gpu_launches = sum(v[1] for v in per_kernel.values())
    peak, peak_kind = load_peaks()
    roofline = None
    if per_kernel:
        dom = max(per_kernel, key=lambda k: per_kernel[k][0])
        tot_ms, launches, units = per_kernel[dom]
        gb = {"bf16": 2, "f32": 4}[wl["grad"]]
        pb2 = 2 * {"bf16": 2, "f32": 4}[wl.get("param", "f32")]     # parameter read + write
        if dom.startswith("fullrank") and dom.endswith(("apply", "noclip", "lag")):
            bpp = gb + pb2 + 4                    # grad + param r/w + M and V codes r/w
        elif dom.startswith("fullrank"):
            bpp = gb + 2                          # statistic pass (fullrank_stat, *_sumsq): grad + both codes
        elif dom == "factored_apply":
            bpp = gb + pb2 + (2 if inner.param_groups[0].get("beta1") is not None else 0)
        elif dom.startswith("factored"):
            bpp = gb                              # statistic passes read the gradient
        elif dom == "apollo_project":
            bpp = gb
        else:
            bpp = gb + 8
        if copy_dtype is not None and dom.endswith(("apply", "noclip", "lag", "scales_apply")):
            bpp += 2                              # the bf16 compute copy written next to the fp32 master
        achieved = units * bpp / (tot_ms * 1e-3) / 1e9
        # DRAM bytes per parameter (read + write) of this kernel: a constant from the committed profiler
        # capture on the four-layer case; every block is independent, so traffic scales with the
        # parameter count.  No entry for the kernel: traffic is null and the note says so.
        entry = None
        if wl.get("param", "f32") == "f32" and copy_dtype is None:
            entry = NCU_TRAFFIC_BPP.get((dom, wl["grad"])) or NCU_TRAFFIC_BPP.get((dom, wl["grad"], bpp))
        traffic = None if entry is None else entry[0] * units / launches
        traffic_note = ("no profiler capture of this kernel and configuration is committed" if entry is None else
                        f"bytes per launch = {entry[0]} B/param from {entry[1]} x parameters of the launch "
                        f"(a constant from that capture, not measured in this run)")
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                    "frac_of_8tbs": achieved / 8000.0,
                    "traffic": traffic, "traffic_unit": traffic_note,
                    "kernel": dom, "launches": launches, "avg_launch_ms": tot_ms / launches,
                    "algorithmic_bytes_per_param": bpp, "peak_source": peak_kind,
                    "all_kernels": {k: {"ms_total": v[0], "launches": v[1]} for k, v in per_kernel.items()}}
        if dom == "apollo_project":
            # the projection is a contraction: 2 * rank flops per parameter as specified, three times that
            # issued (the projection matrix enters as three bf16 planes), against the measured bf16 GEMM rate
            rank_ = int(wl["hp"].get("apollo_rank", 0))
            peak_tf = 1648.3
            try:
                with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                    peak_tf = float(json.load(f)["bf16_tflops"])
            except Exception:
                peak_kind = "fallback"
                peak_tf = 1590.0
            tf = units * 2.0 * rank_ / (tot_ms * 1e-3) / 1e12
            roofline.update({"bound": "tensor", "unit": "TFLOP/s", "peak": peak_tf, "achieved": 3.0 * tf,
                             "frac": 3.0 * tf / peak_tf, "frac_of_8tbs": None, "achieved_as_specified": tf,
                             "flops_note": "achieved = issued bf16 MMA flops (3 planes x 2*rank per parameter); "
                                           "achieved_as_specified = 2*rank per parameter; the launch also transposes "
                                           "left-case gradients and sums channel norms",
                             "traffic": None, "peak_source": peak_kind})

    # ---- end to end: gradients in pinned host memory ----
    e2e = None
    if not args.no_e2e:
        host = [g.cpu().pin_memory() for g in grad_sets[0]]
        dev_grads = [torch.empty_like(g) for g in grad_sets[0]]
        h2d = sum(g.numel() * g.element_size() for g in dev_grads)
        e2e_steps = max(1, min(args.steps, 5))

        def e2e_step():
            for i, dg, hg in zip(owned, dev_grads, host):
                dg.copy_(hg, non_blocking=True)
                params[i].grad = dg
            opt.step()
            return inner.update_norms() if inner is not None else np.zeros(0, np.float32)   # device->host read

        e2e_step()
        barrier()
        ev0.record()
        for _ in range(e2e_steps):
            norms = e2e_step()
        ev1.record()
        barrier()
        ems = ev0.elapsed_time(ev1) / e2e_steps
        tot = torch.tensor([float(h2d), float(norms.nbytes)], device=device, dtype=torch.float64)
        if world > 1:
            t = torch.tensor([ems], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ems = float(t.item())
            dist.all_reduce(tot)
        e2e = {"value": n_params / (ems * 1e-3) / 1e9, "unit": "Gparams/s", "h2d_bytes_per_step": int(tot[0].item()),
               "d2h_bytes_per_step": int(tot[1].item()), "ms_per_step": ems, "steps": e2e_steps}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        # the reference arm in a process of its own (the reference package has the name of this repository's)
        res = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "reference", "--workload", args.workload,
                              "--steps", "3", "--warmup", "1"], capture_output=True, text=True, timeout=900)
        for ln in reversed(res.stdout.strip().splitlines()):
            if ln.startswith("{"):
                cpu = json.loads(ln)["cpu_baseline"]
                break
        if cpu is None:
            raise RuntimeError("the CPU baseline run printed no result:\n" + res.stderr[-2000:])

    if rank == 0:
        line = {
            "metric": "optimizer_step_throughput", "value": value, "unit": "Gparams/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": args.workload, "params": n_params, "tensors": len(params),
                       "grad_dtype": wl["grad"], "param_dtype": wl.get("param", "f32"),
                       "l2_policy": "inputs larger than L2 (whole parameter set streamed every step)",
                       "parallelism": (f"zero1 x{world}: flat block-aligned parameter space in {opt.parts} x {world} cells, "
                                       + ("bf16 compute-copy all-gather, fp32 masters sharded" if copy_dtype is not None
                                          else f"in-place {str(pdtype).replace('torch.', '')} parameter all-gather")
                                       + f", gather of a part overlaps the update of the next") if world > 1 else "single"},
            "hbm_gbs": value * wl["bytes_per_param"], "clocks": clocks.summary(),
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": gpu_launches,
        }
        if world > 1:
            line["allgather_ms_per_step"] = gather_ms          # measured alone; in `value` it overlaps the update
            line["update_ms_per_step"] = update_ms
            line["update_only_value"] = n_params / (max(update_ms, 1e-6) * 1e-3) / 1e9
            line["allgather_bytes_received_per_rank"] = gathered_bytes
            line["allgather_gbs_per_rank"] = gathered_bytes / (max(gather_ms, 1e-6) * 1e-3) / 1e9
            line["allgather_fp32_ms_per_step"] = gather32_ms or None   # the same layout in fp32, measured alone
            line["limiter"] = "parameter all-gather" if gather_ms > update_ms else "update kernels"
            line["cut_tensors"] = sum(len(x) > 1 for x in opt.pieces_of)
            line["exchange_rounds"] = opt.rounds
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--fp32-gather", action="store_true", help="N > 1: gather the fp32 parameters themselves (no bf16 compute copy)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
