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

`--impl reference` times that CPU implementation alone, with all host threads.
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
    # one TinyLlama decoder layer (44 M parameters): the small case used for profiler captures
    "tinyllama_layer_adamw": dict(
        shapes=lambda: llama_shapes(1, 2048, 5632, 256, 32000)[1:-2], grad="bf16", bytes_per_param=14,
        hp=dict(_ADAMW, lr=1e-3, weight_decay=0.01, block_size=2048, m_block_size=256,
                m_quant_type="uf8", v_quant_type="al8")),
    # one 4096x4096 fp32 parameter with fp32 gradients
    "single_4096_adamw": dict(
        shapes=lambda: [("w", (4096, 4096))], grad="f32", bytes_per_param=16,
        hp=dict(_ADAMW, lr=1e-3, weight_decay=0.01, block_size=2048, m_block_size=256,
                m_quant_type="uf8", v_quant_type="al8")),
}
DEFAULT_WORKLOAD = "tinyllama_adamw_fira"


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
def cpu_reference_run(workload, steps, warmup, budget_params=24_000_000):
    """Time the CPU restatement of the reference's step on a bounded sample of
    the workload: its largest tensors are cut to at most `budget_params`
    parameters in total (whole rows), all host threads."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    import af8_oracle as o
    import cases
    wl = WORKLOADS[workload]
    hp = o.hyper(**wl["hp"])
    shapes = wl["shapes"]()
    # sample: one of each distinct shape, in order, until the budget is spent
    seen, sample, total = set(), [], 0
    for name, shp in shapes:
        if shp in seen:
            continue
        seen.add(shp)
        n = int(np.prod(shp))
        if total + n > budget_params and len(shp) == 2:
            rows = max(1, (budget_params - total) // shp[1])
            shp = (min(rows, shp[0]), shp[1])
            n = int(np.prod(shp))
        if n == 0 or total + n > budget_params * 1.05:
            continue
        sample.append(shp)
        total += n
    spec = dict(dist="rowscale", std=1e-3, zero_frac=0.005, dtype="bf16" if wl["grad"] == "bf16" else "f32")
    params = [cases.make_param(s, 100 + i) for i, s in enumerate(sample)]
    states = [o.init_state(s, hp) for s in sample]
    grads = [cases.make_grad(s, 200 + i, 1, spec) for i, s in enumerate(sample)]
    times = []
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        for p, g, st in zip(params, grads, states):
            o.fullrank_step(p.reshape(-1), g.reshape(-1), st, hp)
        dt = time.perf_counter() - t0
        if it >= warmup:
            times.append(dt)
    sec = float(np.mean(times))
    return dict(value=total / sec / 1e9, unit="Gparams/s", cores=o.num_threads(), kind="port",
                sample=f"{len(sample)} tensors of the workload ({total} parameters: one per distinct shape, "
                       f"largest cut to fit), {steps} timed steps after {warmup} warm-up, OpenMP over all host threads",
                ms_per_step=sec * 1e3, sample_params=total)


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    wl = WORKLOADS[args.workload]
    steps = max(1, min(args.steps, 5))
    warm = max(1, min(args.warmup, 2))
    r = cpu_reference_run(args.workload, steps, warm)
    line = {
        "impl": "reference", "metric": "optimizer_step_throughput", "value": r["value"], "unit": "Gparams/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warm, "ms_per_step": r["ms_per_step"],
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "grad_dtype": wl["grad"], "sample_params": r["sample_params"]},
        "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
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
    from adafactor8bit import Adafactor8Bit, _engine

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
    if world > 1:
        # replicas only at this stage: every rank steps the full parameter set
        pass
    gen = torch.Generator(device=device).manual_seed(1234)
    params = []
    for _, shp in shapes:
        p = torch.nn.Parameter(torch.randn(shp, generator=gen, device=device) * 0.02)
        p.grad_dtype = None
        params.append(p)
    n_params = sum(p.numel() for p in params)
    opt = Adafactor8Bit(params, **wl["hp"])
    n_sets = 3
    grad_sets = [make_grad_set(torch, shapes, gdtype, 77 + s, device) for s in range(n_sets)]

    def set_grads(k):
        for p, g in zip(params, grad_sets[k % n_sets]):
            p.grad = g

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
            opt.step()
        ev1.record()
        barrier()
    ms = ev0.elapsed_time(ev1) / args.steps
    log = _engine.LAUNCH_LOG
    _engine.LAUNCH_LOG = None
    if world > 1:
        t = torch.tensor([ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    value = n_params * world / (ms * 1e-3) / 1e9

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
        bpp = wl["bytes_per_param"] if dom.endswith(("apply", "noclip")) else {"bf16": 4, "f32": 6}[wl["grad"]]
        achieved = units * bpp / (tot_ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                    "traffic": None, "kernel": dom, "launches": launches, "avg_launch_ms": tot_ms / launches,
                    "algorithmic_bytes_per_param": bpp, "peak_source": peak_kind,
                    "all_kernels": {k: {"ms_total": v[0], "launches": v[1]} for k, v in per_kernel.items()}}

    # ---- end to end: gradients in pinned host memory ----
    e2e = None
    if not args.no_e2e:
        host_sets = [[g.cpu().pin_memory() for g in grad_sets[0]]]
        dev_grads = [torch.empty_like(g) for g in grad_sets[0]]
        h2d = sum(g.numel() * g.element_size() for g in dev_grads)
        e2e_steps = max(1, min(args.steps, 5))

        def e2e_step():
            for dg, hg, p in zip(dev_grads, host_sets[0], params):
                dg.copy_(hg, non_blocking=True)
                p.grad = dg
            opt.step()
            return opt.update_norms()     # device->host read of the step's result

        e2e_step()
        barrier()
        ev0.record()
        for _ in range(e2e_steps):
            norms = e2e_step()
        ev1.record()
        barrier()
        ems = ev0.elapsed_time(ev1) / e2e_steps
        if world > 1:
            t = torch.tensor([ems], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ems = float(t.item())
        e2e = {"value": n_params * world / (ems * 1e-3) / 1e9, "unit": "Gparams/s", "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": int(norms.nbytes), "ms_per_step": ems, "steps": e2e_steps}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        r = cpu_reference_run(args.workload, 3, 1)
        cpu = {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")}

    if rank == 0:
        line = {
            "metric": "optimizer_step_throughput", "value": value, "unit": "Gparams/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak" if world > 1 else "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": args.workload, "params": n_params, "tensors": len(params),
                       "grad_dtype": wl["grad"], "param_dtype": "f32", "states": "M uf8 block 256, V al8 block 2048",
                       "l2_policy": "inputs larger than L2 (whole parameter set streamed every step)",
                       "parallelism": "replicas" if world > 1 else "single"},
            "hbm_gbs": value * wl["bytes_per_param"], "clocks": clocks.summary(),
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": gpu_launches,
        }
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
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
