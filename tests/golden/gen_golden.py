"""Generate the golden fixtures in this directory by running the REFERENCE
optimizer (its pure-PyTorch path, use_cuda_kernel=False) on the seeded inputs
of cases.py.

Run it where the reference checkout is available:

    python tests/golden/gen_golden.py --reference /path/to/reference [case ...]

With ``--accurate-norm`` the run replaces ``torch.linalg.vector_norm`` (and
``Tensor.norm``) by a version that accumulates in float64 and rounds once, and
writes ``<case>__accnorm.npz`` instead.  The reference's source is untouched;
only the torch routine it calls is swapped.  torch's float32 CPU norm is off by
1e-6 relative at 6e4 elements (5e-3 at 65 M), which is enough to move clip
factors and, through them, an occasional momentum code; the second fixture set
separates that effect from the rest of the arithmetic.

It writes one ``<case>.npz`` per case.  Keys: ``digest`` (sha256 of the inputs),
``t<step>_p<i>_param`` and ``t<step>_p<i>_<state key>`` for every tensor-valued
state entry after that step.  Arrays of 50 000 elements or more are stored only
after steps 1, 2 and the last one; smaller ones after every step.

Cases with ``param_dtype`` "bf16" / "f16" run the reference on parameters of that
dtype (stored in the fixture converted to float32, which is exact).  With
``stochastic_round_writeback`` the reference draws its uniform numbers from a
seeded torch generator, whose stream nothing else can reproduce; for those cases
``torch.rand`` is swapped, during the reference's rounding routine only, for the
counter generator of cases.sr_uniform (the stream of the reference's own CUDA
kernels, kernels.cu:48-65), fed with the seed and step that the reference
passes.  The reference's rounding logic itself (neighbours, probability,
saturation) runs unchanged.
"""
import argparse
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import cases  # noqa: E402

BIG = 50000


def install_accurate_norm():
    import torch
    orig = torch.linalg.vector_norm

    def vector_norm64(x, ord=2, dim=None, keepdim=False, *, dtype=None, out=None):
        if ord != 2 or out is not None:
            return orig(x, ord, dim, keepdim, dtype=dtype)
        r = orig(x.double(), 2, dim, keepdim)
        return r.to(dtype if dtype is not None else x.dtype)

    torch.linalg.vector_norm = vector_norm64

    def tensor_norm(self, p="fro", dim=None, keepdim=False, dtype=None):
        return vector_norm64(self, 2, dim, keepdim, dtype=dtype)

    torch.Tensor.norm = tensor_norm


def install_counter_uniforms():
    """Make the reference's stochastic rounding draw from cases.sr_uniform(seed, step, n)."""
    import torch
    import adafactor8bit.optimizer as ro
    inner = ro._stochastic_round_lowp_pytorch
    real_rand = torch.rand

    def lowp(fp32_tensor, dtype, seed=None, step=None):
        u = torch.from_numpy(cases.sr_uniform(seed, step, fp32_tensor.numel()))
        fn = ro._stochastic_round_bf16_pytorch if dtype == torch.bfloat16 else ro._stochastic_round_fp16_pytorch
        torch.rand = lambda *a, **k: u
        try:
            return fn(fp32_tensor, generator=True)
        finally:
            torch.rand = real_rand

    ro._stochastic_round_lowp_pytorch = lowp
    return inner


def run_case(name, out_dir, suffix=""):
    import torch
    from adafactor8bit import Adafactor8Bit

    c = cases.CASES[name]
    params0, grads = cases.case_inputs(name)
    out = {"digest": np.array(cases.inputs_digest(params0, grads))}
    tdt = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}[c.get("param_dtype", "f32")]
    params = [torch.nn.Parameter(torch.from_numpy(p.copy()).to(tdt)) for p in params0]
    if c["hp"].get("stochastic_round_writeback"):
        install_counter_uniforms()
    for p in params:
        p.grad_dtype = None  # allow bf16 grads on fp32 parameters
    opt = Adafactor8Bit(params, use_cuda_kernel=False, **c["hp"])
    steps = c["steps"]
    for t in range(1, steps + 1):
        for k, v in c.get("changes", {}).get(t, {}).items():     # an option edited between steps
            for group in opt.param_groups:
                group[k] = v
        for p, g in zip(params, grads[t]):
            if g.dtype == np.uint16:
                p.grad = torch.from_numpy(g.view(np.int16).copy()).view(torch.bfloat16).reshape(p.shape)
            else:
                p.grad = torch.from_numpy(g.copy())
        opt.step()
        keep_big = t in (1, 2, steps)
        for i, p in enumerate(params):
            entries = {"param": p.detach().float()}
            for k, v in opt.state[p].items():
                if isinstance(v, torch.Tensor):
                    entries[k] = v
            for k, v in entries.items():
                a = v.detach().cpu().contiguous()
                if a.dtype == torch.int16:
                    a = a.view(torch.uint16) if hasattr(torch, "uint16") else a
                a = a.numpy().reshape(-1) if a.dim() != 0 else a.numpy().reshape(1)
                if a.dtype == np.int16:
                    a = a.view(np.uint16)
                if a.size >= BIG and not keep_big:
                    continue
                if k == "apollo_proj_matrix_T":
                    # keep the matrix only when it changed (refresh steps)
                    prev = out.get(f"_lastP_{i}")
                    if prev is not None and np.array_equal(prev, a):
                        continue
                    out[f"_lastP_{i}"] = a.copy()
                out[f"t{t}_p{i}_{k}"] = a.copy()
    out = {k: v for k, v in out.items() if not k.startswith("_lastP_")}
    path = os.path.join(out_dir, name + suffix + ".npz")
    np.savez_compressed(path, **out)
    print(f"{name}: {len(out)} arrays, {os.path.getsize(path) / 1e6:.2f} MB")


def run_sr_edges(out_dir):
    """Known answers of the reference's two stochastic rounding routines on the values of
    cases.sr_edge_inputs() (zeros, ties, the largest finite numbers, infinities, NaNs, subnormals),
    each with every uniform number of the list."""
    import torch
    import adafactor8bit.optimizer as ro
    x, rnd = cases.sr_edge_inputs()
    real_rand = torch.rand
    out = {"digest": np.array(cases.digest([x, rnd]))}
    torch.rand = lambda *a, **k: torch.from_numpy(rnd.copy())
    try:
        out["bf16"] = ro._stochastic_round_bf16_pytorch(torch.from_numpy(x.copy()), generator=True).view(torch.int16).numpy().view(np.uint16)
        out["f16"] = ro._stochastic_round_fp16_pytorch(torch.from_numpy(x.copy()), generator=True).view(torch.int16).numpy().view(np.uint16)
    finally:
        torch.rand = real_rand
    np.savez_compressed(os.path.join(out_dir, "sr_edges.npz"), **out)
    print("sr_edges:", x.size, "values")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True,
                    help="directory that contains the reference's adafactor8bit package")
    ap.add_argument("--accurate-norm", action="store_true")
    ap.add_argument("cases", nargs="*")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    import torch
    torch.manual_seed(0)
    names = args.cases or (list(cases.CASES) + ["sr_edges"])
    if args.accurate_norm:
        install_accurate_norm()
    for name in names:
        if name == "sr_edges":
            run_sr_edges(HERE)
            continue
        run_case(name, HERE, "__accnorm" if args.accurate_norm else "")


if __name__ == "__main__":
    main()
