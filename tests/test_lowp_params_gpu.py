"""bf16 / fp16 parameters on the CUDA path: nearest rounding after the decay and after the update,
or one stochastic rounding fed by the counter generator (optimizer.py:162-292, 866-881, 2032-2040).
Compared with the CPU oracle step by step and with the fixtures that the reference produced."""
import numpy as np
import pytest
import torch

import cases
import parity
from oracle_runner import OracleRun, golden_entries, load_golden
from test_fullrank_gpu import state_np

pytestmark = pytest.mark.gpu

TORCH_DT = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}
PARAM_FRAC = 1e-4          # share of parameters that may sit on the neighbouring number of the format
CODE_KEYS = ("variance_q", "m_q", "row_var_q", "col_var_q", "conf_row_q", "conf_col_q")


def cuda_grad(g, shape):
    if g.dtype == np.uint16:
        return torch.from_numpy(g.view(np.int16).copy()).view(torch.bfloat16).reshape(shape).cuda()
    return torch.from_numpy(g.copy()).reshape(shape).cuda()


def make(run):
    from adafactor8bit import Adafactor8Bit
    dt = TORCH_DT[run.case["param_dtype"]]
    params = [torch.nn.Parameter(torch.from_numpy(p.copy()).to(dt).cuda()) for p in run.params0]
    for p in params:
        p.grad_dtype = None
    return params, Adafactor8Bit(params, **run.case["hp"])


def check_codes(name, t, i, st_gpu, ref, al16_frac=None):
    for key in CODE_KEYS:
        if key not in ref or key not in st_gpu:
            continue
        b = np.asarray(ref[key]).reshape(-1)
        a = state_np(st_gpu, key)
        al16 = b.dtype == np.uint16
        what = f"{name} t{t} p{i} {key}"
        if al16 and al16_frac is not None:
            s = parity.code_stats(a, b)
            assert s["zero_mismatch"] == 0 and s["max"] <= parity.CODE_SLACK_AL16 and s["neq"] <= max(2, al16_frac * s["n"]), (what, s)
        else:
            parity.assert_codes(a, b, what, al16=al16, zero_reserved=(key != "m_q"))


@pytest.mark.parametrize("name", cases.LOWP_FULLRANK_CASES)
def test_fullrank_low_precision_params(name, oracle):
    run = OracleRun(name)
    fmt = run.case["param_dtype"]
    gold = load_golden(name)
    assert str(gold["digest"]) == cases.inputs_digest(run.params0, run.grads)
    params, opt = make(run)
    steps = run.case["steps"]
    for t in range(1, steps + 1):
        for p, g in zip(params, run.grads[t]):
            p.grad = cuda_grad(g, p.shape)
        opt.step()
        run.step()
        torch.cuda.synchronize()
        for i, p in enumerate(params):
            assert p.dtype == TORCH_DT[fmt]
            got = p.detach().float().cpu().numpy()
            parity.assert_lowp_params(got, run.params[i], fmt, f"{name} t{t} p{i} param", frac=PARAM_FRAC)
            check_codes(name, t, i, opt.state[p], run.states[i])
            if run.hp["stochastic_round_writeback"]:
                assert opt.state[p]["sr_seed"] == i + 1
    for i, p in enumerate(params):     # and against what the reference itself produced
        ref = golden_entries(gold, steps, i)
        parity.assert_lowp_params(p.detach().float().cpu().numpy(), ref["param"], fmt, f"{name} final p{i} vs reference", frac=PARAM_FRAC)
        check_codes(name, steps, i, opt.state[p], ref)


def test_stochastic_rounding_is_unbiased_and_seeded():
    """Statistics of the rounding on a large tensor: the mean of (stored - exact) / unit is zero to
    sampling error, every stored value is one of the two neighbours, and the stream depends on the
    step and on the parameter's seed only."""
    from adafactor8bit import Adafactor8Bit
    n = 1 << 20
    hp = dict(cases.CASES["adamw_sr_bf16p"]["hp"], enable_fira_for_adafactor=False, weight_decay=0.0)
    rng = np.random.default_rng(3)
    p0 = torch.from_numpy((rng.standard_normal(n) * 0.02).astype(np.float32)).to(torch.bfloat16)
    g = torch.from_numpy((rng.standard_normal(n) * 1e-3).astype(np.float32)).to(torch.bfloat16).cuda()
    outs = []
    for rep in range(2):
        p = torch.nn.Parameter(p0.clone().cuda())
        q = torch.nn.Parameter(p0.clone().cuda())          # a second parameter: another seed
        opt = Adafactor8Bit([p, q], **hp)
        p.grad, q.grad = g.clone(), g.clone()
        opt.step()
        torch.cuda.synchronize()
        outs.append((p.detach().clone(), q.detach().clone()))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    assert not torch.equal(outs[0][0], outs[0][1])
    # exact value of the first step: m = 0.1 g, v = 0.001 g^2, bias-corrected: p - lr * g / (|g| + eps')
    pf = p0.float().cuda()
    gf = g.float()
    exact = pf - 1e-3 * gf / (gf.abs() + 1e-8)
    lo = (exact.view(torch.int32) & -65536).view(torch.float32)
    unit = torch.ldexp(torch.ones_like(lo), torch.frexp(lo.abs())[1] - 8)     # spacing of bf16 at lo
    got = outs[0][0].float()
    keep = exact.abs() > 1e-4       # where p and the update nearly cancel, this float32 estimate of the exact value is noise
    dev = ((got - exact) / unit)[keep].cpu().numpy().astype(np.float64)
    n = dev.size
    assert np.abs(dev).max() <= 1.0 + 1e-3
    assert abs(dev.mean()) < 5.0 / np.sqrt(12.0 * n) + 1e-3
    nearest = exact.to(torch.bfloat16)
    assert (outs[0][0] != nearest).float().mean().item() > 0.1      # it is not round-to-nearest


@pytest.mark.parametrize("name", cases.LOWP_FACTORED_CASES)
def test_factored_low_precision_params(name, oracle):
    """Factored Adafactor (bf16 parameters, parameter-scaled relative step) and CAME with stochastic
    rounding, step by step from the oracle's state (AL16 small states move by a code when a mean
    differs in its last bit, so the comparison restarts from identical state every step)."""
    run = OracleRun(name)
    fmt = run.case["param_dtype"]
    params, opt = make(run)
    dt = TORCH_DT[fmt]
    for t in range(1, run.case["steps"] + 1):
        for p, g in zip(params, run.grads[t]):
            p.grad = cuda_grad(g, p.shape)
        if t > 1:
            for i, p in enumerate(params):
                st = opt.state[p]
                p.data.copy_(torch.from_numpy(run.params[i]).reshape(p.shape).to(dt))
                for key, val in run.states[i].items():
                    if isinstance(val, np.ndarray) and key in st and isinstance(st[key], torch.Tensor):
                        src = torch.from_numpy(val.view(np.int16) if val.dtype == np.uint16 else val)
                        st[key].copy_(src.reshape(st[key].shape))
        opt.step()
        run.step()
        torch.cuda.synchronize()
        for i, p in enumerate(params):
            got = p.detach().float().cpu().numpy()
            parity.assert_lowp_params(got, run.params[i], fmt, f"{name} t{t} p{i} param", frac=2e-4)
            check_codes(name, t, i, opt.state[p], run.states[i], al16_frac=3e-2)
            if run.hp["stochastic_round_writeback"]:
                assert opt.state[p]["sr_seed"] == i + 1
    gold = load_golden(name)
    steps = run.case["steps"]
    for i, p in enumerate(params):
        ref = golden_entries(gold, steps, i)
        if "param" in ref:
            parity.assert_lowp_params(p.detach().float().cpu().numpy(), ref["param"], fmt, f"{name} final p{i} vs reference", frac=1e-3)


@pytest.mark.parametrize("name", ["apollo_bf16p", "apollo_sr_bf16p"])
def test_apollo_low_precision_params(name, oracle):
    """APOLLO on bf16 parameters with exact projections (the states then agree with the oracle, see
    test_apollo_gpu.py): parameters equal except for the usual share on a neighbouring bf16 number."""
    from adafactor8bit import _engine, optimizer as opt_mod
    run = OracleRun(name)
    opt_mod.APOLLO_RNG_DEVICE = "cpu"
    saved = _engine.EXACT_PROJECTION
    _engine.EXACT_PROJECTION = True
    try:
        params, opt = make(run)
        for t in range(1, run.case["steps"] + 1):
            for p, g in zip(params, run.grads[t]):
                p.grad = cuda_grad(g, p.shape)
            opt.step()
            run.step()
            torch.cuda.synchronize()
            for i, p in enumerate(params):
                assert p.dtype == torch.bfloat16
                parity.assert_lowp_params(p.detach().float().cpu().numpy(), run.params[i], "bf16", f"{name} t{t} p{i} param", frac=2e-4)
                if "m_low_q" in run.states[i]:
                    parity.assert_codes(state_np(opt.state[p], "m_low_q"), run.states[i]["m_low_q"], f"{name} t{t} p{i} m_low_q", zero_reserved=False)
                    parity.assert_codes(state_np(opt.state[p], "v_low_q"), run.states[i]["v_low_q"], f"{name} t{t} p{i} v_low_q")
        gold = load_golden(name)
        steps = run.case["steps"]
        for i, p in enumerate(params):
            ref = golden_entries(gold, steps, i)
            got = p.detach().float().cpu().numpy()
            s = parity.lowp_stats(got, ref["param"], "bf16")
            assert s["neq"] <= 2e-3 * s["n"] and parity.rel_l2(got, ref["param"]) <= 5e-4, (name, i, s)
    finally:
        opt_mod.APOLLO_RNG_DEVICE = None
        _engine.EXACT_PROJECTION = saved
