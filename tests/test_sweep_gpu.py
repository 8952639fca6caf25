"""A seeded sweep over the option space of the full-rank path (state formats, block sizes, update rules,
parameter and gradient dtypes, limiter and clip) against the CPU oracle: combinations that no fixture names."""
import numpy as np
import pytest
import torch

import cases
import parity
from oracle_runner import OracleRun
from test_fullrank_gpu import state_np

pytestmark = pytest.mark.gpu

TORCH_DT = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}


def _configs(n, seed=2024):
    rng = np.random.default_rng(seed)
    out = []
    for k in range(n):
        block = int(rng.choice([128, 256, 512, 1024, 2048]))
        m_block = int(rng.choice([b for b in (32, 64, 128, 256) if block % b == 0]))
        rule = str(rng.choice(["adam", "rmsprop", "momentum_only", "adafactor_unfactored"]))
        hp = dict(block_size=block, m_block_size=m_block, min_8bit_size=int(rng.choice([1, 4096])),
                  v_quant_type=str(rng.choice(["al8", "al16", "fp32"])), lr=float(rng.choice([1e-3, 1e-2])),
                  weight_decay=float(rng.choice([0.0, 0.01])), factored=False,
                  enable_fira_for_adafactor=bool(rng.integers(0, 2)), maximize=bool(rng.integers(0, 4) == 0))
        if rule == "adam":
            hp.update(beta1=0.9, beta2=0.999, beta2_decay=None, relative_step=False, scale_parameter=False,
                      scale_weight_decay=False, d=float(rng.choice([0.0, 1.0])), eps=(1e-8, 1e-3),
                      m_quant_type=str(rng.choice(["uf8", "uf4", "d8", "d4", "fp32"])))
        elif rule == "rmsprop":
            hp.update(beta1=None, beta2=0.99, beta2_decay=None, relative_step=False, scale_parameter=False,
                      scale_weight_decay=False, d=float(rng.choice([0.0, 1.0])), eps=(1e-8, 1e-3))
        elif rule == "momentum_only":       # Adafactor-style second moment with momentum: the momentum-only rule
            hp.update(beta1=0.9, relative_step=False, scale_parameter=bool(rng.integers(0, 2)), d=1.0,
                      m_quant_type=str(rng.choice(["uf8", "uf4", "d8"])))
        pd = str(rng.choice(["f32", "f32", "bf16", "f16"]))
        gd = {"f32": str(rng.choice(["f32", "bf16"])), "bf16": "bf16", "f16": "f16"}[pd]
        if pd != "f32":
            hp["stochastic_round_writeback"] = bool(rng.integers(0, 2))
        shapes = [tuple(int(x) for x in rng.integers(1, 90, size=int(rng.integers(1, 3)))) for _ in range(3)] + [(int(rng.integers(4096, 9000)),)]
        grad = dict(dist="rowscale", std=1e-3, zero_frac=float(rng.choice([0.0, 0.01])), dtype=gd)
        out.append(dict(shapes=shapes, steps=3, seed=500 + k, grad=grad, hp=hp, param_dtype=pd))
    return out


CONFIGS = _configs(24)


@pytest.mark.parametrize("k", range(len(CONFIGS)))
def test_fullrank_option_sweep(k, oracle):
    from adafactor8bit import Adafactor8Bit, _engine
    case = CONFIGS[k]
    if case["hp"].get("m_quant_type") in ("d8", "d4"):
        for bits in (8, 4):
            oracle.set_dynamic_map(bits, _engine.dynamic_map(bits))
    run = OracleRun(f"sweep{k}", case=case)
    fmt = case["param_dtype"]
    params = [torch.nn.Parameter(torch.from_numpy(p.copy()).to(TORCH_DT[fmt]).cuda()) for p in run.params0]
    for p in params:
        p.grad_dtype = None
    opt = Adafactor8Bit(params, **case["hp"])
    for t in range(1, case["steps"] + 1):
        for p, g in zip(params, run.grads[t]):
            if g.dtype == np.uint16:
                p.grad = torch.from_numpy(g.view(np.int16).copy()).view(torch.bfloat16).reshape(p.shape).cuda()
            else:
                p.grad = torch.from_numpy(g.copy()).reshape(p.shape).cuda()
        opt.step()
        run.step()
        torch.cuda.synchronize()
        for i, p in enumerate(params):
            what = f"sweep {k} {case['hp']} t{t} p{i}"
            st, so = opt.state[p], run.states[i]
            got = p.detach().float().cpu().numpy()
            if fmt == "f32":
                parity.assert_params(got, run.params[i], what, tol=2e-6)
            else:
                parity.assert_lowp_params(got, run.params[i], fmt, what, frac=2e-4)
            for key in ("variance_q", "m_q"):
                if key in so:
                    a, b = state_np(st, key), np.asarray(so[key]).reshape(-1)
                    if key == "m_q" and so.get("m_quant_type") in ("uf4", "d4"):
                        a, b = parity.unpack_nibbles(a), parity.unpack_nibbles(b)
                    parity.assert_codes(a, b, what + " " + key, al16=(b.dtype == np.uint16), zero_reserved=(key != "m_q"))
            for key in ("variance", "m"):
                if key in so:
                    assert parity.rel_l2(state_np(st, key), so[key]) <= 1e-6, what + " " + key


def _factored_configs(n, seed=4048):
    rng = np.random.default_rng(seed)
    out = []
    for k in range(n):
        rule = str(rng.choice(["adafactor", "adafactor_m", "came"]))
        block = int(rng.choice([128, 256, 1024, 2048]))
        hp = dict(block_size=block, m_block_size=int(rng.choice([64, 128, 256])), min_8bit_size=int(rng.choice([1, 4096])),
                  v_quant_type=str(rng.choice(["al8", "al16", "fp32"])), weight_decay=float(rng.choice([0.0, 0.01])),
                  enable_fira_for_adafactor=bool(rng.integers(0, 2)), maximize=bool(rng.integers(0, 4) == 0))
        if rule == "adafactor":
            hp.update(lag_norm=bool(rng.integers(0, 2)), d=float(rng.choice([0.0, 1.0])))
        elif rule == "adafactor_m":
            hp.update(beta1=0.9, relative_step=False, lr=1e-3, m_quant_type=str(rng.choice(["uf8", "uf4", "d8", "fp32"])),
                      lag_norm=bool(rng.integers(0, 2)))
        else:
            hp.update(beta1=0.9, beta2=0.999, beta2_decay=None, beta3=0.9999, relative_step=False, scale_parameter=False,
                      scale_weight_decay=False, d=float(rng.choice([0.0, 1.0])), eps_came=1e-16, lr=1e-4,
                      m_quant_type=str(rng.choice(["uf8", "uf4", "fp32"])), c_quant_type=str(rng.choice(["al8", "al16"])))
        pd = str(rng.choice(["f32", "f32", "bf16"]))
        gd = "bf16" if pd == "bf16" else str(rng.choice(["f32", "bf16"]))
        if pd != "f32":
            hp["stochastic_round_writeback"] = bool(rng.integers(0, 2))
        shapes = []
        for _ in range(3):
            cols = int(rng.integers(1, 40)) * 8 if rng.integers(0, 3) else int(rng.integers(3, 300))
            shapes.append((int(rng.integers(1, 200)), cols))
        shapes.append((int(rng.integers(2, 40)), int(rng.choice([256, 512, 2048, 2304]))))
        grad = dict(dist="rowscale", std=1e-3, zero_frac=float(rng.choice([0.0, 0.01])), dtype=gd)
        out.append(dict(shapes=shapes, steps=3, seed=700 + k, grad=grad, hp=hp, param_dtype=pd))
    return out


FACTORED_CONFIGS = _factored_configs(16)
SMALL_CODE_KEYS = ("row_var_q", "col_var_q", "conf_row_q", "conf_col_q", "m_q")


@pytest.mark.parametrize("k", range(len(FACTORED_CONFIGS)))
def test_factored_option_sweep(k, oracle):
    """The same for the factored path; every step starts from the oracle's state (AL16 small states move by a
    code when a mean differs in its last bit, which would otherwise accumulate over the steps)."""
    from adafactor8bit import Adafactor8Bit, _engine
    case = FACTORED_CONFIGS[k]
    if case["hp"].get("m_quant_type") in ("d8", "d4"):
        for bits in (8, 4):
            oracle.set_dynamic_map(bits, _engine.dynamic_map(bits))
    run = OracleRun(f"fsweep{k}", case=case)
    fmt = case["param_dtype"]
    dt = TORCH_DT[fmt]
    params = [torch.nn.Parameter(torch.from_numpy(p.copy()).to(dt).cuda()) for p in run.params0]
    for p in params:
        p.grad_dtype = None
    opt = Adafactor8Bit(params, **case["hp"])
    for t in range(1, case["steps"] + 1):
        for p, g in zip(params, run.grads[t]):
            if g.dtype == np.uint16:
                p.grad = torch.from_numpy(g.view(np.int16).copy()).view(torch.bfloat16).reshape(p.shape).cuda()
            else:
                p.grad = torch.from_numpy(g.copy()).reshape(p.shape).cuda()
        if t > 1:
            for i, p in enumerate(params):
                st = opt.state[p]
                p.data.copy_(torch.from_numpy(run.params[i]).reshape(p.shape).to(dt))
                for key, val in run.states[i].items():
                    if isinstance(val, np.ndarray) and key in st and isinstance(st[key], torch.Tensor):
                        src = torch.from_numpy(val.view(np.int16) if val.dtype == np.uint16 else val)
                        st[key].copy_(src.reshape(st[key].shape))
                for key in ("fira_prev_norm", "prev_update_norm", "lag_fira_scale"):
                    if key in run.states[i] and key in st:
                        st[key].fill_(float(run.states[i][key]))
        opt.step()
        run.step()
        torch.cuda.synchronize()
        for i, p in enumerate(params):
            what = f"factored sweep {k} {case['hp']} {tuple(p.shape)} t{t}"
            st, so = opt.state[p], run.states[i]
            got = p.detach().float().cpu().numpy()
            if fmt == "f32":
                parity.assert_params(got, run.params[i], what, tol=2e-6)
            else:
                parity.assert_lowp_params(got, run.params[i], fmt, what, frac=3e-4)
            for key in SMALL_CODE_KEYS:
                if key in so:
                    a, b = state_np(st, key), np.asarray(so[key]).reshape(-1)
                    if key == "m_q" and so.get("m_quant_type") in ("uf4", "d4"):
                        a, b = parity.unpack_nibbles(a), parity.unpack_nibbles(b)
                    s = parity.code_stats(a, b)
                    al16 = b.dtype == np.uint16
                    assert (key == "m_q" or s["zero_mismatch"] == 0) and s["max"] <= (parity.CODE_SLACK_AL16 if al16 else 1), (what, key, s)
                    assert s["neq"] <= max(2, (3e-2 if al16 else 1e-4) * s["n"]), (what, key, s)


def _apollo_configs(n, seed=777):
    rng = np.random.default_rng(seed)
    out = []
    for k in range(n):
        rank = int(rng.choice([4, 8, 16, 24, 32]))
        hp = dict(cases._APOLLO, lr=1e-3, weight_decay=float(rng.choice([0.0, 0.01])), apollo_rank=rank,
                  apollo_update_proj_gap=int(rng.choice([1, 2, 5])), m_quant_type=str(rng.choice(["uf8", "uf4", "d8"])),
                  v_quant_type=str(rng.choice(["al8", "al16"])), block_size=int(rng.choice([256, 2048])),
                  apollo_scale_type=str(rng.choice(["channel", "tensor"])), apollo_scale=float(rng.choice([1.0, 128.0])),
                  apollo_scale_front=bool(rng.integers(0, 2)), enable_fira_for_apollo=bool(rng.integers(0, 2)),
                  d=float(rng.choice([0.0, 1.0])), maximize=bool(rng.integers(0, 4) == 0), min_8bit_size=1)
        pd = str(rng.choice(["f32", "f32", "bf16"]))
        if pd != "f32":
            hp["stochastic_round_writeback"] = bool(rng.integers(0, 2))
        shapes = [(int(rng.integers(rank, 160)), int(rng.integers(rank // 8 + 1, 30)) * 8),      # rows or cols may be the larger one
                  (int(rng.integers(rank, 80)), int(rng.integers(rank, 200))),
                  (int(rng.integers(100, 3000)),)]
        grad = dict(dist="normal", std=1e-3, zero_frac=0.0, dtype="bf16")
        out.append(dict(shapes=shapes, steps=4, seed=900 + k, grad=grad, hp=hp, param_dtype=pd))
    return out


APOLLO_CONFIGS = _apollo_configs(10)


@pytest.mark.parametrize("k", range(len(APOLLO_CONFIGS)))
def test_apollo_option_sweep(k, oracle):
    """APOLLO with exact projections (so that the low-rank states are comparable code by code)."""
    from adafactor8bit import Adafactor8Bit, _engine, optimizer as opt_mod
    case = APOLLO_CONFIGS[k]
    if case["hp"].get("m_quant_type") in ("d8", "d4"):
        for bits in (8, 4):
            oracle.set_dynamic_map(bits, _engine.dynamic_map(bits))
    run = OracleRun(f"asweep{k}", case=case)
    fmt = case["param_dtype"]
    opt_mod.APOLLO_RNG_DEVICE = "cpu"
    saved = _engine.EXACT_PROJECTION
    _engine.EXACT_PROJECTION = True
    try:
        params = [torch.nn.Parameter(torch.from_numpy(p.copy()).to(TORCH_DT[fmt]).cuda()) for p in run.params0]
        for p in params:
            p.grad_dtype = None
        opt = Adafactor8Bit(params, **case["hp"])
        for t in range(1, case["steps"] + 1):
            for p, g in zip(params, run.grads[t]):
                p.grad = torch.from_numpy(g.view(np.int16).copy()).view(torch.bfloat16).reshape(p.shape).cuda()
            opt.step()
            run.step()
            torch.cuda.synchronize()
            for i, p in enumerate(params):
                what = f"apollo sweep {k} {case['hp']} {tuple(p.shape)} t{t}"
                got = p.detach().float().cpu().numpy()
                if fmt == "f32":
                    parity.assert_params(got, run.params[i], what, tol=2e-6)
                else:
                    parity.assert_lowp_params(got, run.params[i], fmt, what, frac=3e-4)
                st, so = opt.state[p], run.states[i]
                if "m_low_q" in so:
                    a, b = state_np(st, "m_low_q"), np.asarray(so["m_low_q"]).reshape(-1)
                    if so.get("m_quant_type") in ("uf4", "d4"):
                        a, b = parity.unpack_nibbles(a), parity.unpack_nibbles(b)
                    parity.assert_codes(a, b, what + " m_low_q", zero_reserved=False)
                    b = np.asarray(so["v_low_q"]).reshape(-1)
                    parity.assert_codes(state_np(st, "v_low_q"), b, what + " v_low_q", al16=(b.dtype == np.uint16))
    finally:
        opt_mod.APOLLO_RNG_DEVICE = None
        _engine.EXACT_PROJECTION = saved


def _fast_configs(n, seed=31337):
    """The AdamW UF8/AL8 layout of the specialised kernels (V block 2048, M block 256), everything else varied."""
    rng = np.random.default_rng(seed)
    out = []
    for k in range(n):
        beta1 = float(rng.choice([0.9, 0.9, 0.3, 0.95]))             # 0.3: EMA weight 0.7, the second lerp form
        beta2 = float(rng.choice([0.999, 0.99, 0.4]))
        hp = dict(cases._ADAMW, beta1=beta1, beta2=beta2, lr=float(rng.choice([1e-3, 3e-4])),
                  weight_decay=float(rng.choice([0.0, 0.01, 0.1])), block_size=2048, m_block_size=256,
                  m_quant_type="uf8", v_quant_type="al8", min_8bit_size=int(rng.choice([1, 4096])),
                  d=float(rng.choice([0.0, 0.0, 1.0])), enable_fira_for_adafactor=bool(rng.integers(0, 2)),
                  lag_norm=bool(rng.integers(0, 3) == 0), maximize=bool(rng.integers(0, 2)),
                  eps=(float(rng.choice([1e-8, 1e-6, 1e-12])), 1e-3),
                  bias_correction=None if rng.integers(0, 3) else False,
                  scale_weight_decay=bool(rng.integers(0, 2)))
        pd = str(rng.choice(["f32", "f32", "bf16"]))
        gd = "bf16" if pd == "bf16" else str(rng.choice(["f32", "bf16"]))
        if pd != "f32":
            hp["stochastic_round_writeback"] = bool(rng.integers(0, 2))
        shapes = [(int(rng.integers(1, 40)), int(rng.integers(1, 700))), (int(rng.integers(4096, 20000)),),
                  (2048 * int(rng.integers(1, 4)),), (int(rng.integers(1, 300)),)]
        grad = dict(dist="rowscale", std=float(rng.choice([1e-3, 1e-5, 1.0])), zero_frac=float(rng.choice([0.0, 0.01, 0.3])), dtype=gd)
        if rng.integers(0, 2):
            grad.update(spike_step=2, spike_mult=100.0)
        out.append(dict(shapes=shapes, steps=4, seed=1300 + k, grad=grad, hp=hp, param_dtype=pd))
    return out


FAST_CONFIGS = _fast_configs(32)


@pytest.mark.parametrize("k", range(len(FAST_CONFIGS)))
def test_fast_kernel_option_sweep(k, oracle):
    from adafactor8bit import Adafactor8Bit
    case = FAST_CONFIGS[k]
    run = OracleRun(f"fast{k}", case=case)
    fmt = case["param_dtype"]
    params = [torch.nn.Parameter(torch.from_numpy(p.copy()).to(TORCH_DT[fmt]).cuda()) for p in run.params0]
    for p in params:
        p.grad_dtype = None
    opt = Adafactor8Bit(params, **case["hp"])
    for t in range(1, case["steps"] + 1):
        for p, g in zip(params, run.grads[t]):
            if g.dtype == np.uint16:
                p.grad = torch.from_numpy(g.view(np.int16).copy()).view(torch.bfloat16).reshape(p.shape).cuda()
            else:
                p.grad = torch.from_numpy(g.copy()).reshape(p.shape).cuda()
        opt.step()
        run.step()
        torch.cuda.synchronize()
        for i, p in enumerate(params):
            what = f"fast sweep {k} {case['hp']} {case['grad']} {tuple(p.shape)} t{t}"
            st, so = opt.state[p], run.states[i]
            got = p.detach().float().cpu().numpy()
            if fmt == "f32":
                parity.assert_params(got, run.params[i], what, tol=2e-6)
            else:
                parity.assert_lowp_params(got, run.params[i], fmt, what, frac=2e-4)
            for key in ("variance_q", "m_q"):
                if key in so:
                    parity.assert_codes(state_np(st, key), np.asarray(so[key]).reshape(-1), what + " " + key, zero_reserved=(key != "m_q"))
            for key in ("variance_scale", "variance_min_log", "m_scale"):
                if key in so:
                    parity.assert_ranges(state_np(st, key), so[key], what + " " + key, max_ulp=4)
            for key in ("fira_prev_norm", "prev_update_norm"):
                if key in so:
                    a, b = float(st[key].item()), float(so[key])
                    assert abs(a - b) <= 3e-6 * max(abs(b), 1e-30), (what, key, a, b)


def _migration_configs(n, seed=99):
    """Random sequences of option edits between steps on a group with a matrix and a vector."""
    rng = np.random.default_rng(seed)
    edits = [("quantize", [True, False]), ("m_quant_type", ["uf8", "uf4", "d8", "fp32"]), ("v_quant_type", ["al8", "al16"]),
             ("block_size", [256, 2048]), ("factored", [True, False]), ("beta3", [None, 0.9999]), ("beta1", [None, 0.9]),
             ("min_8bit_size", [1, 4096]), ("weight_decay", [0.0, 0.01])]
    out = []
    for k in range(n):
        hp = dict(beta1=0.9, beta2=0.999, beta2_decay=None, beta3=None if rng.integers(0, 2) else 0.9999,
                  factored=bool(rng.integers(0, 2)), relative_step=False, scale_parameter=False, scale_weight_decay=False,
                  d=1.0, eps=(1e-8, 1e-3), eps_came=1e-16, lr=1e-3, weight_decay=0.01, block_size=256, m_block_size=256,
                  m_quant_type="uf8", v_quant_type="al8", min_8bit_size=4096)
        if hp["beta3"] is not None:
            hp["factored"] = True                          # the constructor refuses CAME without factoring
        changes, now = {}, dict(hp)
        for t in (2, 3, 4, 5):
            if rng.integers(0, 4):
                name, vals = edits[int(rng.integers(0, len(edits)))]
                val = vals[int(rng.integers(0, len(vals)))]
                trial = dict(now, **{name: val})
                if trial["beta3"] is not None and (not trial["factored"] or trial["beta1"] is None):
                    continue                               # keep the edited options a combination the reference accepts
                now = trial
                changes.setdefault(t, {})[name] = val
        shapes = [(int(rng.integers(20, 90)), int(rng.integers(8, 40)) * 8), (int(rng.integers(4096, 6000)),), (300,)]
        out.append(dict(shapes=shapes, steps=5, seed=1700 + k, grad=dict(dist="rowscale", std=1e-3, zero_frac=0.01, dtype="bf16"),
                        hp=hp, changes=changes))
    return out


MIGRATION_CONFIGS = _migration_configs(12)


@pytest.mark.parametrize("k", range(len(MIGRATION_CONFIGS)))
def test_migration_sweep(k, oracle):
    from adafactor8bit import Adafactor8Bit, _engine
    case = MIGRATION_CONFIGS[k]
    for bits in (8, 4):
        oracle.set_dynamic_map(bits, _engine.dynamic_map(bits))
    run = OracleRun(f"mig{k}", case=case)
    params = [torch.nn.Parameter(torch.from_numpy(p.copy()).cuda()) for p in run.params0]
    for p in params:
        p.grad_dtype = None
    opt = Adafactor8Bit(params, **case["hp"])
    for t in range(1, case["steps"] + 1):
        for name, v in case["changes"].get(t, {}).items():
            for group in opt.param_groups:
                group[name] = v
        for p, g in zip(params, run.grads[t]):
            p.grad = torch.from_numpy(g.view(np.int16).copy()).view(torch.bfloat16).reshape(p.shape).cuda()
        opt.step()
        run.step()
        torch.cuda.synchronize()
        for i, p in enumerate(params):
            what = f"migration sweep {k} changes {case['changes']} {tuple(p.shape)} t{t}"
            st, so = opt.state[p], run.states[i]
            skip = ("fira_prev_norm", "prev_update_norm", "lag_fira_scale")
            mine = {key for key, v in st.items() if isinstance(v, torch.Tensor) and key not in skip}
            theirs = {key for key, v in so.items() if isinstance(v, np.ndarray)}
            assert mine == theirs, (what, sorted(mine ^ theirs))
            assert st["step"] == so["step"], what
            parity.assert_params(p.detach().cpu().numpy(), run.params[i], what, tol=5e-6)
            for key in theirs:
                a, b = state_np(st, key), np.asarray(so[key]).reshape(-1)
                if key.endswith("_q"):
                    if key == "m_q" and so.get("m_quant_type") in ("uf4", "d4"):
                        a, b = parity.unpack_nibbles(a), parity.unpack_nibbles(b)
                    s = parity.code_stats(a, b)
                    al16 = b.dtype == np.uint16
                    assert (key == "m_q" or s["zero_mismatch"] == 0) and s["max"] <= (parity.CODE_SLACK_AL16 if al16 else 1), (what, key, s)
                    assert s["neq"] <= max(2, (3e-2 if al16 else 1e-4) * s["n"]), (what, key, s)


CHECKPOINT_CASES = ([("fast", k) for k in range(0, 32, 4)] + [("factored", k) for k in range(0, 16, 3)]
                    + [("apollo", k) for k in range(0, 10, 3)] + [("fullrank", k) for k in range(0, 24, 5)])


@pytest.mark.parametrize("family,k", CHECKPOINT_CASES)
def test_checkpoint_continuity_sweep(family, k):
    """Two steps, state_dict, a fresh optimizer on copies of the parameters, load_state_dict, one more step on
    both: the continued run equals the uninterrupted one bit for bit (every state entry a step needs - limiter and
    lag scalars, rounding seeds, projection seeds and matrices, step counts - travels through the checkpoint)."""
    import copy
    from adafactor8bit import Adafactor8Bit
    case = {"fast": FAST_CONFIGS, "factored": FACTORED_CONFIGS, "apollo": APOLLO_CONFIGS, "fullrank": CONFIGS}[family][k]
    params0, grads = cases.case_inputs(case)
    dt = TORCH_DT[case.get("param_dtype", "f32")]

    def grad_of(g, p):
        if g.dtype == np.uint16:
            return torch.from_numpy(g.view(np.int16).copy()).view(torch.bfloat16).reshape(p.shape).cuda()
        return torch.from_numpy(g.copy()).reshape(p.shape).cuda()

    a = [torch.nn.Parameter(torch.from_numpy(p.copy()).to(dt).cuda()) for p in params0]
    for p in a:
        p.grad_dtype = None
    oa = Adafactor8Bit(a, **case["hp"])
    for t in (1, 2):
        for p, g in zip(a, grads[t]):
            p.grad = grad_of(g, p)
        oa.step()
    sd = copy.deepcopy(oa.state_dict())
    b = [torch.nn.Parameter(p.detach().clone()) for p in a]
    for p in b:
        p.grad_dtype = None
    ob = Adafactor8Bit(b, **case["hp"])
    ob.load_state_dict(sd)
    for opt, ps in ((oa, a), (ob, b)):
        for p, g in zip(ps, grads[3]):
            p.grad = grad_of(g, p)
        opt.step()
    torch.cuda.synchronize()
    for i, (p, q) in enumerate(zip(a, b)):
        assert torch.equal(p.detach(), q.detach()), f"{family} {k} {case['hp']} param {i} {tuple(p.shape)}"
        sa, sb = oa.state[p], ob.state[q]
        assert sorted(sa) == sorted(sb), (family, k, i, sorted(set(sa) ^ set(sb)))
        for key, v in sa.items():
            if isinstance(v, torch.Tensor):
                assert torch.equal(v, sb[key]), (family, k, i, key)
            elif key not in ("variance_shape", "row_var_shape", "col_var_shape", "conf_row_shape", "conf_col_shape", "v_low_shape"):
                assert v == sb[key], (family, k, i, key, v, sb[key])


@pytest.mark.parametrize("family", ["fast", "factored"])
def test_parameters_without_gradient_are_skipped(family, oracle):
    """Parameters whose .grad is None at a step keep their state and step count (optimizer.py:1637): the launch
    plan is rebuilt for the tensors that do have gradients, and their per-tensor step numbers drift apart."""
    from adafactor8bit import Adafactor8Bit
    plain = next(c for c in FACTORED_CONFIGS if not c["hp"].get("stochastic_round_writeback") and not c["hp"].get("lag_norm"))
    case = dict(FAST_CONFIGS[0] if family == "fast" else plain, steps=5)
    case = dict(case, grad=dict(case["grad"]), hp=dict(case["hp"]))
    run = OracleRun(f"skip_{family}", case=case)
    dt = TORCH_DT[case.get("param_dtype", "f32")]
    params = [torch.nn.Parameter(torch.from_numpy(p.copy()).to(dt).cuda()) for p in run.params0]
    for p in params:
        p.grad_dtype = None
    opt = Adafactor8Bit(params, **case["hp"])
    n = len(params)
    active = {1: range(n), 2: [0, 2], 3: [1], 4: range(n), 5: [n - 1]}
    for t in range(1, 6):
        for i, p in enumerate(params):
            p.grad = None
        for i in active[t]:
            g = run.grads[t][i]
            p = params[i]
            p.grad = (torch.from_numpy(g.view(np.int16).copy()).view(torch.bfloat16) if g.dtype == np.uint16
                      else torch.from_numpy(g.copy())).reshape(p.shape).cuda()
            run.step_param(i, run.params[i], g, run.states[i])
        opt.step()
        torch.cuda.synchronize()
        for i, p in enumerate(params):
            what = f"{family} t{t} p{i}"
            if i in active[t] or t > 1:
                assert opt.state[p]["step"] == run.states[i]["step"], what
            got = p.detach().float().cpu().numpy()
            if dt == torch.float32:
                parity.assert_params(got, run.params[i], what, tol=2e-6)
            else:
                parity.assert_lowp_params(got, run.params[i], case["param_dtype"], what, frac=3e-4)
