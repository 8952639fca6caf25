"""Parity of the CUDA full-rank path (through the optimizer class and the C
ABI) with the CPU oracle and with the reference's golden vectors."""
import numpy as np
import pytest
import torch

import cases
import parity
from oracle_runner import FULLRANK_CASES, OracleRun, golden_entries, load_golden

pytestmark = pytest.mark.gpu

CODE_KEYS = ("variance_q", "m_q")
RANGE_KEYS = ("variance_scale", "variance_min_log", "m_scale")


def to_cuda_grad(g, shape):
    if g.dtype == np.uint16:
        return torch.from_numpy(g.view(np.int16).copy()).view(torch.bfloat16).reshape(shape).cuda()
    return torch.from_numpy(g.copy()).reshape(shape).cuda()


def state_np(st, key):
    v = st[key]
    a = v.detach().cpu()
    if a.dtype == torch.int16:
        return a.numpy().view(np.uint16).reshape(-1)
    return a.numpy().reshape(-1)


def make_optimizer(run):
    from adafactor8bit import Adafactor8Bit
    params = [torch.nn.Parameter(torch.from_numpy(p.copy()).cuda()) for p in run.params0]
    for p in params:
        p.grad_dtype = None
    return params, Adafactor8Bit(params, **run.case["hp"])


def compare_state(name, t, i, st_gpu, st_cpu, p_gpu, p_cpu, strict):
    """strict: both sides started this step from identical state."""
    mfmt = st_cpu.get("m_quant_type")
    for key in CODE_KEYS:
        if key not in st_cpu:
            continue
        a, b = state_np(st_gpu, key), np.asarray(st_cpu[key]).reshape(-1)
        if key == "m_q" and mfmt in ("uf4", "d4"):
            a, b = parity.unpack_nibbles(a), parity.unpack_nibbles(b)
        parity.assert_codes(a, b, f"{name} t{t} p{i} {key}", al16=(b.dtype == np.uint16),
                            zero_reserved=(key != "m_q"))
    for key in RANGE_KEYS:
        if key in st_cpu:
            parity.assert_ranges(state_np(st_gpu, key), st_cpu[key], f"{name} t{t} p{i} {key}",
                                 max_ulp=1 if strict else 4)
    for key in ("variance", "m"):
        if key in st_cpu:
            assert parity.rel_l2(state_np(st_gpu, key), st_cpu[key]) <= 1e-6, f"{name} t{t} p{i} {key}"
    parity.assert_params(p_gpu.detach().cpu().numpy(), p_cpu, f"{name} t{t} p{i} param")


@pytest.mark.parametrize("name", FULLRANK_CASES)
def test_free_running_matches_oracle_and_golden(name, oracle):
    from adafactor8bit import _engine
    run = OracleRun(name)
    if run.hp["m_quant_type"] in ("d8", "d4"):
        for bits in (8, 4):
            oracle.set_dynamic_map(bits, _engine.dynamic_map(bits))
    gold = load_golden(name)
    assert str(gold["digest"]) == cases.inputs_digest(run.params0, run.grads)
    params, opt = make_optimizer(run)
    steps = run.case["steps"]
    for t in range(1, steps + 1):
        for p, g in zip(params, run.grads[t]):
            p.grad = to_cuda_grad(g, p.shape)
        opt.step()
        run.step()
        torch.cuda.synchronize()
        for i, p in enumerate(params):
            compare_state(name, t, i, opt.state[p], run.states[i], p, run.params[i], strict=False)
            if "fira_prev_norm" in run.states[i]:
                a = float(opt.state[p]["fira_prev_norm"].item())
                b = float(run.states[i]["fira_prev_norm"])
                assert abs(a - b) <= 2e-6 * abs(b), f"{name} t{t} p{i} fira_prev_norm {a} vs {b}"
    # and against what the reference itself produced
    for i, p in enumerate(params):
        ref = golden_entries(gold, steps, i)
        parity.assert_params(p.detach().cpu().numpy(), ref["param"], f"{name} final p{i} vs reference")
        for key in CODE_KEYS:
            if key in ref:
                a, b = state_np(opt.state[p], key), ref[key]
                if key == "m_q" and run.states[i].get("m_quant_type") in ("uf4", "d4"):
                    a, b = parity.unpack_nibbles(a), parity.unpack_nibbles(b)
                parity.assert_codes(a, b, f"{name} final p{i} {key} vs reference",
                                    al16=(b.dtype == np.uint16), zero_reserved=(key != "m_q"))


@pytest.mark.parametrize("name", ["adamw_uf8_al8", "adamw_fira_bf16", "adamw_uf4_al16"])
def test_teacher_forced_step_matches_oracle(name, oracle):
    """Each step starts from the oracle's state on both sides: block ranges must
    then agree to 1 ulp and codes to the +-1 rule."""
    run = OracleRun(name)
    params, opt = make_optimizer(run)
    for t in range(1, run.case["steps"] + 1):
        for p, g in zip(params, run.grads[t]):
            p.grad = to_cuda_grad(g, p.shape)
        if t > 1:   # overwrite the GPU state and parameters with the oracle's
            for i, p in enumerate(params):
                st = opt.state[p]
                p.data.copy_(torch.from_numpy(run.params[i]).reshape(p.shape))
                for key, val in run.states[i].items():
                    if isinstance(val, np.ndarray) and key in st and isinstance(st[key], torch.Tensor):
                        src = torch.from_numpy(val.view(np.int16) if val.dtype == np.uint16 else val)
                        st[key].copy_(src.reshape(st[key].shape))
                if "fira_prev_norm" in run.states[i]:
                    st["fira_prev_norm"].fill_(float(run.states[i]["fira_prev_norm"]))
        opt.step()
        run.step()
        torch.cuda.synchronize()
        for i, p in enumerate(params):
            compare_state(name, t, i, opt.state[p], run.states[i], p, run.params[i], strict=True)


def test_block_edge_cases(oracle):
    """All-zero gradients, a constant block, one block plus a one-element tail, and
    a tensor shorter than one momentum block."""
    from adafactor8bit import Adafactor8Bit
    hp = dict(cases.CASES["adamw_uf8_al8"]["hp"], min_8bit_size=1)
    shapes = [(2048,), (2049,), (4096 + 255,), (100,), (6144,)]
    rng = np.random.default_rng(3)
    p0 = [rng.standard_normal(s).astype(np.float32) * 0.02 for s in shapes]
    params = [torch.nn.Parameter(torch.from_numpy(p.copy()).cuda()) for p in p0]
    opt = Adafactor8Bit(params, **hp)
    ohp = oracle.hyper(**hp)
    ostates = [oracle.init_state(s, ohp) for s in shapes]
    oparams = [p.copy() for p in p0]
    for t in range(1, 4):
        grads = []
        for k, s in enumerate(shapes):
            g = rng.standard_normal(s).astype(np.float32) * 1e-2
            if k == 0:
                g[:] = 0.0 if t < 3 else 1e-3          # all-zero block, then a constant block
            if k == 4:
                g[2048:4096] = 0.0                      # an all-zero block between live ones
            grads.append(g)
        for p, g in zip(params, grads):
            p.grad = torch.from_numpy(g).cuda()
        opt.step()
        torch.cuda.synchronize()
        for i in range(len(shapes)):
            oracle.fullrank_step(oparams[i], grads[i], ostates[i], ohp)
            compare_state("edges", t, i, opt.state[params[i]], ostates[i], params[i], oparams[i], strict=False)
    st0 = opt.state[params[0]]
    assert int(st0["variance_q"].max()) == 255 and int(st0["variance_q"].min()) == 255   # constant block
    st4 = opt.state[params[4]]
    assert int(st4["variance_q"][2048:4096].max()) == 0                                   # exact zeros kept
    assert abs(float(st4["variance_min_log"][1]) + 127.23327) < 1e-4


def test_cpu_parameters_are_refused():
    from adafactor8bit import Adafactor8Bit
    p = torch.nn.Parameter(torch.zeros(8, 8))
    opt = Adafactor8Bit([p], **cases.CASES["adamw_uf8_al8"]["hp"])
    p.grad = torch.ones(8, 8)
    with pytest.raises(RuntimeError):
        opt.step()


@pytest.mark.parametrize("kind", ["normal_f32", "rowscale_bf16", "narrow_range", "spiky"])
def test_large_tensor_codes_are_exact(kind, oracle):
    """Millions of elements through the specialised kernel: its estimate-then-verify
    code path must reproduce the exact sequence on every element, not just within
    the +-1 allowance."""
    from adafactor8bit import Adafactor8Bit
    hp = dict(cases.CASES["adamw_uf8_al8"]["hp"])
    shape = (1024, 2048)
    rng = np.random.default_rng(hash(kind) % 2 ** 31)
    p0 = (rng.standard_normal(shape) * 0.02).astype(np.float32)
    param = torch.nn.Parameter(torch.from_numpy(p0.copy()).cuda())
    param.grad_dtype = None
    opt = Adafactor8Bit([param], **hp)
    ohp = oracle.hyper(**hp)
    ost = oracle.init_state(shape, ohp)
    op = p0.copy()
    for t in range(1, 5):
        if kind == "normal_f32":
            g = (rng.standard_normal(shape) * 1e-2).astype(np.float32)
            g[rng.random(shape) < 0.01] = 0.0
        elif kind == "rowscale_bf16":
            g = cases.make_grad(shape, 31337, t, cases._G_HEAVY)
        elif kind == "narrow_range":
            g = (1e-3 * (1.0 + 1e-4 * rng.standard_normal(shape))).astype(np.float32)
        else:
            g = (rng.standard_normal(shape) * 1e-4).astype(np.float32)
            g[rng.random(shape) < 1e-3] *= 1e4
            g[:, :7] = 0.0
        param.grad = to_cuda_grad(g, shape)
        opt.step()
        oracle.fullrank_step(op.reshape(-1), g.reshape(-1), ost, ohp)
        torch.cuda.synchronize()
        st = opt.state[param]
        for key in ("variance_q", "m_q"):
            s = parity.code_stats(state_np(st, key), ost[key])
            assert s["neq"] == 0, f"{kind} step {t} {key}: {s}"
        for key in RANGE_KEYS:
            assert int(parity.ulp_diff(state_np(st, key), ost[key]).max()) == 0, f"{kind} step {t} {key}"
        parity.assert_params(param.detach().cpu().numpy(), op, f"{kind} step {t} param", tol=1e-6)


@pytest.mark.parametrize("fira", [False, True], ids=["noclip", "limiter"])
def test_config0_full_size_is_exact(fira, oracle):
    """The reference's own CPU-runnable configuration at its full size: one 4096 x 4096 fp32
    parameter (16.8 M elements, 8192 V blocks), fp32 gradients N(0, 1e-2) with 1 % exact zeros,
    AdamW UF8/AL8 with weight decay; with and without the limiter.  Every code and every block
    range must equal the oracle's; parameters within 1e-6."""
    from adafactor8bit import Adafactor8Bit
    hp = dict(cases.CASES["adamw_uf8_al8"]["hp"])
    if fira:
        hp.update(enable_fira_for_adafactor=True, fira_margin=0.01)
    shape = (4096, 4096)
    rng = np.random.default_rng(4096)
    p0 = (rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02)).astype(np.float32)
    param = torch.nn.Parameter(torch.from_numpy(p0.copy()).cuda())
    opt = Adafactor8Bit([param], **hp)
    ohp = oracle.hyper(**hp)
    ost = oracle.init_state(shape, ohp)
    op = p0.copy()
    for t in range(1, 4):
        g = (rng.standard_normal(shape, dtype=np.float32) * np.float32(1e-2 * (100.0 if (fira and t == 3) else 1.0))).astype(np.float32)
        g[rng.random(shape) < 0.01] = 0.0
        param.grad = torch.from_numpy(g).cuda()
        opt.step()
        oracle.fullrank_step(op.reshape(-1), g.reshape(-1), ost, ohp)
        torch.cuda.synchronize()
        st = opt.state[param]
        for key in ("variance_q", "m_q"):
            s = parity.code_stats(state_np(st, key), ost[key])
            assert s["neq"] == 0, f"step {t} {key}: {s}"
        for key in RANGE_KEYS:
            assert int(parity.ulp_diff(state_np(st, key), ost[key]).max()) == 0, f"step {t} {key}"
        parity.assert_params(param.detach().cpu().numpy(), op, f"step {t} param", tol=1e-6)


def test_device_status_is_clean_after_the_runs_above():
    from adafactor8bit import _native
    assert _native.device_status(torch.cuda.current_stream().cuda_stream) == 0


def test_maximize_equals_negated_gradients(oracle):
    """maximize=True (optimizer.py:1973-1974) is a sign flip of the gradient and nothing else."""
    from adafactor8bit import Adafactor8Bit
    hp = dict(cases.CASES["adamw_fira_bf16"]["hp"])
    shape = (96, 200)
    rng = np.random.default_rng(9)
    p0 = (rng.standard_normal(shape) * 0.02).astype(np.float32)
    a = torch.nn.Parameter(torch.from_numpy(p0.copy()).cuda())
    b = torch.nn.Parameter(torch.from_numpy(p0.copy()).cuda())
    a.grad_dtype = b.grad_dtype = None
    oa, ob = Adafactor8Bit([a], **hp), Adafactor8Bit([b], **dict(hp, maximize=True))
    for t in range(1, 4):
        g = cases.make_grad(shape, 555, t, cases.CASES["adamw_fira_bf16"]["grad"])
        a.grad = to_cuda_grad(g, shape)
        b.grad = -to_cuda_grad(g, shape)
        oa.step()
        ob.step()
    torch.cuda.synchronize()
    assert torch.equal(a.detach(), b.detach())
    for key in CODE_KEYS + RANGE_KEYS:
        assert torch.equal(oa.state[a][key], ob.state[b][key]), key


def test_param_groups_and_closure(oracle):
    """Two groups with different learning rates step like two optimizers; the closure's loss is returned."""
    from adafactor8bit import Adafactor8Bit
    hp = dict(cases.CASES["adamw_uf8_al8"]["hp"])
    rng = np.random.default_rng(10)
    shapes = [(64, 200), (4096,)]
    p0 = [(rng.standard_normal(s) * 0.02).astype(np.float32) for s in shapes]
    pa = [torch.nn.Parameter(torch.from_numpy(x.copy()).cuda()) for x in p0]
    pb = [torch.nn.Parameter(torch.from_numpy(x.copy()).cuda()) for x in p0]
    both = Adafactor8Bit([dict(params=[pa[0]], lr=1e-3), dict(params=[pa[1]], lr=5e-4)], **{k: v for k, v in hp.items() if k != "lr"})
    one = Adafactor8Bit([pb[0]], **dict(hp, lr=1e-3))
    two = Adafactor8Bit([pb[1]], **dict(hp, lr=5e-4))
    for t in range(1, 4):
        gs = [(rng.standard_normal(s) * 1e-2).astype(np.float32) for s in shapes]
        for p, q, g in zip(pa, pb, gs):
            p.grad = torch.from_numpy(g).cuda()
            q.grad = torch.from_numpy(g).cuda()
        assert both.step(lambda: torch.tensor(1.25)) == 1.25
        one.step()
        two.step()
    torch.cuda.synchronize()
    for p, q in zip(pa, pb):
        assert torch.equal(p.detach(), q.detach())


LAG_CASES = {
    # AdamW + limiter + RMS clip, one pass with the previous step's norm
    "lag_adamw_fira_clip": dict(cases.CASES["adamw_fira_bf16"], steps=6,
                                hp=dict(cases.CASES["adamw_fira_bf16"]["hp"], d=1.0, lag_norm=True)),
    # the same on bf16 parameters
    "lag_adamw_bf16p": dict(cases.CASES["adamw_bf16p"], steps=5,
                            hp=dict(cases.CASES["adamw_bf16p"]["hp"], d=1.0, lag_norm=True)),
    # unfactored Adafactor: relative step, alpha from the parameter RMS on the device, clip d = 1, other formats
    "lag_adafactor_unfactored": dict(cases.CASES["adafactor_unfactored"], steps=5,
                                     hp=dict(cases.CASES["adafactor_unfactored"]["hp"], lag_norm=True)),
}


@pytest.mark.parametrize("name", sorted(LAG_CASES))
def test_lag_norm_single_pass(name, oracle):
    """lag_norm=True: the step clips and limits with the previous step's norm (the reference's CUDA
    dispatcher, optimizer.py:1056-1071); compared with the oracle's restatement of that rule, states
    "prev_update_norm", "lag_fira_scale" and "fira_prev_norm" included."""
    case = LAG_CASES[name]
    run = OracleRun(name, case=case)
    fmt = case.get("param_dtype", "f32")
    dt = {"f32": torch.float32, "bf16": torch.bfloat16}[fmt]
    from adafactor8bit import Adafactor8Bit
    params = [torch.nn.Parameter(torch.from_numpy(p.copy()).to(dt).cuda()) for p in run.params0]
    for p in params:
        p.grad_dtype = None
    opt = Adafactor8Bit(params, **case["hp"])
    for t in range(1, case["steps"] + 1):
        for p, g in zip(params, run.grads[t]):
            p.grad = to_cuda_grad(g, p.shape)
        opt.step()
        run.step()
        torch.cuda.synchronize()
        for i, p in enumerate(params):
            st, so = opt.state[p], run.states[i]
            what = f"{name} t{t} p{i}"
            if fmt == "f32":
                compare_state(name, t, i, st, so, p, run.params[i], strict=False)
            else:
                parity.assert_lowp_params(p.detach().float().cpu().numpy(), run.params[i], fmt, what, frac=1e-4)
            assert abs(float(st["prev_update_norm"].item()) - float(so["prev_update_norm"])) <= 2e-6 * abs(float(so["prev_update_norm"])), what
            if "lag_fira_scale" in so:
                assert abs(float(st["lag_fira_scale"].item()) - float(so["lag_fira_scale"])) <= 2e-6, what
                assert abs(float(st["fira_prev_norm"].item()) - float(so["fira_prev_norm"])) <= 2e-6 * abs(float(so["fira_prev_norm"])), what
    # the lagged run is a different algorithm: after the spike it must differ from the exact one
    assert any("prev_update_norm" in opt.state[p] for p in params)


def test_empty_parameter_is_stepped_without_a_launch():
    """A parameter without elements gets a state and a step count, like in the reference, and
    does not disturb the other tensors of its group."""
    from adafactor8bit import Adafactor8Bit
    hp = dict(cases.CASES["adamw_uf8_al8"]["hp"])
    empty = torch.nn.Parameter(torch.zeros(0, 4, device="cuda"))
    full = torch.nn.Parameter(torch.ones(64, 128, device="cuda"))
    alone = torch.nn.Parameter(torch.ones(64, 128, device="cuda"))
    opt, ref = Adafactor8Bit([empty, full], **hp), Adafactor8Bit([alone], **hp)
    for t in range(2):
        g = torch.full((64, 128), 0.01 * (t + 1), device="cuda")
        empty.grad, full.grad, alone.grad = torch.zeros(0, 4, device="cuda"), g.clone(), g.clone()
        opt.step()
        ref.step()
    torch.cuda.synchronize()
    assert opt.state[empty]["step"] == 2 and opt.state[empty]["variance"].shape == (0, 4)
    assert torch.equal(full.detach(), alone.detach())


def test_tensor_beyond_2_31_elements():
    """64-bit indexing: a tensor of 2^31 + 6149 elements (17 GB with its states).  V blocks are
    independent without the limiter, so the first and the last blocks must come out exactly like
    the same values stepped as small tensors."""
    from adafactor8bit import Adafactor8Bit
    if torch.cuda.get_device_properties(0).total_memory < 60 * 2 ** 30:
        pytest.skip("needs 60 GB of device memory")
    hp = dict(cases.CASES["adamw_uf8_al8"]["hp"], min_8bit_size=1)
    n = 2 ** 31 + 6149
    tail0 = (n // 2048 - 1) * 2048                         # the last full block and the ragged one after it

    def fill(t, scale, lo, hi):                            # a value pattern that depends on the global index
        for a in range(lo, hi, 2 ** 27):
            b = min(a + 2 ** 27, hi)
            idx = torch.arange(a, b, device="cuda", dtype=torch.int64)
            t[a - lo:b - lo] = (((idx * 2654435761) % 2001) - 1000).to(torch.float32).mul_(scale).to(t.dtype)
    big = torch.nn.Parameter(torch.empty(n, device="cuda"))
    fill(big.data, 2e-5, 0, n)
    gbig = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    fill(gbig, 1e-6, 0, n)
    head = torch.nn.Parameter(big.detach()[:4096].clone())
    tail = torch.nn.Parameter(big.detach()[tail0:].clone())
    for p in (big, head, tail):
        p.grad_dtype = None
    opt, ref = Adafactor8Bit([big], **hp), Adafactor8Bit([head, tail], **hp)
    for t in range(2):
        big.grad, head.grad, tail.grad = gbig, gbig[:4096].clone(), gbig[tail0:].clone()
        opt.step()
        ref.step()
    torch.cuda.synchronize()
    assert torch.equal(big.detach()[:4096], head.detach())
    assert torch.equal(big.detach()[tail0:], tail.detach())
    sb, st = opt.state[big], ref.state[tail]
    assert torch.equal(sb["variance_q"][tail0:tail0 + st["variance_q"].numel()], st["variance_q"])
    assert torch.equal(sb["m_q"][tail0:tail0 + st["m_q"].numel()], st["m_q"])
    assert torch.equal(sb["variance_scale"][tail0 // 2048:], st["variance_scale"])
    mid = big.detach()[2 ** 31 - 4096:2 ** 31 + 4096]
    assert torch.isfinite(mid).all() and (mid != 0).any()
    from adafactor8bit import _native
    assert _native.device_status(torch.cuda.current_stream().cuda_stream) == 0


def test_step_waits_for_gradients_arriving_on_another_stream():
    """step(grad_ready=[event per group]): gradients copied from pinned host memory on a second stream,
    one event per parameter group; the result equals a plain step on resident gradients."""
    from adafactor8bit import Adafactor8Bit
    hp = dict(cases.CASES["adamw_fira_bf16"]["hp"])
    rng = np.random.default_rng(5)
    shapes = [(300, 200), (4096,), (128, 256), (2048,)]
    p0 = [(rng.standard_normal(s) * 0.02).astype(np.float32) for s in shapes]
    a = [torch.nn.Parameter(torch.from_numpy(x.copy()).cuda()) for x in p0]
    b = [torch.nn.Parameter(torch.from_numpy(x.copy()).cuda()) for x in p0]
    oa = Adafactor8Bit([{"params": a[:2]}, {"params": a[2:]}], **hp)
    ob = Adafactor8Bit([{"params": b[:2]}, {"params": b[2:]}], **hp)
    side = torch.cuda.Stream()
    for t in range(3):
        host = [torch.from_numpy((rng.standard_normal(s) * 1e-3).astype(np.float32)).pin_memory() for s in shapes]
        events = []
        with torch.cuda.stream(side):
            for grp in (a[:2], a[2:]):
                for p in grp:
                    i = next(k for k, q in enumerate(a) if q is p)
                    p.grad = torch.empty_like(p)
                    p.grad.copy_(host[i], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(side)
                events.append(ev)
        oa.step(grad_ready=events)
        for p, h in zip(b, host):
            p.grad = h.cuda()
        ob.step()
        torch.cuda.synchronize()
    for p, q in zip(a, b):
        assert torch.equal(p.detach(), q.detach())
    with pytest.raises(ValueError):
        oa.step(grad_ready=[None])


def test_step_follows_a_parameter_whose_storage_was_replaced(oracle):
    """p.data = <another tensor> keeps the parameter's identity but moves its storage (module.to(),
    flat-parameter wrappers, manual re-materialisation do this).  The launch tables must follow:
    the new storage is updated, the old one is left alone."""
    from adafactor8bit import Adafactor8Bit
    hp = dict(cases.CASES["adamw_fira_bf16"]["hp"])
    shapes = [(96, 200), (4096,)]
    p0 = [cases.make_param(s, 800 + i) for i, s in enumerate(shapes)]
    params = [torch.nn.Parameter(torch.from_numpy(p.copy()).cuda()) for p in p0]
    for p in params:
        p.grad_dtype = None
    opt = Adafactor8Bit(params, **hp)
    ohp = oracle.hyper(**hp)
    ostates = [oracle.init_state(s, ohp) for s in shapes]
    oparams = [p.copy() for p in p0]
    old = None
    for t in range(1, 4):
        grads = [cases.make_grad(s, 850 + i, t, cases.CASES["adamw_fira_bf16"]["grad"]) for i, s in enumerate(shapes)]
        if t == 2:
            old = [p.data for p in params]
            snapshot = [x.clone() for x in old]
            for p in params:
                p.data = p.data.clone()
        for p, g in zip(params, grads):
            p.grad = to_cuda_grad(g, p.shape)
        opt.step()
        torch.cuda.synchronize()
        for i in range(len(shapes)):
            oracle.fullrank_step(oparams[i].reshape(-1), grads[i].reshape(-1), ostates[i], ohp)
        for i, p in enumerate(params):
            parity.assert_params(p.detach().cpu().numpy(), oparams[i], f"step {t} param {i}")
        if t >= 2:
            assert all(torch.equal(a, b) for a, b in zip(old, snapshot)), "the replaced storage was written"
