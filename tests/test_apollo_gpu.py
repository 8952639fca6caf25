"""Parity of the CUDA APOLLO path with the CPU oracle (same projection matrices: both draw
them from the CPU generator) and with the reference's golden vectors."""
import numpy as np
import pytest
import torch

import cases
import parity
from oracle_runner import OracleRun, golden_entries, load_golden
from test_fullrank_gpu import make_optimizer, state_np, to_cuda_grad

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["apollo_r32", "apollo_r8_tensor"])
@pytest.mark.parametrize("exact", [True, False], ids=["exact_projection", "tensor_core_projection"])
def test_apollo_free_running_matches_oracle(oracle, exact, name):
    """exact: correctly rounded projections, states bit-comparable with the oracle.  Tensor
    cores: the projected gradient carries the rounding of a binary32 accumulation (as the
    reference's own matmul does), so ranges and the limiter state move by a few ulp."""
    from adafactor8bit import _engine, optimizer as opt_mod
    run = OracleRun(name)
    opt_mod.APOLLO_RNG_DEVICE = "cpu"
    saved = _engine.EXACT_PROJECTION
    _engine.EXACT_PROJECTION = exact
    norm_tol, param_tol = (3e-6, 2e-6) if exact else (3e-4, 5e-5)   # the bound used against the reference's own fp32 matmul below
    try:
        params, opt = make_optimizer(run)
        for t in range(1, run.case["steps"] + 1):
            for p, g in zip(params, run.grads[t]):
                p.grad = to_cuda_grad(g, p.shape)
            opt.step()
            run.step()
            torch.cuda.synchronize()
            for i, p in enumerate(params):
                st_g, st_c = opt.state[p], run.states[i]
                what = f"{name} t{t} p{i}"
                if "apollo_seed" in st_c:
                    assert np.array_equal(st_g["apollo_proj_matrix_T"].cpu().numpy(), st_c["apollo_proj_matrix_T"]), what
                    assert int(st_g["apollo_seed"]) == int(st_c["apollo_seed"])
                    if exact:
                        parity.assert_codes(state_np(st_g, "v_low_q"), st_c["v_low_q"], what + " v_low_q")
                        parity.assert_codes(state_np(st_g, "m_low_q"), st_c["m_low_q"], what + " m_low_q", zero_reserved=False)
                        for key in ("v_low_scale", "v_low_min_log", "m_low_scale"):
                            parity.assert_ranges(state_np(st_g, key), st_c[key], what + " " + key, max_ulp=1)
                    elif t == 1:
                        # A binary32 accumulation changes the smallest |g_low| of a block by 1e-3
                        # relative and more (it is a sum that cancelled almost completely), hence the
                        # block's min_log and scale by up to a few hundredths, and with them the codes
                        # that sat next to a rounding boundary, by one step.  The reference's own
                        # matmul has the same effect against the exact products.  Later steps start
                        # from these slightly different states, so only the first is compared code by
                        # code; parameters and the limiter state are compared at every step.
                        sv = parity.code_stats(state_np(st_g, "v_low_q"), st_c["v_low_q"])
                        assert sv["zero_mismatch"] == 0 and sv["max"] <= 1 and sv["neq"] <= 0.1 * sv["n"], (what, sv)
                        sm = parity.code_stats(state_np(st_g, "m_low_q"), st_c["m_low_q"])
                        assert sm["max"] <= 1 and sm["neq"] <= 2e-3 * sm["n"], (what, sm)
                        for key, tol in (("v_low_scale", 0.5), ("v_low_min_log", 0.5)):
                            assert np.abs(state_np(st_g, key) - np.asarray(st_c[key]).reshape(-1)).max() <= tol, what + " " + key
                        assert np.allclose(state_np(st_g, "m_low_scale"), np.asarray(st_c["m_low_scale"]).reshape(-1), rtol=1e-5), what
                    a, b = float(st_g["scaled_grad_norm_prev"].item()), float(st_c["scaled_grad_norm_prev"])
                    assert abs(a - b) <= norm_tol * abs(b), f"{what} scaled_grad_norm_prev {a} vs {b}"
                parity.assert_params(p.detach().cpu().numpy(), run.params[i], what + " param", tol=param_tol)
        # against the reference itself: its float32 GEMM rounds the projected gradient differently,
        # which moves low-rank V codes next to a block minimum and, through the channel norms, the
        # limiter state; momentum codes and parameters stay close
        gold = load_golden(name)
        steps = run.case["steps"]
        for i, p in enumerate(params):
            ref = golden_entries(gold, steps, i)
            parity.assert_params(p.detach().cpu().numpy(), ref["param"], f"{name} final p{i} vs reference", tol=5e-5)
            if "m_low_q" in ref:
                s = parity.code_stats(state_np(opt.state[p], "m_low_q"), ref["m_low_q"])
                assert s["max"] <= 1 and s["neq"] <= 1e-3 * s["n"], s
    finally:
        opt_mod.APOLLO_RNG_DEVICE = None
        _engine.EXACT_PROJECTION = saved


@pytest.mark.parametrize("name", ["apollo_fp32_states", "apollo_3d_f16g"])
def test_apollo_variants_match_oracle_and_reference(oracle, name):
    """fp32 low-rank states (quantize=False) and tensors of three dimensions with fp16 gradients, with
    correctly rounded projections on both sides: states and parameters at the full tolerances against the
    oracle, then the final parameters against what the reference itself produced."""
    from adafactor8bit import _engine, optimizer as opt_mod
    run = OracleRun(name)
    opt_mod.APOLLO_RNG_DEVICE = "cpu"
    saved = _engine.EXACT_PROJECTION
    _engine.EXACT_PROJECTION = True
    try:
        params, opt = make_optimizer(run)
        for t in range(1, run.case["steps"] + 1):
            for p, g in zip(params, run.grads[t]):
                p.grad = to_cuda_grad(g, p.shape)
            opt.step()
            run.step()
            torch.cuda.synchronize()
            for i, p in enumerate(params):
                st_g, st_c = opt.state[p], run.states[i]
                what = f"{name} t{t} p{i}"
                assert np.array_equal(st_g["apollo_proj_matrix_T"].cpu().numpy(), st_c["apollo_proj_matrix_T"]), what
                for key in ("v_low", "m_low"):
                    if key in st_c and st_c[key] is not None:
                        assert parity.rel_l2(state_np(st_g, key), st_c[key]) <= 1e-6, (what, key)
                if st_c.get("v_low_q") is not None:
                    parity.assert_codes(state_np(st_g, "v_low_q"), st_c["v_low_q"], what + " v_low_q")
                    parity.assert_codes(state_np(st_g, "m_low_q"), st_c["m_low_q"], what + " m_low_q", zero_reserved=False)
                a, b = float(st_g["scaled_grad_norm_prev"].item()), float(st_c["scaled_grad_norm_prev"])
                assert abs(a - b) <= 3e-6 * abs(b), f"{what} scaled_grad_norm_prev {a} vs {b}"
                parity.assert_params(p.detach().cpu().numpy(), run.params[i], what + " param", tol=2e-6)
        gold = load_golden(name)
        for i, p in enumerate(params):
            ref = golden_entries(gold, run.case["steps"], i)
            parity.assert_params(p.detach().cpu().numpy(), ref["param"], f"{name} final p{i} vs reference", tol=5e-5)
            if name == "apollo_fp32_states":                    # checkpoint layout: the momentum keeps the projected shape
                assert tuple(opt.state[p]["m_low"].shape) in ((p.shape[0], 8), (8, p.shape[1]))
    finally:
        opt_mod.APOLLO_RNG_DEVICE = None
        _engine.EXACT_PROJECTION = saved


@pytest.mark.parametrize("name", cases.APOLLO_RULE_CASES)
def test_apollo_lowrank_rules_match_oracle_and_reference(oracle, name):
    """apollo_factorize, its CAME form, CAME over the projected gradient (AL8-coded and fp32 states) and
    factorisation without momentum (af8_apollo_rule_step), free-running with correctly rounded projections on
    both sides: every state against the oracle (codes exact, fp32 states and block ranges to 1e-6, the
    limiter state to 3e-6, parameters to 2e-6), then the final parameters against what the reference produced."""
    from adafactor8bit import _engine, optimizer as opt_mod
    run = OracleRun(name)
    opt_mod.APOLLO_RNG_DEVICE = "cpu"
    saved = _engine.EXACT_PROJECTION
    _engine.EXACT_PROJECTION = True
    code_keys = ("v_low_q", "res_low_q", "conf_row_low_q", "conf_col_low_q")
    f32_keys = ("v_low", "res_low", "m_low", "row_var_low", "col_var_low", "conf_row_low", "conf_col_low",
                "v_low_scale", "v_low_min_log", "res_low_scale", "res_low_min_log", "m_low_scale",
                "conf_row_low_scale", "conf_row_low_min_log", "conf_col_low_scale", "conf_col_low_min_log")
    try:
        params, opt = make_optimizer(run)
        for t in range(1, run.case["steps"] + 1):
            for p, g in zip(params, run.grads[t]):
                p.grad = to_cuda_grad(g, p.shape)
            opt.step()
            run.step()
            torch.cuda.synchronize()
            for i, p in enumerate(params):
                st_g, st_c = opt.state[p], run.states[i]
                what = f"{name} t{t} p{i}"
                seen = 0
                for key in code_keys:
                    if st_c.get(key) is not None:
                        parity.assert_codes(state_np(st_g, key), st_c[key], f"{what} {key}")
                        seen += 1
                if st_c.get("m_low_q") is not None:
                    parity.assert_codes(state_np(st_g, "m_low_q"), st_c["m_low_q"], what + " m_low_q", zero_reserved=False)
                    seen += 1
                for key in f32_keys:
                    if st_c.get(key) is not None:
                        have = state_np(st_g, key).reshape(-1)
                        assert have.size == np.asarray(st_c[key]).size, (what, key)
                        assert parity.rel_l2(have, np.asarray(st_c[key]).reshape(-1)) <= 1e-6, (what, key, parity.rel_l2(have, np.asarray(st_c[key]).reshape(-1)))
                        seen += 1
                assert seen >= 2, (what, sorted(st_c))
                a, b = float(st_g["scaled_grad_norm_prev"].item()), float(st_c["scaled_grad_norm_prev"])
                assert abs(a - b) <= 3e-6 * abs(b), f"{what} scaled_grad_norm_prev {a} vs {b}"
                parity.assert_params(p.detach().cpu().numpy(), run.params[i], what + " param", tol=2e-6)
        gold = load_golden(name)
        for i, p in enumerate(params):
            ref = golden_entries(gold, run.case["steps"], i)
            parity.assert_params(p.detach().cpu().numpy(), ref["param"], f"{name} final p{i} vs reference", tol=5e-5)
            for key, want in ref.items():            # the checkpoint holds the reference's keys with the reference's sizes
                if key not in ("param", "apollo_proj_matrix_T"):
                    assert key in opt.state[p] and opt.state[p][key].numel() == want.size, (name, i, key)
    finally:
        opt_mod.APOLLO_RNG_DEVICE = None
        _engine.EXACT_PROJECTION = saved


@pytest.mark.parametrize("rows,cols,rank", [(256, 96, 32), (48, 304, 16), (1024, 520, 256), (392, 1024, 256), (128, 128, 8)])
@pytest.mark.parametrize("negate", [0, 1])
def test_tensor_core_projection(rows, cols, rank, negate):
    """af8_apollo_project_ws (bf16 gradients, three-plane split of the projection) against a
    binary64 matmul: errors of a binary32 accumulation, non-finite entries as zero."""
    from adafactor8bit import _native as N
    lib = N.lib()
    rng = np.random.default_rng(rows * 7 + cols)
    g = torch.from_numpy((rng.standard_normal((rows, cols)) * 1e-3).astype(np.float32)).to(torch.bfloat16)
    g[3, 5] = float("inf")
    g[7, 1] = float("nan")
    g[rows - 1, cols - 1] = float("-inf")
    right = rows >= cols
    pt = (rng.standard_normal((cols, rank) if right else (rank, rows)) / np.sqrt(rank)).astype(np.float32)
    gc = g.to(torch.float32).numpy().astype(np.float64)
    gc = np.where(np.isfinite(gc), gc, 0.0)
    want = gc @ pt.astype(np.float64) if right else pt.astype(np.float64) @ gc
    if negate:
        want = -want
    d_g, d_pt = g.cuda(), torch.from_numpy(pt).cuda()
    out = torch.full((want.size,), float("nan"), dtype=torch.float32, device="cuda")
    chan = torch.empty(max(rows, cols), dtype=torch.float64, device="cuda")
    nbytes = int(lib.af8_apollo_project_workspace(rows, cols, rank))
    ws = torch.empty(nbytes + 256, dtype=torch.uint8, device="cuda")
    ws_ptr = (ws.data_ptr() + 255) // 256 * 256
    N.check(lib.af8_apollo_project_ws(d_g.data_ptr(), N.BF16, negate, d_pt.data_ptr(), rows, cols, rank, out.data_ptr(),
                                      chan.data_ptr(), ws_ptr, nbytes, torch.cuda.current_stream().cuda_stream), "project_ws")
    torch.cuda.synchronize()
    got = out.cpu().numpy().reshape(want.shape).astype(np.float64)
    assert np.isfinite(got).all()
    # bound: K accumulations of products of magnitude |g||p| in binary32
    k = cols if right else rows
    bound = 2.0 ** -21 * (np.abs(gc) @ np.abs(pt.astype(np.float64)) if right else np.abs(pt.astype(np.float64)) @ np.abs(gc))
    assert (np.abs(got - want) <= bound + 1e-30).all(), float(np.abs(got - want).max() / np.abs(want).max())
    assert np.abs(got - want).max() <= 4e-6 * np.abs(want).max() * max(1.0, np.sqrt(k / 256.0))
    # the tcgen05 kernel adds the squares of 8 neighbours in binary32 before the binary64 sum (the reference's
    # own channel norm is a binary32 reduction); the mma.sync and exact paths add every square in binary64
    want_ch = (gc ** 2).astype(np.float32).astype(np.float64).sum(axis=1 if right else 0)
    assert np.allclose(chan.cpu().numpy(), want_ch, rtol=1e-6)


def test_tensor_core_projection_batch():
    """af8_apollo_project_batch over mixed shapes: right-case tensors and, through the transposed
    gradient, left-case ones on the tcgen05 kernel; a rank that is no multiple of 16 on mma.sync;
    a scratch too small for the last tensor, which then stays on mma.sync as well."""
    from adafactor8bit import _native as N
    lib = N.lib()
    rng = np.random.default_rng(5)
    shapes = [(512, 256, 64), (128, 640, 64), (64, 1032, 32), (264, 136, 24), (96, 2048, 256)]
    stream = torch.cuda.current_stream().cuda_stream
    descs = np.zeros(len(shapes), dtype=N.APOLLO_PROJ_DESC)
    keep, wants, outs, chans, want_chs = [], [], [], [], []
    for i, (rows, cols, rank) in enumerate(shapes):
        g = torch.from_numpy((rng.standard_normal((rows, cols)) * 1e-3).astype(np.float32)).to(torch.bfloat16)
        g[1, 2] = float("nan")
        right = rows >= cols
        pt = (rng.standard_normal((cols, rank) if right else (rank, rows)) / np.sqrt(rank)).astype(np.float32)
        gc = g.to(torch.float32).numpy().astype(np.float64)
        gc = np.where(np.isfinite(gc), gc, 0.0)
        wants.append(gc @ pt.astype(np.float64) if right else pt.astype(np.float64) @ gc)
        d_g, d_pt = g.cuda(), torch.from_numpy(pt).cuda()
        out = torch.full((wants[-1].size,), float("nan"), dtype=torch.float32, device="cuda")
        chan = torch.empty(max(rows, cols), dtype=torch.float64, device="cuda")
        nbytes = int(lib.af8_apollo_project_workspace(rows, cols, rank))
        ws = torch.empty(nbytes + 256, dtype=torch.uint8, device="cuda")
        keep += [d_g, d_pt, chan, ws]
        outs.append(out)
        chans.append(chan)
        want_chs.append((gc ** 2).sum(axis=1 if right else 0))
        descs["grad"][i], descs["pt"][i], descs["g_low"][i], descs["chan_g2"][i] = d_g.data_ptr(), d_pt.data_ptr(), out.data_ptr(), chan.data_ptr()
        descs["workspace"][i], descs["workspace_bytes"][i] = (ws.data_ptr() + 255) // 256 * 256, nbytes
        descs["rows"][i], descs["cols"][i], descs["rank"][i] = rows, cols, rank
    tb = int(lib.af8_apollo_project_task_bytes()) * len(shapes)
    h = torch.empty(tb, dtype=torch.uint8).pin_memory()
    d = torch.empty(tb, dtype=torch.uint8, device="cuda")
    t_bytes = 200 * 1024                      # fits tensors 1 and 2 one at a time (160 KB, 129 KB), not tensor 4 (384 KB)
    t = torch.empty(t_bytes + 256, dtype=torch.uint8, device="cuda")
    N.check(lib.af8_apollo_project_batch(descs.ctypes.data, len(shapes), N.BF16, h.data_ptr(), d.data_ptr(),
                                         (t.data_ptr() + 255) // 256 * 256, t_bytes, stream), "project_batch")
    torch.cuda.synchronize()
    assert N.device_status(stream) == 0
    for (rows, cols, rank), want, out in zip(shapes, wants, outs):
        got = out.cpu().numpy().reshape(want.shape).astype(np.float64)
        assert np.isfinite(got).all(), (rows, cols, rank)
        assert np.abs(got - want).max() <= 4e-6 * np.abs(want).max(), (rows, cols, rank, float(np.abs(got - want).max() / np.abs(want).max()))
    for shape, chan, want_ch in zip(shapes, chans, want_chs):       # squared channel norms, the NaN entry counted as zero
        assert np.allclose(chan.cpu().numpy(), want_ch, rtol=1e-6), shape


def test_projection_is_correctly_rounded():
    """af8_apollo_project against a binary64 matmul, both sides."""
    from adafactor8bit import _native as N
    lib = N.lib()
    rng = np.random.default_rng(7)
    for rows, cols, rank in ((200, 96, 32), (48, 300, 16)):
        g = (rng.standard_normal((rows, cols)) * 1e-3).astype(np.float32)
        g[3, 5] = np.inf
        g[7, 1] = np.nan
        right = rows >= cols
        pt = (rng.standard_normal((cols, rank) if right else (rank, rows)) / np.sqrt(rank)).astype(np.float32)
        gc = np.where(np.isfinite(g), g, 0.0).astype(np.float64)
        want = (gc @ pt.astype(np.float64) if right else pt.astype(np.float64) @ gc).astype(np.float32)
        d_g, d_pt = torch.from_numpy(g).cuda(), torch.from_numpy(pt).cuda()
        out = torch.empty(want.size, dtype=torch.float32, device="cuda")
        chan = torch.empty(max(rows, cols), dtype=torch.float64, device="cuda")
        N.check(lib.af8_apollo_project(d_g.data_ptr(), N.F32, 0, d_pt.data_ptr(), rows, cols, rank, out.data_ptr(),
                                       chan.data_ptr(), torch.cuda.current_stream().cuda_stream), "project")
        torch.cuda.synchronize()
        got = out.cpu().numpy().reshape(want.shape)
        assert np.array_equal(got, want)
        want_ch = (gc.astype(np.float32).astype(np.float64) ** 2).astype(np.float32).astype(np.float64).sum(axis=1 if right else 0)
        assert np.allclose(chan.cpu().numpy(), want_ch, rtol=1e-12)


@pytest.mark.parametrize("param_dtype,grad_dtype", [("f32", "bf16"), ("f32", "f32"), ("bf16", "bf16")])
@pytest.mark.parametrize("aligned", [True, False], ids=["vector_path", "one_odd_tensor"])
def test_apply_batch_equals_per_tensor_calls(param_dtype, grad_dtype, aligned):
    """af8_apollo_apply_batch writes what af8_apollo_apply writes tensor by tensor, bit for bit: right- and
    left-case tensors, channel- and tensor-wise scaling, every decay mode, a bf16 compute copy, a tensor that
    ends inside a 2048-element chunk; with one tensor whose columns are no multiple of 8 the table takes the
    per-tensor route."""
    import ctypes
    from adafactor8bit import _native as N
    lib = N.lib()
    dev = torch.device("cuda:0")
    gen = torch.Generator(device="cpu").manual_seed(77)
    shapes = [(512, 256), (64, 1032), (264, 136), (96, 2048), (40, 72)]
    if not aligned:
        shapes[2] = (250, 36)
    pdt = dict(f32=torch.float32, bf16=torch.bfloat16)[param_dtype]
    gdt = dict(f32=torch.float32, bf16=torch.bfloat16)[grad_dtype]
    n = len(shapes)
    p0 = [torch.randn(s, generator=gen).to(pdt).to(dev) for s in shapes]
    grads = [(torch.randn(s, generator=gen) * 0.01).to(gdt).to(dev) for s in shapes]
    grads[0][3, 5] = float("inf")                     # non-finite gradients count as zero
    sfs = [(torch.rand(max(s), generator=gen) + 0.5).to(dev) for s in shapes]
    scal = torch.zeros(n, 4, dtype=torch.float32)
    scal[:, 0] = -torch.rand(n, generator=gen) * 1e-2     # update_scale
    scal[:, 1] = 0.5 + torch.rand(n, generator=gen)       # fira
    scal[:, 3] = 0.99                                     # decay computed on the device
    scal = scal.to(dev)
    sins = []
    for i in range(n):
        sin = N.ApolloScalarsIn()
        sin.scale_tensor, sin.fira, sin.scale_front, sin.sqrt_scale = int(i == 3), int(i % 2 == 0), int(i == 1), 1.25
        sins.append(sin)
    decay = [0.999, 0.0, 0.98, 0.0, 0.97]
    has_decay = [1, 0, 2, 0, 1]
    sr = [int(param_dtype != "f32" and i == 4) for i in range(n)]
    copies = [torch.zeros(s, dtype=torch.bfloat16, device=dev) if (param_dtype == "f32" and i in (0, 3)) else None
              for i, s in enumerate(shapes)]
    PD, GD = dict(f32=N.F32, bf16=N.BF16)[param_dtype], dict(f32=N.F32, bf16=N.BF16)[grad_dtype]
    s = torch.cuda.current_stream(dev).cuda_stream

    want_p = [p.clone() for p in p0]
    want_c = [c.clone() if c is not None else None for c in copies]
    for i in range(n):
        N.check(lib.af8_apollo_apply(want_p[i].data_ptr(), PD, sr[i], 1234 + i, grads[i].data_ptr(), GD, 1, sfs[i].data_ptr(),
                                     scal.data_ptr() + 16 * i, shapes[i][0], shapes[i][1], ctypes.byref(sins[i]), decay[i],
                                     has_decay[i], want_c[i].data_ptr() if want_c[i] is not None else None, s), "af8_apollo_apply")
    got_p = [p.clone() for p in p0]
    got_c = [c.clone() if c is not None else None for c in copies]
    host = torch.zeros(n * N.APOLLO_APPLY_TENSOR.itemsize, dtype=torch.uint8).pin_memory()
    devt = torch.empty(n * N.APOLLO_APPLY_TENSOR.itemsize, dtype=torch.uint8, device=dev)
    t = np.frombuffer(host.numpy(), dtype=N.APOLLO_APPLY_TENSOR, count=n)
    first = 0
    for i in range(n):
        t["param"][i], t["grad"][i], t["sf"][i] = got_p[i].data_ptr(), grads[i].data_ptr(), sfs[i].data_ptr()
        t["scalars"][i] = scal.data_ptr() + 16 * i
        t["param_copy"][i] = got_c[i].data_ptr() if got_c[i] is not None else 0
        t["rows"][i], t["cols"][i], t["first_chunk"][i] = shapes[i][0], shapes[i][1], first
        first += (shapes[i][0] * shapes[i][1] + 2047) // 2048
        t["sr_base"][i], t["stochastic_round"][i] = 1234 + i, sr[i]
        t["sqrt_scale"][i], t["decay"][i], t["has_decay"][i] = sins[i].sqrt_scale, decay[i], has_decay[i]
        t["scale_tensor"][i], t["fira"][i], t["scale_front"][i] = sins[i].scale_tensor, sins[i].fira, sins[i].scale_front
    N.check(lib.af8_apollo_apply_batch(host.data_ptr(), devt.data_ptr(), n, first, PD, GD, 1, s), "af8_apollo_apply_batch")
    torch.cuda.synchronize(dev)
    for i in range(n):
        assert not torch.equal(want_p[i], p0[i])
        assert torch.equal(got_p[i].view(torch.int16 if pdt == torch.bfloat16 else torch.int32),
                           want_p[i].view(torch.int16 if pdt == torch.bfloat16 else torch.int32)), shapes[i]
        if want_c[i] is not None:
            assert torch.equal(got_c[i].view(torch.int16), want_c[i].view(torch.int16)), shapes[i]
    # a table whose chunk numbering is wrong is refused before anything is launched
    t["first_chunk"][1] += 1
    assert lib.af8_apollo_apply_batch(host.data_ptr(), devt.data_ptr(), n, first, PD, GD, 1, s) == N.ERR_INVALID
