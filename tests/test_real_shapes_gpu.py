"""Parity at the layer shapes of the benchmark configurations.

The fixtures and the other GPU tests use tensors of at most a few hundred thousand elements.
Here every path steps real layers against the CPU oracle, free-running for a few steps:

  * factored Adafactor (constructor defaults, AL8 block 256) and AdamW UF8/AL8 with the limiter
    and a x100 gradient spike on the TinyLlama-1.1B shapes: the 32000 x 2048 embedding (125
    row-state blocks of 256, 32000 V blocks), a 5632 x 2048 MLP matrix, a 256 x 2048 k/v
    projection and a 2048-element norm vector;
  * CAME (UF8 momentum, AL16 second moment and confidence, block 2048) on the Llama-2-7B shapes
    11008 x 4096, 4096 x 11008 and 4096 x 4096;
  * APOLLO rank 256 on the Llama-3-8B shapes 14336 x 4096 (projection from the right),
    4096 x 14336 and 1024 x 4096 (from the left), three ways: with correctly rounded projections
    at the full tolerances; the tensor-core projection alone against a binary64 product with a
    contraction length of 4096; and the whole step with the tensor-core projection, where the
    oracle is handed the projected gradient the GPU produced, so that everything after the
    contraction is held to the full tolerances.

Inputs are seeded numpy arrays drawn in float32 (the generators of tests/golden/cases.py draw in
float64, which is too slow for 65 M elements).
"""
import numpy as np
import pytest
import torch

import cases
import parity
from test_factored_gpu import compare as compare_factored
from test_fullrank_gpu import compare_state as compare_fullrank, state_np, to_cuda_grad

pytestmark = pytest.mark.gpu
f32 = np.float32

TINYLLAMA = [(32000, 2048), (5632, 2048), (256, 2048), (2048,)]
LLAMA2_7B = [(11008, 4096), (4096, 11008), (4096, 4096)]
LLAMA3_8B = [(14336, 4096), (4096, 14336), (1024, 4096)]


def quick_param(shape, seed):
    rng = np.random.default_rng(seed)
    return rng.standard_normal(shape, dtype=f32) * f32(0.02)


def quick_grad(shape, seed, step, spec):
    """Same distributions as cases.make_grad (per-row log-normal scale, exact zeros, spike), bf16 bits."""
    rng = np.random.default_rng([seed, step])
    g = rng.standard_normal(shape, dtype=f32)
    g *= f32(spec["std"])
    if spec.get("dist") == "rowscale" and len(shape) >= 2:
        g *= np.exp(rng.standard_normal((shape[0], 1), dtype=f32))
    zf = spec.get("zero_frac", 0.0)
    if zf > 0:
        g[rng.random(shape, dtype=f32) < zf] = 0.0
    if spec.get("spike_step") == step:
        g *= f32(spec.get("spike_mult", 100.0))
    return cases.f32_to_bf16_bits(g).reshape(shape)


def make(shapes, hp, seed):
    from adafactor8bit import Adafactor8Bit
    p0 = [quick_param(s, seed + i) for i, s in enumerate(shapes)]
    params = [torch.nn.Parameter(torch.from_numpy(p.copy()).cuda()) for p in p0]
    for p in params:
        p.grad_dtype = None
    return p0, params, Adafactor8Bit(params, **hp)


def oracle_step(oracle, p, g, st, hp, **kw):
    if hp["apollo_rank"] > 0 and p.ndim >= 2:
        return oracle.apollo_step(p, g, st, hp, **kw)
    if p.ndim >= 2 and hp["factored"]:
        return oracle.factored_step(p, g, st, hp)
    return oracle.fullrank_step(p.reshape(-1), g.reshape(-1), st, hp)


def run_free(oracle, name, shapes, hp, spec, steps, seed, compare):
    ohp = oracle.hyper(**hp)
    p0, params, opt = make(shapes, hp, seed)
    oparams = [p.copy() for p in p0]
    ostates = [oracle.init_state(s, ohp) for s in shapes]
    k = 1
    for st in ostates:                       # projection seeds in parameter order (optimizer.py:1727-1728)
        if "apollo_seed" in st:
            st["apollo_seed"] = k
            k += 1
    for t in range(1, steps + 1):
        grads = [quick_grad(s, seed + 100 + i, t, spec) for i, s in enumerate(shapes)]
        for p, g in zip(params, grads):
            p.grad = to_cuda_grad(g, p.shape)
        opt.step()
        for i in range(len(shapes)):
            oracle_step(oracle, oparams[i], grads[i], ostates[i], ohp)
        torch.cuda.synchronize()
        for i, p in enumerate(params):
            compare(name, t, i, opt.state[p], ostates[i], p, oparams[i])
            if "fira_prev_norm" in ostates[i]:
                a, b = float(opt.state[p]["fira_prev_norm"].item()), float(ostates[i]["fira_prev_norm"])
                assert abs(a - b) <= 2e-6 * abs(b), f"{name} t{t} p{i} fira_prev_norm {a} vs {b}"
    from adafactor8bit import _native
    assert _native.device_status(torch.cuda.current_stream().cuda_stream) == 0


def _cmp_mixed(name, t, i, st_gpu, st_cpu, p_gpu, p_cpu):
    """Factored comparison for matrices, full-rank comparison for vectors; parameters at 2e-6."""
    if "row_var_q" in st_cpu or "row_var" in st_cpu:
        compare_factored(name, t, i, st_gpu, st_cpu, p_gpu, p_cpu, param_tol=2e-6)
    else:
        compare_fullrank(name, t, i, st_gpu, st_cpu, p_gpu, p_cpu, strict=False)


def test_adafactor_on_tinyllama_shapes(oracle):
    """Factored Adafactor, constructor defaults (relative step, parameter scaling, clip d = 1), AL8 block 256."""
    run_free(oracle, "adafactor_tinyllama", TINYLLAMA, dict(block_size=256), cases.CASES["adafactor_factored"]["grad"],
             3, 7100, _cmp_mixed)


def test_adamw_limiter_on_tinyllama_shapes(oracle):
    """AdamW UF8/AL8 with the limiter; the gradients of step 3 are 100 times larger."""
    spec = dict(cases.CASES["adamw_fira_bf16"]["grad"], spike_step=3, spike_mult=100.0)
    run_free(oracle, "adamw_fira_tinyllama", TINYLLAMA, cases.CASES["adamw_fira_bf16"]["hp"], spec, 4, 7200,
             lambda *a: compare_fullrank(*a, strict=False))


def test_came_on_llama2_shapes(oracle):
    run_free(oracle, "came_llama2", LLAMA2_7B, cases.CASES["came_al16"]["hp"], cases.CASES["came_al16"]["grad"],
             3, 7300, _cmp_mixed)


def test_came_rows_that_end_inside_a_box(oracle):
    """The residual pass brings four rows in per copy: row counts that are no multiple of 4, of a warp's 32-row
    stride or of the 512-row tile (the rows past the end arrive as zeros and must not count), one tile column
    and several, against the oracle."""
    run_free(oracle, "came_ragged_rows", [(517, 512), (1030, 256), (3, 768), (33, 256)], cases.CASES["came_al16"]["hp"],
             cases.CASES["came_al16"]["grad"], 3, 7400, _cmp_mixed)


APOLLO_HP = dict(cases.CASES["apollo_r32"]["hp"], apollo_rank=256, apollo_update_proj_gap=200)
APOLLO_GRAD = dict(dist="normal", std=1e-3, zero_frac=0.0, dtype="bf16")


def compare_apollo(name, t, i, st_g, st_c, p_gpu, p_cpu, param_tol=2e-6, norm_tol=3e-6):
    what = f"{name} t{t} p{i}"
    assert np.array_equal(st_g["apollo_proj_matrix_T"].cpu().numpy(), st_c["apollo_proj_matrix_T"]), what
    parity.assert_codes(state_np(st_g, "v_low_q"), st_c["v_low_q"], what + " v_low_q")
    parity.assert_codes(state_np(st_g, "m_low_q"), st_c["m_low_q"], what + " m_low_q", zero_reserved=False)
    for key in ("v_low_scale", "v_low_min_log", "m_low_scale"):
        parity.assert_ranges(state_np(st_g, key), st_c[key], what + " " + key, max_ulp=1)
    a, b = float(st_g["scaled_grad_norm_prev"].item()), float(st_c["scaled_grad_norm_prev"])
    assert abs(a - b) <= norm_tol * abs(b), f"{what} scaled_grad_norm_prev {a} vs {b}"
    parity.assert_params(p_gpu.detach().cpu().numpy(), p_cpu, what + " param", tol=param_tol)


def test_apollo_exact_projection_on_llama3_shapes(oracle):
    """Correctly rounded projections on both sides: every quantity at the full tolerances."""
    from adafactor8bit import _engine, optimizer as opt_mod
    opt_mod.APOLLO_RNG_DEVICE = "cpu"
    saved = _engine.EXACT_PROJECTION
    _engine.EXACT_PROJECTION = True
    try:
        run_free(oracle, "apollo_exact_llama3", LLAMA3_8B, APOLLO_HP, APOLLO_GRAD, 2, 7400, compare_apollo)
    finally:
        opt_mod.APOLLO_RNG_DEVICE = None
        _engine.EXACT_PROJECTION = saved


@pytest.mark.parametrize("rows,cols", LLAMA3_8B)
def test_tensor_core_projection_at_k4096(rows, cols):
    """The tcgen05 projection of one real layer (rank 256) against a binary64 product: the error of
    every element stays inside the bound of a binary32 accumulation of its own products."""
    from adafactor8bit import _native as N
    lib = N.lib()
    rank = 256
    rng = np.random.default_rng(rows + cols)
    g = torch.from_numpy(rng.standard_normal((rows, cols), dtype=f32) * f32(1e-3)).to(torch.bfloat16)
    right = rows >= cols
    pt = (rng.standard_normal((cols, rank) if right else (rank, rows), dtype=f32) / f32(np.sqrt(rank))).astype(f32)
    gc = g.to(torch.float32).numpy().astype(np.float64)
    p64 = pt.astype(np.float64)
    want = gc @ p64 if right else p64 @ gc
    bound = 2.0 ** -21 * (np.abs(gc) @ np.abs(p64) if right else np.abs(p64) @ np.abs(gc))
    d_g, d_pt = g.cuda(), torch.from_numpy(pt).cuda()
    out = torch.full((want.size,), float("nan"), dtype=torch.float32, device="cuda")
    chan = torch.empty(max(rows, cols), dtype=torch.float64, device="cuda")
    descs = np.zeros(1, dtype=N.APOLLO_PROJ_DESC)
    nbytes = int(lib.af8_apollo_project_workspace(rows, cols, rank))
    ws = torch.empty(nbytes + 256, dtype=torch.uint8, device="cuda")
    descs["grad"][0], descs["pt"][0], descs["g_low"][0], descs["chan_g2"][0] = d_g.data_ptr(), d_pt.data_ptr(), out.data_ptr(), chan.data_ptr()
    descs["workspace"][0], descs["workspace_bytes"][0] = (ws.data_ptr() + 255) // 256 * 256, nbytes
    descs["rows"][0], descs["cols"][0], descs["rank"][0] = rows, cols, rank
    tb = int(lib.af8_apollo_project_task_bytes())
    h = torch.empty(tb, dtype=torch.uint8).pin_memory()
    d = torch.empty(tb, dtype=torch.uint8, device="cuda")
    t_bytes = 0 if right else rows * cols * 2 + 512      # room for the transposed gradient of a left-case tensor
    t = torch.empty(t_bytes + 256, dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    N.check(lib.af8_apollo_project_batch(descs.ctypes.data, 1, N.BF16, h.data_ptr(), d.data_ptr(),
                                         (t.data_ptr() + 255) // 256 * 256, t_bytes, stream), "project_batch")
    torch.cuda.synchronize()
    assert N.device_status(stream) == 0
    got = out.cpu().numpy().reshape(want.shape).astype(np.float64)
    assert np.isfinite(got).all()
    err = np.abs(got - want)
    assert (err <= bound + 1e-30).all(), float((err / (bound + 1e-30)).max())
    rms = float(np.sqrt((err ** 2).mean()) / np.sqrt((want ** 2).mean()))
    assert rms <= 2e-6, rms                           # the class of a binary32 product, not of a truncating accumulator
    want_ch = (gc ** 2).astype(f32).astype(np.float64).sum(axis=1 if right else 0)
    assert np.allclose(chan.cpu().numpy(), want_ch, rtol=1e-6)      # 8 neighbouring squares are added in binary32 first


def test_apollo_tensor_core_step_teacher_forced_on_g_low(oracle):
    """The product path (tcgen05 projection).  The oracle takes the projected gradient from the GPU,
    and before the second step the GPU takes the oracle's state: everything after the contraction
    (low-rank states, channel scaling, limiter, parameter write) must then meet the full tolerances."""
    from adafactor8bit import _engine, optimizer as opt_mod
    opt_mod.APOLLO_RNG_DEVICE = "cpu"
    assert not _engine.EXACT_PROJECTION
    shapes, hp, seed = LLAMA3_8B, APOLLO_HP, 7500
    try:
        ohp = oracle.hyper(**hp)
        p0, params, opt = make(shapes, hp, seed)
        oparams = [p.copy() for p in p0]
        ostates = [oracle.init_state(s, ohp) for s in shapes]
        for k, st in enumerate(ostates):
            st["apollo_seed"] = k + 1
        for t in (1, 2):
            grads = [quick_grad(s, seed + 100 + i, t, APOLLO_GRAD) for i, s in enumerate(shapes)]
            for p, g in zip(params, grads):
                p.grad = to_cuda_grad(g, p.shape)
            if t > 1:
                for i, p in enumerate(params):
                    st = opt.state[p]
                    p.data.copy_(torch.from_numpy(oparams[i]))
                    for key in ("v_low_q", "v_low_scale", "v_low_min_log", "m_low_q", "m_low_scale"):
                        st[key].copy_(torch.from_numpy(np.asarray(ostates[i][key])).reshape(st[key].shape))
                    st["scaled_grad_norm_prev"].fill_(float(ostates[i]["scaled_grad_norm_prev"]))
            opt.step()
            torch.cuda.synchronize()
            plans = [pl for pl in opt._plans.values() if isinstance(pl, _engine.ApolloPlan)]
            assert len(plans) == 1
            for i, p in enumerate(params):
                g_low = plans[0].g_low[i].cpu().numpy()
                oracle.apollo_step(oparams[i], grads[i], ostates[i], ohp, g_low=g_low)
                compare_apollo("apollo_forced_llama3", t, i, opt.state[p], ostates[i], p, oparams[i], param_tol=1e-5)
        from adafactor8bit import _native
        assert _native.device_status(torch.cuda.current_stream().cuda_stream) == 0
    finally:
        opt_mod.APOLLO_RNG_DEVICE = None
