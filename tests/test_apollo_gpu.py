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


def test_apollo_free_running_matches_oracle(oracle):
    from adafactor8bit import optimizer as opt_mod
    name = "apollo_r32"
    run = OracleRun(name)
    opt_mod.APOLLO_RNG_DEVICE = "cpu"
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
                    parity.assert_codes(state_np(st_g, "v_low_q"), st_c["v_low_q"], what + " v_low_q")
                    parity.assert_codes(state_np(st_g, "m_low_q"), st_c["m_low_q"], what + " m_low_q", zero_reserved=False)
                    for key in ("v_low_scale", "v_low_min_log", "m_low_scale"):
                        parity.assert_ranges(state_np(st_g, key), st_c[key], what + " " + key, max_ulp=1)
                    a, b = float(st_g["scaled_grad_norm_prev"].item()), float(st_c["scaled_grad_norm_prev"])
                    assert abs(a - b) <= 3e-6 * abs(b), f"{what} scaled_grad_norm_prev {a} vs {b}"
                parity.assert_params(p.detach().cpu().numpy(), run.params[i], what + " param", tol=2e-6)
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
