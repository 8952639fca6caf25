"""Parity of the CUDA factored path (Adafactor, CAME) with the CPU oracle and the
reference's golden vectors, through the optimizer class."""
import numpy as np
import pytest
import torch

import cases
import parity
from oracle_runner import FACTORED_CASES, OracleRun, golden_entries, load_golden
from test_fullrank_gpu import make_optimizer, state_np, to_cuda_grad

pytestmark = pytest.mark.gpu

CODE_KEYS = ("row_var_q", "col_var_q", "conf_row_q", "conf_col_q", "variance_q", "m_q")
RANGE_KEYS = ("row_var_scale", "row_var_min_log", "col_var_scale", "col_var_min_log", "conf_row_scale",
              "conf_row_min_log", "conf_col_scale", "conf_col_min_log", "variance_scale", "variance_min_log", "m_scale")
F32_KEYS = ("row_var", "col_var", "conf_row", "conf_col", "variance", "m")


def compare(name, t, i, st_gpu, st_cpu, p_gpu, p_cpu, param_tol):
    for key in CODE_KEYS:
        if key in st_cpu:
            a, b = state_np(st_gpu, key), np.asarray(st_cpu[key]).reshape(-1)
            parity.assert_codes(a, b, f"{name} t{t} p{i} {key}", al16=(b.dtype == np.uint16),
                                zero_reserved=(key != "m_q"))
    for key in RANGE_KEYS:
        if key in st_cpu:
            parity.assert_ranges(state_np(st_gpu, key), st_cpu[key], f"{name} t{t} p{i} {key}", max_ulp=4)
    for key in F32_KEYS:
        if key in st_cpu:
            assert parity.rel_l2(state_np(st_gpu, key), st_cpu[key]) <= 1e-6, f"{name} t{t} p{i} {key}"
    parity.assert_params(p_gpu.detach().cpu().numpy(), p_cpu, f"{name} t{t} p{i} param", tol=param_tol)


# Cases without fixtures.  "odd": column counts that are not multiples of 8 take the
# element-wise kernels; "tiles": several statistic tiles per tensor with ragged edges and
# chunks that end inside a momentum block, through the 128-bit kernels.
EXTRA_CASES = {
    "adafactor_odd": dict(shapes=[(37, 131), (50, 100)], steps=3, seed=31, grad=cases.CASES["adafactor_factored"]["grad"],
                          hp=cases.CASES["adafactor_factored"]["hp"]),
    "adafactor_m_odd": dict(shapes=[(37, 131), (130, 273)], steps=3, seed=32, grad=cases.CASES["adafactor_factored_m"]["grad"],
                            hp=cases.CASES["adafactor_factored_m"]["hp"]),
    "came_odd": dict(shapes=[(33, 77), (129, 300)], steps=3, seed=33, grad=cases.CASES["came_al16"]["grad"],
                     hp=cases.CASES["came_al16"]["hp"]),
    "adafactor_tiles": dict(shapes=[(200, 520), (70, 264), (3, 8)], steps=3, seed=34,
                            grad=cases.CASES["adafactor_factored"]["grad"], hp=cases.CASES["adafactor_factored"]["hp"]),
    "adafactor_m_tiles": dict(shapes=[(200, 520), (70, 264), (3, 8)], steps=3, seed=35,
                              grad=cases.CASES["adafactor_factored_m"]["grad"], hp=cases.CASES["adafactor_factored_m"]["hp"]),
    "adafactor_m_uf4_tiles": dict(shapes=[(200, 520), (5, 24)], steps=3, seed=36,
                                  grad=cases.CASES["adafactor_factored_m"]["grad"],
                                  hp=dict(cases.CASES["adafactor_factored_m"]["hp"], m_quant_type="uf4")),
    "came_tiles": dict(shapes=[(200, 520), (70, 264), (3, 8)], steps=3, seed=37, grad=cases.CASES["came_al16"]["grad"],
                       hp=dict(cases.CASES["came_al16"]["hp"], block_size=256)),
}


# column counts that are multiples of 2048: the apply pass walks such tensors strip by strip
EXTRA_CASES.update({
    "adafactor_strips": dict(shapes=[(5, 2048), (70, 4096), (1, 2048), (33, 6144)], steps=3, seed=39,
                             grad=cases.CASES["adafactor_factored"]["grad"], hp=cases.CASES["adafactor_factored"]["hp"]),
    "adafactor_m_strips": dict(shapes=[(5, 2048), (70, 4096), (33, 6144)], steps=3, seed=40,
                               grad=cases.CASES["adafactor_factored_m"]["grad"], hp=cases.CASES["adafactor_factored_m"]["hp"]),
    "came_strips": dict(shapes=[(5, 2048), (70, 4096), (33, 6144)], steps=3, seed=41, grad=cases.CASES["came_al16"]["grad"],
                        hp=cases.CASES["came_al16"]["hp"]),
})

# lag_norm=True (one pass with the previous step's norm; optimizer.py:1056-1071): the vector kernels, the
# element-wise kernels (odd column counts) and the limiter on top of the clip
EXTRA_CASES.update({
    "adafactor_lag": dict(cases.CASES["adafactor_factored"], steps=5,
                          hp=dict(cases.CASES["adafactor_factored"]["hp"], lag_norm=True)),
    "adafactor_m_lag_fira": dict(shapes=[(200, 520), (37, 131)], steps=5, seed=38,
                                 grad=dict(cases.CASES["adafactor_factored_m"]["grad"], spike_step=3, spike_mult=50.0),
                                 hp=dict(cases.CASES["adafactor_factored_m"]["hp"], lag_norm=True,
                                         enable_fira_for_adafactor=True)),
})


@pytest.mark.parametrize("name", FACTORED_CASES + cases.FACTORED_3D_CASES + sorted(EXTRA_CASES))
def test_factored_free_running_matches_oracle(name, oracle):
    run = OracleRun(name, EXTRA_CASES.get(name))
    params, opt = make_optimizer(run)
    steps = run.case["steps"]
    for t in range(1, steps + 1):
        for p, g in zip(params, run.grads[t]):
            p.grad = to_cuda_grad(g, p.shape)
        opt.step()
        run.step()
        torch.cuda.synchronize()
        for i, p in enumerate(params):
            compare(name, t, i, opt.state[p], run.states[i], p, run.params[i], param_tol=2e-6)
            for key in ("prev_update_norm", "lag_fira_scale"):
                if key in run.states[i]:
                    a, b = float(opt.state[p][key].item()), float(run.states[i][key])
                    assert abs(a - b) <= 2e-6 * max(abs(b), 1.0), f"{name} t{t} p{i} {key}: {a} vs {b}"
    if run.hp["lag_norm"]:
        assert all("prev_update_norm" in opt.state[p] for p in params if p.dim() == 2)
    from adafactor8bit import _native
    assert _native.device_status(torch.cuda.current_stream().cuda_stream) == 0


@pytest.mark.parametrize("name", ["adafactor_factored", "adafactor_factored_m"] + cases.FACTORED_3D_CASES)
def test_factored_matches_reference_golden(name, oracle):
    run = OracleRun(name)
    gold = load_golden(name)
    params, opt = make_optimizer(run)
    steps = run.case["steps"]
    for t in range(1, steps + 1):
        for p, g in zip(params, run.grads[t]):
            p.grad = to_cuda_grad(g, p.shape)
        opt.step()
    torch.cuda.synchronize()
    for i, p in enumerate(params):
        ref = golden_entries(gold, steps, i)
        # (CAME with the limiter: torch's float32 norm puts the reference's limiter state 2e-5 off the accurately
        # summed one, which the parameters then carry)
        parity.assert_params(p.detach().cpu().numpy(), ref["param"], f"{name} final p{i} vs reference",
                             tol=5e-5 if name == "came_3d" else 1e-6)
        for key in CODE_KEYS:
            if key in ref:
                parity.assert_codes(state_np(opt.state[p], key), ref[key], f"{name} final p{i} {key} vs reference",
                                    al16=(ref[key].dtype == np.uint16), zero_reserved=(key != "m_q"))
