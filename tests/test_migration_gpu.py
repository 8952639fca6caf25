"""Group options edited between steps on the CUDA path: the optimizer converts, resets or re-creates
the per-parameter states as the reference's _init_group does (optimizer.py:1650-1860, 976-1045).
Compared step by step with the CPU oracle (itself pinned to the reference's fixtures for these cases)."""
import numpy as np
import pytest
import torch

import cases
import parity
from oracle_runner import OracleRun, golden_entries, load_golden
from test_fullrank_gpu import make_optimizer, state_np, to_cuda_grad

pytestmark = pytest.mark.gpu

CODE_KEYS = ("variance_q", "m_q", "row_var_q", "col_var_q", "conf_row_q", "conf_col_q")
SKIP = ("fira_prev_norm", "prev_update_norm", "lag_fira_scale")


@pytest.mark.parametrize("name", cases.MIGRATION_CASES)
def test_state_migration_matches_oracle(name, oracle):
    run = OracleRun(name)
    params, opt = make_optimizer(run)
    changes = run.case["changes"]
    for t in range(1, run.case["steps"] + 1):
        for k, v in changes.get(t, {}).items():
            for group in opt.param_groups:
                group[k] = v
        for p, g in zip(params, run.grads[t]):
            p.grad = to_cuda_grad(g, p.shape)
        opt.step()
        run.step()
        torch.cuda.synchronize()
        for i, p in enumerate(params):
            st, so = opt.state[p], run.states[i]
            mine = {k for k, v in st.items() if isinstance(v, torch.Tensor) and k not in SKIP}
            theirs = {k for k, v in so.items() if isinstance(v, np.ndarray)}
            assert mine == theirs, f"{name} t{t} p{i}: state entries {sorted(mine ^ theirs)} differ"
            assert st["step"] == so["step"] == t
            assert bool(st["is_quantized"]) == bool(so["is_quantized"])
            for key in theirs:
                what = f"{name} t{t} p{i} {key}"
                a, b = state_np(st, key), np.asarray(so[key]).reshape(-1)
                if key in CODE_KEYS:
                    if key == "m_q" and so.get("m_quant_type") in ("uf4", "d4"):
                        a, b = parity.unpack_nibbles(a), parity.unpack_nibbles(b)
                    parity.assert_codes(a, b, what, al16=(b.dtype == np.uint16), zero_reserved=(key != "m_q"))
                elif key.endswith(("_scale", "_min_log")):
                    parity.assert_ranges(a, b, what, max_ulp=4)
                else:
                    assert parity.rel_l2(a, b) <= 1e-6, what
            parity.assert_params(p.detach().cpu().numpy(), run.params[i], f"{name} t{t} p{i} param", tol=2e-6)
    gold = load_golden(name)            # and the end state against the reference itself
    steps = run.case["steps"]
    for i, p in enumerate(params):
        ref = golden_entries(gold, steps, i)
        parity.assert_params(p.detach().cpu().numpy(), ref["param"], f"{name} final p{i} vs reference")
        theirs = {k for k in ref if k not in ("param",) + SKIP}
        mine = {k for k, v in opt.state[p].items() if isinstance(v, torch.Tensor) and k not in SKIP}
        assert mine == theirs, f"{name} final p{i}: state entries differ from the reference's: {sorted(mine ^ theirs)}"


def test_checkpoint_then_option_change(oracle):
    """A state dict loaded into an optimizer whose group asks for another format is migrated at the
    next step (the loaded states are checked against the options again)."""
    from adafactor8bit import Adafactor8Bit
    name = "migrate_quantize_off_on"
    run = OracleRun(name)
    params, opt = make_optimizer(run)
    for t in (1, 2):
        for p, g in zip(params, run.grads[t]):
            p.grad = to_cuda_grad(g, p.shape)
        opt.step()
    sd = opt.state_dict()
    params2 = [torch.nn.Parameter(p.detach().clone()) for p in params]
    opt2 = Adafactor8Bit(params2, **dict(run.case["hp"], quantize=False))
    sd["param_groups"][0]["quantize"] = False
    opt2.load_state_dict(sd)
    for p, g in zip(params2, run.grads[3]):
        p.grad = to_cuda_grad(g, p.shape)
    opt2.step()
    torch.cuda.synchronize()
    for p in params2:
        st = opt2.state[p]
        assert not st["is_quantized"] and "variance" in st and "variance_q" not in st and "m" in st and st["step"] == 3
