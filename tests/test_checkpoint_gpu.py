"""state_dict / load_state_dict of the CUDA optimizer: a save-load round trip continues
bit-identically, and a step that starts from the REFERENCE's saved state (the golden
fixtures hold its per-step state tensors) lands on the reference's next state."""
import numpy as np
import pytest
import torch

import parity
from oracle_runner import OracleRun, golden_entries, load_golden
from test_fullrank_gpu import make_optimizer, state_np, to_cuda_grad

pytestmark = pytest.mark.gpu


def _step(params, opt, grads):
    for p, g in zip(params, grads):
        p.grad = to_cuda_grad(g, p.shape)
    opt.step()


@pytest.mark.parametrize("name", ["adamw_fira_bf16", "adamw_uf4_al16", "adafactor_factored_m", "came_al16"])
def test_round_trip_continues_bit_identically(name, oracle):
    from adafactor8bit import Adafactor8Bit
    run = OracleRun(name)
    params, opt = make_optimizer(run)
    steps = run.case["steps"]
    half = steps // 2
    for t in range(1, half + 1):
        _step(params, opt, run.grads[t])
    saved = opt.state_dict()
    # a second optimizer over copies of the parameters, restored from the saved state
    params2 = [torch.nn.Parameter(p.detach().clone()) for p in params]
    for p in params2:
        p.grad_dtype = None                              # bf16 gradients on fp32 parameters
    opt2 = Adafactor8Bit(params2, **run.case["hp"])
    opt2.load_state_dict({"state": {k: {kk: (vv.clone() if isinstance(vv, torch.Tensor) else vv) for kk, vv in v.items()}
                                    for k, v in saved["state"].items()},
                          "param_groups": saved["param_groups"],
                          **{k: v for k, v in saved.items() if k not in ("state", "param_groups")}})
    for t in range(half + 1, steps + 1):
        _step(params, opt, run.grads[t])
        _step(params2, opt2, run.grads[t])
    torch.cuda.synchronize()
    for p, q in zip(params, params2):
        assert torch.equal(p.detach(), q.detach())
        for key, val in opt.state[p].items():
            other = opt2.state[q][key]
            if isinstance(val, torch.Tensor):
                assert val.dtype == other.dtype and torch.equal(val, other), (name, key)
            else:
                assert val == other, (name, key)


@pytest.mark.parametrize("name", ["adamw_uf8_al8", "adamw_fira_bf16", "adafactor_factored_m"])
def test_step_from_the_reference_state(name, oracle):
    """Reference state after step t in, one CUDA step, reference state after step t+1 out."""
    run = OracleRun(name)
    gold = load_golden(name)
    params, opt = make_optimizer(run)
    _step(params, opt, run.grads[1])                     # creates the state entries and their metadata
    steps = run.case["steps"]
    for t in range(1, steps):
        for i, p in enumerate(params):                   # overwrite parameters and state with the reference's at step t
            ref, st = golden_entries(gold, t, i), opt.state[p]
            p.data.copy_(torch.from_numpy(ref["param"]).reshape(p.shape))
            for key, val in ref.items():
                if key in st and isinstance(st[key], torch.Tensor):
                    src = torch.from_numpy(val.view(np.int16) if val.dtype == np.uint16 else val)
                    st[key].copy_(src.reshape(st[key].shape))
            st["step"] = t
        _step(params, opt, run.grads[t + 1])
        torch.cuda.synchronize()
        for i, p in enumerate(params):
            ref = golden_entries(gold, t + 1, i)
            what = f"{name} t{t + 1} p{i}"
            parity.assert_params(p.detach().cpu().numpy(), ref["param"], what + " param", tol=1e-6)
            for key in ("variance_q", "m_q", "row_var_q", "col_var_q"):
                if key in ref:
                    a, b = state_np(opt.state[p], key), np.asarray(ref[key]).reshape(-1)
                    if key == "m_q" and run.hp.get("m_quant_type") in ("uf4", "d4"):
                        a, b = parity.unpack_nibbles(a), parity.unpack_nibbles(b)
                    parity.assert_codes(a, b, what + " " + key, al16=(b.dtype == np.uint16), zero_reserved=(key != "m_q"))
            for key in ("variance_scale", "variance_min_log", "m_scale"):
                if key in ref:
                    parity.assert_ranges(state_np(opt.state[p], key), ref[key], what + " " + key, max_ulp=1)
