"""load_state_dict with checkpoints of older formats, as the reference handles them
(adafactor8bit/optimizer.py:1469-1553): groups saved without a stochastic-rounding policy inherit the
current one, counters that the checkpoint lacks start from 0, and full-size momentum left in an
APOLLO state is dropped.  Runs without a GPU (loading touches no kernel)."""
import torch


def _opt(**kw):
    from adafactor8bit import Adafactor8Bit
    p = [torch.nn.Parameter(torch.zeros(8, 4)), torch.nn.Parameter(torch.zeros(16))]
    return p, Adafactor8Bit(p, **kw)


def test_groups_saved_without_sr_policy_inherit_the_current_one():
    _, opt = _opt(stochastic_round_writeback=True)
    sd = opt.state_dict()
    for g in sd["param_groups"]:
        del g["stochastic_round_writeback"]
    opt.load_state_dict(sd)
    assert opt.param_groups[0]["stochastic_round_writeback"] is True
    sd = opt.state_dict()
    sd["param_groups"][0]["stochastic_round_writeback"] = False     # a saved policy wins
    opt.load_state_dict(sd)
    assert opt.param_groups[0]["stochastic_round_writeback"] is False


def test_missing_counters_start_from_zero():
    _, opt = _opt()
    opt._apollo_seed_counter, opt._sr_seed_counter = 7, 9
    sd = opt.state_dict()
    assert sd["_apollo_seed_counter"] == 7 and sd["_sr_seed_counter"] == 9
    del sd["_apollo_seed_counter"], sd["_sr_seed_counter"]
    opt.load_state_dict(sd)
    assert opt._apollo_seed_counter == 0 and opt._sr_seed_counter == 0
    opt._apollo_seed_counter = 5
    opt.load_state_dict(opt.state_dict())
    assert opt._apollo_seed_counter == 5


def test_stale_full_size_momentum_of_an_apollo_state_is_dropped():
    params, opt = _opt(apollo_rank=2, beta1=0.9, beta2=0.999, relative_step=False, scale_parameter=False)
    sd = opt.state_dict()
    sd["state"] = {
        0: {"step": 3, "apollo_seed": 11, "apollo_rank": 2, "is_quantized": True, "m_q": torch.zeros(256, dtype=torch.uint8),
            "m_scale": torch.ones(1), "m": torch.zeros(8, 4), "m_low_q": torch.full((256,), 128, dtype=torch.uint8),
            "m_low_scale": torch.ones(1), "m_quant_type": "uf8", "v_quant_type": "al8"},
        1: {"step": 3, "is_quantized": False, "m": torch.ones(16), "variance": torch.ones(16), "m_quant_type": "fp32"},
    }
    opt.load_state_dict(sd)
    st = opt.state[params[0]]
    assert "m_q" not in st and "m_scale" not in st and "m" not in st
    assert st["m_low_q"].dtype == torch.uint8 and st["step"] == 3 and st["apollo_seed"] == 11
    assert "m" in opt.state[params[1]]                       # other states keep their momentum
