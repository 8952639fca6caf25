"""build_param_groups / policies against what the reference package returns for the same
models and arguments (tests/golden/routing_golden.json, recorded by gen_routing_golden.py)."""
import json
import os

import pytest

import routing_cases as rc

GOLDEN = json.load(open(os.path.join(os.path.dirname(os.path.abspath(rc.__file__)), "routing_golden.json")))


@pytest.mark.parametrize("name,model,kwargs", rc.SCENARIOS, ids=[s[0] for s in rc.SCENARIOS])
def test_groups_match_reference(name, model, kwargs):
    from adafactor8bit import build_param_groups
    got, want = rc.run_scenario(build_param_groups, model, kwargs), GOLDEN[name]
    if "error" in want:
        assert got == want                          # the same exception type
        return
    assert "error" not in got, got
    assert [g["group_name"] for g in got["groups"]] == [g["group_name"] for g in want["groups"]]
    for a, b in zip(got["groups"], want["groups"]):
        assert a == b, (a["group_name"], {k: (a.get(k), b.get(k)) for k in set(a) | set(b) if a.get(k) != b.get(k)})
    assert got["warnings"] == want["warnings"]


def test_presets_table_matches_reference_values():
    from adafactor8bit.presets import PRESETS
    assert tuple(PRESETS) == ("sgd", "adafactor", "adamw", "rmsprop", "came", "apollo")
    assert PRESETS["adamw"].primary["eps"] == (1e-8, 1e-3) and PRESETS["adamw"].primary["beta2"] == 0.999
    assert PRESETS["came"].primary["beta3"] == 0.9999 and PRESETS["came"].primary["d"] == 1.0
    assert PRESETS["apollo"].default_apollo_rank == 256 and PRESETS["apollo"].fallback["eps"] == (1e-6, 1e-3)
    assert all(s.default_grouping == "G1" for s in PRESETS.values())


def test_groups_feed_the_constructor_validation():
    """Generated groups are accepted by the optimizer's constructor on CPU parameters
    (no launch happens before step())."""
    from adafactor8bit import Adafactor8Bit, build_param_groups
    model = rc.MODELS["llama"]()
    for preset in ("adamw", "came", "adafactor", "rmsprop", "sgd"):
        opt = Adafactor8Bit(build_param_groups(model, preset), lr=1e-3)
        assert [g["group_name"] for g in opt.param_groups][0] == "one_d"
