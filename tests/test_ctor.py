"""The constructor against the reference's: same keyword names, order and defaults, and the same
verdict (accepted with the same group defaults, or refused with the same exception type) on every
scenario of tests/golden/ctor_cases.py (recorded by gen_ctor_golden.py)."""
import json
import os

import pytest

import ctor_cases as cc

GOLDEN = json.load(open(os.path.join(os.path.dirname(os.path.abspath(cc.__file__)), "ctor_golden.json")))


def test_signature_matches_reference():
    from adafactor8bit import Adafactor8Bit
    assert cc.signature_of(Adafactor8Bit) == GOLDEN["signature"]


@pytest.mark.parametrize("name,kwargs", cc.SCENARIOS, ids=[s[0] for s in cc.SCENARIOS])
def test_constructor_verdict_matches_reference(name, kwargs):
    from adafactor8bit import Adafactor8Bit
    got, want = cc.run_scenario(Adafactor8Bit, kwargs), GOLDEN["scenarios"][name]
    if "error" in want:
        assert got == want
        return
    assert "ok" in got, got
    for k, v in want["ok"].items():
        assert got["ok"].get(k) == v, (k, got["ok"].get(k), v)
