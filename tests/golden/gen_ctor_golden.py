"""Record the reference constructor's signature and its verdict on every scenario of
ctor_cases.py into ctor_golden.json.

    python tests/golden/gen_ctor_golden.py --reference <checkout of the reference>
"""
import argparse
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="directory that contains the reference's adafactor8bit package")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    sys.path.insert(0, HERE)
    import adafactor8bit
    assert os.path.abspath(adafactor8bit.__file__).startswith(os.path.abspath(args.reference))
    import ctor_cases as cc
    out = {"signature": cc.signature_of(adafactor8bit.Adafactor8Bit),
           "scenarios": {name: cc.run_scenario(adafactor8bit.Adafactor8Bit, kw) for name, kw in cc.SCENARIOS}}
    with open(os.path.join(HERE, "ctor_golden.json"), "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)
    print(len(cc.SCENARIOS), "scenarios,", sum("error" in v for v in out["scenarios"].values()), "refused")


if __name__ == "__main__":
    main()
