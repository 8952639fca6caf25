"""Record what the reference package's build_param_groups returns for every scenario of
routing_cases.py into routing_golden.json.

    python tests/golden/gen_routing_golden.py --reference <checkout of the reference>

The reference is imported from the given directory; nothing of it is copied.
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
    import adafactor8bit                      # the reference
    assert os.path.abspath(adafactor8bit.__file__).startswith(os.path.abspath(args.reference))
    import routing_cases as rc
    out = {name: rc.run_scenario(adafactor8bit.build_param_groups, model, kwargs) for name, model, kwargs in rc.SCENARIOS}
    out["__reference_version__"] = adafactor8bit.__version__
    with open(os.path.join(HERE, "routing_golden.json"), "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)
    errs = sum(1 for v in out.values() if isinstance(v, dict) and "error" in v)
    print(f"{len(rc.SCENARIOS)} scenarios recorded ({errs} raise)")


if __name__ == "__main__":
    main()
