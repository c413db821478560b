"""Packs the multi-rank plan files the reference ships (examples/tutorial/allreduce-sm/plan_gpu{0..7}.json and
examples/tutorial/allreduce-packet/plan_gpu{0..7}.json) into tests/golden/ref_allreduce_plans.json.gz, byte for byte, so
that the tests can load and run them where no reference checkout exists.

    python tests/golden/make_ref_plans.py <reference checkout>
"""
import gzip
import json
import os
import sys


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("ARK_REFERENCE_DIR", "")
    base = os.path.join(ref, "examples", "tutorial")
    out = {}
    for d in ("allreduce-sm", "allreduce-packet"):
        for r in range(8):
            with open(os.path.join(base, d, f"plan_gpu{r}.json")) as f:
                out[f"{d}/plan_gpu{r}.json"] = f.read()
    here = os.path.dirname(os.path.abspath(__file__))
    with gzip.open(os.path.join(here, "ref_allreduce_plans.json.gz"), "wt", compresslevel=9) as f:
        json.dump(out, f)
    print(f"packed {len(out)} plans")


if __name__ == "__main__":
    main()
