"""Generates tests/golden/ref_baselines.npz from the reference's own host
baselines (oracle/_ref/libark_ref.so, compiled from the reference checkout by
oracle/Makefile). Run in a container that has the reference checkout:

    make -C oracle && python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
from oracle import oracle as O  # noqa: E402
from tests.golden.cases import build_cases  # noqa: E402


def main():
    out = {}
    for c in build_cases(O):
        o = np.zeros(c["out_shape"], dtype=c["out_np"])
        O.ref_call(c["ref"], [o], c["ins"])
        out[c["name"]] = o
    path = os.path.join(HERE, "ref_baselines.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {len(out)} cases to {path} ({os.path.getsize(path)} bytes)")


if __name__ == "__main__":
    main()
