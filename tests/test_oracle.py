"""Pins the C restatement (oracle/ark_oracle.c) to the reference's own host
baselines: against the committed golden vectors (generated from the compiled
reference baselines by tests/golden/make_golden.py) and, when that compiled
library is present, against it live. Also checks the restated matmul and
all_reduce against the closed-form cases the reference tests use."""
import os

import numpy as np
import pytest

from oracle import oracle as O
from tests.golden.cases import build_cases

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_baselines.npz"))
CASES = build_cases(O)


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_oracle_matches_golden(case):
    got = case["oracle"](case["ins"])
    want = GOLD[case["name"]]
    assert got.shape == want.shape
    # bit-exact: compare raw storage
    assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), case["name"]


@pytest.mark.skipif(O.ref_lib() is None, reason="compiled reference baselines not present")
def test_golden_matches_live_reference():
    for c in CASES:
        o = np.zeros(c["out_shape"], dtype=c["out_np"])
        O.ref_call(c["ref"], [o], c["ins"])
        assert np.array_equal(o.view(np.uint8), GOLD[c["name"]].view(np.uint8)), c["name"]


@pytest.mark.parametrize("dt", ["fp32", "fp16", "bf16"])
def test_matmul_constant_inputs(dt):
    # ops_matmul_test.cpp:343-360: all-0.1 inputs, every output equals k * 0.1 * 0.1
    m, n, k = 64, 48, 32
    a = O.to_storage(np.full((m, k), 0.1, np.float32), dt)
    b = O.to_storage(np.full((k, n), 0.1, np.float32), dt)
    c = O.to_f32(O.matmul(a, b, dt), dt)
    a0 = float(O.to_f32(a, dt).flat[0])
    want = O.to_f32(O.to_storage(np.float32(k) * np.float32(a0) * np.float32(a0), dt), dt)
    assert np.allclose(c, want, rtol=2e-3 if dt != "fp32" else 1e-6)


@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
def test_matmul_vs_numpy(ta, tb):
    rng = np.random.default_rng(7)
    m, n, k = 33, 20, 50
    a = rng.uniform(-0.1, 0.1, (k, m) if ta else (m, k)).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, (n, k) if tb else (k, n)).astype(np.float32)
    c = O.matmul(a, b, "fp32", ta, tb)
    want = (a.T if ta else a).astype(np.float64) @ (b.T if tb else b).astype(np.float64)
    assert np.allclose(c, want, atol=1e-5)


def test_matmul_batched_broadcast():
    rng = np.random.default_rng(8)
    a = rng.uniform(-0.1, 0.1, (2, 3, 8, 16)).astype(np.float16)
    b = rng.uniform(-0.1, 0.1, (1, 3, 16, 4)).astype(np.float16)
    c = O.matmul(a, b, "fp16")
    want = np.matmul(a.astype(np.float32), b.astype(np.float32))
    assert c.shape == (2, 3, 8, 4)
    assert np.allclose(c.astype(np.float32), want, atol=2e-3)


@pytest.mark.parametrize("nranks", [2, 4, 8])
def test_all_reduce_closed_form(nranks):
    # ops_all_reduce_test.cpp:9-24: rank r holds r+1 everywhere; result is the exact sum
    ins = [np.full(1024, r + 1, np.float16) for r in range(nranks)]
    out = O.all_reduce(ins, "fp16")
    assert np.all(out == np.float16(nranks * (nranks + 1) / 2))


def test_fused_rows_match_compositions():
    rng = np.random.default_rng(9)
    x = rng.normal(0, 1, (6, 256)).astype(np.float32)
    w = rng.normal(1, 0.1, (256,)).astype(np.float32)
    y = O.rmsnorm(x, w, "fp32", eps=1e-5)
    want = x / np.sqrt((x * x).mean(-1, keepdims=True) + 1e-5) * w
    assert np.allclose(y, want, rtol=1e-5, atol=1e-6)
    s = O.softmax(x, "fp32")
    e = np.exp(x - x.max(-1, keepdims=True))
    assert np.allclose(s, e / e.sum(-1, keepdims=True), rtol=1e-5, atol=1e-7)
    ln = O.layernorm(x, "fp32")
    want = (x - x.mean(-1, keepdims=True)) / np.sqrt(x.var(-1, keepdims=True) + 1e-5)
    assert np.allclose(ln, want, rtol=1e-4, atol=1e-5)
