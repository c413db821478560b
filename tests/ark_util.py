"""Helpers for the GPU parity tests: build a model with the ark_b200 front end,
run it through the C ABI (Executor) and hand back numpy arrays to compare with
the CPU oracle."""
import numpy as np

import ark_b200 as ark
from oracle import oracle as O

NAME = {"fp32": ark.fp32, "fp16": ark.fp16, "bf16": ark.bf16, "int32": ark.int32}


def rand(rng, shape, dt, lo=-0.1, hi=0.1):
    """Uniform values like the reference's op_test (ark/ops/ops_test_common.cpp:52-66), in storage type."""
    return O.to_storage(rng.uniform(lo, hi, size=shape).astype(np.float32), dt)


def execute(outputs, feeds, loop_mode=False, iters=1, plan=None, wait_limit_ns=3_000_000_000, keep=False):
    plan = plan if plan is not None else ark.Planner(0).plan()
    ex = ark.Executor(0, 0, "test", str(plan), loop_mode)
    try:
        ex.set_wait_limit(wait_limit_ns)
        ex.compile()
        for t, arr in feeds.items():
            ex.tensor_from_numpy(t, arr)
        ex.launch()
        ex.run(iters)
        ex.wait()
        outs = [ex.tensor_to_numpy(t) for t in outputs]
        ex.stop()
    finally:
        if not keep:
            ex.destroy()
    return outs if not keep else (outs, ex)


def ulp_tol(dt):
    return {"fp32": 4e-6, "fp16": 2.0 ** -9, "bf16": 2.0 ** -7}[dt]


def assert_close(got, want, dt, rtol=None, atol=0.0, what=""):
    """Element check |got - want| <= atol + rtol * |want| on fp32 views."""
    g, w = O.to_f32(got, dt).astype(np.float64), O.to_f32(want, dt).astype(np.float64)
    rtol = ulp_tol(dt) if rtol is None else rtol
    err = np.abs(g - w)
    bad = err > (atol + rtol * np.abs(w))
    assert not bad.any(), f"{what}: {bad.sum()} of {bad.size} off; max abs err {err.max():.3e}, at {np.argmax(err)}: got {g.flat[np.argmax(err)]} want {w.flat[np.argmax(err)]}"


def assert_matmul_close(got, want, dt, what=""):
    """The tolerance stated for fp16/bf16 matmul with fp32 accumulation:
    max relative error <= 1e-2 or mean absolute error <= 2e-3."""
    g, w = O.to_f32(got, dt).astype(np.float64), O.to_f32(want, dt).astype(np.float64)
    err = np.abs(g - w)
    denom = np.maximum(np.abs(w), 1e-3)
    max_rel = float((err / denom).max())
    mean_abs = float(err.mean())
    assert max_rel <= 1e-2 or mean_abs <= 2e-3, f"{what}: max rel {max_rel:.3e}, mean abs {mean_abs:.3e}"
    # and never grossly wrong anywhere
    assert float(err.max()) <= 0.05 * max(1.0, float(np.abs(w).max())), f"{what}: max abs err {err.max():.3e}"
