"""The allocation-free skinny matmul entry point (arkb_matvec_splitk_static) against the
engine's regular Matmul path, through the C ABI. It serves callers that must not allocate
device memory when they need the product (a stream capture in progress, a pre-allocated
real-time loop, a plug-in inside someone else's memory pool): its split-K partial sums
live in a fixed 4 MiB array inside the library. Two calls in a row with different inputs
check that what the first call left in that shared array does not leak into the second;
a problem too large for the array must be refused, not truncated.

This file sorts last on purpose: a run that stops at the first failure has already run
every other test."""
import ctypes

import numpy as np
import pytest

import ark_b200 as ark
from ark_b200.executor import matvec_splitk_static
from oracle import oracle as O
from tests.ark_util import NAME, assert_matmul_close, execute, rand

pytestmark = pytest.mark.gpu


def engine_matmul(x, w, dt):
    """Reference result from the existing entry points (Executor + Matmul plan)."""
    ark.init()
    tx, tw = ark.tensor(list(x.shape), NAME[dt]), ark.tensor(list(w.shape), NAME[dt])
    out = ark.matmul(tx, tw, transpose_other=True)
    (got,) = execute([out], {tx: x, tw: w})
    return got


@pytest.mark.parametrize("dt", ["fp16", "bf16"])
def test_static_scratch_matvec_matches_engine_twice(dt):
    import torch
    tdt = torch.float16 if dt == "fp16" else torch.bfloat16
    rng = np.random.default_rng(71)
    for call, (m, n, k) in enumerate([(4, 4096, 2048), (1, 1376, 4096)]):
        x, w = rand(rng, (m, k), dt, -1.0, 1.0), rand(rng, (n, k), dt, -0.05, 0.05)
        want = engine_matmul(x, w, dt)
        dx = torch.from_numpy(x.view(np.int16)).cuda().view(tdt)
        dw = torch.from_numpy(w.view(np.int16)).cuda().view(tdt)
        dy = torch.empty((m, n), dtype=tdt, device="cuda")
        torch.cuda.synchronize()
        matvec_splitk_static(dx.data_ptr(), dw.data_ptr(), dy.data_ptr(), m, n, k, dt)
        torch.cuda.synchronize()
        got = dy.view(torch.int16).cpu().numpy().view(O.NP[dt])
        assert_matmul_close(got, want, dt, f"static-scratch matvec, call {call}")
        assert_matmul_close(got, O.matmul(x, w, dt, trans_b=True), dt, f"static-scratch matvec vs oracle, call {call}")


@pytest.mark.parametrize("m,n,k", [(16, 1000, 1096), (3, 64, 8), (16, 264, 520)])
def test_static_scratch_matvec_ragged_k_and_full_rows(m, n, k):
    """K that is not a multiple of the 256-element lane stride (the tail of the last k-range, a K below one
    stride) and all 16 accumulator rows, on random data, against the engine and the oracle."""
    import torch
    dt = "fp16"
    rng = np.random.default_rng(73 + m + k)
    x, w = rand(rng, (m, k), dt, -1.0, 1.0), rand(rng, (n, k), dt, -0.05, 0.05)
    dx = torch.from_numpy(x.view(np.int16)).cuda().view(torch.float16)
    dw = torch.from_numpy(w.view(np.int16)).cuda().view(torch.float16)
    dy = torch.empty((m, n), dtype=torch.float16, device="cuda")
    torch.cuda.synchronize()
    for call in range(2):
        dy.zero_()
        matvec_splitk_static(dx.data_ptr(), dw.data_ptr(), dy.data_ptr(), m, n, k, dt)
        torch.cuda.synchronize()
        got = dy.view(torch.int16).cpu().numpy().view(O.NP[dt])
        assert_matmul_close(got, O.matmul(x, w, dt, trans_b=True), dt, f"static-scratch matvec {m}x{n}x{k} vs oracle, call {call}")
    assert_matmul_close(got, engine_matmul(x, w, dt), dt, f"static-scratch matvec {m}x{n}x{k} vs engine")


def test_static_scratch_rejects_oversized_and_bad_arguments():
    import torch
    x = torch.zeros((16, 512), dtype=torch.float16, device="cuda")
    w = torch.zeros((8, 512), dtype=torch.float16, device="cuda")
    y = torch.zeros((16, 8), dtype=torch.float16, device="cuda")
    with pytest.raises(ark.InvalidUsageError):  # 16 x 200000 partials exceed 4 MiB
        matvec_splitk_static(x.data_ptr(), w.data_ptr(), y.data_ptr(), 16, 200000, 512, "fp16")
    with pytest.raises(ark.InvalidUsageError):
        matvec_splitk_static(x.data_ptr(), w.data_ptr(), y.data_ptr(), 17, 8, 512, "fp16")
    with pytest.raises(ark.InvalidUsageError):
        matvec_splitk_static(x.data_ptr(), w.data_ptr(), y.data_ptr(), 16, 8, 500, "fp16")
    matvec_splitk_static(x.data_ptr(), w.data_ptr(), y.data_ptr(), 16, 8, 512, "fp16")  # still usable afterwards
    torch.cuda.synchronize()
    assert float(y.abs().max()) == 0.0
