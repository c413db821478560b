"""GPU tests of the executor protocol through the C ABI: loop mode, repeated
runs, error behaviour pinned by the reference's executor tests
(ark/api/executor_test.cpp:47-59, 149-155, 171-183), the idle exit of the
resident kernel and serialised kernel launches. (The bounded-wait status path
is in tests/test_gpu_multi.py: it needs a peer that stays silent.)"""
import os
import subprocess
import sys
import time

import numpy as np
import pytest

import ark_b200 as ark
from oracle import oracle as O
from tests.ark_util import assert_close, execute, rand

pytestmark = pytest.mark.gpu


def build_chain():
    ark.init()
    t = ark.tensor([64, 1024], ark.fp16)
    o = ark.add(t, 1.0, t)  # in place: x += 1 every iteration
    return t, o


def test_device_info():
    di = ark.device_info(0)
    assert di["arch"] == "CUDA_100" and di["num_sm"] >= 100


@pytest.mark.parametrize("loop_mode", [False, True])
def test_iterations_accumulate(loop_mode):
    t, o = build_chain()
    x = np.zeros((64, 1024), np.float16)
    ex = ark.Executor(0, 0, "t", str(ark.Planner(0).plan()), loop_mode)
    ex.set_wait_limit(3_000_000_000)
    ex.compile()
    ex.tensor_from_numpy(t, x)
    ex.launch()
    ex.run(3)
    ex.wait()
    ex.run(2)
    ex.wait()
    got = ex.tensor_to_numpy(o)
    ms = ex.stop()
    st = ex.status()
    ex.destroy()
    assert np.all(got == 5.0)
    assert ms >= 0 and st["code"] == 0 and st["iterations"] == 5
    assert st["n_launches"] == (1 if loop_mode else 2)


def test_relaunch_after_stop():
    t, o = build_chain()
    ex = ark.Executor(0, 0, "t", str(ark.Planner(0).plan()), True)
    ex.compile()
    ex.tensor_from_numpy(t, np.zeros((64, 1024), np.float16))
    for expect in (1.0, 2.0):
        ex.launch()
        ex.run(1)
        ex.wait()
        ex.stop()
        assert np.all(ex.tensor_to_numpy(o) == expect)
    ex.destroy()
    assert ex.destroyed()


def test_idle_exit_is_followed_by_a_relaunch():
    """The resident kernel leaves after the idle limit; the next request brings it back and every requested
    iteration runs (the count the kernel reports is checked by wait())."""
    t, o = build_chain()
    ex = ark.Executor(0, 0, "t", str(ark.Planner(0).plan()), True)
    ex.set_wait_limit(3_000_000_000)
    ex.set_idle_limit(30_000_000)  # 30 ms
    ex.compile()
    ex.tensor_from_numpy(t, np.zeros((64, 1024), np.float16))
    ex.launch()
    time.sleep(0.3)
    ex.run(2)
    ex.wait()
    time.sleep(0.3)
    ex.run(1)
    ex.wait()
    ex.run(4)  # back to back: the kernel is still there
    ex.wait()
    got = ex.tensor_to_numpy(o)
    ex.stop()
    st = ex.status()
    ex.destroy()
    assert np.all(got == 7.0)
    assert st["iterations"] == 7 and st["n_launches"] >= 3 and st["code"] in (0, 4)


_BLOCKING = r"""
import sys
sys.path.insert(0, sys.argv[1])
import numpy as np
import __graft_entry__ as g
import ark_b200 as ark
g.smoke()  # loop mode: FFN block + rmsnorm against the oracle
ark.init()
t = ark.tensor([64, 1024], ark.fp16)
o = ark.add(t, 1.0, t)
ex = ark.Executor(0, 0, "t", str(ark.Planner(0).plan()), True)
ex.set_idle_limit(50_000_000)
ex.compile()
ex.tensor_from_numpy(t, np.zeros((64, 1024), np.float16))
ex.launch()
ex.run(3); ex.wait()
ex.run(2); ex.wait()
got = ex.tensor_to_numpy(o)
ex.stop()
st = ex.status()
ex.destroy()
assert np.all(got == 5.0), got[0, :4]
assert st["iterations"] == 5 and st["code"] == 0, st
print("blocking ok", st["n_launches"])
"""


def test_serialised_launches_give_right_numbers(tmp_path):
    """With CUDA_LAUNCH_BLOCKING=1 (as under a profiler) a launch only returns when the kernel has ended, so a
    resident kernel can never see a request posted after its launch: the executor notices and serves every
    run() with a launch of its own. Right numbers, never a silent success without work."""
    script = tmp_path / "blocking.py"
    script.write_text(_BLOCKING)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, CUDA_LAUNCH_BLOCKING="1")
    t0 = time.perf_counter()
    p = subprocess.run([sys.executable, str(script), root], capture_output=True, text=True, timeout=600, env=env)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    assert "smoke ok" in p.stdout and "blocking ok" in p.stdout
    assert time.perf_counter() - t0 < 120


def test_usage_errors():
    t, o = build_chain()
    plan = str(ark.Planner(0).plan())
    with pytest.raises(ark.InvalidUsageError):
        ark.Executor(-1, 0, "t", plan, True)
    ex = ark.Executor(0, 0, "t", plan, True)
    with pytest.raises(ark.InvalidUsageError):
        ex.launch()  # launch before compile
    ex.compile()
    ex.launch()
    ex.launch()  # second launch is ignored
    with pytest.raises(ark.InvalidUsageError):
        ex.tensor_to_numpy(o, np.zeros(3, np.float16))  # size mismatch
    ex.stop()
    ex.destroy()
    with pytest.raises(ark.PlanError):
        ark.Executor(0, 0, "t", "{not json", True)


def test_tensor_io_strided_roundtrip():
    ark.init()
    t = ark.tensor([4, 3, 10, 20], ark.fp32, strides=[4, 3, 16, 32], offsets=[0, 0, 2, 8], padded_shape=[4, 3, 10, 20])
    o = ark.mul(t, 2.0)
    x = np.random.default_rng(41).normal(size=(4, 3, 10, 20)).astype(np.float32)
    (got,) = execute([o], {t: x})
    assert np.array_equal(got, x * 2)


def test_multi_op_plan_ffn_block():
    """Config 1 of the benchmark set: Y = ReLU(X W1) W2, fp16 with fp32 accumulate."""
    rng = np.random.default_rng(0)
    x = O.to_storage(rng.normal(0, 1, (128, 1024)).astype(np.float32), "fp16")
    w1 = O.to_storage(rng.normal(0, 0.02, (1024, 4096)).astype(np.float32), "fp16")
    w2 = O.to_storage(rng.normal(0, 0.02, (4096, 1024)).astype(np.float32), "fp16")
    ark.init()
    tx, t1, t2 = ark.tensor([128, 1024], ark.fp16), ark.tensor([1024, 4096], ark.fp16), ark.tensor([4096, 1024], ark.fp16)
    with ark.PlannerContext(sync=False):
        h = ark.relu(ark.matmul(tx, t1))
    y = ark.matmul(h, t2)
    (got,) = execute([y], {tx: x, t1: w1, t2: w2}, loop_mode=True)
    hh = O.matmul(x, w1, "fp16", act="relu")
    want = O.matmul(hh, w2, "fp16")
    from tests.ark_util import assert_matmul_close
    assert_matmul_close(got, want, "fp16", "ffn block")


def test_streaming_rings_feed_and_drain_a_resident_kernel():
    """Input and output rings walked by the iteration number: iteration i reads slot (i-1) % 2 and leaves its
    result in the same slot, so the host can fill / drain the other slot meanwhile (what bench.py's end-to-end leg does)."""
    from ark_b200.ffn import build_ffn_streaming
    from ark_b200.model import Tensor
    from tests.ark_util import assert_matmul_close
    tokens, d, f = 256, 512, 1024
    rng = np.random.default_rng(11)
    w1 = O.to_storage(rng.normal(0, 0.02, (d, f)).astype(np.float32), "fp16")
    w2 = O.to_storage(rng.normal(0, 0.02, (f, d)).astype(np.float32), "fp16")
    xs = [O.to_storage(rng.normal(0, 1, (tokens, d)).astype(np.float32), "fp16") for _ in range(3)]
    ark.init()
    x_ring, t1, t2, y_ring = build_ffn_streaming(tokens, d, f, ark.fp16)
    m = ark.Model.get_model()
    x_slot = [Tensor(m, ark.fp16, x_ring.buffer, [tokens, d], [2 * tokens, d], [s * tokens, 0]) for s in range(2)]
    y_slot = [Tensor(m, ark.fp16, y_ring.buffer, [tokens, d], [2 * tokens, d], [s * tokens, 0]) for s in range(2)]
    ex = ark.Executor(0, 0, "rings", str(ark.Planner(0).plan()), True)
    ex.set_wait_limit(3_000_000_000)
    ex.compile()
    ex.tensor_from_numpy(t1, w1)
    ex.tensor_from_numpy(t2, w2)
    ex.launch()
    ex.tensor_from_numpy(x_slot[0], xs[0])
    ex.tensor_from_numpy(x_slot[1], xs[1])
    ex.run(2)  # iterations 1 and 2: slots 0 and 1
    ex.wait()
    got = [ex.tensor_to_numpy(y_slot[0]), ex.tensor_to_numpy(y_slot[1])]
    ex.tensor_from_numpy(x_slot[0], xs[2])
    ex.run(1)  # iteration 3: slot 0 again
    ex.wait()
    got.append(ex.tensor_to_numpy(y_slot[0]))
    ex.stop()
    ex.destroy()
    for i in range(3):
        want = O.matmul(O.matmul(xs[i], w1, "fp16", act="gelu"), w2, "fp16")
        assert_matmul_close(got[i], want, "fp16", f"streamed batch {i}")
