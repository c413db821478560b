"""GPU parity: reductions, fused row operators, transpose and embedding
(reference tests: ark/ops/ops_reduce_test.cpp, ops_transpose_test.cpp,
ops_embedding_test.cpp)."""
import numpy as np
import pytest

import ark_b200 as ark
from oracle import oracle as O
from tests.ark_util import ulp_tol, NAME, assert_close, execute, rand

pytestmark = pytest.mark.gpu
FLOATS = ["fp32", "fp16", "bf16"]


def red_tol(dt, k):
    # reduction_abs_error_bound (ark/ops/ops_test_common.hpp:52-69), halved: the oracle is exact fp32
    bits = {"fp32": 23, "fp16": 10, "bf16": 7}[dt]
    return k * 2 * 0.1 / (1 << (bits + 1)) * 2


@pytest.mark.parametrize("dt", FLOATS)
@pytest.mark.parametrize("axis", [0, 1, 2, 3])
@pytest.mark.parametrize("kind", ["sum", "mean", "max"])
def test_reduce_axes(kind, axis, dt):
    rng = np.random.default_rng(21)
    shape = (7, 2, 4, 1024)
    x = rand(rng, shape, dt)
    ark.init()
    t = ark.tensor(list(shape), NAME[dt])
    out = getattr(ark, "reduce_" + kind)(t, axis=axis)
    (got,) = execute([out], {t: x})
    want = O.reduce(kind, x, axis, dt)
    assert_close(got, want, dt, rtol=2 * (2.0 ** -9 if dt == "fp16" else 2.0 ** -7 if dt == "bf16" else 1e-6),
                 atol=red_tol(dt, shape[axis]), what=f"reduce_{kind}_axis{axis}_{dt}")


@pytest.mark.parametrize("dt", FLOATS)
def test_reduce_no_keepdims_and_odd_width(dt):
    rng = np.random.default_rng(22)
    x = rand(rng, (5, 3, 1001), dt)
    ark.init()
    t = ark.tensor([5, 3, 1001], NAME[dt])
    o1 = ark.reduce_sum(t, axis=-1, keepdims=False)
    o2 = ark.reduce_sum(t, axis=0, keepdims=False)
    g1, g2 = execute([o1, o2], {t: x})
    assert g1.shape == (5, 3) and g2.shape == (3, 1001)
    assert_close(g1, O.reduce("sum", x, 2, dt, keepdims=False), dt, rtol=4e-3 if dt != "fp32" else 1e-5,
                 atol=red_tol(dt, 1001), what="sum -1")
    assert_close(g2, O.reduce("sum", x, 0, dt, keepdims=False), dt, rtol=1e-2 if dt == "bf16" else 4e-3, atol=red_tol(dt, 5), what="sum 0")


@pytest.mark.parametrize("dt", FLOATS)
@pytest.mark.parametrize("rows,cols", [(64, 4096), (7, 8192), (2048, 128), (3, 40000)])
def test_rmsnorm_softmax_layernorm(dt, rows, cols):
    rng = np.random.default_rng(23)
    x = O.to_storage(rng.normal(0, 1, (rows, cols)).astype(np.float32), dt)
    w = O.to_storage(rng.normal(1, 0.1, (cols,)).astype(np.float32), dt)
    ark.init()
    t, tw = ark.tensor([rows, cols], NAME[dt]), ark.tensor([cols], NAME[dt])
    o1 = ark.rmsnorm(t, tw, eps=1e-5)
    o2 = ark.softmax(t)
    o3 = ark.layernorm(t)
    g1, g2, g3 = execute([o1, o2, o3], {t: x, tw: w})
    tol = {"fp32": 2e-5, "fp16": 2e-3, "bf16": 1.6e-2}[dt]
    assert_close(g1, O.rmsnorm(x, w, dt, 1e-5), dt, rtol=tol, atol=tol, what="rmsnorm")
    assert_close(g2, O.softmax(x, dt), dt, rtol=tol, atol=1e-7 if dt == "fp32" else 1e-5, what="softmax")
    assert_close(g3, O.layernorm(x, dt), dt, rtol=tol, atol=tol, what="layernorm")


@pytest.mark.parametrize("dt", ["fp16", "bf16", "fp32"])
@pytest.mark.parametrize("shape,mrows", [((2, 3, 64, 512), 64), ((1, 4, 1024, 1024), 1024), ((1, 2, 8, 20000), 8), ((1, 1, 40, 256), 1)])
def test_softmax_with_scale_and_additive_mask(dt, shape, mrows):
    """One row kernel for softmax(x * scale + mask): each variant of the kernel (rows in registers, rows streamed
    through shared memory, two-pass) against the oracle's scalar-mul, add, softmax with their per-op rounding."""
    rng = np.random.default_rng(26)
    cols = shape[-1]
    x = O.to_storage(rng.normal(0, 3, shape).astype(np.float32), dt)
    m = np.where(rng.random((1, 1, mrows, cols)) < 0.3, -np.inf, 0.0).astype(np.float32)
    m[..., 0] = 0.0  # no fully masked row
    mk = O.to_storage(m, dt)
    scale = 0.125
    ark.init()
    t, tm = ark.tensor(list(shape), NAME[dt]), ark.tensor([1, 1, mrows, cols], NAME[dt])
    out = ark.softmax(t, scale=scale, mask=tm)
    (got,) = execute([out], {t: x, tm: mk})
    logits = O.binary("add", O.scalar("mul", x, scale, dt), np.broadcast_to(mk, shape).copy(), dt)
    want = O.softmax(logits, dt)
    tol = {"fp32": 2e-5, "fp16": 2e-3, "bf16": 1.6e-2}[dt]
    assert_close(got, want, dt, rtol=tol, atol=1e-7 if dt == "fp32" else 1e-5, what="masked softmax")


def test_fused_rows_match_the_reference_compositions(monkeypatch):
    """softmax/layernorm as the reference composes them (python/ark/ops.py:491-513), run operator by operator
    (chain recognition switched off), vs the fused kernels."""
    monkeypatch.setenv("ARKB_FUSE_CHAINS", "0")
    rng = np.random.default_rng(24)
    x = rng.normal(0, 1, (16, 512)).astype(np.float32)
    ark.init()
    t = ark.tensor([16, 512], ark.fp32)
    f1, f2 = ark.softmax(t, fused=True), ark.layernorm(t, fused=True)
    c1, c2 = ark.softmax(t, fused=False), ark.layernorm(t, fused=False)
    plan = ark.Planner(0).plan()
    assert ark.plan_dump(str(plan)).count("ReduceM") >= 3  # the compositions stay operator by operator
    g = execute([f1, f2, c1, c2], {t: x}, plan=plan)
    assert np.allclose(g[0], g[2], rtol=1e-5, atol=1e-7)
    assert np.allclose(g[1], g[3], rtol=1e-4, atol=1e-5)


def _ref_softmax(x):
    m = ark.reduce_max(x, axis=-1)
    o = ark.sub(x, m)
    o = ark.exp(o, o)
    s = ark.reduce_sum(o, axis=-1)
    return ark.div(o, s, o)


def _ref_layernorm(x, eps):
    mean = ark.reduce_mean(x, axis=-1)
    c = ark.sub(x, mean)
    var = ark.reduce_mean(ark.mul(c, c), axis=-1)
    return ark.mul(c, ark.rsqrt(ark.add(var, eps)))


def _ref_rmsnorm(x, w, dt):
    f = ark.cast(x, ark.fp32)
    r = ark.rsqrt(ark.reduce_mean(ark.mul(f, f), axis=-1))
    f2 = ark.mul(f, r)
    return ark.cast(ark.mul(f2, w, f2), NAME[dt])


@pytest.mark.parametrize("merged", [False, True])
@pytest.mark.parametrize("dt", ["fp16", "bf16"])
def test_reference_op_chains_run_as_one_row_kernel(dt, merged):
    """The op chains an unmodified reference model emits for softmax (python/ark/ops.py:491-500), layernorm
    (:503-513) and the llama example's RMSNorm (examples/llama/model.py:92-99: fp32 weight, no epsilon) are
    recognised, whether the planner left every operator in its own task or merged them (Sync=false), and lowered to
    the fused row kernel; results against the oracle's per-operator composition in the reference's op order."""
    rng = np.random.default_rng(27)
    rows, cols = 96, 2048
    x = rand(rng, (rows, cols), dt, -2.0, 2.0)
    w = rng.normal(1.0, 0.1, (1, cols)).astype(np.float32)
    ark.init()
    tx, tw = ark.tensor([rows, cols], NAME[dt]), ark.tensor([1, cols], ark.fp32)

    def build():
        return _ref_softmax(tx), _ref_layernorm(tx, 1e-5), _ref_rmsnorm(tx, tw, dt)
    if merged:
        outs = []
        for f in (lambda: _ref_softmax(tx), lambda: _ref_layernorm(tx, 1e-5), lambda: _ref_rmsnorm(tx, tw, dt)):
            with ark.PlannerContext(sync=False):
                outs.append(f())
    else:
        outs = list(build())
    plan = ark.Planner(0).plan()
    text = ark.plan_dump(str(plan))
    assert "Softmax reduce_max...div" in text and "LayerNorm reduce_mean" in text and "RMSNorm cast" in text, text
    assert "ReduceMax" not in text and " Exp " not in text and " Cast " not in text
    got = execute(outs, {tx: x, tw: w}, plan=plan)
    # the reference's own arithmetic: every operator rounds to the storage type
    m = O.reduce("max", x, -1, dt)
    e = O.unary("exp", O.binary("sub", x, m, dt), dt)
    want_sm = O.binary("div", e, O.reduce("sum", e, -1, dt), dt)
    c = O.binary("sub", x, O.reduce("mean", x, -1, dt), dt)
    var = O.reduce("mean", O.binary("mul", c, c, dt), -1, dt)
    want_ln = O.binary("mul", c, O.unary("rsqrt", O.scalar("add", var, 1e-5, dt), dt), dt)
    f = O.cast(x, dt, "fp32")
    r = O.unary("rsqrt", O.reduce("mean", O.binary("mul", f, f, "fp32"), -1, "fp32"), "fp32")
    want_rn = O.cast(O.binary("mul", O.binary("mul", f, r, "fp32"), w, "fp32"), "fp32", dt)
    tol = 4 * ulp_tol(dt)  # the chain rounds its intermediates, the row kernel rounds once
    assert_close(got[0], want_sm, dt, rtol=tol, atol=tol * 0.01, what="softmax chain")
    assert_close(got[1], want_ln, dt, rtol=tol, atol=tol * 2.0, what="layernorm chain")
    assert_close(got[2], want_rn, dt, rtol=tol, atol=tol * 0.1, what="rmsnorm chain")


@pytest.mark.parametrize("dt", ["fp32", "fp16"])
@pytest.mark.parametrize("perm", [[0, 1, 3, 2], [0, 2, 3, 1], [0, 2, 1, 3], [3, 2, 1, 0], [1, 0, 2, 3], [2, 3, 0, 1]])
def test_transpose_exact(dt, perm):
    rng = np.random.default_rng(25)
    x = rand(rng, (5, 3, 32, 128), dt)
    ark.init()
    t = ark.tensor([5, 3, 32, 128], NAME[dt])
    out = ark.transpose(t, perm)
    (got,) = execute([out], {t: x})
    assert np.array_equal(got, O.transpose(x, perm))


@pytest.mark.parametrize("dt", FLOATS)
def test_embedding_exact(dt):
    rng = np.random.default_rng(26)
    w = rand(rng, (100, 4096), dt)
    idx = rng.integers(-100, 100, size=(8, 3, 64)).astype(np.int32)
    ark.init()
    ti, tw = ark.tensor([8, 3, 64], ark.int32), ark.tensor([100, 4096], NAME[dt])
    out = ark.embedding(ti, tw)
    (got,) = execute([out], {ti: idx, tw: w})
    assert np.array_equal(got.view(np.uint8), O.embedding(idx, w).view(np.uint8))


def _split_plan(split):
    """Gives every operator's tasks to two processor groups' worth of CTAs: [0, n/3) + [n/3, n), or even / odd."""
    import json
    plan = ark.Planner(0).plan().plan
    groups = []
    for ti in plan["TaskInfos"]:
        nt = ti["Ops"][0]["Config"]["NumTasks"]
        ranges = ([0, nt // 3], [nt // 3, nt]) if split == "halves" else ([0, nt, 2], [1, nt, 2])
        rgs = [{"ProcessorRange": pr, "WarpRange": [0, 1], "SramRange": [0, 0],
                "TaskGroups": [{"TaskId": ti["Id"], "TaskRange": tr, "Granularity": 1}]}
               for pr, tr in zip(([0, 48], [48, 148]), ranges)]
        groups.append({"ProcessorRange": [0, 148], "ResourceGroups": rgs})
    plan["ProcessorGroups"] = groups
    plan["NumProcessors"] = 148
    return json.dumps(plan)


@pytest.mark.parametrize("split", ["halves", "interleaved"])
def test_partial_task_ranges_of_reductions_rows_transposes_and_gathers(split):
    """A plan may hand any operator's tasks to several groups of processors (ark/codegen.cpp:318-385): a reduction's
    task is one output element, a row operator's one row, a transpose's one 8 x 8 tile of the output, an embedding's
    one index. Each group writes exactly its share; together they give the whole result."""
    rng = np.random.default_rng(46)
    x = O.to_storage(rng.normal(0, 1, (3, 20, 72)).astype(np.float32), "fp16")
    w = O.to_storage(rng.normal(0, 1, (50, 64)).astype(np.float32), "fp16")
    idx = rng.integers(-50, 50, size=(2, 9), dtype=np.int32)
    ark.init()
    tx, tw, ti = ark.tensor([3, 20, 72], ark.fp16), ark.tensor([50, 64], ark.fp16), ark.tensor([2, 9], ark.int32)
    outs = [ark.reduce_sum(tx, axis=-1), ark.reduce_max(tx, axis=1), ark.reduce_mean(tx, axis=0), ark.softmax(tx),
            ark.rmsnorm(tx), ark.transpose(tx, [1, 0, 2]), ark.transpose(tx, [0, 2, 1]), ark.embedding(ti, tw)]
    plan = _split_plan(split)
    text = ark.plan_dump(plan)
    assert text.count("tasks ") == 2 * len(outs), text
    got = execute(outs, {tx: x, tw: w, ti: idx}, plan=plan)
    want = [O.reduce("sum", x, 2, "fp16"), O.reduce("max", x, 1, "fp16"), O.reduce("mean", x, 0, "fp16"),
            O.softmax(x, "fp16"), O.rmsnorm(x, None, "fp16", 1e-5)]
    for g, wv, name in zip(got[:5], want, ("sum w", "max h", "mean c", "softmax", "rmsnorm")):
        err = np.abs(O.to_f32(g, "fp16").reshape(wv.shape) - O.to_f32(wv, "fp16"))
        assert float(err.max()) <= 2e-2, (name, float(err.max()))
    assert np.array_equal(got[5], x.transpose(1, 0, 2)) and np.array_equal(got[6], x.transpose(0, 2, 1))
    assert np.array_equal(got[7], w[idx])


@pytest.mark.parametrize("dt", ["fp16", "bf16"])
@pytest.mark.parametrize("rows,cols", [(8, 512), (1024, 2048), (700, 4096)])
def test_rmsnorm_with_residual(dt, rows, cols):
    """h, x1 = rmsnorm(x, weight, residual=r): x1 = x + r (rounded, kept for the next block), h = rmsnorm(x1) * weight.
    Few rows run in registers, many rows stream through shared memory (the residual is added when a row lands)."""
    rng = np.random.default_rng(47)
    x, r = rand(rng, (rows, cols), dt, -2.0, 2.0), rand(rng, (rows, cols), dt, -2.0, 2.0)
    w = rand(rng, (cols,), dt, 0.5, 1.5)
    ark.init()
    tx, tr, tw = ark.tensor([rows, cols], NAME[dt]), ark.tensor([rows, cols], NAME[dt]), ark.tensor([cols], NAME[dt])
    h, x1 = ark.rmsnorm(tx, tw, residual=tr)
    text = ark.plan_dump(str(ark.Planner(0).plan()))
    assert ("staged" in text) == (rows >= 4 * 148), text
    got_h, got_x1 = execute([h, x1], {tx: x, tr: r, tw: w})
    want_x1 = O.binary("add", x, r, dt)
    assert np.array_equal(got_x1.view(np.uint16), want_x1.view(np.uint16))
    tol = 2e-3 if dt == "fp16" else 1.6e-2
    assert_close(got_h, O.rmsnorm(want_x1, w, dt, 1e-5), dt, rtol=tol, atol=tol, what=f"rmsnorm + residual {rows}x{cols}")
