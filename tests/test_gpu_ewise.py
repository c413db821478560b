"""GPU parity: elementwise, scalar, cast, copy and rope stages against the CPU
oracle on the same seeded inputs. Shapes follow the reference's op tests
(ark/ops/ops_math_test.cpp, ops_arithmetic_test.cpp, ops_scalar_test.cpp,
ops_cast_test.cpp, ops_copy_test.cpp, ops_rope_test.cpp)."""
import numpy as np
import pytest

import ark_b200 as ark
from oracle import oracle as O
from tests.ark_util import NAME, assert_close, execute, rand

pytestmark = pytest.mark.gpu
FLOATS = ["fp32", "fp16", "bf16"]


@pytest.mark.parametrize("dt", FLOATS)
@pytest.mark.parametrize("op", ["gelu", "exp", "relu", "sigmoid", "sqrt", "rsqrt"])
def test_unary(op, dt):
    rng = np.random.default_rng(11)
    lo, hi = (0.1, 10.0) if op in ("sqrt", "rsqrt") else (-4.0, 4.0)
    x = rand(rng, (4, 2, 1024), dt, lo, hi)
    ark.init()
    t = ark.tensor([4, 2, 1024], NAME[dt])
    out = getattr(ark, op)(t)
    (got,) = execute([out], {t: x})
    assert_close(got, O.unary(op, x, dt), dt, what=f"{op}_{dt}")


@pytest.mark.parametrize("dt", FLOATS)
@pytest.mark.parametrize("op", ["add", "sub", "mul", "div"])
@pytest.mark.parametrize("shapes", [((4, 2, 1024), (4, 2, 1024)), ((4, 2, 1024), (1, 1024)), ((4, 2, 1024), (4, 2, 1)),
                                    ((3, 1, 1024), (1, 4, 1)), ((2, 64, 33), (2, 64, 33)), ((8192, 512), (8192, 512))])
def test_binary_broadcast(op, dt, shapes):
    rng = np.random.default_rng(12)
    sa, sb = shapes
    a = rand(rng, sa, dt, -1.0, 1.0)
    b = rand(rng, sb, dt, 0.5, 2.0) if op == "div" else rand(rng, sb, dt, -1.0, 1.0)
    ark.init()
    ta, tb = ark.tensor(list(sa), NAME[dt]), ark.tensor(list(sb), NAME[dt])
    out = getattr(ark, op)(ta, tb)
    (got,) = execute([out], {ta: a, tb: b})
    assert_close(got, O.binary(op, a, b, dt), dt, what=f"{op}_{dt}_{sa}_{sb}")


@pytest.mark.parametrize("dt", FLOATS)
def test_scalar_ops(dt):
    rng = np.random.default_rng(13)
    x = rand(rng, (4, 2, 1024), dt, -1.0, 1.0)
    ark.init()
    t = ark.tensor([4, 2, 1024], NAME[dt])
    o1 = ark.add(t, 0.7)
    o2 = ark.mul(t, 0.7)
    o3 = ark.constant(7.0, [4, 2, 50], NAME[dt])
    g1, g2, g3 = execute([o1, o2, o3], {t: x})
    assert_close(g1, O.scalar("add", x, 0.7, dt), dt, what="scalar_add")
    assert_close(g2, O.scalar("mul", x, 0.7, dt), dt, what="scalar_mul")
    assert np.array_equal(g3.view(np.uint8), O.fill((4, 2, 50), 7.0, dt).view(np.uint8))


@pytest.mark.parametrize("pair", [("fp16", "fp32"), ("fp32", "fp16"), ("bf16", "fp32"), ("fp32", "bf16"),
                                  ("fp16", "int32"), ("int32", "fp16"), ("fp32", "int32"), ("int32", "fp32")])
def test_cast_exact(pair):
    frm, to = pair
    rng = np.random.default_rng(14)
    if frm == "int32":
        x = rng.integers(-2000, 2000, size=(4, 2, 1024)).astype(np.int32)
    else:
        x = rand(rng, (4, 2, 1024), frm, -100.0, 100.0)
    ark.init()
    t = ark.tensor([4, 2, 1024], NAME[frm])
    out = ark.cast(t, NAME[to])
    (got,) = execute([out], {t: x})
    want = O.cast(x, frm, to)
    assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), f"cast {frm}->{to}"  # ops_cast_test.cpp: max_diff == 0


@pytest.mark.parametrize("dt", ["fp32", "fp16", "int32"])
def test_copy_exact(dt):
    rng = np.random.default_rng(15)
    x = rng.integers(-9, 9, size=(4, 2, 1000)).astype(O.NP[dt])
    ark.init()
    t = ark.tensor([4, 2, 1000], NAME[dt])
    out = ark.copy(t)
    (got,) = execute([out], {t: x})
    assert np.array_equal(got, x)


@pytest.mark.parametrize("dt", FLOATS)
def test_rope(dt):
    rng = np.random.default_rng(16)
    a = rand(rng, (1, 32, 32, 256), dt, -1.0, 1.0)
    b = rand(rng, (1, 32, 32, 256), dt, -1.0, 1.0)
    ark.init()
    ta, tb = ark.tensor([1, 32, 32, 256], NAME[dt]), ark.tensor([1, 32, 32, 256], NAME[dt])
    out = ark.rope(ta, tb)
    (got,) = execute([out], {ta: a, tb: b})
    # the host baseline rounds each product to the storage type; the kernel rounds once
    assert_close(got, O.rope(a, b, dt), dt, rtol=4 * (2.0 ** -9 if dt == "fp16" else 2.0 ** -7 if dt == "bf16" else 1e-6),
                 atol={"fp32": 1e-6, "fp16": 2e-3, "bf16": 1.6e-2}[dt], what="rope")


def test_strided_and_offset_views():
    """Padded / offset tensors (cases of ark/ops/ops_matmul_test.cpp:527-561 applied to elementwise ops)."""
    rng = np.random.default_rng(17)
    a = rand(rng, (64, 100), "fp16", -1.0, 1.0)
    b = rand(rng, (64, 100), "fp16", -1.0, 1.0)
    ark.init()
    ta = ark.tensor([64, 100], ark.fp16, strides=[128, 256], offsets=[32, 64], padded_shape=[64, 128])
    tb = ark.tensor([64, 100], ark.fp16)
    out = ark.add(ta, tb)
    (got,) = execute([out], {ta: a, tb: b})
    assert_close(got, O.binary("add", a, b, "fp16"), "fp16", what="strided add")


@pytest.mark.parametrize("dt,npdt", [("int32", np.int32), ("uint32", np.uint32), ("int8", np.int8), ("uint8", np.uint8)])
def test_integer_arithmetic_is_exact(dt, npdt):
    """Add / Sub / Mul / Div and the scalar forms on integer tensors run in the tensors' own arithmetic (wrap-around,
    truncating division): bit-exact over the whole range, also beyond 2^24 where fp32 could not hold the values."""
    rng = np.random.default_rng(44)
    info = np.iinfo(npdt)
    a = rng.integers(info.min, info.max, size=(3, 5, 64, 96), dtype=npdt, endpoint=True)
    b = rng.integers(info.min, info.max, size=(1, 5, 1, 96), dtype=npdt, endpoint=True)
    b[b == 0] = 1
    adt = getattr(ark, dt)
    ark.init()
    ta, tb = ark.tensor(list(a.shape), adt), ark.tensor(list(b.shape), adt)
    outs = [ark.add(ta, tb), ark.sub(ta, tb), ark.mul(ta, tb), ark.div(ta, tb), ark.add(ta, 3.0), ark.mul(ta, 5.0)]
    got = execute(outs, {ta: a, tb: b})
    with np.errstate(over="ignore"):
        q = (np.trunc(a.astype(np.float64) / b.astype(np.float64))).astype(np.int64).astype(npdt)  # C++ division truncates
        want = [a + b, a - b, a * b, q, a + npdt(3), a * npdt(5)]
    for g, w, name in zip(got, want, ("add", "sub", "mul", "div", "scalar add", "scalar mul")):
        assert np.array_equal(g, w.astype(npdt)), f"{dt} {name}"


@pytest.mark.parametrize("split", ["halves", "interleaved"])
def test_elementwise_partial_task_ranges_follow_plan_tiles(split):
    """A plan may give one operator's tasks to several processor groups (TaskRange [b, e) or [b, e, step]); task id ->
    output tile (n, c, tile row, tile column), column fastest. Each group writes exactly its tiles; together they
    give the whole result (hand-edited plan, as ark/codegen.cpp:318-385 allows for any operator)."""
    import json
    rng = np.random.default_rng(45)
    a, b = rand(rng, (3, 40, 200), "fp16"), rand(rng, (3, 40, 200), "fp16")
    ark.init()
    ta, tb = ark.tensor([3, 40, 200], ark.fp16), ark.tensor([3, 40, 200], ark.fp16)
    out = ark.gelu(ark.add(ta, tb))
    plan = ark.Planner(0).plan().plan
    new_groups = []
    for ti in plan["TaskInfos"]:
        nt = ti["Ops"][0]["Config"]["NumTasks"]
        assert ti["Ops"][0]["Config"]["Tile"] == [1, 64] and nt == 3 * 40 * 4
        ranges = ([0, nt // 3], [nt // 3, nt]) if split == "halves" else ([0, nt, 2], [1, nt, 2])
        rgs = [{"ProcessorRange": pr, "WarpRange": [0, 1], "SramRange": [0, 0],
                "TaskGroups": [{"TaskId": ti["Id"], "TaskRange": tr, "Granularity": 1}]}
               for pr, tr in zip(([0, 48], [48, 148]), ranges)]
        new_groups.append({"ProcessorRange": [0, 148], "ResourceGroups": rgs})
    plan["ProcessorGroups"] = new_groups
    plan["NumProcessors"] = 148
    text = ark.plan_dump(json.dumps(plan))
    assert text.count("tasks [") == 4, text
    (got,) = execute([out], {ta: a, tb: b}, plan=json.dumps(plan))
    want = O.unary("gelu", O.binary("add", a, b, "fp16"), "fp16")
    assert_close(got, want, "fp16", what=f"partial task ranges ({split})")
