"""GPU parity: tensor-core matmul (tcgen05) and the CUDA-core fallback against
the oracle's fp32-accumulate restatement. Cases follow
ark/ops/ops_matmul_test.cpp:330-561 (plain, transposed, batched with N/C
broadcast, padded/offset operands, constant inputs)."""
import numpy as np
import pytest

import ark_b200 as ark
from oracle import oracle as O
from tests.ark_util import NAME, assert_matmul_close, execute, rand

pytestmark = pytest.mark.gpu


def run_mm(ash, bsh, dt, ta=False, tb=False, seed=31, fuse=None):
    rng = np.random.default_rng(seed)
    a, b = rand(rng, ash, dt), rand(rng, bsh, dt)
    ark.init()
    t_a, t_b = ark.tensor(list(ash), NAME[dt]), ark.tensor(list(bsh), NAME[dt])
    if fuse:
        with ark.PlannerContext(sync=False):
            out = getattr(ark, fuse)(ark.matmul(t_a, t_b, transpose_input=ta, transpose_other=tb))
    else:
        out = ark.matmul(t_a, t_b, transpose_input=ta, transpose_other=tb)
    (got,) = execute([out], {t_a: a, t_b: b})
    want = O.matmul(a, b, dt, ta, tb, act=fuse)
    return got, want


@pytest.mark.parametrize("dt", ["fp16", "bf16"])
@pytest.mark.parametrize("mnk", [(128, 256, 64), (128, 256, 256), (256, 512, 1024), (128, 64, 64), (4096, 256, 128),
                                 (64, 48, 96), (1, 256, 512), (200, 1000, 136)])
def test_matmul_nn(dt, mnk):
    m, n, k = mnk
    got, want = run_mm((m, k), (k, n), dt)
    assert_matmul_close(got, want, dt, f"nn {mnk}")


@pytest.mark.parametrize("dt", ["fp16", "bf16"])
@pytest.mark.parametrize("ta,tb", [(False, True), (True, False), (True, True)])
@pytest.mark.parametrize("mnk", [(128, 256, 64), (256, 384, 512), (72, 200, 264)])
def test_matmul_transposed(dt, ta, tb, mnk):
    m, n, k = mnk
    got, want = run_mm((k, m) if ta else (m, k), (n, k) if tb else (k, n), dt, ta, tb)
    assert_matmul_close(got, want, dt, f"t{int(ta)}{int(tb)} {mnk}")


@pytest.mark.parametrize("dt", ["fp16"])
@pytest.mark.parametrize("ash,bsh", [((3, 128, 64), (3, 64, 256)), ((2, 3, 128, 64), (1, 3, 64, 128)),
                                     ((2, 1, 64, 64), (1, 3, 64, 64)), ((4, 128, 128), (128, 64))])
def test_matmul_batched_broadcast(dt, ash, bsh):
    got, want = run_mm(ash, bsh, dt)
    assert got.shape == want.shape
    assert_matmul_close(got, want, dt, f"batched {ash}x{bsh}")


@pytest.mark.parametrize("fuse", ["relu", "gelu"])
def test_matmul_fused_activation(fuse):
    got, want = run_mm((256, 512), (512, 768), "fp16", fuse=fuse)
    assert_matmul_close(got, want, "fp16", f"fused {fuse}")


def test_matmul_constant_inputs():
    # ops_matmul_test.cpp:343-360: all 0.1 -> every output is k * 0.01
    ark.init()
    m, n, k = 256, 256, 512
    t_a, t_b = ark.tensor([m, k], ark.fp16), ark.tensor([k, n], ark.fp16)
    out = ark.matmul(t_a, t_b)
    a = np.full((m, k), 0.1, np.float16)
    b = np.full((k, n), 0.1, np.float16)
    (got,) = execute([out], {t_a: a, t_b: b})
    want = O.matmul(a, b, "fp16")
    assert np.array_equal(got, want)  # exact: identical products, fp32 accumulation


def test_matmul_padded_offset_operands():
    """Operands that are windows of larger buffers (ops_matmul_test.cpp:527-561)."""
    rng = np.random.default_rng(33)
    a, b = rand(rng, (128, 64), "fp16"), rand(rng, (64, 256), "fp16")
    ark.init()
    t_a = ark.tensor([128, 64], ark.fp16, strides=[256, 128], offsets=[128, 64], padded_shape=[128, 64])
    t_b = ark.tensor([64, 256], ark.fp16, strides=[128, 512], offsets=[64, 256], padded_shape=[64, 256])
    out = ark.matmul(t_a, t_b)
    (got,) = execute([out], {t_a: a, t_b: b})
    assert_matmul_close(got, O.matmul(a, b, "fp16"), "fp16", "padded/offset")


@pytest.mark.parametrize("dt,mnk", [("fp32", (128, 256, 64)), ("fp32", (100, 70, 130)), ("fp16", (64, 50, 70))])
def test_matmul_cuda_core_fallback(dt, mnk):
    """fp32, and fp16 rows that are not 16-byte multiples, run on the CUDA-core path."""
    m, n, k = mnk
    got, want = run_mm((m, k), (k, n), dt)
    if dt == "fp32":
        assert np.allclose(got, want, rtol=1e-4, atol=1e-5)
    else:
        assert_matmul_close(got, want, dt, "simt fp16")


def test_matmul_partial_task_range_follows_plan_tiles():
    """A hand-written plan that splits one Matmul's tiles over two processor groups
    (as examples/tutorial/plan_tutorial.py does) must compute the same result."""
    import json
    rng = np.random.default_rng(34)
    a, b = rand(rng, (256, 128), "fp16"), rand(rng, (128, 512), "fp16")
    ark.init()
    t_a, t_b = ark.tensor([256, 128], ark.fp16), ark.tensor([128, 512], ark.fp16)
    out = ark.matmul(t_a, t_b)
    plan = ark.Planner(0).plan().plan
    assert plan["TaskInfos"][0]["Ops"][0]["Config"]["NumTasks"] == 4  # 128x256 tiles
    pg = plan["ProcessorGroups"][0]
    rg = pg["ResourceGroups"][0]
    pg["ProcessorRange"] = [0, 4]
    rg["ProcessorRange"] = [0, 2]
    rg["TaskGroups"][0]["TaskRange"] = [0, 4, 2]
    rg2 = json.loads(json.dumps(rg))
    rg2["ProcessorRange"] = [2, 4]
    rg2["TaskGroups"][0]["TaskRange"] = [1, 4, 2]
    pg["ResourceGroups"].append(rg2)
    plan["NumProcessors"] = 4
    (got,) = execute([out], {t_a: a, t_b: b}, plan=ark.Plan(plan))
    assert_matmul_close(got, O.matmul(a, b, "fp16"), "fp16", "partial ranges")


# ---- few activation rows against a weight matrix: the CUDA-core weight-streaming stage ----
@pytest.mark.parametrize("dt", ["fp16", "bf16"])
@pytest.mark.parametrize("tb", [True, False])
@pytest.mark.parametrize("mnk", [(1, 4096, 4096), (1, 1000, 520), (2, 2048, 1024), (3, 264, 3072), (4, 8192, 2048),
                                 (5, 1536, 1288), (8, 4096, 8192), (8, 512, 512), (1, 256, 16384)])
def test_matmul_few_rows_stream_weights(dt, tb, mnk):
    m, n, k = mnk
    got, want = run_mm((m, k), (n, k) if tb else (k, n), dt, tb=tb, seed=37)
    assert_matmul_close(got, want, dt, f"gemv {mnk} tb={tb}")


@pytest.mark.parametrize("tb", [True, False])
def test_matmul_few_rows_fused_activation(tb):
    got, want = run_mm((2, 2048), (4096, 2048) if tb else (2048, 4096), "fp16", tb=tb, seed=38, fuse="gelu")
    assert_matmul_close(got, want, "fp16", "gemv + gelu")


def test_matmul_few_rows_uses_the_streaming_stage():
    ark.init()
    x, w = ark.tensor([1, 4096], ark.fp16), ark.tensor([4096, 4096], ark.fp16)
    ark.matmul(x, w, transpose_other=True)
    ex = ark.Executor(0, 0, "gemv", str(ark.Planner(0).plan()), loop_mode=False)
    ex.compile()
    assert "Matmul(gemv)" in ex.program_dump()
    ex.destroy()


# ---- operators of the same task folded into the weight-streaming stage ----
@pytest.mark.parametrize("dt", ["fp16", "bf16"])
@pytest.mark.parametrize("tb", [True, False])
@pytest.mark.parametrize("m", [1, 2])
def test_rmsnorm_folded_into_weight_streaming_matmul(dt, tb, m):
    n, k = 2048, 4096
    rng = np.random.default_rng(41)
    x, r = rand(rng, (m, k), dt), rand(rng, (m, k), dt)
    g = O.to_storage(rng.normal(1, 0.1, (k,)).astype(np.float32), dt)
    w = O.to_storage(rng.normal(0, 0.02, (n, k) if tb else (k, n)).astype(np.float32), dt)
    ark.init()
    tx, tr, tg, tw = (ark.tensor(list(a.shape), NAME[dt]) for a in (x, r, g, w))
    with ark.PlannerContext(sync=False):
        y1 = ark.matmul(ark.rmsnorm(tx, tg, eps=1e-5), tw, transpose_other=tb)
    with ark.PlannerContext(sync=False):
        h, xr = ark.rmsnorm(tx, tg, eps=1e-5, residual=tr)
        y2 = ark.matmul(h, tw, transpose_other=tb)
    plan = ark.Planner(0).plan()
    assert ark.plan_dump(str(plan)).count("<-rmsnorm") == 2
    g1, g2, gxr = execute([y1, y2, xr], {tx: x, tr: r, tg: g, tw: w})
    assert_matmul_close(g1, O.matmul(O.rmsnorm(x, g, dt, 1e-5), w, dt, False, tb), dt, "rmsnorm -> gemv")
    xs = O.binary("add", x, r, dt)
    assert np.array_equal(gxr.view(np.uint16), xs.view(np.uint16)), "x + residual kept for later"
    assert_matmul_close(g2, O.matmul(O.rmsnorm(xs, g, dt, 1e-5), w, dt, False, tb), dt, "rmsnorm(residual) -> gemv")


@pytest.mark.parametrize("dt", ["fp16", "bf16"])
@pytest.mark.parametrize("tb", [True, False])
def test_mul_and_residual_add_folded_into_weight_streaming_matmul(dt, tb):
    m, n, k = 1, 4096, 2048
    rng = np.random.default_rng(42)
    a, b, res = rand(rng, (m, k), dt), rand(rng, (m, k), dt), rand(rng, (m, n), dt)
    w = O.to_storage(rng.normal(0, 0.02, (n, k) if tb else (k, n)).astype(np.float32), dt)
    ark.init()
    ta_, tb_, tres, tw = (ark.tensor(list(t.shape), NAME[dt]) for t in (a, b, res, w))
    with ark.PlannerContext(sync=False):
        y = ark.add(ark.matmul(ark.mul(ta_, tb_), tw, transpose_other=tb), tres)
    text = ark.plan_dump(str(ark.Planner(0).plan()))
    assert "<-mul" in text and "+residual" in text and "Add" not in text
    (got,) = execute([y], {ta_: a, tb_: b, tres: res, tw: w})
    want = O.binary("add", O.matmul(O.binary("mul", a, b, dt), w, dt, False, tb), res, dt)
    assert_matmul_close(got, want, dt, "mul -> gemv -> add")



@pytest.mark.parametrize("dt", ["fp16", "bf16"])
@pytest.mark.parametrize("kind", ["add", "mul"])
@pytest.mark.parametrize("mnk", [(256, 512, 256), (1000, 1376, 512)])
def test_add_and_mul_folded_into_tensor_core_matmul_epilogue(dt, kind, mnk):
    """Matmul -> Add / Mul with a tensor of the result's shape in one task: the tensor is read in the epilogue and
    combined with the fp32 accumulator (one rounding), the product itself is never stored. Against the oracle's
    matmul and add / mul on fp32 values."""
    m, n, k = mnk
    rng = np.random.default_rng(43)
    a, other = rand(rng, (m, k), dt), rand(rng, (m, n), dt)
    w = O.to_storage(rng.normal(0, 0.05, (n, k)).astype(np.float32), dt)
    ark.init()
    ta_, to_, tw = (ark.tensor(list(t.shape), NAME[dt]) for t in (a, other, w))
    with ark.PlannerContext(sync=False):
        mm = ark.matmul(ta_, tw, transpose_other=True)
        y = ark.add(mm, to_) if kind == "add" else ark.mul(to_, mm)
    text = ark.plan_dump(str(ark.Planner(0).plan()))
    assert ("+operand" if kind == "add" else "*operand") in text and " Add " not in text and " Mul " not in text
    (got,) = execute([y], {ta_: a, to_: other, tw: w})
    acc = O.matmul(O.to_f32(a, dt), O.to_f32(w, dt), "fp32", False, True)
    want = O.to_storage(O.binary(kind, acc, O.to_f32(other, dt), "fp32"), dt)
    assert_matmul_close(got, want, dt, f"matmul -> {kind} {mnk}")


def test_gate_times_up_needs_no_barrier_between_the_two_matmuls():
    """SwiGLU: gate = silu(x W1) and g = gate * (x W3) have the same tiles on the same CTAs, so the W3 epilogue reads
    the gate tile its own CTA stored: no barrier between the two stages. Run twice in loop mode (the second iteration
    overwrites what the first one read)."""
    m, d, f = 512, 512, 1536
    rng = np.random.default_rng(44)
    x = rand(rng, (m, d), "fp16")
    w1, w3 = (O.to_storage(rng.normal(0, 0.05, (f, d)).astype(np.float32), "fp16") for _ in range(2))
    ark.init()
    tx, t1, t3 = ark.tensor([m, d], ark.fp16), ark.tensor([f, d], ark.fp16), ark.tensor([f, d], ark.fp16)
    with ark.PlannerContext(sync=False):
        gate = ark.silu(ark.matmul(tx, t1, transpose_other=True))
    with ark.PlannerContext(sync=False):
        g = ark.mul(gate, ark.matmul(tx, t3, transpose_other=True))
    text = ark.plan_dump(str(ark.Planner(0).plan()))
    lines = text.splitlines()
    i = next(k for k, l in enumerate(lines) if "act=4" in l)
    assert "*operand" in lines[i + 1], text
    (got,) = execute([g], {tx: x, t1: w1, t3: w3}, loop_mode=True, iters=2)
    a32 = O.matmul(O.to_f32(x, "fp16"), O.to_f32(w1, "fp16"), "fp32", False, True)
    gate_ref = O.to_storage(O.binary("mul", a32, O.unary("sigmoid", a32, "fp32"), "fp32"), "fp16")
    up32 = O.matmul(O.to_f32(x, "fp16"), O.to_f32(w3, "fp16"), "fp32", False, True)
    want = O.to_storage(O.binary("mul", O.to_f32(gate_ref, "fp16"), up32, "fp32"), "fp16")
    assert_matmul_close(got, want, "fp16", "silu(x W1) * (x W3)")


@pytest.mark.parametrize("dt", ["fp16", "bf16"])
@pytest.mark.parametrize("b,seq,heads,k", [(2, 128, 4, 256), (1, 300, 3, 512)])
def test_rope_folded_into_tensor_core_matmul_epilogue(dt, b, seq, heads, k):
    """Projection -> reshape to [b, seq, heads, 128] -> RoPE in one task: the (cos, sin) table is read in the matmul's
    epilogue and the rotation applied to the fp32 accumulator; tiles of 240 columns straddle head boundaries."""
    hd = 128
    rng = np.random.default_rng(45)
    x = rand(rng, (b * seq, k), dt)
    w = O.to_storage(rng.normal(0, 0.05, (heads * hd, k)).astype(np.float32), dt)
    tab = O.to_storage(rng.uniform(-1, 1, (1, seq, 1, hd)).astype(np.float32), dt)
    ark.init()
    tx, tw, tt = ark.tensor([b * seq, k], NAME[dt]), ark.tensor([heads * hd, k], NAME[dt]), ark.tensor([1, seq, 1, hd], NAME[dt])
    with ark.PlannerContext(sync=False):
        q = ark.rope(ark.reshape(ark.matmul(tx, tw, transpose_other=True), [b, seq, heads, hd]), tt)
    text = ark.plan_dump(str(ark.Planner(0).plan()))
    assert " rope " in text and "Rope" not in text, text
    (got,) = execute([q], {tx: x, tw: w, tt: tab})
    acc = O.matmul(O.to_f32(x, dt), O.to_f32(w, dt), "fp32", False, True).reshape(b, seq, heads, hd)
    want = O.to_storage(O.rope(acc, np.ascontiguousarray(np.broadcast_to(O.to_f32(tab, dt), acc.shape)), "fp32"), dt)
    assert_matmul_close(got.reshape(b * seq, heads * hd), want.reshape(b * seq, heads * hd), dt, "matmul -> rope")


@pytest.mark.parametrize("dt", ["fp16", "bf16"])
@pytest.mark.parametrize("mnk,tb,fuse", [((512, 256, 4096), True, None), ((512, 128, 8192), False, "relu"), ((300, 200, 2056), True, "gelu")])
def test_matmul_few_long_tiles_split_k(dt, mnk, tb, fuse):
    """A narrow output with a long K gives few tiles with long main loops: K is cut into ranges, the fp32 partials go to
    scratch and a sum stage adds them in range order (deterministic), applies the activation and rounds once."""
    m, n, k = mnk
    got, want = run_mm((m, k), (n, k) if tb else (k, n), dt, False, tb, fuse=fuse)
    assert_matmul_close(got, want, dt, f"split-K tiles {mnk}")


def test_matmul_split_k_tiles_are_chosen():
    """The lowering cuts K only where the model says it pays (a [4096, 128] output over K = 8192), and an Add folded into
    the epilogue moves to the sum stage."""
    rng = np.random.default_rng(48)
    m, n, k = 1024, 128, 8192
    a, other = rand(rng, (m, k), "fp16"), rand(rng, (m, n), "fp16")
    w = O.to_storage(rng.normal(0, 0.05, (n, k)).astype(np.float32), "fp16")
    ark.init()
    ta_, to_, tw = (ark.tensor(list(t.shape), ark.fp16) for t in (a, other, w))
    with ark.PlannerContext(sync=False):
        y = ark.add(ark.matmul(ta_, tw, transpose_other=True), to_)
    text = ark.plan_dump(str(ark.Planner(0).plan()))
    assert "splitK=" in text and "split-K sum" in text and " Add " not in text, text
    (got,) = execute([y], {ta_: a, to_: other, tw: w})
    acc = O.matmul(O.to_f32(a, "fp16"), O.to_f32(w, "fp16"), "fp32", False, True)
    want = O.to_storage(O.binary("add", acc, O.to_f32(other, "fp16"), "fp32"), "fp16")
    assert_matmul_close(got, want, "fp16", "split-K + added operand")


@pytest.mark.parametrize("dt", ["fp16", "bf16"])
@pytest.mark.parametrize("mnk,ta,tb,fuse", [((600, 400, 320), False, True, None), ((512, 256, 1024), False, False, "relu"),
                                            ((304, 264, 136), True, True, None)])
def test_matmul_tall_tiles(monkeypatch, dt, mnk, ta, tb, fuse):
    """Optional tile form of the one-CTA-per-tile matmul: 256 rows per CTA as two 128-row halves that share every
    block of B and take one accumulator buffer each (rows past M arrive as zeros and are clipped by the epilogue)."""
    monkeypatch.setenv("ARKB_NO_PAIR", "1")
    monkeypatch.setenv("ARKB_TALL", "2")
    m, n, k = mnk
    rng = np.random.default_rng(77)
    a, b = rand(rng, (k, m) if ta else (m, k), dt), rand(rng, (n, k) if tb else (k, n), dt)
    ark.init()
    t_a, t_b = ark.tensor(list(a.shape), NAME[dt]), ark.tensor(list(b.shape), NAME[dt])
    if fuse:
        with ark.PlannerContext(sync=False):
            out = getattr(ark, fuse)(ark.matmul(t_a, t_b, transpose_input=ta, transpose_other=tb))
    else:
        out = ark.matmul(t_a, t_b, transpose_input=ta, transpose_other=tb)
    plan = ark.Planner(0).plan()
    assert " tall " in ark.plan_dump(str(plan))
    (got,) = execute([out], {t_a: a, t_b: b}, plan=plan)
    assert_matmul_close(got, O.matmul(a, b, dt, ta, tb, act=fuse), dt, f"tall {mnk}")
