"""Seeded cases shared by the golden-vector generator and the oracle tests.

Each case names a reference baseline (exported by oracle/ref_shim.cpp), builds
its inputs from a fixed seed and says how the oracle restatement computes the
same thing. Shapes follow the reference's own op tests where they are small
enough to keep the fixture file at a few hundred KB.
"""
import numpy as np

FLOATS = ("fp32", "fp16", "bf16")


def _rand(rng, shape, dt, lo=-0.1, hi=0.1, O=None):
    # ops_test_common.cpp:52-66 draws uniform(-0.1, 0.1) for float inputs
    return O.to_storage(rng.uniform(lo, hi, size=shape).astype(np.float32), dt)


def build_cases(O):
    """Returns a list of dicts: name, ref (symbol suffix), ins, out_shape,
    out_dtype, oracle (callable on ins)."""
    cases = []
    seed = [1000]

    def add(name, ref, ins, out_shape, out_np, fn):
        cases.append(dict(name=name, ref=ref, ins=ins, out_shape=tuple(out_shape), out_np=out_np, oracle=fn))

    def rng():
        seed[0] += 1
        return np.random.default_rng(seed[0])

    for dt in FLOATS:
        npdt = O.NP[dt]
        # reductions: ops_reduce_test.cpp uses {7,2,4,1024}-like shapes; smaller here
        x = _rand(rng(), (3, 2, 4, 96), dt, O=O)
        for ax in range(4):
            osh = list(x.shape)
            osh[ax] = 1
            add(f"reduce_sum_axis{ax}_{dt}", f"reduce_sum_axis{ax}_{dt}", [x], osh, npdt,
                lambda ins, ax=ax, dt=dt: O.reduce("sum", ins[0], ax, dt))
        add(f"reduce_max_axis3_{dt}", f"reduce_max_axis3_{dt}", [x], [3, 2, 4, 1], npdt,
            lambda ins, dt=dt: O.reduce("max", ins[0], 3, dt))
        add(f"reduce_mean_axis3_{dt}", f"reduce_mean_axis3_{dt}", [x], [3, 2, 4, 1], npdt,
            lambda ins, dt=dt: O.reduce("mean", ins[0], 3, dt))
        # unary math: ops_math_test.cpp uses {4,2,1024}
        for op in ("gelu", "exp", "relu", "sigmoid"):
            xi = _rand(rng(), (2, 2, 256), dt, -4.0, 4.0, O=O)
            add(f"{op}_{dt}", f"{op}_{dt}", [xi], xi.shape, npdt, lambda ins, op=op, dt=dt: O.unary(op, ins[0], dt))
        for op in ("rsqrt", "sqrt"):
            xi = _rand(rng(), (2, 2, 256), dt, 0.1, 10.0, O=O)
            add(f"{op}_{dt}", f"{op}_{dt}", [xi], xi.shape, npdt, lambda ins, op=op, dt=dt: O.unary(op, ins[0], dt))
        xi = _rand(rng(), (2, 2, 256), dt, O=O)
        add(f"copy_{dt}", f"copy_{dt}", [xi], xi.shape, npdt, lambda ins, dt=dt: O.unary("copy", ins[0], dt))
        # binary with broadcast: ops_arithmetic_test.cpp (same-shape and broadcast cases)
        for op in ("add", "sub", "mul", "div"):
            lo, hi = (0.5, 2.0) if op == "div" else (-1.0, 1.0)
            a = _rand(rng(), (2, 3, 4, 64), dt, -1.0, 1.0, O=O)
            b = _rand(rng(), (2, 3, 4, 64), dt, lo, hi, O=O)
            add(f"{op}_{dt}", f"{op}_{dt}", [a, b], a.shape, npdt, lambda ins, op=op, dt=dt: O.binary(op, ins[0], ins[1], dt))
            b1 = _rand(rng(), (1, 3, 1, 64), dt, lo, hi, O=O)
            add(f"{op}_bcast_{dt}", f"{op}_{dt}", [a, b1], a.shape, npdt,
                lambda ins, op=op, dt=dt: O.binary(op, ins[0], ins[1], dt))
            b2 = _rand(rng(), (4, 1), dt, lo, hi, O=O)
            add(f"{op}_bcast2_{dt}", f"{op}_{dt}", [a, b2], a.shape, npdt,
                lambda ins, op=op, dt=dt: O.binary(op, ins[0], ins[1], dt))
        # scalar ops with the reference's factor 0.7
        for op in ("add", "sub", "mul", "div"):
            xi = _rand(rng(), (2, 2, 128), dt, -1.0, 1.0, O=O)
            add(f"scalar_{op}_{dt}", f"scalar_{op}_{dt}", [xi], xi.shape, npdt,
                lambda ins, op=op, dt=dt: O.scalar(op, ins[0], 0.7, dt))
        # rope: ops_rope_test.cpp uses {1,32,32,256}
        a = _rand(rng(), (1, 4, 8, 64), dt, -1.0, 1.0, O=O)
        b = _rand(rng(), (1, 4, 8, 64), dt, -1.0, 1.0, O=O)
        add(f"rope_{dt}", f"rope_{dt}", [a, b], a.shape, npdt, lambda ins, dt=dt: O.rope(ins[0], ins[1], dt))
        # transpose: ops_transpose_test.cpp ({5,3,32,128})
        xi = _rand(rng(), (2, 3, 8, 16), dt, O=O)
        add(f"transpose_0132_{dt}", f"transpose_0132_{dt}", [xi], (2, 3, 16, 8), npdt,
            lambda ins: O.transpose(ins[0], [0, 1, 3, 2]))
        add(f"transpose_0231_{dt}", f"transpose_0231_{dt}", [xi], (2, 8, 16, 3), npdt,
            lambda ins: O.transpose(ins[0], [0, 2, 3, 1]))
        # embedding: ops_embedding_test.cpp (100 x 4096 table, negative indices allowed)
        r = rng()
        w = _rand(r, (50, 64), dt, O=O)
        idx = r.integers(-50, 50, size=(2, 3, 5)).astype(np.int32)
        add(f"embedding_{dt}", f"embedding_{dt}", [idx, w], (2, 3, 5, 64), npdt,
            lambda ins: O.embedding(ins[0], ins[1]))

    # casts: ops_cast_test.cpp
    for frm, to in (("fp16", "fp32"), ("fp32", "fp16"), ("bf16", "fp32"), ("fp32", "bf16"), ("fp16", "int32"),
                    ("int32", "fp16"), ("fp32", "int32"), ("int32", "fp32")):
        r = rng()
        if frm == "int32":
            xi = r.integers(-10000, 10000, size=(2, 2, 128)).astype(np.int32)
        else:
            xi = _rand(r, (2, 2, 128), frm, -100.0, 100.0, O=O)
        add(f"cast_{frm}_{to}", f"cast_{frm}_{to}", [xi], xi.shape, O.NP[to],
            lambda ins, frm=frm, to=to: O.cast(ins[0], frm, to))
    return cases
