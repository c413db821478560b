"""ctypes front-end of the CPU oracle (TEST INFRASTRUCTURE, not product code).

Two libraries sit behind it:

* ``libark_oracle.so``  — the C restatement of the reference's host baselines
  (``oracle/ark_oracle.c``); every function there cites the reference lines
  it follows.
* ``_ref/libark_ref.so`` — the reference's own baseline templates compiled
  from the reference checkout (``oracle/ref_shim.cpp``); optional, used to pin
  the restatement and to generate ``tests/golden``.

Only ``tests/``, ``__graft_entry__.smoke()`` and the ``cpu_baseline`` /
``--impl reference`` legs of ``bench.py`` may import this module.

Arrays are numpy; ``bf16`` tensors are carried as ``uint16`` bit patterns
(numpy has no bfloat16), ``fp16`` as ``float16``.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
DT = {"fp32": 0, "fp16": 1, "bf16": 2, "int32": 3, "uint32": 4, "int8": 5, "uint8": 6, "byte": 6}
NP = {"fp32": np.float32, "fp16": np.float16, "bf16": np.uint16, "int32": np.int32, "uint32": np.uint32,
      "int8": np.int8, "uint8": np.uint8, "byte": np.uint8}
UNARY = {"gelu": 0, "exp": 1, "relu": 2, "rsqrt": 3, "sigmoid": 4, "sqrt": 5, "copy": 6}
BINARY = {"add": 0, "sub": 1, "mul": 2, "div": 3}
REDUCE = {"sum": 0, "max": 1, "mean": 2}


def build(force=False):
    """Compile the oracle libraries (and the reference baselines when the
    reference checkout is present)."""
    if force or not os.path.exists(os.path.join(_HERE, "libark_oracle.so")):
        subprocess.check_call(["make", "-s", "-C", _HERE, "-f", os.path.join(_HERE, "Makefile")])


_lib = None
_ref = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(os.path.join(_HERE, "libark_oracle.so"))
    return _lib


def ref_lib():
    """The compiled reference baselines, or None when they were never built."""
    global _ref
    if _ref is None:
        p = os.path.join(_HERE, "_ref", "libark_ref.so")
        if not os.path.exists(p):
            return None
        _ref = ctypes.CDLL(p)
    return _ref


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _i64(v):
    return (ctypes.c_int64 * len(v))(*[int(x) for x in v])


def dims4(shape):
    shape = list(shape)
    return [1] * (4 - len(shape)) + shape


# ---- bf16 helpers -----------------------------------------------------------
def f32_to_bf16_bits(x):
    """fp32 -> bf16 bit patterns, round to nearest even."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    nan = np.isnan(x)
    if np.any(nan):
        r = np.where(nan, np.uint16(0x7FFF), r)
    return r


def bf16_bits_to_f32(b):
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def to_storage(x, dt):
    """fp32 values -> storage array of dtype ``dt``."""
    if dt == "bf16":
        return f32_to_bf16_bits(np.asarray(x, dtype=np.float32))
    return np.ascontiguousarray(np.asarray(x).astype(NP[dt]))


def to_f32(a, dt):
    if dt == "bf16":
        return bf16_bits_to_f32(a)
    return np.asarray(a).astype(np.float32)


# ---- ops ---------------------------------------------------------------------
def unary(op, x, dt):
    x = np.ascontiguousarray(x)
    out = np.empty_like(x)
    lib().orc_unary(UNARY[op], DT[dt], _p(out), _p(x), ctypes.c_size_t(x.size))
    return out


def binary(op, a, b, dt):
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b)
    osh = np.broadcast_shapes(a.shape, b.shape)
    out = np.empty(osh, dtype=a.dtype)
    lib().orc_binary(BINARY[op], DT[dt], _p(out), _i64(dims4(osh)), _p(a), _i64(dims4(a.shape)), _p(b),
                     _i64(dims4(b.shape)))
    return out


def scalar(op, x, val, dt):
    x = np.ascontiguousarray(x)
    out = np.empty_like(x)
    lib().orc_scalar(BINARY[op], DT[dt], _p(out), _p(x), ctypes.c_size_t(x.size), ctypes.c_float(val))
    return out


def fill(shape, val, dt):
    out = np.empty(shape, dtype=NP[dt])
    lib().orc_fill(DT[dt], _p(out), ctypes.c_size_t(out.size), ctypes.c_float(val))
    return out


def cast(x, frm, to):
    x = np.ascontiguousarray(x)
    out = np.empty(x.shape, dtype=NP[to])
    lib().orc_cast(DT[frm], DT[to], _p(out), _p(x), ctypes.c_size_t(x.size))
    return out


def reduce(kind, x, axis, dt, keepdims=True):
    x = np.ascontiguousarray(x)
    nd = x.ndim
    if axis < 0:
        axis += nd
    ax4 = axis + 4 - nd
    osh = list(x.shape)
    osh[axis] = 1
    out = np.empty(osh, dtype=x.dtype)
    lib().orc_reduce(REDUCE[kind], DT[dt], ax4, _p(out), _p(x), _i64(dims4(x.shape)))
    if not keepdims:
        out = out.reshape([s for i, s in enumerate(osh) if i != axis])
    return out


def rope(x, other, dt):
    x = np.ascontiguousarray(x)
    other = np.ascontiguousarray(other)
    out = np.empty_like(x)
    lib().orc_rope(DT[dt], _p(out), _p(x), _p(other), ctypes.c_size_t(x.size))
    return out


def transpose(x, perm):
    x = np.ascontiguousarray(x)
    nd = x.ndim
    perm4 = list(range(4 - nd)) + [p + 4 - nd for p in perm]
    ish = dims4(x.shape)
    osh = [ish[p] for p in perm4]
    out = np.empty(osh[4 - nd:], dtype=x.dtype)
    lib().orc_transpose(ctypes.c_size_t(x.itemsize), _p(out), _p(x), _i64(ish), (ctypes.c_int * 4)(*perm4))
    return out


def embedding(idx, weight):
    idx = np.ascontiguousarray(idx, dtype=np.int32)
    weight = np.ascontiguousarray(weight)
    out = np.empty(tuple(idx.shape) + (weight.shape[-1],), dtype=weight.dtype)
    lib().orc_embedding(ctypes.c_size_t(weight.itemsize), _p(out), _p(idx), _p(weight), ctypes.c_size_t(idx.size),
                        ctypes.c_int64(weight.shape[-2]), ctypes.c_int64(weight.shape[-1]))
    return out


def matmul(a, b, dt, trans_a=False, trans_b=False, act=None):
    """C = A·B with NumPy-style broadcast over the leading (N,C) batch dims,
    fp32 accumulation in k order, one rounding to ``dt``."""
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b)
    a2 = a.reshape((1,) * max(0, 2 - a.ndim) + a.shape)
    b2 = b.reshape(b.shape + (1,)) if b.ndim == 1 else b
    m, k = (a2.shape[-1], a2.shape[-2]) if trans_a else (a2.shape[-2], a2.shape[-1])
    n, k2 = (b2.shape[-2], b2.shape[-1]) if trans_b else (b2.shape[-1], b2.shape[-2])
    assert k == k2, (a.shape, b.shape)
    ba, bb = a2.shape[:-2], b2.shape[:-2]
    bo = np.broadcast_shapes(ba, bb)
    out = np.empty(tuple(bo) + (m, n), dtype=a.dtype)
    nb = int(np.prod(bo)) if bo else 1
    a3 = a2.reshape((-1,) + a2.shape[-2:])
    b3 = b2.reshape((-1,) + b2.shape[-2:])
    o3 = out.reshape((-1, m, n))
    idx = np.arange(nb).reshape(bo if bo else (1,))
    ia = np.broadcast_to(np.arange(a3.shape[0]).reshape(ba if ba else (1,)), idx.shape).reshape(-1)
    ib = np.broadcast_to(np.arange(b3.shape[0]).reshape(bb if bb else (1,)), idx.shape).reshape(-1)
    actc = {None: 0, "relu": 1, "gelu": 2}[act]
    for i in range(nb):
        lib().orc_matmul(DT[dt], _p(o3[i]), _p(a3[ia[i]]), _p(b3[ib[i]]), ctypes.c_int64(1), ctypes.c_int64(m),
                         ctypes.c_int64(n), ctypes.c_int64(k), int(trans_a), int(trans_b),
                         ctypes.c_int64(a3.shape[-1]), ctypes.c_int64(b3.shape[-1]), ctypes.c_int64(n),
                         ctypes.c_int64(0), ctypes.c_int64(0), ctypes.c_int64(0), actc)
    return out


def all_reduce(inputs, dt):
    inputs = [np.ascontiguousarray(x) for x in inputs]
    out = np.empty_like(inputs[0])
    ptrs = (ctypes.c_void_p * len(inputs))(*[x.ctypes.data for x in inputs])
    lib().orc_all_reduce(DT[dt], _p(out), ptrs, len(inputs), ctypes.c_size_t(out.size))
    return out


def rmsnorm(x, weight, dt, eps=1e-5):
    x = np.ascontiguousarray(x)
    out = np.empty_like(x)
    cols = x.shape[-1]
    w = None if weight is None else np.ascontiguousarray(weight)
    lib().orc_rmsnorm(DT[dt], _p(out), _p(x), _p(w) if w is not None else None, ctypes.c_int64(x.size // cols),
                      ctypes.c_int64(cols), ctypes.c_float(eps))
    return out


def softmax(x, dt):
    x = np.ascontiguousarray(x)
    out = np.empty_like(x)
    cols = x.shape[-1]
    lib().orc_softmax(DT[dt], _p(out), _p(x), ctypes.c_int64(x.size // cols), ctypes.c_int64(cols))
    return out


def layernorm(x, dt, eps=1e-5):
    x = np.ascontiguousarray(x)
    out = np.empty_like(x)
    cols = x.shape[-1]
    lib().orc_layernorm(DT[dt], _p(out), _p(x), ctypes.c_int64(x.size // cols), ctypes.c_int64(cols),
                        ctypes.c_float(eps))
    return out


# ---- the compiled reference baselines ---------------------------------------
def ref_call(name, outs, ins):
    """Run reference baseline ``ref_<name>`` (see oracle/ref_shim.cpp) on numpy
    arrays; ``outs`` are preallocated and filled in place."""
    r = ref_lib()
    if r is None:
        raise RuntimeError("oracle/_ref/libark_ref.so was not built")
    fn = getattr(r, "ref_" + name)
    no, ni = len(outs), len(ins)
    osh = []
    for o in outs:
        osh += list(o.shape) + [0] * (4 - o.ndim)
    ish = []
    for i in ins:
        ish += list(i.shape) + [0] * (4 - i.ndim)
    fn((ctypes.c_void_p * no)(*[o.ctypes.data for o in outs]), _i64(osh), (ctypes.c_int * no)(*[o.ndim for o in outs]),
       no, (ctypes.c_void_p * ni)(*[i.ctypes.data for i in ins]), _i64(ish),
       (ctypes.c_int * ni)(*[i.ndim for i in ins]), ni)
    return outs
