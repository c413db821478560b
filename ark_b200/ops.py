"""Functional operator API — same names and argument meaning as the reference
front end (python/ark/ops.py), building ops on the global Model.

Engine extensions (no counterpart op in the reference, which composes them
from several ops): `rmsnorm`, `silu`, fused `softmax`/`layernorm` row kernels
(selected with `fused=True`), and `all_reduce` as one collective op.
"""
import math

from . import data_type as dt
from .error import ModelError
from .model import Model, Tensor, Buffer

NullTensor = None


def _m():
    return Model.get_model()


def _broadcast_shape(a, b):
    ra, rb = list(a)[::-1], list(b)[::-1]
    out = []
    for i in range(max(len(ra), len(rb))):
        x = ra[i] if i < len(ra) else 1
        y = rb[i] if i < len(rb) else 1
        if x != y and x != 1 and y != 1:
            raise ModelError(f"shapes {a} and {b} do not broadcast")
        out.append(max(x, y))
    return out[::-1]


def _out_like(shape, dtype, output, padded_shape=None):
    m = _m()
    if output is not None:
        if list(output.shape) != list(shape):
            raise ModelError(f"output shape {output.shape} does not match {shape}")
        return output
    return Tensor(m, dtype, Buffer(m), shape, padded_shape=padded_shape)


def _result_of(output):
    return output.clone_view()


# ---- tensors -----------------------------------------------------------------
def tensor(shape, dtype=dt.fp32, strides=None, offsets=None, padded_shape=None, rank=-1, name="tensor"):
    """ark.tensor (python/ark/ops.py:418-431)."""
    return _m().new_tensor(list(shape), dtype, strides, offsets, padded_shape, rank, name)


def parameter(shape, dtype=dt.fp32, strides=None, offsets=None, padded_shape=None, name="parameter"):
    return tensor(shape, dtype, strides, offsets, padded_shape, -1, name)


def reshape(input, shape, allowzero=False, name="reshape"):
    """View with a new shape over the same buffer (ark/ops/ops_reshape.cpp). Dense inputs only."""
    shape = list(shape)
    n = input.nelems()
    if -1 in shape:
        known = 1
        for s in shape:
            if s != -1:
                known *= s
        shape[shape.index(-1)] = n // known
    p = 1
    for s in shape:
        p *= s
    if p != n:
        raise ModelError(f"cannot reshape {input.shape} to {shape}")
    if not input.is_dense():
        raise ModelError("reshape needs a dense tensor")
    t = Tensor(_m(), input.dtype, input.buffer, shape)
    _m().add_op("Reshape", name, [input], [], [t], virtual=True)
    return t


def identity(input, deps=(), name="identity"):
    """Same view, new id; `deps` only express ordering (ark/ops/ops_identity.cpp)."""
    t = input.clone_view()
    _m().add_op("Identity", name, [input] + list(deps), [], [t], virtual=True)
    return t


def refer(input, shape, strides, offsets, padded_shape, dtype=None, name="refer"):
    t = Tensor(_m(), dtype or input.dtype, input.buffer, shape, strides, offsets, padded_shape)
    _m().add_op("Refer", name, [input], [], [t], virtual=True)
    return t


def sharding(input, axis, dim_per_shard, name="sharding"):
    """Splits a tensor along `axis` into views (ark/ops/ops_sharding.cpp)."""
    if axis < 0:
        axis += len(input.shape)
    out = []
    pos = 0
    while pos < input.shape[axis]:
        d = min(dim_per_shard, input.shape[axis] - pos)
        shape = list(input.shape)
        shape[axis] = d
        offs = list(input.offsets)
        offs[axis] += pos
        out.append(refer(input, shape, input.strides, offs, shape, name=f"{name}_{len(out)}"))
        pos += d
    return out


def noop(input, name="noop"):
    _m().add_op("Noop", name, [input], [], [])


# ---- elementwise ----------------------------------------------------------------
def _unary(type_, input, output, name):
    out = _out_like(input.shape, input.dtype, output)
    res = _result_of(out)
    _m().add_op(type_, name, [input], [out], [res])
    return res


def _binary(type_, input, other, output, name):
    if isinstance(other, (int, float)):
        raise ModelError("scalar operands go through scalar ops")
    if input.dtype is not other.dtype:
        raise ModelError("operand data types differ")
    out = _out_like(_broadcast_shape(input.shape, other.shape), input.dtype, output)
    res = _result_of(out)
    _m().add_op(type_, name, [input, other], [out], [res])
    return res


def add(input, other, output=None, name="add"):
    if isinstance(other, (int, float)):
        return _scalar("ScalarAdd", input, float(other), output, name)
    return _binary("Add", input, other, output, name)


def sub(input, other, output=None, name="sub"):
    if isinstance(other, (int, float)):
        return _scalar("ScalarAdd", input, -float(other), output, name)
    return _binary("Sub", input, other, output, name)


def mul(input, other, output=None, name="mul"):
    if isinstance(other, (int, float)):
        return _scalar("ScalarMul", input, float(other), output, name)
    return _binary("Mul", input, other, output, name)


def div(input, other, output=None, name="div"):
    if isinstance(other, (int, float)):
        return _scalar("ScalarMul", input, 1.0 / float(other), output, name)
    return _binary("Div", input, other, output, name)


def _scalar(type_, input, factor, output, name):
    out = _out_like(input.shape, input.dtype, output)
    res = _result_of(out)
    _m().add_op(type_, name, [input], [out], [res], {"Factor": float(factor)})
    return res


def constant(value, shape, dtype=dt.fp32, name="constant"):
    out = Tensor(_m(), dtype, Buffer(_m()), list(shape))
    res = _result_of(out)
    _m().add_op("ScalarAssign", name, [], [out], [res], {"Value": float(value)})
    return res


def ones(shape, dtype=dt.fp32, name="ones"):
    return constant(1.0, shape, dtype, name)


def zeros(shape, dtype=dt.fp32, name="zeros"):
    return constant(0.0, shape, dtype, name)


def exp(input, output=None, name="exp"):
    return _unary("Exp", input, output, name)


def gelu(input, output=None, name="gelu"):
    return _unary("Gelu", input, output, name)


def relu(input, output=None, name="relu"):
    return _unary("Relu", input, output, name)


def rsqrt(input, output=None, name="rsqrt"):
    return _unary("Rsqrt", input, output, name)


def sigmoid(input, output=None, name="sigmoid"):
    return _unary("Sigmoid", input, output, name)


def sqrt(input, output=None, name="sqrt"):
    return _unary("Sqrt", input, output, name)


def silu(input, output=None, name="silu"):
    """x * sigmoid(x) in one pass (engine extension; the reference composes sigmoid and mul)."""
    return _unary("Silu", input, output, name)


def copy(input, output=None, name="copy"):
    return _unary("Copy", input, output, name)


def cast(input, dtype, output=None, name="cast"):
    """ark.cast (ark/ops/ops_cast.cpp). Casting to/from `byte` reinterprets the bytes."""
    if dtype is input.dtype:
        return input
    if dtype is dt.byte or input.dtype is dt.byte:
        if not input.is_dense():
            raise ModelError("byte casts need a dense tensor")
        shape = list(input.shape)
        if dtype is dt.byte:
            shape[-1] *= input.dtype.nbytes
        else:
            if shape[-1] % dtype.nbytes:
                raise ModelError("byte tensor length is not a multiple of the element size")
            shape[-1] //= dtype.nbytes
        t = Tensor(_m(), dtype, input.buffer, shape)
        _m().add_op("Refer", name, [input], [], [t], virtual=True)
        return t
    out = _out_like(input.shape, dtype, output)
    res = _result_of(out)
    _m().add_op("Cast", name, [input], [out], [res])
    return res


def rope(input, other, output=None, name="rope"):
    return _binary("Rope", input, other, output, name)


# ---- reductions ----------------------------------------------------------------------
def _reduce(type_, input, axis, keepdims, output, name):
    nd = len(input.shape)
    ax = axis + nd if axis < 0 else axis
    if ax < 0 or ax >= nd:
        raise ModelError(f"invalid reduction axis {axis}")
    shape = list(input.shape)
    if keepdims:
        shape[ax] = 1
    else:
        shape.pop(ax)
    out = _out_like(shape, input.dtype, output)
    if out is input:
        raise ModelError("output tensor cannot be the same as input tensor for a reduce op")
    res = _result_of(out)
    _m().add_op(type_, name, [input], [out], [res], {"Axis": int(ax), "KeepDim": bool(keepdims)})
    return res


def reduce_sum(input, axis, keepdims=True, output=None, name="reduce_sum"):
    return _reduce("ReduceSum", input, axis, keepdims, output, name)


def reduce_mean(input, axis, keepdims=True, output=None, name="reduce_mean"):
    return _reduce("ReduceMean", input, axis, keepdims, output, name)


def reduce_max(input, axis, keepdims=True, output=None, name="reduce_max"):
    return _reduce("ReduceMax", input, axis, keepdims, output, name)


def mean(input, axis, keepdims=True, output=None, name="mean"):
    return reduce_mean(input, axis, keepdims, output, name)


# ---- matmul -----------------------------------------------------------------------------
def matmul(input, other, output=None, transpose_input=False, transpose_other=False, name="matmul"):
    """ark.matmul (ark/ops/ops_matmul.cpp:13-106): [N,C,H,W] batches broadcast over N and C."""
    if input.dtype is not other.dtype:
        raise ModelError("operand data types differ")

    def mnk(a, b):
        m = 1 if len(a) == 1 else a[-2]
        k = a[-1]
        n = 1 if len(b) == 1 else b[-1]
        k2 = b[0] if len(b) == 1 else b[-2]
        if transpose_input:
            m, k = k, m
        if transpose_other:
            n, k2 = k2, n
        if k != k2:
            raise ModelError(f"inner dimensions mismatch: {k} and {k2}")
        return m, n, k

    def oshape(a, b):
        m, n, _ = mnk(a, b)
        nd = max(len(a), len(b))
        if nd < 3:
            return [m, n]
        a4 = [1] * (4 - len(a)) + list(a)
        b4 = [1] * (4 - len(b)) + list(b)
        nc = _broadcast_shape(a4[:2], b4[:2])
        return [nc[0], nc[1], m, n] if nd == 4 else [nc[1], m, n]

    shape = oshape(input.shape, other.shape)
    padded = oshape(input.padded_shape, other.padded_shape)
    out = _out_like(shape, input.dtype, output, padded)
    res = _result_of(out)
    _m().add_op("Matmul", name, [input, other], [out], [res],
                {"TransposeInput": bool(transpose_input), "TransposeOther": bool(transpose_other)})
    return res


# ---- layout ------------------------------------------------------------------------------
def transpose(input, perm, output=None, name="transpose"):
    nd = len(input.shape)
    perm = [int(p) for p in perm]
    if sorted(perm) != list(range(nd)):
        raise ModelError(f"invalid permutation {perm}")
    shape = [input.shape[p] for p in perm]
    out = _out_like(shape, input.dtype, output)
    res = _result_of(out)
    _m().add_op("Transpose", name, [input], [out], [res], {"Permutation": perm})
    return res


def embedding(input, weight, output=None, name="embedding"):
    """Row gather (ark/ops/ops_embedding.cpp:11-70): input INT32 indices, weight [num_emb, dim]."""
    if input.dtype is not dt.int32:
        raise ModelError("embedding indices must be int32")
    if len(input.shape) > 3:
        raise ModelError("embedding input has at most 3 dimensions")
    shape = list(input.shape) + [weight.shape[-1]]
    out = _out_like(shape, weight.dtype, output)
    res = _result_of(out)
    _m().add_op("Embedding", name, [input, weight], [out], [res])
    return res


# ---- compositions / fused rows ----------------------------------------------------------------
def softmax(input, output=None, name="softmax", fused=True, scale=1.0, mask=None):
    """Softmax over the last axis of `input * scale + mask`. The reference composes five ops
    (python/ark/ops.py:491-500) after a separate scale and mask add; `fused=True` runs one row
    kernel instead. `mask` is additive, shaped [1, 1, rows, cols] or [1, 1, 1, cols]; the masked
    logits are rounded to the storage type before the softmax, like the separate ops would."""
    if fused:
        out = _out_like(input.shape, input.dtype, output)
        res = _result_of(out)
        reads = [input] if mask is None else [input, mask]
        _m().add_op("Softmax", name, reads, [out], [res], {"Scale": float(scale), "Mask": mask is not None})
        return res
    x = input if scale == 1.0 else mul(input, float(scale))
    if mask is not None:
        x = add(x, mask)
    mx = reduce_max(x, axis=-1)
    e = exp(sub(x, mx))
    s = reduce_sum(e, axis=-1)
    return div(e, s, output)


def decode_attention(q, k_cache, v_cache, scale=1.0, output=None, name="decode_attention"):
    """softmax(scale * q . K^T) . V for ONE query row per head against a K/V cache: q [B, Hq, 1, 128],
    k_cache and v_cache [B, Hkv, T, 128] with Hq / Hkv in {1, 2, 4, 8} (grouped-query attention).
    Engine extension: the reference example builds it from two matmuls, a scale and a softmax
    (examples/llama/model.py:336-444); here the cache is read once."""
    if len(q.shape) != 4 or q.shape[2] != 1 or len(k_cache.shape) != 4 or list(k_cache.shape) != list(v_cache.shape):
        raise ModelError("decode_attention: q [B, Hq, 1, D], k_cache and v_cache [B, Hkv, T, D]")
    out = _out_like(q.shape, q.dtype, output)
    res = _result_of(out)
    _m().add_op("DecodeAttention", name, [q, k_cache, v_cache], [out], [res], {"Scale": float(scale)})
    return res


def prefill_attention(q, k, v, scale=1.0, causal=True, token_major=False, mask=None, output=None, name="prefill_attention"):
    """softmax(scale * q . k^T [+ causal mask]) . v for many query rows per head, head dimension 128:
    q [B, Hq, Tq, 128], k and v [B, Hkv, Tkv, 128] (Hq a multiple of Hkv: grouped-query attention), result as q.
    With token_major=True all four tensors are [B, T, H, 128], the layout the projection matmuls leave behind, so
    no transpose is needed on either side. causal=True: row i attends to keys [0, i + Tkv - Tq] (key tiles past the
    diagonal are skipped). mask: an additive mask [B or 1, Hq or 1, Tq, Tkv] of the operands' type (the tensor
    examples/llama/model.py:419-420 adds to the scores), added to scale * q . k^T; every key tile is computed then.
    Engine extension: the reference example builds the block from two matmuls, a scale, a mask add and a softmax
    (examples/llama/model.py:336-444) and writes the [B, H, T, T] scores to memory twice; here the scores stay
    in tensor memory (S = q k^T and O = P v on tcgen05, online softmax in fp32, P rounded to the storage type)."""
    hx, tx = (2, 1) if token_major else (1, 2)
    if len(q.shape) != 4 or len(k.shape) != 4 or list(k.shape) != list(v.shape) or q.shape[3] != 128 or k.shape[3] != 128 \
            or q.shape[0] != k.shape[0] or q.shape[hx] % k.shape[hx]:
        raise ModelError("prefill_attention: q [B, Hq, Tq, 128], k and v [B, Hkv, Tkv, 128], Hq a multiple of Hkv")
    if mask is not None:
        ms = [1] * (4 - len(mask.shape)) + list(mask.shape)
        if ms[2] != q.shape[tx] or ms[3] != k.shape[tx] or ms[0] not in (1, q.shape[0]) or ms[1] not in (1, q.shape[hx]):
            raise ModelError("prefill_attention: mask [B or 1, Hq or 1, Tq, Tkv]")
    out = _out_like(q.shape, q.dtype, output)
    res = _result_of(out)
    _m().add_op("PrefillAttention", name, [q, k, v] + ([mask] if mask is not None else []), [out], [res],
                {"Scale": float(scale), "Causal": int(bool(causal)), "TokenMajor": int(bool(token_major))})
    return res


def layernorm(input, eps=1e-5, output=None, name="layernorm", fused=True):
    """Layer normalisation over the last axis (python/ark/ops.py:503-513 composes six ops)."""
    if fused:
        out = _out_like(input.shape, input.dtype, output)
        res = _result_of(out)
        _m().add_op("LayerNorm", name, [input], [out], [res], {"Eps": float(eps)})
        return res
    mu = reduce_mean(input, axis=-1)
    x = sub(input, mu)
    var = reduce_mean(mul(x, x), axis=-1)
    return mul(x, rsqrt(add(var, float(eps))), output)


def rmsnorm(input, weight=None, eps=1e-5, output=None, residual=None, name="rmsnorm"):
    """RMSNorm row kernel for the pattern examples/llama/model.py:92-99 builds
    from cast/mul/reduce_mean/rsqrt/mul. With `residual`, normalises
    input + residual and also returns the sum: (normed, summed)."""
    out = _out_like(input.shape, input.dtype, output)
    res = _result_of(out)
    reads = [input] + ([weight] if weight is not None else [])
    args = {"Eps": float(eps)}
    if residual is None:
        _m().add_op("RMSNorm", name, reads, [out], [res], args)
        return res
    summed = Tensor(_m(), input.dtype, Buffer(_m()), input.shape)
    sres = _result_of(summed)
    args["Residual"] = True
    _m().add_op("RMSNorm", name, reads + [residual], [out, summed], [res, sres], args)
    return res, sres


# ---- communication ------------------------------------------------------------------------------
def send(input, remote_rank, tag, output=None, name="send"):
    """ark::Model::send (ark/ops/ops_communication.cpp:18-43)."""
    m = _m()
    if output is None:
        output = Tensor(m, input.dtype, Buffer(m, remote_rank), input.shape, input.strides, input.offsets,
                        input.padded_shape)
    elif output.buffer.rank != remote_rank:
        raise ModelError(f"invalid buffer rank: {output.buffer.rank}, expected: {remote_rank}")
    input.buffer.tag_send(remote_rank, tag)
    output.buffer.tag_recv(-1, tag)
    res = _result_of(output)
    m.add_op("Send", name, [input], [output], [res])
    return res


def send_done(input, name="send_done"):
    res = input.clone_view()
    _m().add_op("SendDone", name, [input], [], [res])
    return res


def recv(output, remote_rank, tag, name="recv"):
    """ark::Model::recv (ark/ops/ops_communication.cpp:122-139)."""
    m = _m()
    res = _result_of(output)
    stand_in = Tensor(m, output.dtype, Buffer(m, remote_rank), output.shape, output.strides, output.offsets,
                      output.padded_shape)
    stand_in.buffer.tag_send(-1, tag)
    output.buffer.tag_recv(remote_rank, tag)
    m.add_op("Recv", name, [stand_in], [output], [res])
    return res


def device_sync(input, rank, rank_num, name="device_sync"):
    res = input.clone_view()
    _m().add_op("DeviceSync", name, [input], [input], [res], {"Rank": int(rank), "PeerNum": int(rank_num) - 1})
    return res


def _nbytes(t):
    return t.nelems() * t.dtype.nbytes


def send_packet(input, remote_rank, tag, flag, output=None, name="send_packet"):
    """ark::Model::send_packet (ark/ops/ops_communication.cpp:171-197, 612-619): `input` goes to `output`, a UINT8
    packet tensor on `remote_rank` twice the size of the data (payload and flag words travel together)."""
    m = _m()
    if output is None:
        output = Tensor(m, dt.uint8, Buffer(m, remote_rank), [_nbytes(input) * 2])
    elif output.buffer.rank != remote_rank:
        raise ModelError(f"invalid buffer rank: {output.buffer.rank}, expected: {remote_rank}")
    output.buffer.tag_recv(-1, tag)
    res = _result_of(output)
    m.add_op("SendPacket", name, [input], [output], [res], {"Flag": int(flag)})
    return res


def recv_packet(output, remote_rank, tag, flag, scratch=None, name="recv_packet"):
    """ark::Model::recv_packet (ops_communication.cpp:262-292, 621-628): waits for the packets `remote_rank` wrote into
    the local packet tensor `scratch` and unpacks them into `output`."""
    m = _m()
    if scratch is None:
        scratch = Tensor(m, dt.uint8, Buffer(m, output.buffer.rank), [_nbytes(output) * 2])
    elif scratch.buffer.rank not in (-1, output.buffer.rank, m.rank):
        raise ModelError(f"invalid buffer rank: {scratch.buffer.rank}")
    sender = Tensor(m, output.dtype, Buffer(m, remote_rank), output.shape)  # names the sender only
    scratch.buffer.tag_recv(remote_rank, tag)
    res = _result_of(output)
    m.add_op("RecvPacket", name, [sender, scratch], [output], [res], {"Flag": int(flag)})
    return res


def _recv_reduce_send(type_, input, remote_ranks, recv_tag, output_tag, flag, output, peer_outputs, scratch, name):
    m = _m()
    n = len(remote_ranks)
    packets = flag is not None
    if scratch is None:
        if packets:
            scratch = Tensor(m, dt.uint8, Buffer(m, m.rank), [_nbytes(input) * 2 * n])
        else:
            scratch = Tensor(m, input.dtype, Buffer(m, m.rank), [input.nelems() * n])
    elif scratch.buffer.rank not in (-1, m.rank):
        raise ModelError(f"invalid buffer rank: {scratch.buffer.rank}, expected: {m.rank}")
    if output is None:
        output = Tensor(m, input.dtype, Buffer(m, m.rank), input.shape, input.strides, input.offsets, input.padded_shape)
    if not peer_outputs:
        if packets:
            peer_outputs = [Tensor(m, dt.uint8, Buffer(m, r), [_nbytes(input) * 2]) for r in remote_ranks]
        else:
            peer_outputs = [Tensor(m, input.dtype, Buffer(m, r), input.shape, input.strides, input.offsets, input.padded_shape)
                            for r in remote_ranks]
    for r, po in zip(remote_ranks, peer_outputs):
        scratch.buffer.tag_recv(r, recv_tag)
        po.buffer.tag_recv(-1, output_tag)
    res = _result_of(output)
    args = {"NPeers": n, "Rank": int(m.rank)}
    if packets:
        args["Flag"] = int(flag)
    m.add_op(type_, name, [input, scratch], [output] + list(peer_outputs), [res], args)
    return res


def recv_reduce_send_packet(input, remote_ranks, recv_tag, output_tag, flag, output=None, peer_outputs=None, scratch=None,
                            name="recv_reduce_send_packet"):
    """ark::Model::recv_reduce_send_packet (ops_communication.cpp:353-399, 630-661): sums `input` with the packets the
    peers sent into `scratch`, stores the sum in `output` and sends it, as packets, to every peer's output tensor."""
    return _recv_reduce_send("RecvReduceSendPacket", input, list(remote_ranks), recv_tag, output_tag, int(flag), output,
                             peer_outputs, scratch, name)


def recv_reduce_send(input, remote_ranks, recv_tag, output_tag, output=None, peer_outputs=None, scratch=None,
                     name="recv_reduce_send"):
    """ark::Model::recv_reduce_send (ops_communication.cpp:455-500, 663-692): the same step on plain data; a
    device_sync before it says that the peers' shards have arrived."""
    return _recv_reduce_send("RecvReduceSend", input, list(remote_ranks), recv_tag, output_tag, None, output, peer_outputs,
                             scratch, name)


def all_reduce_packet(input, rank, rank_num, flag=1, output=None):
    """The packet all_reduce the reference composes in its tests (ark/ops/ops_all_reduce_test.cpp:52-118): every rank
    sends shard i to rank i as packets, reduces its own shard with the n-1 it received and sends the sum to every
    peer, then unpacks the n-1 sums it receives. Scratch halves alternate with the parity of `flag`."""
    from .planner import PlannerContext
    m = _m()
    tag_send_reduce, tag_output = m.unique_tag(), m.unique_tag()
    if output is None:
        output = tensor(input.shape, input.dtype, input.strides, input.offsets, input.padded_shape)
    peers = [i for i in range(rank_num) if i != rank]
    flat_in, flat_out = reshape(input, [input.nelems()]), reshape(output, [output.nelems()])
    per = flat_in.nelems() // rank_num
    nb = per * flat_in.dtype.nbytes
    ins, outs = sharding(flat_in, 0, per), sharding(flat_out, 0, per)
    npeer = rank_num - 1
    scratch_off = 0 if flag % 2 == 0 else nb * npeer * 2
    scratch_strides = [nb * 2 * npeer * 2]
    for i in peers:
        slot = rank - 1 if i < rank else rank
        dst = tensor([nb * 2], dt.uint8, scratch_strides, [scratch_off + nb * slot * 2], [nb * 2], i)
        send_packet(ins[i], i, tag_send_reduce, flag, dst)
    scratch = tensor([nb * 2 * npeer], dt.uint8, scratch_strides, [scratch_off], [nb * 2 * npeer])
    out_off = 0 if flag % 2 == 0 else nb * 2
    peer_outs = [tensor([nb * 2], dt.uint8, [nb * 4], [out_off], [nb * 2], i) for i in peers]
    deps = [recv_reduce_send_packet(ins[rank], peers, tag_send_reduce, tag_output, flag, outs[rank], peer_outs, scratch)]
    for i in peers:
        mine = tensor([nb * 2], dt.uint8, [nb * 4], [out_off], [nb * 2])
        deps.append(recv_packet(outs[i], i, tag_output, flag, mine))
    return identity(output, deps)


def all_reduce_sm(input, rank, rank_num, output=None):
    """The plain-data all_reduce of the reference's tests (ark/ops/ops_all_reduce_test.cpp:139-187): put shard i into
    rank i's scratch, device_sync, recv_reduce_send of the own shard (sum stored into every rank's tensor),
    device_sync. In place on `input` (as the reference test uses it)."""
    from .planner import PlannerContext
    m = _m()
    send_tag, recv_tag = m.unique_tag(), m.unique_tag()
    peers = [i for i in range(rank_num) if i != rank]
    flat_in = reshape(input, [input.nelems()])
    per = flat_in.nelems() // rank_num
    npeer = rank_num - 1
    ins = sharding(flat_in, 0, per)
    with PlannerContext(config={"ChannelType": "Sm", "Signal": False}):
        for i in peers:
            slot = rank - 1 if i < rank else rank
            dst = tensor([per], flat_in.dtype, [per * npeer], [per * slot], [per], i)
            send(ins[i], i, send_tag, dst)
    device_sync(flat_in, rank, rank_num)
    recv_reduce_send(ins[rank], peers, send_tag, recv_tag, ins[rank])
    with PlannerContext(config={"ChannelType": "Sm", "Wait": False}):
        for i in peers:
            recv(ins[i], i, recv_tag)
    return device_sync(input, rank, rank_num)


def all_reduce(input, rank, world_size, output=None, name="all_reduce", naive=False, gather=True):
    """Sum over ranks. The reference composes world_size-1 rounds of
    send/send_done/recv/add (ark/ops/ops_all_reduce.cpp:8-37, kept as
    `naive=True`); by default this is one in-kernel collective on `output`
    (in place on a copy of `input` when `output` is None). `gather=False`
    (only with a Matmul planned into the same task): rank r keeps the sum of
    rows [r*M/p, (r+1)*M/p) only, the rest of `output` is undefined."""
    m = _m()
    if output is None:
        output = copy(input)
    elif output is not input:
        output = copy(input, output)
    if world_size == 1:
        return output
    if naive:
        tags = [m.unique_tag() for _ in range(world_size)]
        prev_recv = None
        cumulate = output
        for i in range(1, world_size):
            dst = (rank + i) % world_size
            src = (rank + world_size - i) % world_size
            send_data = input if prev_recv is None else identity(input, [prev_recv])
            send_data = send(send_data, dst, tags[rank])
            sd = send_done(send_data)
            recv_buf = tensor(output.shape, output.dtype)
            recv_t = identity(recv_buf, [sd])
            recv_t = recv(recv_buf, src, tags[src])
            prev_recv = recv_t
            cumulate = add(cumulate, recv_t, cumulate)
        return cumulate
    res = output.clone_view()
    tag = m.unique_tag()
    args = {"Tag": int(tag), "Rank": int(rank), "RankNum": int(world_size)}
    if not gather:
        args["Gather"] = False
    m.add_op("AllReduce", name, [output], [output], [res], args)
    return res
