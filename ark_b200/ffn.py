"""Megatron-split feed-forward block: Y = act(X W1) W2 with W1 split by columns
and W2 by rows over the ranks, partial outputs summed by all_reduce
(the layout of examples/transformer/megatron_ark.py:14-33 and
examples/llama/model.py:316-333 in the reference)."""
from . import ops
from .planner import PlannerContext


def build_ffn(tokens, d_model, d_ff, dtype, rank=0, world_size=1, act="gelu", fuse_act=True, weights_nk=False,
              fuse_all_reduce=True):
    """Adds the block to the global model. Returns (x, w1_shard, w2_shard, out).
    w1_shard is [d_model, d_ff / world_size], w2_shard is [d_ff / world_size, d_model]."""
    if d_ff % world_size:
        raise ValueError("d_ff must be divisible by the world size")
    shard = d_ff // world_size
    x = ops.tensor([tokens, d_model], dtype, name="x")
    # weights_nk stores the weights [out_features, in_features] (as nn.Linear / the llama example do)
    w1 = ops.tensor([shard, d_model] if weights_nk else [d_model, shard], dtype, name="w1")
    w2 = ops.tensor([d_model, shard] if weights_nk else [shard, d_model], dtype, name="w2")
    actf = getattr(ops, act)
    if fuse_act:
        with PlannerContext(sync=False):  # one task: the activation runs in the GEMM epilogue
            h = actf(ops.matmul(x, w1, transpose_other=weights_nk))
    else:
        h = actf(ops.matmul(x, w1, transpose_other=weights_nk))
    if world_size > 1 and fuse_all_reduce:
        # one task: the W2 matmul's epilogue stores its tiles on the rank that sums them (needs tokens to be a
        # multiple of 256 x world size; otherwise the two run one after the other as below)
        with PlannerContext(sync=False):
            y = ops.matmul(h, w2, transpose_other=weights_nk)
            y = ops.all_reduce(y, rank, world_size, output=y)
        return x, w1, w2, y
    y = ops.matmul(h, w2, transpose_other=weights_nk)
    if world_size > 1:
        y = ops.all_reduce(y, rank, world_size, output=y)
    return x, w1, w2, y


def build_ffn_streaming(tokens, d_model, d_ff, dtype, rank=0, world_size=1, act="gelu", slots=2):
    """The same block fed and drained through rings of `slots` buffers, for a resident loop kernel that takes a new
    batch every iteration: iteration i reads its rows of X from slot (i-1) % slots of `x_ring` and leaves its rows of
    Y in the same slot of `y_ring`, so the host fills and drains the other slots meanwhile. With several ranks each
    rank feeds rows [r*T/p, (r+1)*T/p) only; the ranks exchange them over NVLink (peer stores into every rank's X),
    and the all_reduce keeps each rank's own rows of the sum (no gather: the host reads Y shard by shard).
    Returns (x_ring [slots, T/p, d_model], w1_shard, w2_shard, y_ring [slots, T/p, d_model])."""
    p = world_size
    if d_ff % p or tokens % p:
        raise ValueError("d_ff and tokens must be divisible by the world size")
    shard, rows = d_ff // p, tokens // p
    x_ring = ops.tensor([slots, rows, d_model], dtype, name="x_ring")
    y_ring = ops.tensor([slots, rows, d_model], dtype, name="y_ring")
    x = ops.tensor([tokens, d_model], dtype, name="x")
    w1 = ops.tensor([d_model, shard], dtype, name="w1")
    w2 = ops.tensor([shard, d_model], dtype, name="w2")
    x_rows = ops.sharding(x, 0, rows)
    slot0 = ops.refer(x_ring, [rows, d_model], [slots * rows, d_model], [0, 0], [rows, d_model])  # slot 0 as a 2-D view
    ring = {"IterSlots": slots, "InIterStride": rows * d_model}
    deps = []
    with PlannerContext(config=ring):
        deps.append(ops.copy(slot0, x_rows[rank]))
    tag = Model_unique_tag()
    for q in range(p):
        if q == rank:
            continue
        dst = ops.tensor([rows, d_model], dtype, [tokens, d_model], [rank * rows, 0], [rows, d_model], rank=q)
        with PlannerContext(config=dict(ring, ChannelType="Sm", Signal=False)):
            deps.append(ops.send(slot0, q, tag, dst))
        x_rows[q].buffer.tag_recv(q, tag)  # the peers' rows land in this rank's X
    xin = ops.identity(x, deps)
    if p > 1:
        xin = ops.device_sync(xin, rank, p)
    with PlannerContext(sync=False):
        h = getattr(ops, act)(ops.matmul(xin, w1))
    if p > 1:
        with PlannerContext(sync=False):
            y = ops.matmul(h, w2)
            y = ops.all_reduce(y, rank, p, output=y, gather=False)
    else:
        y = ops.matmul(h, w2)
    y_rows = ops.sharding(y, 0, rows)[rank]
    with PlannerContext(config={"IterSlots": slots, "OutIterStride": rows * d_model}):
        ops.copy(y_rows, ops.refer(y_ring, [rows, d_model], [slots * rows, d_model], [0, 0], [rows, d_model]))
    return x_ring, w1, w2, y_ring


def Model_unique_tag():
    from .model import Model
    return Model.get_model().unique_tag()
