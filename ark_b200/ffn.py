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
