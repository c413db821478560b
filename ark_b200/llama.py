"""Llama-2-shaped decoder layers, tensor-parallel (Megatron split), built from the
engine's operators. Shapes follow examples/llama/model.py of the reference
(RMSNorm :79-99, Column/RowParallelLinear :102-216, FeedForward :316-333,
Attention :336-444): weights are stored [out_features, in_features]; QKV and
W1/W3 are split by output features, Wo and W2 by input features, and the two
partial outputs per layer are summed over the ranks.

Differences from the reference example, all inside one rank's graph:
RMSNorm and softmax (with the score scale and the causal mask folded in) are
single row kernels, SiLU runs in the W1 epilogue, the
two all_reduces are single in-kernel collectives, and a decode step reads a
K/V cache (the reference example has none).
"""
import math

from . import ops
from .planner import DEFAULT_NUM_SM, PlannerContext


class LlamaConfig:
    def __init__(self, dim=4096, n_heads=32, n_kv_heads=None, head_dim=128, ffn_dim=11008, norm_eps=1e-5, rope_theta=10000.0):
        self.dim, self.n_heads, self.head_dim = dim, n_heads, head_dim
        self.n_kv_heads = n_kv_heads or n_heads
        self.ffn_dim, self.norm_eps, self.rope_theta = ffn_dim, norm_eps, rope_theta


LLAMA2_7B = dict(dim=4096, n_heads=32, n_kv_heads=32, ffn_dim=11008)
LLAMA2_70B = dict(dim=8192, n_heads=64, n_kv_heads=8, ffn_dim=28672)


def layer_weights(cfg, dtype, world_size, prefix=""):
    """Creates this rank's weight tensors of one layer. Returns a dict name -> Tensor."""
    p = world_size
    hl, kvl, hd = cfg.n_heads // p, max(1, cfg.n_kv_heads // p), cfg.head_dim
    if cfg.ffn_dim % p or cfg.n_heads % p:
        raise ValueError("heads and ffn_dim must be divisible by the world size")
    f = cfg.ffn_dim // p
    t = ops.tensor
    return {
        "attn_norm": t([cfg.dim], dtype, name=prefix + "attn_norm"),
        "wq": t([hl * hd, cfg.dim], dtype, name=prefix + "wq"),
        "wk": t([kvl * hd, cfg.dim], dtype, name=prefix + "wk"),
        "wv": t([kvl * hd, cfg.dim], dtype, name=prefix + "wv"),
        "wo": t([cfg.dim, hl * hd], dtype, name=prefix + "wo"),
        "ffn_norm": t([cfg.dim], dtype, name=prefix + "ffn_norm"),
        "w1": t([f, cfg.dim], dtype, name=prefix + "w1"),
        "w3": t([f, cfg.dim], dtype, name=prefix + "w3"),
        "w2": t([cfg.dim, f], dtype, name=prefix + "w2"),
    }


def decoder_layer(x, w, cfg, batch, seq, rank, world_size, rope=None, mask=None, k_cache=None, v_cache=None, causal=False,
                  qkv_side_by_side=None, fused_attention=False, num_sm=DEFAULT_NUM_SM):
    """One layer on `x` [batch*seq, dim].

    Prefill: `mask` [1, 1, seq, seq] (additive, -inf above the diagonal) and `rope` [1, seq, 1, head_dim]
    (interleaved cos/sin pairs, examples/llama/model_test.py:379-384). Decode (seq == 1): `k_cache`/`v_cache`
    [batch, kv_heads_local, t_kv, head_dim] hold the keys/values attended to; `rope` is [1, 1, 1, head_dim].
    Prefill with causal=True (and no `mask` tensor; head_dim 128): the attention block is one fused stage that reads
    q, k, v in the [batch, seq, heads, head_dim] layout the projections leave and keeps the scores on chip, so the
    four transposes, the scores tensor and the mask tensor of the reference's chain disappear. fused_attention=True
    with a `mask` tensor: the same stage in its general form, the mask added to the scaled scores on chip (every key
    tile is computed, the stage cannot know which ones the mask hides, unless causal=True is given as well: key tiles
    past the diagonal are then skipped and the mask only acts below it); the default for a mask tensor stays the
    reference's operator chain (matmul, scale + mask + softmax, matmul: examples/llama/model.py:403-444).
    qkv_side_by_side (fused-attention prefill only; None = decide here): projections run next to each other on a share
    of the processors each instead of one after the other on all of them: Wq, Wk, Wv on a third each when there are as
    many K/V heads as query heads, else Wk and Wv on a half each after Wq. That pays when a projection has too few
    columns per rank to fill half the grid (a quarter for the K/V pair) with 128 x 256 tiles (the 7B shape from
    tensor-parallel degree 4 on, the K/V projections of the 70B shape from degree 4 on): a narrow tile costs as much per k-block as a wide one, so 49 CTAs
    with 176-wide tiles finish a projection in the time 148 CTAs with 64-wide tiles need (measured on one rank's
    share of the 7B shape at degree 8: 98 -> 42 microseconds for the three). num_sm: the processors the plan will be
    made for (the Planner's num_sm), which the shares are cut from.
    Returns the layer output [batch*seq, dim]."""
    p = world_size
    hl, kvl, hd = cfg.n_heads // p, max(1, cfg.n_kv_heads // p), cfg.head_dim
    bt = batch * seq
    # Decode: the small operators around each weight matrix are planned into the matmul's task (Sync=false); with one
    # or two rows of activations the engine folds them into the weight-streaming stage (norm and gate*up while the
    # activations are staged, the residual add on the way out) and otherwise runs them one after the other.
    decode = seq == 1 and k_cache is not None
    fused_prefill = ((causal and mask is None) or (fused_attention and mask is not None)) and k_cache is None and seq > 1
    if qkv_side_by_side is None:
        # 128 x 256 tiles of one K/V projection against the share of the grid it would get (measured: the 70B shape at
        # degree 2, 64 tiles per projection on a half each, gains nothing; at degree 8, 32 tiles, 2.6 %)
        qkv_side_by_side = -(-bt // 128) * -(-(kvl * hd) // 256) <= num_sm // (2 if kvl == hl else 4)
    side = fused_prefill and qkv_side_by_side
    third, half = num_sm // 3, num_sm // 2
    if kvl == hl:
        rq, rk, rv = [0, third], [third, 2 * third], [2 * third, 3 * third]
    else:
        rq, rk, rv = None, [0, half], [half, 2 * half]
    if side:
        h = ops.rmsnorm(x, w["attn_norm"], eps=cfg.norm_eps)   # on all processors; the projections share them out
    with PlannerContext(sync=False, processor_range=rq if side else None):  # prefill: RoPE in the projection's epilogue
        if not side:
            h = ops.rmsnorm(x, w["attn_norm"], eps=cfg.norm_eps)
        q = ops.matmul(h, w["wq"], transpose_other=True)   # [bt, hl*hd]
        q = ops.reshape(q, [batch, seq, hl, hd])
        if rope is not None:
            q = ops.rope(q, rope)
    scale = 1.0 / math.sqrt(hd)
    if fused_prefill:
        if hd != 128 or hl % kvl:
            raise ValueError("the fused attention stage needs head_dim 128 and a whole number of query heads per K/V head; "
                             "pass a mask tensor (and fused_attention=False) otherwise")
        with PlannerContext(sync=False, processor_range=rk if side else None):
            k = ops.reshape(ops.matmul(h, w["wk"], transpose_other=True), [batch, seq, kvl, hd])
            if rope is not None:
                k = ops.rope(k, rope)
        with PlannerContext(sync=False, processor_range=rv if side else None):
            v = ops.reshape(ops.matmul(h, w["wv"], transpose_other=True), [batch, seq, kvl, hd])
        o = ops.prefill_attention(q, k, v, scale, causal=causal, token_major=True, mask=mask)   # [b, seq, hl, hd]
        return _after_attention(ops.reshape(o, [bt, hl * hd]), x, w, cfg, rank, p)
    # [b, hl, seq, hd]; with one token per sequence the two layouts are the same memory
    q = ops.reshape(q, [batch, hl, 1, hd]) if seq == 1 else ops.transpose(q, [0, 2, 1, 3])
    if k_cache is None:
        with PlannerContext(sync=False):
            k = ops.reshape(ops.matmul(h, w["wk"], transpose_other=True), [batch, seq, kvl, hd])
            if rope is not None:
                k = ops.rope(k, rope)
        v = ops.matmul(h, w["wv"], transpose_other=True)
        k = ops.transpose(k, [0, 2, 1, 3])             # [b, kvl, seq, hd]
        v = ops.transpose(ops.reshape(v, [batch, seq, kvl, hd]), [0, 2, 1, 3])
    else:
        k, v = k_cache, v_cache
    if seq == 1 and k_cache is not None and hd == 128 and hl % kvl == 0 and hl // kvl in (1, 2, 4, 8):
        o = ops.decode_attention(q, k, v, scale)            # one pass over the cache: scores, softmax, output
    elif kvl == hl or kvl == 1:
        scores = ops.matmul(q, k, transpose_other=True)     # [b, hl, seq, t_kv]; C broadcasts when kvl == 1
        probs = ops.softmax(scores, scale=scale, mask=mask)  # scale, causal mask and softmax in one pass over the scores
        o = ops.matmul(probs, v)                            # [b, hl, seq, hd]
    else:
        raise ValueError("grouped-query attention needs 1 or n_heads KV heads per rank")
    o = ops.reshape(o if seq == 1 else ops.transpose(o, [0, 2, 1, 3]), [bt, hl * hd])
    if decode:
        with PlannerContext(sync=False):                    # matmul [-> all_reduce] -> residual add: one task
            attn = ops.matmul(o, w["wo"], transpose_other=True)
            if p > 1:
                attn = ops.all_reduce(attn, rank, p, output=attn)
            x1 = ops.add(attn, x)
        with PlannerContext(sync=False):                    # the norm is recomputed per consumer: it costs one row
            gate = ops.silu(ops.matmul(ops.rmsnorm(x1, w["ffn_norm"], eps=cfg.norm_eps), w["w1"], transpose_other=True))
        with PlannerContext(sync=False):
            up = ops.matmul(ops.rmsnorm(x1, w["ffn_norm"], eps=cfg.norm_eps), w["w3"], transpose_other=True)
        with PlannerContext(sync=False):
            down = ops.matmul(ops.mul(gate, up), w["w2"], transpose_other=True)
            if p > 1:
                down = ops.all_reduce(down, rank, p, output=down)
            return ops.add(down, x1)
    return _after_attention(o, x, w, cfg, rank, p)


def _after_attention(o, x, w, cfg, rank, p):
    """Output projection, residual, and the feed-forward block of a prefill layer; `o` is [batch*seq, heads_local*head_dim]."""
    if p == 1:
        with PlannerContext(sync=False):                    # one rank: the residual is added in the Wo epilogue ...
            x1 = ops.add(ops.matmul(o, w["wo"], transpose_other=True), x)
        h2 = ops.rmsnorm(x1, w["ffn_norm"], eps=cfg.norm_eps)  # ... and the norm streams plain rows
    else:
        with PlannerContext(sync=False):                    # one task: the all_reduce starts in the matmul epilogue
            attn = ops.matmul(o, w["wo"], transpose_other=True)  # partial [bt, dim]
            attn = ops.all_reduce(attn, rank, p, output=attn)
        h2, x1 = ops.rmsnorm(attn, w["ffn_norm"], eps=cfg.norm_eps, residual=x)
    with PlannerContext(sync=False):                        # SiLU in the W1 epilogue
        gate = ops.silu(ops.matmul(h2, w["w1"], transpose_other=True))
    with PlannerContext(sync=False):                        # gate * up in the W3 epilogue: `up` is never stored
        g = ops.mul(gate, ops.matmul(h2, w["w3"], transpose_other=True))
    with PlannerContext(sync=False):
        down = ops.matmul(g, w["w2"], transpose_other=True)  # partial [bt, dim]
        if p > 1:
            down = ops.all_reduce(down, rank, p, output=down)
        return ops.add(x1, down)                            # one rank: the residual is added in the W2 epilogue
