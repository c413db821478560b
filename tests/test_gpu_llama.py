"""GPU parity of Llama-shaped decoder layers (prefill with causal mask and RoPE,
decode against a K/V cache) against the per-op oracle composition, one GPU."""
import numpy as np
import pytest

import ark_b200 as ark
from ark_b200.llama import LlamaConfig, decoder_layer, layer_weights
from oracle import oracle as O
from tests.ark_util import NAME, execute
from tests.llama_ref import causal_mask, layer, rope_table

pytestmark = pytest.mark.gpu


def make_weights(cfg, dt, world, rng):
    hl, kvl, hd, f = cfg.n_heads // world, max(1, cfg.n_kv_heads // world), cfg.head_dim, cfg.ffn_dim // world
    shapes = {"attn_norm": (cfg.dim,), "wq": (hl * hd, cfg.dim), "wk": (kvl * hd, cfg.dim), "wv": (kvl * hd, cfg.dim),
              "wo": (cfg.dim, hl * hd), "ffn_norm": (cfg.dim,), "w1": (f, cfg.dim), "w3": (f, cfg.dim), "w2": (cfg.dim, f)}
    out = {}
    for k, sh in shapes.items():
        if "norm" in k:
            out[k] = O.to_storage(rng.normal(1.0, 0.05, sh).astype(np.float32), dt)
        else:
            out[k] = O.to_storage(rng.normal(0.0, 0.02, sh).astype(np.float32), dt)
    return out


def check(got, want, dt, spacings=1.5, tail_limit=2e-3):
    """The stated tolerance (mean abs error <= 2e-3 or max relative error <= 1e-2), and for bf16 layers, whose
    outputs of magnitude ~1-2 are spaced 2^-7 .. 2^-6 apart, its equivalent in units of that spacing: a layer
    rounds a dozen intermediates to bf16, and wherever the engine's fp32 sums (tensor-core accumulation order)
    and the oracle's (k order) straddle a rounding boundary the intermediate moves by a whole spacing, i.e. by
    0.4-0.8 %, which the rest of the layer carries on. The mean error may therefore reach `spacings` spacings at
    the mean magnitude of the output (1.5 at small widths; 2.5 at d_model 8192, where every sum has 8192 terms:
    the same layer in fp16, eight times finer, passes the stated tolerance, see the fp16 case of the test); errors
    of more than 6 spacings must stay rare (`tail_limit`: 2 in 1000; 2 in 100 for the unfused bf16 attention chain
    at d_model 8192, which rounds its [T, T] scores of magnitude ~4-8 to bf16 before the softmax: a score that lands
    on the other side of a rounding boundary moves a probability by 3-6 %, and 1.2 % of the outputs were measured
    beyond 6 spacings; the fused attention stage, which keeps the scores in fp32, stays within 2 in 1000)."""
    g, w = O.to_f32(got, dt), O.to_f32(want, dt)
    err = np.abs(g - w)
    rel = err / np.maximum(np.abs(w), 1e-2)
    # the stated bound is for results of magnitude ~1: the residual stream of a layer has a mean magnitude of ~2,
    # the bound is taken relative to it
    ok = float(err.mean()) <= 2e-3 * max(1.0, float(np.abs(w).mean())) or float(rel.max()) <= 1e-2
    if not ok and dt == "bf16":
        step = 2.0 ** -7 * max(float(np.abs(w).mean()), 2.0 ** -7)
        tail = float((err > 6 * 2.0 ** -7 * np.maximum(np.abs(w), 1.0)).mean())
        ok = float(err.mean()) <= spacings * step and tail <= tail_limit
        assert ok, (float(err.mean()), spacings * step, tail, float(np.abs(w).mean()))
    assert ok, (float(err.mean()), float(rel.max()), float(np.abs(w).mean()))
    # never grossly wrong anywhere: a few spacings of the storage type at the element's own magnitude
    spacing = (2.0 ** -10 if dt == "fp16" else 2.0 ** -7) * np.maximum(np.abs(w), 1.0)
    worst = int(np.argmax(err / spacing))
    assert float((err / spacing).max()) <= (48 if dt == "fp16" else 32), (float(err.flat[worst]), float(w.flat[worst]), float(g.flat[worst]))


@pytest.mark.parametrize("dt,heads,kv,reuse", [("fp16", 4, 4, False), ("bf16", 8, 1, False), ("fp16", 4, 4, True)])
def test_prefill_layer(dt, heads, kv, reuse):
    """reuse: the plan lets intermediates with disjoint lifetimes share arena space; two layers, so that the
    second one's activations land on memory the first one used."""
    cfg = LlamaConfig(dim=512, n_heads=heads, n_kv_heads=kv, ffn_dim=1376)
    batch, seq = 2, 128
    rng = np.random.default_rng(51)
    w = make_weights(cfg, dt, 1, rng)
    x = O.to_storage(rng.normal(0, 1, (batch * seq, cfg.dim)).astype(np.float32), dt)
    rope = O.to_storage(rope_table(seq, cfg.head_dim), dt)
    mask = O.to_storage(causal_mask(seq, dt), dt)
    ark.init()
    tw = layer_weights(cfg, NAME[dt], 1)
    tx = ark.tensor([batch * seq, cfg.dim], NAME[dt])
    tr, tm = ark.tensor([1, seq, 1, cfg.head_dim], NAME[dt]), ark.tensor([1, 1, seq, seq], NAME[dt])
    ty = decoder_layer(tx, tw, cfg, batch, seq, 0, 1, rope=tr, mask=tm)
    feeds = {tx: x, tr: rope, tm: mask}
    feeds.update({tw[k]: w[k] for k in w})
    want = layer(x, [w], cfg, batch, seq, dt, rope=rope, mask=mask)
    if reuse:
        w2 = make_weights(cfg, dt, 1, rng)
        tw2 = layer_weights(cfg, NAME[dt], 1)
        ty = decoder_layer(ty, tw2, cfg, batch, seq, 0, 1, rope=tr, mask=tm)
        feeds.update({tw2[k]: w2[k] for k in w2})
        want = layer(want, [w2], cfg, batch, seq, dt, rope=rope, mask=mask)
        plan = ark.Planner(0, reuse_memory=True).plan()
        text = ark.plan_dump(str(plan))
        assert "intermediates share space by lifetime" in text
        _, arena_reuse, _ = ark.plan_check(str(plan))
        _, arena_plain, _ = ark.plan_check(str(ark.Planner(0).plan()))
        assert arena_reuse < 0.7 * arena_plain, (arena_reuse, arena_plain)
        (got,) = execute([ty], feeds, loop_mode=True, iters=2, plan=plan)
    else:
        (got,) = execute([ty], feeds, loop_mode=True)
    check(got, want, dt)


@pytest.mark.parametrize("dt,dim,heads,kv,batch,seq,side", [("fp16", 512, 4, 4, 2, 128, False), ("bf16", 1024, 8, 2, 2, 200, False),
                                                            ("fp16", 512, 4, 4, 2, 640, True), ("bf16", 1024, 8, 2, 2, 200, True)])
def test_prefill_layer_with_fused_attention(dt, dim, heads, kv, batch, seq, side):
    """causal=True: q, k, v go from the projections (and RoPE) straight into the fused attention stage, no mask
    tensor, no transposes; grouped-query heads and a sequence that is not a multiple of the tile. side: the three
    projections run next to each other on a third of the processors each (Wk and Wv on a half each when there are fewer
    K/V heads than query heads), with no barrier between them."""
    cfg = LlamaConfig(dim=dim, n_heads=heads, n_kv_heads=kv, ffn_dim=1376)
    rng = np.random.default_rng(54)
    w = make_weights(cfg, dt, 1, rng)
    x = O.to_storage(rng.normal(0, 1, (batch * seq, cfg.dim)).astype(np.float32), dt)
    rope = O.to_storage(rope_table(seq, cfg.head_dim), dt)
    ark.init()
    tw = layer_weights(cfg, NAME[dt], 1)
    tx, tr = ark.tensor([batch * seq, cfg.dim], NAME[dt]), ark.tensor([1, seq, 1, cfg.head_dim], NAME[dt])
    ty = decoder_layer(tx, tw, cfg, batch, seq, 0, 1, rope=tr, causal=True, qkv_side_by_side=side)
    text = ark.plan_dump(str(ark.Planner(0).plan()))
    assert "PrefillAttention" in text and "Transpose" not in text and "Softmax" not in text
    lines = text.splitlines()
    first = next(i for i, l in enumerate(lines) if " Matmul " in l)
    if side:
        want_ranges = ["[0,49)", "[49,98)", "[98,147)"] if kv == heads else ["[0,148)", "[0,74)", "[74,148)"]
        assert want_ranges == [l.split()[1] for l in lines[first:first + 3]], lines[first:first + 3]
        assert all(" Matmul " in l for l in lines[first:first + 3])
    feeds = {tx: x, tr: rope}
    feeds.update({tw[k]: w[k] for k in w})
    (got,) = execute([ty], feeds, loop_mode=True)
    want = layer(x, [w], cfg, batch, seq, dt, rope=rope, causal=True)
    check(got, want, dt)


@pytest.mark.parametrize("dt,heads,kv,causal", [("fp16", 4, 4, False), ("bf16", 8, 2, True)])
def test_prefill_layer_with_mask_tensor_in_the_fused_stage(dt, heads, kv, causal):
    """The reference's call (a mask tensor, examples/llama/model.py:419-420) with the attention block as one stage: the
    mask is added on chip; with causal=True besides, key tiles past the diagonal are skipped. Reference: the oracle's
    per-operator composition with the same mask tensor."""
    cfg = LlamaConfig(dim=128 * heads, n_heads=heads, n_kv_heads=kv, ffn_dim=1376)
    batch, seq = 2, 200
    rng = np.random.default_rng(57)
    w = make_weights(cfg, dt, 1, rng)
    x = O.to_storage(rng.normal(0, 1, (batch * seq, cfg.dim)).astype(np.float32), dt)
    rope = O.to_storage(rope_table(seq, cfg.head_dim), dt)
    mask = O.to_storage(causal_mask(seq, dt), dt)
    ark.init()
    tw = layer_weights(cfg, NAME[dt], 1)
    tx = ark.tensor([batch * seq, cfg.dim], NAME[dt])
    tr, tm = ark.tensor([1, seq, 1, cfg.head_dim], NAME[dt]), ark.tensor([1, 1, seq, seq], NAME[dt])
    ty = decoder_layer(tx, tw, cfg, batch, seq, 0, 1, rope=tr, mask=tm, causal=causal, fused_attention=True)
    text = ark.plan_dump(str(ark.Planner(0).plan()))
    assert "+mask" in text and "Softmax" not in text and "Transpose" not in text and (" causal" in text) == causal
    feeds = {tx: x, tr: rope, tm: mask}
    feeds.update({tw[k]: w[k] for k in w})
    (got,) = execute([ty], feeds, loop_mode=True)
    check(got, layer(x, [w], cfg, batch, seq, dt, rope=rope, causal=True), dt)


@pytest.mark.parametrize("dt,heads,kv,batch", [("fp16", 4, 4, 1), ("bf16", 8, 1, 16)])
def test_decode_layer_with_kv_cache(dt, heads, kv, batch):
    cfg = LlamaConfig(dim=512, n_heads=heads, n_kv_heads=kv, ffn_dim=1376)
    t_kv = 256
    rng = np.random.default_rng(52)
    w = make_weights(cfg, dt, 1, rng)
    x = O.to_storage(rng.normal(0, 1, (batch, cfg.dim)).astype(np.float32), dt)
    rope = O.to_storage(rope_table(1, cfg.head_dim, start=t_kv), dt)
    kc = O.to_storage(rng.normal(0, 1, (batch, kv, t_kv, cfg.head_dim)).astype(np.float32), dt)
    vc = O.to_storage(rng.normal(0, 1, (batch, kv, t_kv, cfg.head_dim)).astype(np.float32), dt)
    ark.init()
    tw = layer_weights(cfg, NAME[dt], 1)
    tx = ark.tensor([batch, cfg.dim], NAME[dt])
    tr = ark.tensor([1, 1, 1, cfg.head_dim], NAME[dt])
    tk, tv = ark.tensor(list(kc.shape), NAME[dt]), ark.tensor(list(vc.shape), NAME[dt])
    ty = decoder_layer(tx, tw, cfg, batch, 1, 0, 1, rope=tr, k_cache=tk, v_cache=tv)
    feeds = {tx: x, tr: rope, tk: kc, tv: vc}
    feeds.update({tw[k]: w[k] for k in w if k not in ("wk", "wv")})  # K/V come from the cache
    (got,) = execute([ty], feeds, loop_mode=True)
    want = layer(x, [w], cfg, batch, 1, dt, rope=rope, k_caches=[kc], v_caches=[vc])
    check(got, want, dt)


@pytest.mark.parametrize("dt,b,hq,hkv,t", [("fp16", 1, 4, 4, 2048), ("bf16", 16, 8, 1, 1000), ("fp16", 3, 8, 2, 333),
                                           ("bf16", 2, 4, 2, 4096), ("fp16", 1, 32, 32, 40)])
def test_decode_attention_against_float64(dt, b, hq, hkv, t):
    """One query row per head against a K/V cache, grouped-query heads, cache lengths that do not divide into chunks."""
    rng = np.random.default_rng(53)
    q = O.to_storage(rng.normal(0, 1, (b, hq, 1, 128)).astype(np.float32), dt)
    k = O.to_storage(rng.normal(0, 1, (b, hkv, t, 128)).astype(np.float32), dt)
    v = O.to_storage(rng.normal(0, 1, (b, hkv, t, 128)).astype(np.float32), dt)
    scale = 1.0 / np.sqrt(128.0)
    ark.init()
    tq, tk, tv = ark.tensor(list(q.shape), NAME[dt]), ark.tensor(list(k.shape), NAME[dt]), ark.tensor(list(v.shape), NAME[dt])
    out = ark.decode_attention(tq, tk, tv, scale)
    (got,) = execute([out], {tq: q, tk: k, tv: v}, loop_mode=True)
    g = hq // hkv
    qf, kf, vf = (O.to_f32(x, dt).astype(np.float64) for x in (q, k, v))
    kf, vf = np.repeat(kf, g, axis=1), np.repeat(vf, g, axis=1)
    s = np.einsum("bhqd,bhtd->bhqt", qf, kf) * scale
    p = np.exp(s - s.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    want = np.einsum("bhqt,bhtd->bhqd", p, vf)
    err = np.abs(O.to_f32(got, dt).astype(np.float64) - want)
    tol = 2e-3 if dt == "fp16" else 1.6e-2   # one rounding of outputs of magnitude <= ~1
    assert float(err.max()) <= tol, float(err.max())


@pytest.mark.parametrize("dt,b,hq,hkv,tq,tkv,causal,token_major", [
    ("fp16", 1, 4, 4, 256, 256, True, False),     # two tiles, every head its own K/V
    ("bf16", 2, 8, 2, 384, 384, True, True),      # grouped-query heads, [B, T, H, 128] storage
    ("fp16", 1, 3, 1, 333, 333, True, False),     # ragged last tile
    ("bf16", 1, 2, 2, 200, 456, False, False),    # no mask, more keys than rows, both ragged
    ("fp16", 1, 2, 1, 128, 640, True, True),      # a block of new rows against a longer history (row i sees keys up to i + 512)
    ("fp16", 1, 32, 32, 2048, 2048, True, True),  # more units than CTAs: several units per CTA, barriers wrap
    ("fp16", 1, 1, 1, 40, 40, True, False),       # a single partial tile
])
def test_prefill_attention_against_float64(dt, b, hq, hkv, tq, tkv, causal, token_major):
    """S = q k^T and O = P v on the tensor cores with the scores kept on chip, against softmax attention in float64
    on the same (rounded) inputs. Tolerance: P is rounded to the storage type before P v (as the unfused chain rounds
    its probabilities) and the output once more: outputs of magnitude <= ~1, a few spacings of the type."""
    rng = np.random.default_rng(71)
    shape = lambda h, t: (b, t, h, 128) if token_major else (b, h, t, 128)
    q = O.to_storage(rng.normal(0, 1, shape(hq, tq)).astype(np.float32), dt)
    k = O.to_storage(rng.normal(0, 1, shape(hkv, tkv)).astype(np.float32), dt)
    v = O.to_storage(rng.normal(0, 1, shape(hkv, tkv)).astype(np.float32), dt)
    scale = 1.0 / np.sqrt(128.0)
    ark.init()
    tq_, tk_, tv_ = ark.tensor(list(q.shape), NAME[dt]), ark.tensor(list(k.shape), NAME[dt]), ark.tensor(list(v.shape), NAME[dt])
    out = ark.prefill_attention(tq_, tk_, tv_, scale, causal=causal, token_major=token_major)
    (got,) = execute([out], {tq_: q, tk_: k, tv_: v}, loop_mode=True)
    g = hq // hkv
    qf, kf, vf = (O.to_f32(x, dt).astype(np.float64) for x in (q, k, v))
    if token_major:
        qf, kf, vf = (x.transpose(0, 2, 1, 3) for x in (qf, kf, vf))
    kf, vf = np.repeat(kf, g, axis=1), np.repeat(vf, g, axis=1)
    s = np.einsum("bhqd,bhtd->bhqt", qf, kf) * scale
    if causal:
        visible = np.arange(tkv)[None, :] <= (np.arange(tq)[:, None] + tkv - tq)
        s = np.where(visible[None, None], s, -np.inf)
    p = np.exp(s - s.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    want = np.einsum("bhqt,bhtd->bhqd", p, vf)
    gotf = O.to_f32(got, dt).astype(np.float64)
    if token_major:
        gotf = gotf.transpose(0, 2, 1, 3)
    err = np.abs(gotf - want)
    tol = 4e-3 if dt == "fp16" else 3e-2
    assert float(err.max()) <= tol, (float(err.max()), np.unravel_index(err.argmax(), err.shape))
    assert float(err.mean()) <= tol / 20, float(err.mean())


@pytest.mark.parametrize("dt,b,hq,hkv,tq,tkv,mshape,token_major,causal", [
    ("fp16", 1, 4, 4, 256, 256, (1, 1), False, False),  # the llama example's mask: one [T, T] tensor for every head
    ("bf16", 2, 4, 2, 200, 328, (2, 4), True, False),   # one mask per sequence and head, ragged tiles, [B, T, H, 128] storage
    ("fp16", 2, 2, 1, 136, 136, (2, 1), False, False),  # per sequence (padding masks), broadcast over the heads
    ("fp16", 1, 2, 2, 384, 384, (1, 1), True, True),    # the caller also says causal: key tiles past the diagonal are skipped
])
def test_prefill_attention_with_additive_mask(dt, b, hq, hkv, tq, tkv, mshape, token_major, causal):
    """The general form of the fused stage: an additive mask tensor (here the causal -inf triangle plus finite biases
    plus, per sequence, a block of padded keys) joins scale * q k^T before the softmax; every key tile is computed.
    Reference: softmax attention in float64 on the same rounded inputs and the same rounded mask."""
    rng = np.random.default_rng(73)
    shape = lambda h, t: (b, t, h, 128) if token_major else (b, h, t, 128)
    q = O.to_storage(rng.normal(0, 1, shape(hq, tq)).astype(np.float32), dt)
    k = O.to_storage(rng.normal(0, 1, shape(hkv, tkv)).astype(np.float32), dt)
    v = O.to_storage(rng.normal(0, 1, shape(hkv, tkv)).astype(np.float32), dt)
    mb, mh = mshape
    m = rng.normal(0, 1, (mb, mh, tq, tkv)).astype(np.float32)
    visible = np.arange(tkv)[None, :] <= (np.arange(tq)[:, None] + tkv - tq)
    m = np.where(visible[None, None], m, -np.inf).astype(np.float32)
    for i in range(mb):
        m[i, :, :, 3 + 5 * i: 40 + 9 * i] = -np.inf       # a block of keys nobody sees (key 0 stays visible to every row)
    m = O.to_storage(m, dt)
    scale = 1.0 / np.sqrt(128.0)
    ark.init()
    tq_, tk_, tv_ = ark.tensor(list(q.shape), NAME[dt]), ark.tensor(list(k.shape), NAME[dt]), ark.tensor(list(v.shape), NAME[dt])
    tm_ = ark.tensor(list(m.shape), NAME[dt])
    out = ark.prefill_attention(tq_, tk_, tv_, scale, causal=causal, token_major=token_major, mask=tm_)
    plan = ark.Planner(0).plan()
    assert "+mask" in ark.plan_dump(str(plan))
    (got,) = execute([out], {tq_: q, tk_: k, tv_: v, tm_: m}, loop_mode=True, plan=plan)
    g = hq // hkv
    qf, kf, vf = (O.to_f32(x, dt).astype(np.float64) for x in (q, k, v))
    if token_major:
        qf, kf, vf = (x.transpose(0, 2, 1, 3) for x in (qf, kf, vf))
    kf, vf = np.repeat(kf, g, axis=1), np.repeat(vf, g, axis=1)
    s = np.einsum("bhqd,bhtd->bhqt", qf, kf) * scale + O.to_f32(m, dt).astype(np.float64)
    p = np.exp(s - s.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    want = np.einsum("bhqt,bhtd->bhqd", p, vf)
    gotf = O.to_f32(got, dt).astype(np.float64)
    if token_major:
        gotf = gotf.transpose(0, 2, 1, 3)
    err = np.abs(gotf - want)
    tol = 4e-3 if dt == "fp16" else 3e-2
    assert float(err.max()) <= tol, (float(err.max()), np.unravel_index(err.argmax(), err.shape))
    assert float(err.mean()) <= tol / 20, float(err.mean())


# Per-rank shapes of the two Llama-shaped benchmark configurations at tensor-parallel degree 8 (one rank's share of
# the heads and of the feed-forward width, full d_model, full sequence / cache lengths), against the oracle's per-op
# composition of the whole layer. (The sum over ranks is covered by the multi-GPU tests.)
REAL = {
    "7b": dict(cfg=dict(dim=4096, n_heads=4, n_kv_heads=4, ffn_dim=1376), dt="fp16", prefill=(1, 2048), decode=(1, 2048)),
    "70b": dict(cfg=dict(dim=8192, n_heads=8, n_kv_heads=1, ffn_dim=3584), dt="bf16", prefill=(4, 1024), decode=(16, 4096)),
}


@pytest.mark.parametrize("model", ["7b", "70b"])
def test_decode_layer_at_benchmark_shapes(model):
    spec = REAL[model]
    dt, (batch, t_kv) = spec["dt"], spec["decode"]
    cfg = LlamaConfig(**spec["cfg"])
    rng = np.random.default_rng(61)
    w = make_weights(cfg, dt, 1, rng)
    x = O.to_storage(rng.normal(0, 1, (batch, cfg.dim)).astype(np.float32), dt)
    rope = O.to_storage(rope_table(1, cfg.head_dim, start=t_kv), dt)
    kc = O.to_storage(rng.normal(0, 1, (batch, cfg.n_kv_heads, t_kv, cfg.head_dim)).astype(np.float32), dt)
    vc = O.to_storage(rng.normal(0, 1, (batch, cfg.n_kv_heads, t_kv, cfg.head_dim)).astype(np.float32), dt)
    ark.init()
    tw = layer_weights(cfg, NAME[dt], 1)
    tx, tr = ark.tensor([batch, cfg.dim], NAME[dt]), ark.tensor([1, 1, 1, cfg.head_dim], NAME[dt])
    tk, tv = ark.tensor(list(kc.shape), NAME[dt]), ark.tensor(list(vc.shape), NAME[dt])
    ty = decoder_layer(tx, tw, cfg, batch, 1, 0, 1, rope=tr, k_cache=tk, v_cache=tv)
    feeds = {tx: x, tr: rope, tk: kc, tv: vc}
    feeds.update({tw[k]: w[k] for k in w if k not in ("wk", "wv")})
    (got,) = execute([ty], feeds, loop_mode=True, iters=2)
    want = layer(x, [w], cfg, batch, 1, dt, rope=rope, k_caches=[kc], v_caches=[vc])
    check(got, want, dt, spacings=2.5 if cfg.dim >= 8192 else 1.5)


@pytest.mark.parametrize("model,dt_override,fused", [("7b", None, False), ("70b", None, False), ("70b", "fp16", False),
                                                     ("7b", None, True), ("70b", None, True)])
def test_prefill_layer_at_benchmark_shapes(model, dt_override, fused):
    spec = REAL[model]
    dt, (batch, seq) = dt_override or spec["dt"], spec["prefill"]
    cfg = LlamaConfig(**spec["cfg"])
    rng = np.random.default_rng(62)
    w = make_weights(cfg, dt, 1, rng)
    x = O.to_storage(rng.normal(0, 1, (batch * seq, cfg.dim)).astype(np.float32), dt)
    rope = O.to_storage(rope_table(seq, cfg.head_dim), dt)
    mask = O.to_storage(causal_mask(seq, dt), dt)
    ark.init()
    tw = layer_weights(cfg, NAME[dt], 1)
    tx = ark.tensor([batch * seq, cfg.dim], NAME[dt])
    tr, tm = ark.tensor([1, seq, 1, cfg.head_dim], NAME[dt]), ark.tensor([1, 1, seq, seq], NAME[dt])
    if fused:
        ty = decoder_layer(tx, tw, cfg, batch, seq, 0, 1, rope=tr, causal=True)
        feeds = {tx: x, tr: rope}
    else:
        ty = decoder_layer(tx, tw, cfg, batch, seq, 0, 1, rope=tr, mask=tm)
        feeds = {tx: x, tr: rope, tm: mask}
    feeds.update({tw[k]: w[k] for k in w})
    (got,) = execute([ty], feeds, loop_mode=True)
    # the oracle composes the whole layer of ONE sequence on the host cores (sequences are independent); the engine
    # ran all of them, the last one is compared
    b = batch - 1
    want = layer(np.ascontiguousarray(x[b * seq:(b + 1) * seq]), [w], cfg, 1, seq, dt, rope=rope,
                 mask=None if fused else mask, causal=fused)
    check(got[b * seq:(b + 1) * seq], want, dt, spacings=2.5 if cfg.dim >= 8192 else 1.5,
          tail_limit=2e-2 if (dt == "bf16" and cfg.dim >= 8192 and not fused) else 2e-3)


def test_decode_chain_folds_keep_the_bits(monkeypatch):
    """The folds of the decode chain (rotary embedding applied by the attention stage, attention chunks merged by the
    output projection, W1 and W3 as one stage) reproduce the roundings of the separate operators: the layer's output is
    bit-identical with and without them."""
    cfg = LlamaConfig(dim=1024, n_heads=8, n_kv_heads=2, ffn_dim=2752)
    t_kv, batch = 700, 2
    rng = np.random.default_rng(55)
    w = make_weights(cfg, "fp16", 1, rng)
    x = O.to_storage(rng.normal(0, 1, (batch, cfg.dim)).astype(np.float32), "fp16")
    rope = O.to_storage(rope_table(1, cfg.head_dim, start=t_kv), "fp16")
    kc = O.to_storage(rng.normal(0, 1, (batch, cfg.n_kv_heads, t_kv, cfg.head_dim)).astype(np.float32), "fp16")
    vc = O.to_storage(rng.normal(0, 1, (batch, cfg.n_kv_heads, t_kv, cfg.head_dim)).astype(np.float32), "fp16")
    outs, texts = [], []
    for folds in ("1", "0"):
        monkeypatch.setenv("ARKB_FOLD_DECODE", folds)
        monkeypatch.setenv("ARKB_PAIR_GEMV", folds)
        ark.init()
        tw = layer_weights(cfg, ark.fp16, 1)
        tx, tr = ark.tensor([batch, cfg.dim], ark.fp16), ark.tensor([1, 1, 1, cfg.head_dim], ark.fp16)
        tk, tv = ark.tensor(list(kc.shape), ark.fp16), ark.tensor(list(vc.shape), ark.fp16)
        ty = decoder_layer(tx, tw, cfg, batch, 1, 0, 1, rope=tr, k_cache=tk, v_cache=tv)
        texts.append(ark.plan_dump(str(ark.Planner(0).plan())))
        feeds = {tx: x, tr: rope, tk: kc, tv: vc}
        feeds.update({tw[k]: w[k] for k in w if k not in ("wk", "wv")})
        (got,) = execute([ty], feeds, loop_mode=True, iters=2)
        outs.append(got)
    assert "<-rope" in texts[0] and "<-attention merge" in texts[0] and "(second matrix" in texts[0]
    assert "<-rope" not in texts[1] and "merge of the chunks" in texts[1] and "(second matrix" not in texts[1]
    assert np.array_equal(outs[0].view(np.uint16), outs[1].view(np.uint16))
