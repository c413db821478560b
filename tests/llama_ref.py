"""CPU composition of one tensor-parallel Llama decoder layer from the oracle's
per-op functions, in the op order of ark_b200/llama.py (which follows
examples/llama/model.py of the reference). Storage type roundings happen where
the engine materialises a tensor; fused kernels keep fp32 inside (rmsnorm,
softmax, matmul + SiLU)."""
import math

import numpy as np

from oracle import oracle as O


def rope_table(seq, head_dim, theta=10000.0, start=0):
    """Interleaved (cos, sin) pairs per position (examples/llama/generator.py:20-27,
    model_test.py:379-384), shape [1, seq, 1, head_dim] in fp32."""
    freqs = 1.0 / (theta ** (np.arange(0, head_dim, 2)[: head_dim // 2].astype(np.float32) / head_dim))
    t = np.arange(start, start + seq, dtype=np.float32)
    ang = np.outer(t, freqs)
    tab = np.stack([np.cos(ang), np.sin(ang)], axis=-1).reshape(seq, head_dim)
    return tab.reshape(1, seq, 1, head_dim).astype(np.float32)


def causal_mask(seq, dt):
    m = np.triu(np.full((seq, seq), -np.inf, np.float32), k=1)
    m = np.where(np.isinf(m), np.float32(-60000.0 if dt == "fp16" else -1e30), m)
    return m.reshape(1, 1, seq, seq)


def layer(x, ws, cfg, batch, seq, dt, rope=None, mask=None, k_caches=None, v_caches=None, causal=False):
    """Full layer over all ranks: ws is a list (one dict of numpy weights per rank);
    returns the layer output (identical on all ranks)."""
    p = len(ws)
    hl, kvl, hd = cfg.n_heads // p, max(1, cfg.n_kv_heads // p), cfg.head_dim
    bt = batch * seq
    f32 = lambda a: O.to_f32(a, dt)
    st = lambda a: O.to_storage(a, dt)
    scale = 1.0 / math.sqrt(hd)
    attn_parts = []
    for r in range(p):
        w = ws[r]
        h = O.rmsnorm(x, w["attn_norm"], dt, cfg.norm_eps)
        def project(wn, heads):
            """x W^T [+ RoPE]. Prefill: the rotation is applied to the fp32 accumulator in the matmul's epilogue (one
            rounding); decode: the projection is stored and a separate operator rotates it."""
            if rope is not None and seq > 1:
                a32 = O.matmul(f32(h), f32(w[wn]), "fp32", trans_b=True).reshape(batch, seq, heads, hd)
                return st(O.rope(a32, np.ascontiguousarray(np.broadcast_to(f32(rope), a32.shape)), "fp32"))
            a = O.matmul(h, w[wn], dt, trans_b=True).reshape(batch, seq, heads, hd)
            if rope is not None:
                a = O.rope(a, np.ascontiguousarray(np.broadcast_to(rope, a.shape)), dt)
            return a
        q = project("wq", hl)
        q = np.ascontiguousarray(q.transpose(0, 2, 1, 3))
        if k_caches is None:
            k = project("wk", kvl)
            v = O.matmul(h, w["wv"], dt, trans_b=True).reshape(batch, seq, kvl, hd)
            k = np.ascontiguousarray(k.transpose(0, 2, 1, 3))
            v = np.ascontiguousarray(v.transpose(0, 2, 1, 3))
        else:
            k, v = k_caches[r], v_caches[r]
        if causal:
            # the fused attention stage: scores, scale and mask in fp32 (never stored), probabilities rounded once
            if k.shape[1] != q.shape[1]:
                k, v = np.repeat(k, q.shape[1] // k.shape[1], axis=1), np.repeat(v, q.shape[1] // v.shape[1], axis=1)
            s32 = O.scalar("mul", O.matmul(f32(q), f32(k), "fp32", trans_b=True), scale, "fp32")
            s32 = np.where(np.tril(np.ones((seq, seq), bool))[None, None], s32, np.float32(-np.inf))
            scores, probs = None, st(O.softmax(s32, "fp32"))
        else:
            scores = O.matmul(q, k, dt, trans_b=True)
        if causal:
            pass
        elif mask is not None:
            scores = O.scalar("mul", scores, scale, dt)
            scores = O.binary("add", scores, mask, dt)
            probs = O.softmax(scores, dt)
        else:
            # the engine's softmax multiplies by the scale in fp32 before the max/exp: the oracle's operators on the
            # fp32 values, one rounding at the end
            probs = st(O.softmax(O.scalar("mul", f32(scores), scale, "fp32"), "fp32"))
        o = O.matmul(probs, v, dt)
        o = np.ascontiguousarray(o.transpose(0, 2, 1, 3)).reshape(bt, hl * hd)
        attn_parts.append(O.matmul(o, w["wo"], dt, trans_b=True))
        if seq > 1 and p == 1:
            # prefill on one rank: the residual is added to the fp32 accumulator of the output projection
            o32 = O.matmul(f32(o), f32(w["wo"]), "fp32", trans_b=True)
    if seq > 1 and p == 1:
        x1 = st(O.binary("add", o32, f32(x), "fp32"))
    else:
        attn = O.all_reduce(attn_parts, dt) if p > 1 else attn_parts[0]
        x1 = O.binary("add", attn, x, dt)
    down_parts = []
    for r in range(p):
        w = ws[r]
        h2 = O.rmsnorm(x1, w["ffn_norm"], dt, cfg.norm_eps)
        # SiLU runs on the fp32 accumulator in the epilogue: the oracle's matmul, sigmoid and mul on fp32 values
        a32 = O.matmul(f32(h2), f32(w["w1"]), "fp32", trans_b=True)
        gate = st(O.binary("mul", a32, O.unary("sigmoid", a32, "fp32"), "fp32"))
        if seq > 1:
            # prefill: gate * up happens on the fp32 accumulator of the W3 matmul (its epilogue reads the gate)
            up32 = O.matmul(f32(h2), f32(w["w3"]), "fp32", trans_b=True)
            g = st(O.binary("mul", f32(gate), up32, "fp32"))
        else:
            up = O.matmul(h2, w["w3"], dt, trans_b=True)
            g = O.binary("mul", gate, up, dt)
        if seq > 1 and p == 1:
            # one rank: the residual is added to the fp32 accumulator of the W2 matmul
            d32 = O.matmul(f32(g), f32(w["w2"]), "fp32", trans_b=True)
            return st(O.binary("add", f32(x1), d32, "fp32"))
        down_parts.append(O.matmul(g, w["w2"], dt, trans_b=True))
    down = O.all_reduce(down_parts, dt) if p > 1 else down_parts[0]
    return O.binary("add", x1, down, dt)
