"""Per-kernel-class measurements of the loop-kernel engine on one GPU: achieved
HBM GB/s for elementwise / reduce / norm / softmax / gemv-shaped matmul stages
and TFLOP/s for matmul shapes, each as a fraction of the measured peak
(MEASURED_PEAKS.json). One JSON line per case. bench.py remains the headline
benchmark; this script produces the numbers quoted in profiles/.

  python bench_ops.py [--iters 20] [--only name-substring]
"""
import argparse
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


def time_plan(ark, torch, build, iters, warm=3):
    """Builds a model with `build()` (returns algorithmic bytes, flops), runs `iters`
    iterations in one launch and returns milliseconds per iteration."""
    ark.init()
    nbytes, flops = build()
    plan = ark.Planner(0).plan()
    ex = ark.Executor(0, 0, "bench_ops", str(plan), loop_mode=False)
    ex.compile()
    stream = torch.cuda.ExternalStream(ex.stream())
    ex.launch()
    ex.run(warm)
    ex.wait()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    ex.run(iters)
    e1.record(stream)
    ex.wait()
    ms = e0.elapsed_time(e1) / iters
    n_stages = ex.status()["n_stages"]
    ex.stop()
    ex.destroy()
    return ms, nbytes, flops, n_stages


def time_ffn_cfg1(ark, iters, flush_l2=True):
    """Config 1 (Y = ReLU(X W1) W2, X [128, 1024], W1 [1024, 4096], W2 [4096, 1024], fp16): its 16.5 MiB fit in L2,
    so every iteration ends with a read of 256 MiB that flushes L2, and the block is timed with the engine's own
    per-stage time stamps (first CTA entering the first matmul -> last CTA leaving the second), median over the
    iterations' last one of several launches. Returns (microseconds, bytes, flops, stage texts)."""
    ark.init()
    x, w1, w2 = ark.tensor([128, 1024], ark.fp16), ark.tensor([1024, 4096], ark.fp16), ark.tensor([4096, 1024], ark.fp16)
    with ark.PlannerContext(sync=False):
        h = ark.relu(ark.matmul(x, w1))
    y = ark.matmul(h, w2)
    # the flush READS 256 MiB (a row reduction): L2 ends up full of clean lines of another buffer. A flush that writes
    # leaves 126 MB of dirty lines behind, and the first stage of the next iteration then waits for their write-back
    # (measured: 30 us for the first matmul instead of 8)
    if flush_l2:
        flush = ark.tensor([16384, 8192], ark.fp16)
        ark.reduce_sum(ark.identity(flush, [y]), axis=-1)
    plan = ark.Planner(0).plan()
    ex = ark.Executor(0, 0, "cfg1", str(plan), loop_mode=False)
    ex.compile()
    rng = np.random.default_rng(0)
    ex.tensor_from_numpy(x, rng.standard_normal((128, 1024)).astype(np.float16))
    ex.tensor_from_numpy(w1, (rng.standard_normal((1024, 4096)) * 0.02).astype(np.float16))
    ex.tensor_from_numpy(w2, (rng.standard_normal((4096, 1024)) * 0.02).astype(np.float16))
    notes = ex.program_dump().splitlines()[1:]
    last_ffn = max(i for i, n in enumerate(notes) if "Matmul" in n or "split-K" in n)
    ex.enable_stage_times(True)
    ex.launch()
    spans = []
    for _ in range(max(3, iters)):
        ex.run(3)
        ex.wait()
        t = ex.stage_times()
        first = t[0, :, 0][t[0, :, 0] > 0].min()
        spans.append((t[last_ffn, :, 1].max() - first) / 1e3)
    # when the CTAs entered and left every stage of the block in the last iteration measured (microseconds after `first`)
    table = []
    for si in range(last_ffn + 1):
        m = t[si, :, 0] > 0
        if m.any():
            table.append([round(float((t[si, m, 0].min() - first) / 1e3), 1), round(float((t[si, m, 1].max() - first) / 1e3), 1)])
    ex.stop()
    ex.destroy()
    nbytes = (128 * 1024 + 2 * 1024 * 4096 + 128 * 1024) * 2
    return float(np.median(spans)), nbytes, 2.0 * 2 * 128 * 1024 * 4096, [f"{n}  {b}" for n, b in zip(notes[:last_ffn + 1], table)]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--only", default="")
    ap.add_argument("--mib", type=int, default=256,
                    help="size of the tensors of the HBM-bound cases in MiB (256: the per-iteration barrier is ~10 %% of the time; "
                         "1024 shows the streaming rate)")
    args = ap.parse_args()
    import torch
    import ark_b200 as ark
    pk, which = peaks()
    MB = 1 << 20
    SC = max(1, args.mib // 256)  # row-count multiplier of the HBM-bound cases
    cases = []

    def case(name, fn):
        if args.only in name:
            cases.append((name, fn))

    # ---- HBM-bound stages: tensors of 256 MiB so that nothing fits in L2 ----
    def ew_unary(op, dt, es):
        def b():
            n = args.mib * MB // es
            t = ark.tensor([n // 8192, 8192], dt)
            getattr(ark, op)(t)
            return 2 * n * es, 0
        return b

    def ew_binary(op, dt, es):
        def b():
            n = args.mib * MB // es
            a, c = ark.tensor([n // 8192, 8192], dt), ark.tensor([n // 8192, 8192], dt)
            getattr(ark, op)(a, c)
            return 3 * n * es, 0
        return b
    case("relu_fp16", ew_unary("relu", ark.fp16, 2))
    case("gelu_fp16", ew_unary("gelu", ark.fp16, 2))
    case("copy_fp32", ew_unary("copy", ark.fp32, 4))
    case("add_fp16", ew_binary("add", ark.fp16, 2))
    case("mul_bf16", ew_binary("mul", ark.bf16, 2))

    def add_bcast():
        a, c = ark.tensor([16384 * SC, 8192], ark.fp16), ark.tensor([1, 8192], ark.fp16)
        ark.add(a, c)
        return 2 * 16384 * SC * 8192 * 2, 0
    case("add_broadcast_row_fp16", add_bcast)

    def reduce_last(rows, cols, dt, es):
        def b():
            t = ark.tensor([rows, cols], dt)
            ark.reduce_sum(t, axis=-1)
            return rows * cols * es, 0
        return b
    case("reduce_sum_w_fp16_32768x4096", reduce_last(32768 * SC, 4096, ark.fp16, 2))
    case("reduce_sum_w_fp32_16384x4096", reduce_last(16384 * SC, 4096, ark.fp32, 4))

    def reduce_h():
        t = ark.tensor([64 * SC, 1024, 2048], ark.fp16)
        ark.reduce_sum(t, axis=1)
        return 64 * SC * 1024 * 2048 * 2, 0
    case("reduce_sum_h_fp16", reduce_h)

    def rows(opname, r, c, dt, es):
        def b():
            t = ark.tensor([r, c], dt)
            if opname == "rmsnorm":
                w = ark.tensor([c], dt)
                ark.rmsnorm(t, w)
            elif opname == "softmax":
                ark.softmax(t)
            else:
                ark.layernorm(t)
            return 2 * r * c * es, 0
        return b
    case("rmsnorm_fp16_32768x4096", rows("rmsnorm", 32768 * SC, 4096, ark.fp16, 2))
    case("rmsnorm_bf16_16384x8192", rows("rmsnorm", 16384 * SC, 8192, ark.bf16, 2))
    case("softmax_fp16_65536x2048", rows("softmax", 65536 * SC, 2048, ark.fp16, 2))
    case("layernorm_fp16_32768x4096", rows("layernorm", 32768 * SC, 4096, ark.fp16, 2))

    # ---- fixed cost of a stage: 16 dependent tiny operators (time / 16 = one stage + one grid barrier) ----
    def chain16():
        t = ark.tensor([148, 2048], ark.fp16)
        for _ in range(16):
            t = ark.relu(t)
        return 16 * 2 * 148 * 2048 * 2, 0
    case("chain16_relu_148x2048", chain16)

    # ---- weight-streaming matmuls (decode shapes): bytes = weights ----
    def gemv(m, n, k, dt, es, nk=True):
        def b():
            x = ark.tensor([m, k], dt)
            w = ark.tensor([n, k] if nk else [k, n], dt)
            ark.matmul(x, w, transpose_other=nk)
            return (n * k + m * k + m * n) * es, 2.0 * m * n * k
        return b
    case("gemv_m1_fp16_28672x8192", gemv(1, 28672, 8192, ark.fp16, 2))
    case("gemv_m16_bf16_28672x8192", gemv(16, 28672, 8192, ark.bf16, 2))
    case("gemv_m1_fp16_4096x4096", gemv(1, 4096, 4096, ark.fp16, 2))
    case("gemv_m1_fp16_65536x8192", gemv(1, 65536, 8192, ark.fp16, 2))
    case("gemv_m2_bf16_32768x8192", gemv(2, 32768, 8192, ark.bf16, 2))
    case("gemv_m1_fp16_kn_8192x28672", gemv(1, 28672, 8192, ark.fp16, 2, nk=False))

    # ---- tensor-core matmuls ----
    def mm(m, n, k, dt, es, nk=False):
        def b():
            x = ark.tensor([m, k], dt)
            w = ark.tensor([n, k] if nk else [k, n], dt)
            ark.matmul(x, w, transpose_other=nk)
            return (n * k + m * k + m * n) * es, 2.0 * m * n * k
        return b
    case("matmul_fp16_8192x8192x8192", mm(8192, 8192, 8192, ark.fp16, 2))
    case("matmul_bf16_nk_4096x8192x8192", mm(4096, 8192, 8192, ark.bf16, 2, nk=True))
    case("matmul_fp16_2048x4096x4096", mm(2048, 4096, 4096, ark.fp16, 2))
    case("matmul_fp16_nk_2048x4096x4096", mm(2048, 4096, 4096, ark.fp16, 2, nk=True))     # Llama-7B Q/K/V/O projection, 2048 tokens
    case("matmul_fp16_nk_2048x11008x4096", mm(2048, 11008, 4096, ark.fp16, 2, nk=True))   # W1 / W3
    case("matmul_fp16_nk_2048x4096x11008", mm(2048, 4096, 11008, ark.fp16, 2, nk=True))   # W2
    case("matmul_fp16_nk_2048x512x4096", mm(2048, 512, 4096, ark.fp16, 2, nk=True))       # Llama-7B Q/K/V projection of one rank at TP8
    case("matmul_fp16_nk_2048x4096x512", mm(2048, 4096, 512, ark.fp16, 2, nk=True))       # ... output projection
    case("matmul_fp16_nk_2048x1376x4096", mm(2048, 1376, 4096, ark.fp16, 2, nk=True))     # ... W1 / W3
    case("matmul_fp16_nk_2048x4096x1376", mm(2048, 4096, 1376, ark.fp16, 2, nk=True))     # ... W2
    case("matmul_fp16_kn_4096x4096x8192", mm(4096, 4096, 8192, ark.fp16, 2))              # one rank's W1 of the FFN block at TP8
    case("matmul_fp16_kn_4096x8192x4096", mm(4096, 8192, 4096, ark.fp16, 2))              # one rank's W2
    case("matmul_fp16_128x4096x1024", mm(128, 4096, 1024, ark.fp16, 2))

    # ---- fused prefill attention: FLOPs = the (causal) part of q k^T and p v that is needed ----
    def attn(b, hq, hkv, t, dt):
        def f():
            q = ark.tensor([b, t, hq, 128], dt)
            k, v = ark.tensor([b, t, hkv, 128], dt), ark.tensor([b, t, hkv, 128], dt)
            ark.prefill_attention(q, k, v, 1.0 / 128 ** 0.5, causal=True, token_major=True)
            return (2 * b * t * hq * 128 + 2 * b * t * hkv * 128) * 2, 4.0 * b * hq * (t * (t + 1) / 2) * 128
        return f
    case("prefill_attn_fp16_32h_1x2048", attn(1, 32, 32, 2048, ark.fp16))
    case("prefill_attn_bf16_gqa_64h_8kv_4x1024", attn(4, 64, 8, 1024, ark.bf16))
    case("prefill_attn_fp16_32h_1x8192", attn(1, 32, 32, 8192, ark.fp16))

    if args.only and args.only in "ffn_cfg1":
        # cold: L2 flushed between iterations (operands AND the kernel's own code come from HBM); warm: the 16.5 MiB of
        # operands stay in L2 between iterations, which is how a block of this size runs in a loop
        for flush_l2 in (True, False):
            us, nbytes, flops, notes = time_ffn_cfg1(ark, args.iters, flush_l2)
            gbs = nbytes / (us * 1e-6) / 1e9
            print(json.dumps({"case": "ffn_cfg1_128x1024x4096_relu_fp16", "us": us, "algorithmic_bytes": nbytes, "GB/s": gbs,
                              "hbm_frac": gbs / pk["hbm_gbs"], "TFLOP/s": flops / (us * 1e-6) / 1e12, "peak": which,
                              "l2": "flushed by a 256 MiB read (row reduction) at the end of every iteration" if flush_l2
                                    else "warm: the operands (16.5 MiB) stay in L2 between iterations",
                              "stages": notes}))
        return
    for name, fn in cases:
        try:
            ms, nbytes, flops, n_stages = time_plan(ark, torch, fn, args.iters)
        except Exception as e:  # keep going: one failing case must not hide the others
            print(json.dumps({"case": name, "error": f"{type(e).__name__}: {e}"[:300]}))
            continue
        gbs = nbytes / (ms * 1e-3) / 1e9
        line = {"case": name, "ms": ms, "stages": n_stages, "algorithmic_bytes": nbytes, "GB/s": gbs,
                "hbm_frac": gbs / pk["hbm_gbs"], "peak": which}
        if flops:
            tf = flops / (ms * 1e-3) / 1e12
            line["TFLOP/s"] = tf
            line["tensor_frac"] = tf / pk["bf16_tflops"]
        print(json.dumps(line))


if __name__ == "__main__":
    main()
