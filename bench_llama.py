"""Llama-shaped decoder layers through the loop-kernel engine: prefill and decode
throughput of a stack of tensor-parallel layers (random-init weights, synthetic
activations and K/V caches), one process per GPU:

  python bench_llama.py --model 7b --phase prefill            # one GPU, TP1
  python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
      --master-port P bench_llama.py --model 70b --phase decode

--model 7b : d_model 4096, 32 heads of 128, SwiGLU 11008, fp16, 4 layers;
             prefill = batch 1 x 2048 tokens, decode = batch 1 against 2048 cached tokens.
--model 70b: d_model 8192, 64 query / 8 KV heads of 128, SwiGLU 28672, bf16, 2 layers;
             prefill = batch 4 x 1024 tokens, decode = batch 16 against 4096 cached tokens.

Rank 0 prints one JSON line: tokens/s over all layers (device time of one launch
of K iterations, max over ranks), the per-rank roofline the phase is bound by
(tensor FLOP/s for prefill, HBM bytes of weights + K/V cache for decode), and
the number of stages of the lowered program.
"""
import argparse
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODELS = {
    "7b": dict(cfg=dict(dim=4096, n_heads=32, n_kv_heads=32, ffn_dim=11008), dtype="fp16", layers=4,
               prefill=(1, 2048), decode=(1, 2048)),
    "70b": dict(cfg=dict(dim=8192, n_heads=64, n_kv_heads=8, ffn_dim=28672), dtype="bf16", layers=2,
                prefill=(4, 1024), decode=(16, 4096)),
}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


def to_storage(a, dt):
    """fp32 array -> the engine's storage type: float16, or bfloat16 bits (round to nearest even) as uint16."""
    a = np.ascontiguousarray(a, np.float32)
    if dt == "fp16":
        return a.astype(np.float16)
    u = a.view(np.uint32).astype(np.uint64)
    inf_nan = (u & 0x7F800000) == 0x7F800000
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    r[inf_nan] = (u[inf_nan] >> 16).astype(np.uint16)
    return r


def to_f32(a, dt):
    if dt == "fp16":
        return a.astype(np.float32)
    return (a.astype(np.uint32) << 16).view(np.float32)


def run_case(model, phase, rank=0, world=1, local=0, ag=None, host_group=None, layers=0, iters=10, warmup=3,
             stage_times=False, attention="fused", qkv_side_by_side=None):
    """Builds the layer stack, runs it and returns the result line (a dict) on rank 0, None on the other ranks.
    attention: "fused" = the prefill attention block is one stage with the scores kept on chip; "chain" = the
    reference's matmul -> scale/mask/softmax -> matmul chain with a mask tensor. The caller owns the process group (`ag`: bootstrap callback, `host_group`: a gloo group for host rendezvous)."""
    import torch
    import ark_b200 as ark
    from ark_b200.llama import LlamaConfig, decoder_layer, layer_weights

    class A:
        pass
    args = A()
    args.model, args.phase, args.layers, args.iters, args.warmup, args.stage_times = model, phase, layers, iters, warmup, stage_times
    spec = MODELS[args.model]
    cfg = LlamaConfig(**spec["cfg"])
    dt, nlayers = spec["dtype"], args.layers or spec["layers"]
    adt = ark.fp16 if dt == "fp16" else ark.bf16
    decode = args.phase == "decode"
    batch, span = spec[args.phase]          # prefill: tokens per sequence; decode: cached tokens
    seq = 1 if decode else span
    hl, kvl, hd = cfg.n_heads // world, max(1, cfg.n_kv_heads // world), cfg.head_dim

    ark.init()
    ark.set_rank(rank)
    ark.set_world_size(world)
    x = ark.tensor([batch * seq, cfg.dim], adt)
    rope = ark.tensor([1, seq, 1, hd], adt)
    fused = attention in ("fused", "fused-mask") and not decode and hd == 128
    with_mask = not decode and (not fused or attention == "fused-mask")
    mask = ark.tensor([1, 1, seq, seq], adt) if with_mask else None
    layers, caches = [], []
    h = x
    for li in range(nlayers):
        w = layer_weights(cfg, adt, world, prefix=f"l{li}.")
        kc = vc = None
        if decode:
            kc, vc = ark.tensor([batch, kvl, span, hd], adt), ark.tensor([batch, kvl, span, hd], adt)
            caches.append((kc, vc))
        h = decoder_layer(h, w, cfg, batch, seq, rank, world, rope=rope, mask=mask, k_cache=kc, v_cache=vc, causal=fused and mask is None,
                          qkv_side_by_side=qkv_side_by_side, fused_attention=fused and mask is not None)
        layers.append(w)
    ex = ark.Executor(local, 0, "llama", str(ark.Planner(local).plan()), loop_mode=False, allgather=ag)
    ex.compile()
    rng = np.random.default_rng(100 + rank)
    made = {}

    def synth(shape, std, mean=0.0):
        key = (tuple(shape), std, mean)
        if key not in made:  # one block per distinct shape: the values do not matter for the timing, the buffers do
            made[key] = to_storage(rng.normal(mean, std, shape).astype(np.float32), dt)
        return made[key]
    for w in layers:
        for k, t in w.items():
            if decode and k in ("wk", "wv"):
                continue  # keys and values come from the cache
            ex.tensor_from_numpy(t, synth(t.shape, 0.05, 1.0) if "norm" in k else synth(t.shape, 0.02))
    for kc, vc in caches:
        ex.tensor_from_numpy(kc, synth(kc.shape, 1.0))
        ex.tensor_from_numpy(vc, synth(vc.shape, 1.0))
    ex.tensor_from_numpy(x, synth(x.shape, 1.0))
    ex.tensor_from_numpy(rope, synth(rope.shape, 0.5))
    if mask is not None:
        m = np.triu(np.full((seq, seq), -np.inf, np.float32), 1).reshape(1, 1, seq, seq)
        ex.tensor_from_numpy(mask, to_storage(m, dt))
    if args.stage_times:
        ex.enable_stage_times(True)
        ex.launch()
        ex.barrier()
        ex.run(3)
        ex.wait()
        t = ex.stage_times()
        notes = ex.program_dump().splitlines()[1:]
        if rank == 0:
            t0 = t[t > 0].min()
            print(f"stages of {nlayers} layer(s), {args.phase}: first entry -> last exit over the CTAs, microseconds")
            for si in range(t.shape[0]):
                m = t[si, :, 0] > 0
                if not m.any():
                    continue
                b, e = (t[si, m, 0].min() - t0) / 1e3, (t[si, m, 1].max() - t0) / 1e3
                print(f"{si:4d} {b:9.1f} -> {e:9.1f}  {e - b:8.1f}  {notes[si] if si < len(notes) else ''}")
        ex.barrier()
        ex.stop()
        ex.destroy()
        return None
    stream = torch.cuda.ExternalStream(ex.stream())
    ex.launch()
    ex.barrier()
    ex.run(args.warmup)
    ex.wait()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if host_group is not None:
        import torch.distributed as dist
        dist.barrier(group=host_group)
    torch.cuda.synchronize()
    e0.record(stream)
    ex.run(args.iters)
    e1.record(stream)
    ex.wait()
    ms = e0.elapsed_time(e1) / args.iters
    n_stages = ex.status()["n_stages"]
    out = ex.tensor_to_numpy(h)
    finite = bool(np.isfinite(to_f32(out, dt)).all())
    ex.barrier()
    ex.stop()
    ex.destroy()
    if world > 1:
        import torch.distributed as dist
        v = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(v, op=dist.ReduceOp.MAX)
        ms = float(v[0])
    if rank == 0:
        pk, which = peaks()
        f = cfg.ffn_dim // world
        t = batch * seq
        w_elems = cfg.dim * (hl + (0 if decode else 2 * kvl)) * hd + hl * hd * cfg.dim + 3 * cfg.dim * f
        t_kv = span
        flops = nlayers * (2.0 * t * w_elems + 4.0 * batch * hl * seq * t_kv * hd)
        wbytes = nlayers * 2.0 * (w_elems + (2 * batch * kvl * t_kv * hd if decode else 0))
        line = {"metric": f"llama_{args.model}_{args.phase}_tokens_per_s", "value": t / (ms * 1e-3), "unit": "tokens/s",
                "n_gpus": world, "ms_per_step": ms, "layers": nlayers, "dtype": dt, "data": "synthetic",
                "config": {"workload": f"llama2-{args.model}-shaped x{nlayers} layers, tp{world}, {args.phase} batch {batch} "
                                       f"x {seq} tokens, {t_kv} keys", "stages": n_stages, "timed_iterations": args.iters},
                "output_finite": finite}
        if not decode:
            line["config"]["attention"] = ("fused, additive mask tensor" if mask is not None else "fused") if fused else "chain"
        if decode:
            gbs = wbytes / (ms * 1e-3) / 1e9
            line["roofline"] = {"bound": "hbm", "achieved": gbs, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": gbs / pk["hbm_gbs"],
                                "note": f"per-rank weights + K/V bytes per step, of {which} peak"}
        else:
            tf = flops / (ms * 1e-3) / 1e12
            line["roofline"] = {"bound": "tensor", "achieved": tf, "peak": pk["bf16_tflops"], "unit": "TFLOP/s",
                                "frac": tf / pk["bf16_tflops"], "note": f"per-rank matmul FLOPs per step, of {which} peak"}
        return line
    return None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", choices=list(MODELS), default="7b")
    ap.add_argument("--phase", choices=["prefill", "decode"], default="prefill")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--stage-times", action="store_true",
                    help="instead of timing, print when the CTAs entered and left every stage of the last of 3 iterations")
    ap.add_argument("--attention", choices=["fused", "fused-mask", "chain"], default="fused",
                    help="prefill: one fused attention stage (scores on chip; causal from indices, or 'fused-mask': the mask "
                         "tensor added on chip, every key tile computed) or the reference's matmul/softmax/matmul chain")
    ap.add_argument("--qkv", choices=["auto", "side", "sequential"], default="auto",
                    help="prefill with fused attention: Wq, Wk, Wv next to each other on a third of the processors each, "
                         "or one after the other on all of them (auto: side by side from tensor-parallel degree 4 on)")
    args = ap.parse_args()
    import torch
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank, local = int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    ag = host_group = None
    if world > 1:
        import torch.distributed as dist
        from ark_b200.executor import torch_allgather
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        host_group = dist.new_group(backend="gloo")
        ag = torch_allgather(host_group)
    line = run_case(args.model, args.phase, rank, world, local, ag, host_group, args.layers, args.iters, args.warmup, args.stage_times,
                    args.attention, {"auto": None, "side": True, "sequential": False}[args.qkv])
    if line is not None:
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.barrier(group=host_group)
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
