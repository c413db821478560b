"""Worker of the multi-GPU tests: one process per GPU under torch.distributed.run.
Checks, on every rank, the in-kernel all_reduce (one-shot and two-shot) against
the exact fp32 sum of the rank inputs (bit-exact), send/recv between
neighbours, the reference's naive all_reduce composition, and the
tensor-parallel FFN block against the oracle."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import ark_b200 as ark  # noqa: E402
from ark_b200.executor import torch_allgather  # noqa: E402
from ark_b200.ffn import build_ffn  # noqa: E402
from oracle import oracle as O  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    # host-side rendezvous over gloo: a resident loop kernel owns every SM, so NCCL kernels could not start
    host_group = dist.new_group(backend="gloo")
    ag = torch_allgather(host_group)

    def run(outputs, feeds, iters=1, loop_mode=True):
        plan = ark.Planner(local).plan()
        ex = ark.Executor(local, 0, "multi", str(plan), loop_mode, allgather=ag)
        ex.set_wait_limit(5_000_000_000)
        ex.compile()
        for t, a in feeds.items():
            ex.tensor_from_numpy(t, a)
        ex.barrier()
        ex.launch()
        ex.run(iters)
        ex.wait()
        outs = [ex.tensor_to_numpy(t) for t in outputs]
        ex.barrier()
        ex.stop()
        ex.destroy()
        return outs

    def fresh():
        ark.init()
        ark.set_rank(rank)
        ark.set_world_size(world)

    # ---- all_reduce sweep: values ~ U(-1,1) from seed+rank, exact fp32 sum then one rounding ----
    for n in (512, 4096, 64 * 1024, 128 * 1024, 1024 * 1024, 8 * 1024 * 1024):
        for dt, adt in (("fp16", ark.fp16), ("bf16", ark.bf16), ("fp32", ark.fp32)):
            if dt != "fp16" and n not in (4096, 1024 * 1024):
                continue
            ins = [O.to_storage(np.random.default_rng(1000 + r).uniform(-1, 1, n).astype(np.float32), dt) for r in range(world)]
            fresh()
            t = ark.tensor([n], adt)
            out = ark.all_reduce(t, rank, world, output=t)
            (got,) = run([out], {t: ins[rank]})
            want = O.all_reduce(ins, dt)
            assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), f"all_reduce {dt} n={n} rank {rank}"
    # closed form of the reference tests: rank r holds r+1 (ops_all_reduce_test.cpp:9-24), 3 iterations in place
    fresh()
    t = ark.tensor([8192], ark.fp16)
    out = ark.all_reduce(t, rank, world, output=t)
    (got,) = run([out], {t: np.full(8192, rank + 1, np.float16)}, iters=1)
    assert np.all(got == np.float16(world * (world + 1) / 2)), "closed-form all_reduce"

    # ---- weight-streaming matmul whose K is cut into ranges, then the one-shot all_reduce of the same task: the push
    # stage follows the sum stage after a barrier (it splits the tensor over the CTAs differently) ----
    rng = np.random.default_rng(31)
    xs = [O.to_storage(rng.normal(0, 1, (1, 8192)).astype(np.float32), "fp16") for _ in range(world)]
    wk = [O.to_storage(rng.normal(0, 0.02, (8192, 1024)).astype(np.float32), "fp16") for _ in range(world)]
    fresh()
    tx, tw = ark.tensor([1, 8192], ark.fp16), ark.tensor([8192, 1024], ark.fp16)
    with ark.PlannerContext(sync=False):
        ty = ark.matmul(tx, tw)
        ty = ark.all_reduce(ty, rank, world, output=ty)
    text = ark.plan_dump(str(ark.Planner(local).plan()))
    assert "split-K sum" in text and "one-shot push" in text, text
    (got,) = run([ty], {tx: xs[rank], tw: wk[rank]}, iters=3)
    want = O.all_reduce([O.matmul(xs[r], wk[r], "fp16") for r in range(world)], "fp16")
    err = np.abs(got.astype(np.float32) - want.astype(np.float32))
    assert err.max() <= 1e-2 * max(1.0, float(np.abs(want.astype(np.float32)).max())), ("split-K matmul + all_reduce", err.max())

    # ---- the reference's two all_reduce compositions (ops_all_reduce_test.cpp:52-187), built with the front end:
    # packets (SendPacket / RecvReduceSendPacket / RecvPacket) and plain data (Send / DeviceSync / RecvReduceSend) ----
    for kind, sizes in (("packet", (2048, 8192)), ("sm", (16 * 1024 * world, 256 * 1024 * world))):
        for n in sizes:
            for closed_form in (True, False):
                if closed_form:  # rank r holds r + 1 everywhere: the sum is exact (ops_all_reduce_test.cpp:9-24)
                    ins = [np.full(n, r + 1, np.float16) for r in range(world)]
                else:
                    ins = [O.to_storage(np.random.default_rng(2000 + r).uniform(-1, 1, n).astype(np.float32), "fp16") for r in range(world)]
                fresh()
                t = ark.tensor([n], ark.fp16)
                out = ark.all_reduce_packet(t, rank, world, 1, t) if kind == "packet" else ark.all_reduce_sm(t, rank, world)
                # 3 iterations in place would sum the sums: run one, then a second executor life is covered by the next case
                (got,) = run([t], {t: ins[rank]}, iters=1)
                want = O.all_reduce(ins, "fp16")
                if closed_form:
                    assert np.all(got == np.float16(world * (world + 1) / 2)), f"all_reduce_{kind} closed form n={n}"
                else:  # own shard first, then the peers': same fp32 sums up to the last bit of the rounding
                    err = np.abs(got.astype(np.float32) - want.astype(np.float32))
                    assert err.max() <= 2.0 ** -9 * max(1.0, float(np.abs(want.astype(np.float32)).max())), (kind, n, err.max())
    # packets over several iterations of one launch: out of place, so that every iteration sums the same inputs
    fresh()
    t = ark.tensor([4096], ark.fp16)
    o = ark.tensor([4096], ark.fp16)
    ark.all_reduce_packet(t, rank, world, 1, o)
    (got,) = run([o], {t: np.full(4096, rank + 1, np.float16)}, iters=5)
    assert np.all(got == np.float16(world * (world + 1) / 2)), "all_reduce_packet, 5 iterations"

    # ---- the plan files the reference ships for 8 ranks, unmodified (examples/tutorial/allreduce-{sm,packet}) ----
    if world == 8:
        import gzip
        import json
        with gzip.open(os.path.join(ROOT, "tests", "golden", "ref_allreduce_plans.json.gz"), "rt") as f:
            plans = json.load(f)
        for d, nelem in (("allreduce-sm", 8 * 1024 * 1024), ("allreduce-packet", 8192)):
            text = plans[f"{d}/plan_gpu{rank}.json"]
            data = json.dumps({"Id": 0, "DataType": "FP16", "Shape": [nelem], "Strides": [nelem], "Offsets": [0],
                               "PaddedShape": [nelem], "Buffer": {"Id": 0, "Rank": -1, "SendTags": [], "RecvTags": []}})
            ex = ark.Executor(local, 0, d, text, True, allgather=ag)
            ex.set_wait_limit(5_000_000_000)
            ex.compile()
            x = np.full(nelem, rank + 1, np.float16)
            ex.tensor_write(data, x.ctypes.data, x.nbytes)
            ex.barrier()
            ex.launch()
            ex.run(1)
            ex.wait()
            ex.barrier()  # every rank has finished: the sums the peers stored here have landed
            got = np.zeros(nelem, np.float16)
            ex.tensor_read(data, got.ctypes.data, got.nbytes)
            ex.barrier()
            ex.stop()
            ex.destroy()
            assert np.all(got == np.float16(36.0)), f"reference plan set {d} on rank {rank}: {np.unique(got)[:8]}"

    # ---- send / recv ring: every rank sends its tensor to rank+1 ----
    fresh()
    src = ark.tensor([4, 1024], ark.fp16)
    dstbuf = ark.tensor([4, 1024], ark.fp16)
    s = ark.send(src, (rank + 1) % world, tag=7)
    ark.send_done(s)
    r = ark.recv(dstbuf, (rank - 1) % world, tag=7)
    res = ark.add(r, 0.0)
    (got,) = run([res], {src: np.full((4, 1024), rank + 1, np.float16)})
    assert np.all(got == np.float16((rank - 1) % world + 1)), f"send/recv on rank {rank}"

    # ---- the reference's naive all_reduce composition (send/send_done/recv/add rounds) ----
    fresh()
    t = ark.tensor([2048], ark.fp16)
    out = ark.all_reduce(t, rank, world, naive=True)
    (got,) = run([out], {t: np.full(2048, rank + 1, np.float16)})
    assert np.all(got == np.float16(world * (world + 1) / 2)), "naive all_reduce"

    # ---- tensor-parallel FFN: partial products summed in-kernel ----
    # fused: the W2 matmul's epilogue stores its tiles into staging slots on the rank that sums them
    # (tokens a multiple of 256 x world); unfused: matmul, then the two-shot all_reduce. Same sums, same order.
    tokens, d, f = 256 * world, 512, 2048
    rng = np.random.default_rng(5)
    x = O.to_storage(rng.normal(0, 1, (tokens, d)).astype(np.float32), "fp16")
    w1 = O.to_storage(rng.normal(0, 0.02, (d, f)).astype(np.float32), "fp16")
    w2 = O.to_storage(rng.normal(0, 0.02, (f, d)).astype(np.float32), "fp16")
    sh = f // world
    parts = [O.matmul(O.matmul(x, np.ascontiguousarray(w1[:, r * sh:(r + 1) * sh]), "fp16", act="gelu"),
                      np.ascontiguousarray(w2[r * sh:(r + 1) * sh, :]), "fp16") for r in range(world)]
    want = O.all_reduce(parts, "fp16")
    results = {}
    for fused in (True, False):
        fresh()
        tx, t1, t2, ty = build_ffn(tokens, d, f, ark.fp16, rank, world, fuse_all_reduce=fused)
        (got,) = run([ty], {tx: x, t1: np.ascontiguousarray(w1[:, rank * sh:(rank + 1) * sh]),
                            t2: np.ascontiguousarray(w2[rank * sh:(rank + 1) * sh, :])}, iters=2)
        err = np.abs(got.astype(np.float32) - want.astype(np.float32))
        assert err.mean() <= 2e-3 and err.max() <= 5e-2, ("tp ffn", fused, err.mean(), err.max())
        results[fused] = got
    assert np.array_equal(results[True].view(np.uint16), results[False].view(np.uint16)), "fused and two-shot sums differ"

    # ---- the same block fed through rings: every rank feeds its tokens/p rows, the ranks exchange them in-kernel, and
    # the all_reduce keeps each rank's rows of the sum (what bench.py's end-to-end leg runs) ----
    from ark_b200.ffn import build_ffn_streaming
    from ark_b200.model import Tensor
    fresh()
    rows = tokens // world
    x_ring, t1, t2, y_ring = build_ffn_streaming(tokens, d, f, ark.fp16, rank, world)
    mdl = ark.Model.get_model()
    x_slot = [Tensor(mdl, ark.fp16, x_ring.buffer, [rows, d], [2 * rows, d], [s_ * rows, 0]) for s_ in range(2)]
    y_slot = [Tensor(mdl, ark.fp16, y_ring.buffer, [rows, d], [2 * rows, d], [s_ * rows, 0]) for s_ in range(2)]
    x2 = O.to_storage(np.random.default_rng(6).normal(0, 1, (tokens, d)).astype(np.float32), "fp16")
    ex = ark.Executor(local, 0, "rings", str(ark.Planner(local).plan()), True, allgather=ag)
    ex.set_wait_limit(5_000_000_000)
    ex.compile()
    ex.tensor_from_numpy(t1, np.ascontiguousarray(w1[:, rank * sh:(rank + 1) * sh]))
    ex.tensor_from_numpy(t2, np.ascontiguousarray(w2[rank * sh:(rank + 1) * sh, :]))
    ex.tensor_from_numpy(x_slot[0], np.ascontiguousarray(x[rank * rows:(rank + 1) * rows]))
    ex.tensor_from_numpy(x_slot[1], np.ascontiguousarray(x2[rank * rows:(rank + 1) * rows]))
    ex.barrier()
    ex.launch()
    ex.run(2)
    ex.wait()
    got0, got1 = ex.tensor_to_numpy(y_slot[0]), ex.tensor_to_numpy(y_slot[1])
    ex.barrier()
    ex.stop()
    ex.destroy()
    assert np.array_equal(got0.view(np.uint16), results[True][rank * rows:(rank + 1) * rows].view(np.uint16)), "streamed rows differ from the fused all_reduce"
    parts2 = [O.matmul(O.matmul(x2, np.ascontiguousarray(w1[:, r * sh:(r + 1) * sh]), "fp16", act="gelu"),
                       np.ascontiguousarray(w2[r * sh:(r + 1) * sh, :]), "fp16") for r in range(world)]
    want2 = O.all_reduce(parts2, "fp16")[rank * rows:(rank + 1) * rows]
    err = np.abs(got1.astype(np.float32) - want2.astype(np.float32))
    assert err.mean() <= 2e-3 and err.max() <= 5e-2, ("streamed tp ffn, second slot", err.mean(), err.max())

    # ---- one tensor-parallel Llama-shaped decoder layer (prefill), against the per-op oracle composition ----
    from ark_b200.llama import LlamaConfig, decoder_layer, layer_weights
    from tests.llama_ref import causal_mask, layer, rope_table
    from tests.test_gpu_llama import make_weights
    cfg = LlamaConfig(dim=512, n_heads=8, n_kv_heads=8, ffn_dim=1024 * world)
    batch, seq = 1, 64
    rng = np.random.default_rng(77)
    ws = [make_weights(cfg, "fp16", world, rng) for _ in range(world)]
    for r in range(1, world):  # the norm weights are replicated
        ws[r]["attn_norm"], ws[r]["ffn_norm"] = ws[0]["attn_norm"], ws[0]["ffn_norm"]
    x = O.to_storage(rng.normal(0, 1, (batch * seq, cfg.dim)).astype(np.float32), "fp16")
    rope = O.to_storage(rope_table(seq, cfg.head_dim), "fp16")
    mask = O.to_storage(causal_mask(seq, "fp16"), "fp16")
    fresh()
    tw = layer_weights(cfg, ark.fp16, world)
    tx = ark.tensor([batch * seq, cfg.dim], ark.fp16)
    tr, tm = ark.tensor([1, seq, 1, cfg.head_dim], ark.fp16), ark.tensor([1, 1, seq, seq], ark.fp16)
    ty = decoder_layer(tx, tw, cfg, batch, seq, rank, world, rope=tr, mask=tm)
    feeds = {tx: x, tr: rope, tm: mask}
    feeds.update({tw[k]: ws[rank][k] for k in tw})
    (got,) = run([ty], feeds)
    want = layer(x, ws, cfg, batch, seq, "fp16", rope=rope, mask=mask)
    err = np.abs(got.astype(np.float32) - want.astype(np.float32))
    assert err.mean() <= 2e-3 and err.max() <= 5e-2, ("llama layer", err.mean(), err.max())

    # ---- the same layer with the fused attention stage (causal=True: no mask tensor, no CTA pairs), 512 tokens: the
    # output projection and W2 push their tiles into the summing rank's slots when 512 splits into 128-row blocks per rank
    seq = 512
    x = O.to_storage(rng.normal(0, 1, (batch * seq, cfg.dim)).astype(np.float32), "fp16")
    rope = O.to_storage(rope_table(seq, cfg.head_dim), "fp16")
    fresh()
    tw = layer_weights(cfg, ark.fp16, world)
    tx, tr = ark.tensor([batch * seq, cfg.dim], ark.fp16), ark.tensor([1, seq, 1, cfg.head_dim], ark.fp16)
    ty = decoder_layer(tx, tw, cfg, batch, seq, rank, world, rope=tr, causal=True)
    text = ark.plan_dump(str(ark.Planner(local).plan()))
    assert "PrefillAttention" in text and text.count(" rope ") == 2 and "*operand" in text, text
    # a rank's projections are narrow here: they run side by side on a third of the processors each
    assert [l.split()[1] for l in text.splitlines() if " Matmul " in l][:3] == ["[0,49)", "[49,98)", "[98,147)"], text
    feeds = {tx: x, tr: rope}
    feeds.update({tw[k]: ws[rank][k] for k in tw})
    (got,) = run([ty], feeds)
    want = layer(x, ws, cfg, batch, seq, "fp16", rope=rope, causal=True)
    err = np.abs(got.astype(np.float32) - want.astype(np.float32))
    assert err.mean() <= 2e-3 and err.max() <= 5e-2, ("llama layer, fused attention", err.mean(), err.max())

    # ---- the same layer, one token against a K/V cache (decode): the one-shot all_reduces ride on the weight-streaming
    # matmuls (result stored straight into every rank's staging slots) and the residual adds on their sum stages ----
    # 4 heads per rank so that every weight matrix keeps >= 512 columns per rank at any world size
    cfg = LlamaConfig(dim=512 * world, n_heads=4 * world, n_kv_heads=4 * world, ffn_dim=1024 * world)
    t_kv, hd = 256, cfg.head_dim
    hl = cfg.n_heads // world
    rng = np.random.default_rng(78)
    ws = [make_weights(cfg, "fp16", world, rng) for _ in range(world)]
    for r in range(1, world):
        ws[r]["attn_norm"], ws[r]["ffn_norm"] = ws[0]["attn_norm"], ws[0]["ffn_norm"]
    xd = O.to_storage(rng.normal(0, 1, (1, cfg.dim)).astype(np.float32), "fp16")
    rope1 = O.to_storage(rope_table(1, hd, start=t_kv), "fp16")
    kcs = [O.to_storage(rng.normal(0, 1, (1, hl, t_kv, hd)).astype(np.float32), "fp16") for _ in range(world)]
    vcs = [O.to_storage(rng.normal(0, 1, (1, hl, t_kv, hd)).astype(np.float32), "fp16") for _ in range(world)]
    fresh()
    tw = layer_weights(cfg, ark.fp16, world)
    tx, tr = ark.tensor([1, cfg.dim], ark.fp16), ark.tensor([1, 1, 1, hd], ark.fp16)
    tk, tv = ark.tensor([1, hl, t_kv, hd], ark.fp16), ark.tensor([1, hl, t_kv, hd], ark.fp16)
    # two layers (the second with its own weights, the same caches): the sum of a layer's last all_reduce is left to the
    # next layer's query projection
    ws2 = [make_weights(cfg, "fp16", world, rng) for _ in range(world)]
    for r in range(1, world):
        ws2[r]["attn_norm"], ws2[r]["ffn_norm"] = ws2[0]["attn_norm"], ws2[0]["ffn_norm"]
    tw2 = layer_weights(cfg, ark.fp16, world, prefix="l1.")
    ty1 = decoder_layer(tx, tw, cfg, 1, 1, rank, world, rope=tr, k_cache=tk, v_cache=tv)
    ty = decoder_layer(ty1, tw2, cfg, 1, 1, rank, world, rope=tr, k_cache=tk, v_cache=tv)
    text = ark.plan_dump(str(ark.Planner(local).plan()))
    # the sums (+ residual) of the first three all_reduces are added up by the stages that consume them (W1 and W3 as one
    # stage over both matrices, the next layer's Wq); the last one keeps its sum stage
    assert text.count("->all_reduce slots") == 4 and text.count("one-shot reduce +residual") == 1 and \
        text.count("<-all_reduce sum +residual") == 3 and text.count("(second matrix") == 2, text
    feeds = {tx: xd, tr: rope1, tk: kcs[rank], tv: vcs[rank]}
    feeds.update({tw[k]: ws[rank][k] for k in tw if k not in ("wk", "wv")})
    feeds.update({tw2[k]: ws2[rank][k] for k in tw2 if k not in ("wk", "wv")})
    got1, got = run([ty1, ty], feeds, iters=3)
    want1 = layer(xd, ws, cfg, 1, 1, "fp16", rope=rope1, k_caches=kcs, v_caches=vcs)
    want = layer(want1, ws2, cfg, 1, 1, "fp16", rope=rope1, k_caches=kcs, v_caches=vcs)
    for g, w_, name in ((got1, want1, "first"), (got, want, "second")):
        err = np.abs(g.astype(np.float32) - w_.astype(np.float32))
        assert err.mean() <= 2e-3 * max(1.0, float(np.abs(w_.astype(np.float32)).mean())) and err.max() <= 1e-1, \
            (f"llama decode, {name} layer", err.mean(), err.max())

    dist.barrier()
    dist.destroy_process_group()
    print(f"rank {rank}: multi-GPU checks passed")


if __name__ == "__main__":
    main()
