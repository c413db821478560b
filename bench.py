"""Benchmark of the loop-kernel engine on the tensor-parallel FFN block
(X[4096,8192] · W1[8192,32768/p] -> GeLU -> · W2[32768/p,8192], fp16, fp32
accumulate, partial outputs summed by the in-kernel all_reduce for p > 1).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One JSON line on stdout (rank 0). `value` is whole-job TFLOP/s with operands
resident in HBM (median of several launches of K iterations); `e2e` goes through
the public Executor API with host buffers (H2D of X and D2H of Y inside the timed
region, every step); `parity` compares sampled rows of the result with the CPU
oracle at the full shape on every rank (exit code 3 when it fails).
`--impl reference` times the CPU host-baseline port (the oracle) on a bounded sample.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

TOKENS, D_MODEL, D_FF = 4096, 8192, 32768
FLOPS_PER_STEP = 4.0 * TOKENS * D_MODEL * D_FF  # two GEMMs, 2 flops per MAC
METRIC, UNIT = "ffn_tflops", "TFLOP/s"
# dram__bytes_read.sum + dram__bytes_write.sum of one iteration of the loop kernel, from ncu captures of this file's
# device-timed leg (key: (tokens, GPUs)); the summaries are in profiles/loop_kernel_ffn_tp1.md
NCU_DRAM_BYTES_PER_STEP = {(1024, 1): 1.520e9, (4096, 1): 6.831e9}


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return d, "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs
    (one streaming nvidia-smi process, a line every 20 ms)."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.index, self.rows, self.proc, self.th = index, [], None, None
        self.t_rows = []

    def _run(self):
        for line in self.proc.stdout:
            c = [x.strip() for x in line.split(",")]
            if len(c) >= 7:
                self.rows.append(c)
                self.t_rows.append(time.perf_counter())

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-i",
                                          str(self.index), "-lms", "20"], stdout=subprocess.PIPE, text=True)
            self.th = threading.Thread(target=self._run, daemon=True)
            self.th.start()
            time.sleep(0.3)  # let the first lines arrive before the timed region starts
        except Exception:
            self.proc = None

    def stop(self, t_begin=None, t_end=None):
        time.sleep(0.05)
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                pass
        if self.th:
            self.th.join(timeout=5)
        rows = self.rows
        if t_begin is not None:
            sel = [r for r, t in zip(self.rows, self.t_rows) if t_begin <= t <= t_end]
            rows = sel if sel else rows
        sm = sorted(int(float(r[0])) for r in rows if r[0].replace(".", "").isdigit())
        mx = [int(float(r[1])) for r in rows if r[1].replace(".", "").isdigit()]
        pw = [float(r[2]) for r in rows if r[2].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[3 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_min_mhz": sm[0] if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "power_w_max": max(pw) if pw else None, "reasons": reasons,
                "samples": len(rows)}


def synth(rank, world):
    """Seeded synthetic operands: X ~ N(0,1) (same on every rank), weight shards ~ N(0,0.02)."""
    shard = D_FF // world
    rng = np.random.default_rng(0)
    x = rng.standard_normal((TOKENS, D_MODEL), dtype=np.float32).astype(np.float16)
    rng = np.random.default_rng(100 + rank)
    w1 = (rng.standard_normal((D_MODEL, shard), dtype=np.float32) * 0.02).astype(np.float16)
    w2 = (rng.standard_normal((shard, D_MODEL), dtype=np.float32) * 0.02).astype(np.float16)
    return x, w1, w2


def cpu_sample(rows, threads_note=True):
    """Times the oracle (CPU port of the reference host baselines) on `rows` rows of X
    through the full-width FFN. Returns (TFLOP/s, seconds)."""
    from oracle import oracle as O
    try:  # launchers set OMP_NUM_THREADS=1; the CPU baseline uses every host core
        import ctypes
        ctypes.CDLL("libgomp.so.1").omp_set_num_threads(os.cpu_count() or 1)
    except OSError:
        pass
    x, w1, w2 = synth(0, 1)
    xs = np.ascontiguousarray(x[:rows])
    t0 = time.perf_counter()
    h = O.matmul(xs, w1, "fp16", act="gelu")
    y = O.matmul(h, w2, "fp16")
    dt = time.perf_counter() - t0
    flops = 4.0 * rows * D_MODEL * D_FF
    return flops / dt / 1e12, dt, y


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    rows = 8
    tf, dt, _ = cpu_sample(rows)  # calibration
    per_row = dt / rows
    rows = int(max(8, min(TOKENS, 2.0 / per_row)))  # ~2 s of CPU work per step
    for _ in range(max(0, min(args.warmup, 1))):
        cpu_sample(rows)
    times = []
    for _ in range(max(1, min(args.steps, 5))):
        tf, dt, _ = cpu_sample(rows)
        times.append(dt)
    dt = float(np.mean(times))
    val = 4.0 * rows * D_MODEL * D_FF / dt / 1e12
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": len(times),
            "warmup": min(args.warmup, 1), "ms_per_step": dt * 1e3 * TOKENS / rows, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "fp16", "data": "synthetic",
            "config": {"workload": "tp_ffn_4096x8192x32768_gelu_fp16", "tokens": TOKENS, "d_model": D_MODEL, "d_ff": D_FF},
            "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port",
                             "sample": f"{rows} of {TOKENS} token rows through the full-width FFN per step (OpenMP over rows)"},
            "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def oracle_partial_rows(x_rows, w1, w2):
    """CPU oracle of one rank's partial product on some rows of X: fp16(gelu(x W1_r)) W2_r, fp16 (as the engine rounds)."""
    from oracle import oracle as O
    h = O.matmul(np.ascontiguousarray(x_rows), w1, "fp16", act="gelu")
    return O.matmul(h, w2, "fp16")


def parity_check(y_dev, x, w1, w2, world, rank, host_group, rows=16):
    """Compares `rows` sampled rows of this rank's copy of Y with the oracle at the full shape of the workload:
    every rank computes its own partial product of those rows on the CPU, the partials are exchanged and summed in
    rank order in fp32 with one rounding (the oracle's all_reduce), and each rank checks its own device result."""
    import torch
    from oracle import oracle as O
    try:
        import ctypes
        ctypes.CDLL("libgomp.so.1").omp_set_num_threads(max(1, (os.cpu_count() or 1) // world))
    except OSError:
        pass
    tokens = x.shape[0]
    sel = np.sort(np.random.default_rng(7).choice(tokens, size=min(rows, tokens), replace=False))
    part = oracle_partial_rows(x[sel], w1, w2)
    if world > 1:
        t = torch.from_numpy(np.ascontiguousarray(part).view(np.uint8).reshape(-1).copy())  # gloo moves bytes
        outs = [torch.empty_like(t) for _ in range(world)]
        torch.distributed.all_gather(outs, t, group=host_group)
        want = O.all_reduce([o.numpy().view(np.float16).reshape(part.shape) for o in outs], "fp16")
    else:
        want = part
    got = y_dev[sel].astype(np.float64)
    w = want.astype(np.float64)
    err = np.abs(got - w)
    max_rel = float((err / np.maximum(np.abs(w), 1e-3)).max())
    mean_abs = float(err.mean())
    # the tolerance stated for fp16 results with fp32 accumulation: max rel <= 1e-2 or mean abs <= 2e-3
    ok = bool(np.isfinite(got).all() and (max_rel <= 1e-2 or mean_abs <= 2e-3))
    if world > 1:
        f = torch.tensor([1.0 if ok else 0.0, max_rel, mean_abs], dtype=torch.float64)
        fs = [torch.empty_like(f) for _ in range(world)]
        torch.distributed.all_gather(fs, f, group=host_group)
        ranks_ok = int(sum(float(v[0]) for v in fs))
        max_rel, mean_abs = max(float(v[1]) for v in fs), max(float(v[2]) for v in fs)
    else:
        ranks_ok = int(ok)
    return {"rows": int(len(sel)), "max_rel": max_rel, "mean_abs": mean_abs, "ok": ranks_ok == world, "ranks_ok": ranks_ok,
            "against": "CPU oracle composition matmul -> gelu -> matmul -> all_reduce at the full shape, sampled rows, every rank"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ark_b200")
    ap.add_argument("--repeats", type=int, default=5, help="timed launches of --steps iterations each; the median is reported")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-fused-all-reduce", action="store_true",
                    help="run the W2 matmul and the all_reduce as separate stages (two-shot) instead of fusing them")
    ap.add_argument("--no-e2e", action="store_true", help="device-timed leg only (profiler captures)")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle check of the result (profiler captures)")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the other two parts of the metric (Llama-shaped layers, all_reduce sweep points)")
    ap.add_argument("--tokens", type=int, default=TOKENS, help="reduced size for profiler captures only")
    ap.add_argument("--procs", type=int, default=0, help="experiment: plan for this many SMs instead of all")
    ap.add_argument("--weights-nk", action="store_true", help="store the weights [out, in] (K-major B operands)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import ark_b200 as ark
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    allgather, host_group = None, None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        from ark_b200.executor import torch_allgather
        # host-side rendezvous goes over gloo: while a loop kernel is resident it owns every SM,
        # so an NCCL kernel issued for a barrier could not start
        host_group = dist.new_group(backend="gloo")
        allgather = torch_allgather(host_group)
    tokens = args.tokens
    flops = 4.0 * tokens * D_MODEL * D_FF
    warm = max(args.warmup, 3)
    repeats = max(1, args.repeats)

    from ark_b200.ffn import build_ffn, build_ffn_streaming
    x, w1, w2 = synth(rank, world)
    x = x[:tokens]
    if args.weights_nk:
        w1, w2 = np.ascontiguousarray(w1.T), np.ascontiguousarray(w2.T)

    def barrier():
        if world > 1:
            torch.distributed.barrier(group=host_group)
        torch.cuda.synchronize()

    # ---- device-resident timing: one launch runs all K iterations of the stage program; `repeats` launches ----
    ark.init()
    ark.set_rank(rank)
    ark.set_world_size(world)
    tx, t1, t2, ty = build_ffn(tokens, D_MODEL, D_FF, ark.fp16, rank, world, act="gelu", weights_nk=args.weights_nk,
                               fuse_all_reduce=not args.no_fused_all_reduce)
    plan = ark.Planner(local, num_sm=args.procs or None).plan()
    ex = ark.Executor(local, 0, "bench", str(plan), loop_mode=False, allgather=allgather)
    ex.compile()
    ex.tensor_from_numpy(tx, x)
    ex.tensor_from_numpy(t1, w1)
    ex.tensor_from_numpy(t2, w2)
    stream = torch.cuda.ExternalStream(ex.stream())
    ex.launch()
    ex.run(warm)
    ex.wait()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()  # before the barrier: every rank must enter the timed region together
    ms_all = []
    t_b = time.perf_counter()
    for _ in range(repeats):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record(stream)
        ex.run(args.steps)
        e1.record(stream)
        ex.wait()
        barrier()
        ms_all.append(e0.elapsed_time(e1))
    t_e = time.perf_counter()
    clocks = sampler.stop(t_b, t_e) if rank == 0 else None
    st = ex.status()
    n_stages = st["n_stages"]
    y_value_leg = ex.tensor_to_numpy(ty)
    ex.stop()
    ex.destroy()
    if world > 1:  # per repeat, the slowest rank
        t = torch.tensor(ms_all, device="cuda", dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms_all = [float(v) for v in t]
    ms = float(np.median(ms_all))

    parity = None
    if not args.no_parity:
        if args.weights_nk:
            parity = parity_check(y_value_leg, x, np.ascontiguousarray(w1.T), np.ascontiguousarray(w2.T), world, rank, host_group)
        else:
            parity = parity_check(y_value_leg, x, w1, w2, world, rank, host_group)

    if args.no_e2e:
        value = flops / (ms / args.steps * 1e-3) / 1e12
        if rank == 0:
            print(json.dumps({"metric": METRIC, "value": value, "unit": UNIT, "ms_per_step": ms / args.steps,
                              "tokens": tokens, "clocks": clocks, "parity": parity, "note": "device-timed leg only"}))
        if world > 1:
            torch.distributed.destroy_process_group()
        if parity is not None and not parity["ok"]:
            sys.exit(3)
        return

    # ---- end to end through the Executor API with host buffers: ONE resident loop kernel per rank, the same method
    # at every N. Iteration i reads its input from slot (i-1) % 2 of a ring in the arena and leaves its result in the
    # same slot of an output ring, so while it runs the host copies the next batch in (pinned memory -> device) and
    # the previous result out, all inside the timed region. Each rank feeds and drains only its T/p rows: the ranks
    # exchange the rows of X over NVLink inside the kernel, and the all_reduce keeps each rank's rows of the sum. ----
    rows = tokens // world
    ark.init()
    ark.set_rank(rank)
    ark.set_world_size(world)
    x_ring, s1, s2, y_ring = build_ffn_streaming(tokens, D_MODEL, D_FF, ark.fp16, rank, world, act="gelu")
    plan2 = ark.Planner(local, num_sm=args.procs or None).plan()
    from ark_b200.model import Tensor
    m = ark.Model.get_model()
    x_slot = [Tensor(m, ark.fp16, x_ring.buffer, [rows, D_MODEL], [2 * rows, D_MODEL], [s * rows, 0]) for s in range(2)]
    y_slot = [Tensor(m, ark.fp16, y_ring.buffer, [rows, D_MODEL], [2 * rows, D_MODEL], [s * rows, 0]) for s in range(2)]
    ex2 = ark.Executor(local, 0, "bench_e2e", str(plan2), loop_mode=True, allgather=allgather)
    ex2.compile()
    ex2.tensor_from_numpy(s1, w1)
    ex2.tensor_from_numpy(s2, w2)
    hx = torch.from_numpy(np.ascontiguousarray(x[rank * rows:(rank + 1) * rows])).pin_memory()
    hy = [torch.empty((rows, D_MODEL), dtype=torch.float16).pin_memory() for _ in range(2)]
    nby = hx.numel() * 2
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    from concurrent.futures import ThreadPoolExecutor
    pool = ThreadPoolExecutor(2)
    ex2.barrier()
    ex2.launch()
    done = [ex2.status()["iterations"]]

    def e2e_steps(n):
        slot = done[0] % 2  # iteration done+1 uses slot (done+1-1) % 2
        ex2.tensor_write(x_slot[slot], hx.data_ptr(), nby, s_in.cuda_stream)
        for i in range(n):
            ex2.run(1)
            wr = pool.submit(ex2.tensor_write, x_slot[slot ^ 1], hx.data_ptr(), nby, s_in.cuda_stream) if i + 1 < n else None
            rd = pool.submit(ex2.tensor_read, y_slot[slot ^ 1], hy[slot ^ 1].data_ptr(), nby, s_out.cuda_stream) if i > 0 else None
            ex2.wait()
            if wr:
                wr.result()
            if rd:
                rd.result()
            slot ^= 1
        ex2.tensor_read(y_slot[slot ^ 1], hy[slot ^ 1].data_ptr(), nby, s_out.cuda_stream)
        done[0] += n
        return slot ^ 1

    e2e_steps(warm)
    if world > 1:
        torch.distributed.barrier(group=host_group)
    t0 = time.perf_counter()
    last = e2e_steps(args.steps)
    e2e_s = time.perf_counter() - t0
    if world > 1:
        torch.distributed.barrier(group=host_group)
    y_e2e = hy[last].numpy()
    # the streamed result is the same arithmetic as the device-resident leg: bit for bit
    same = bool(np.array_equal(y_e2e.view(np.uint16), y_value_leg[rank * rows:(rank + 1) * rows].view(np.uint16)))
    checksum = float(np.abs(y_e2e.astype(np.float32)).mean())
    ex2.stop()
    ex2.destroy()

    # ---- the other two parts of the metric, measured in the same run with their own drivers' code: Llama-shaped layer
    # stacks (tokens/s; tensor-parallel over all ranks) and points of the in-kernel all_reduce sweep (bus GB/s) ----
    extras = {}
    if not args.no_extras and tokens == TOKENS:
        import bench_llama
        extras["llama"] = []
        for model, phase in (("7b", "decode"), ("7b", "prefill"), ("70b", "decode"), ("70b", "prefill")):
            try:
                if model == "70b" and world not in (1, 2, 4, 8):
                    # 64 query / 8 KV heads: every rank needs a whole number of query heads per K/V head
                    raise ValueError("needs a tensor-parallel degree that divides 8 K/V heads")
                line = bench_llama.run_case(model, phase, rank, world, local, allgather, host_group)
            except Exception as e:  # one failing case must not lose the headline
                line = {"metric": f"llama_{model}_{phase}_tokens_per_s", "error": f"{type(e).__name__}: {e}"[:200]}
            if rank == 0:
                extras["llama"].append(line)
        if world > 1:
            import bench_allreduce
            extras["all_reduce"] = []
            for size in (8 << 10, 256 << 10, 16 << 20, 64 << 20, 1 << 30):
                try:
                    line = bench_allreduce.run_size(size, rank, world, local, allgather, host_group)
                except Exception as e:
                    line = {"bytes": size, "error": f"{type(e).__name__}: {e}"[:200]}
                if rank == 0:
                    extras["all_reduce"].append(line)
            # the same points through the NVSwitch (multicast-bound arena, multimem.ld_reduce / multimem.st) where the
            # GPUs offer it; from 4 ranks on (with 2 the direct exchange moves fewer bytes)
            if world >= 4:
                os.environ["ARKB_NVLS"] = "1"
                extras["all_reduce_nvls"] = []
                for size in (16 << 20, 64 << 20, 1 << 30):
                    try:
                        line = bench_allreduce.run_size(size, rank, world, local, allgather, host_group)
                    except Exception as e:
                        line = {"bytes": size, "error": f"{type(e).__name__}: {e}"[:200]}
                    if rank == 0:
                        extras["all_reduce_nvls"].append(line)
                os.environ.pop("ARKB_NVLS", None)

    if world > 1:
        t = torch.tensor([e2e_s, 0.0 if same else 1.0], device="cuda", dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        e2e_s, same = float(t[0]), float(t[1]) == 0.0
    bad = (parity is not None and not parity["ok"]) or not same
    if rank != 0:
        if world > 1:
            torch.distributed.destroy_process_group()
        if bad:
            sys.exit(3)
        return
    ms_step = ms / args.steps
    value = flops / (ms_step * 1e-3) / 1e12
    peaks, which = measured_peaks()
    # Denominator: the cuBLAS peak measured in the same regime. The timed launches run back to back for a few tenths
    # of a second; when that drives the GPU into its power cap (reason active, SM clock well below its maximum) the
    # seconds-long sustained figure applies, otherwise the burst figure.
    capped = bool(clocks and clocks.get("sm_mhz") and clocks.get("sm_max_mhz") and "sw_power_cap" in clocks["reasons"] and
                  clocks["sm_mhz"] < 0.9 * clocks["sm_max_mhz"])
    timed_s = ms * 1e-3
    peak = peaks["bf16_tflops_sustained"] if (capped or timed_s >= 1.0) else peaks["bf16_tflops"]
    per_gpu = value / world
    # DRAM traffic of one launch (K iterations), from the ncu capture summarised in profiles/loop_kernel_ffn_tp1.md:
    # dram__bytes_read.sum + dram__bytes_write.sum per iteration at this shape, one GPU
    traffic = NCU_DRAM_BYTES_PER_STEP.get((tokens, world))
    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warm,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp16",
            "data": "synthetic",
            "config": {"workload": "tp_ffn_4096x8192x32768_gelu_fp16", "tokens": tokens, "d_model": D_MODEL, "d_ff": D_FF,
                       "parallelism": f"tp{world}", "l2": "operands (1.1 GiB of weights per step) exceed the 126 MB L2",
                       "stages": n_stages, "checksum_mean_abs": checksum, "timed_launches": repeats,
                       "ms_per_step_each_launch": [round(v / args.steps, 4) for v in ms_all]},
            "clocks": clocks,
            "parity": dict(parity or {}, e2e_bit_identical_to_value_leg=same),
            "e2e": {"value": flops / (e2e_s / args.steps) / 1e12, "unit": UNIT, "h2d_bytes_per_step": nby * world,
                    "d2h_bytes_per_step": nby * world,
                    "method": "one resident loop kernel per rank; input and output rings of 2 slots, copies of step i+1 / "
                              "i-1 under the kernel of step i; each rank moves its tokens/p rows"},
            "gpu_launches": repeats,
            "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": peak, "unit": "TFLOP/s", "frac": per_gpu / peak,
                         "frac_of_burst_peak": per_gpu / peaks["bf16_tflops"],
                         "frac_of_sustained_peak": per_gpu / peaks["bf16_tflops_sustained"],
                         "traffic": traffic * args.steps if traffic else None,
                         "algorithmic_flops_per_launch": flops / world * args.steps,
                         "nvlink_peak_gbs": {"nominal_per_direction": 900.0, "measured_peer_copy": 770.0},
                         "note": f"per-GPU tensor-core rate of the loop kernel (both GEMMs of the step), of {which} "
                                 f"{'sustained' if (capped or timed_s >= 1.0) else 'burst'} cuBLAS bf16 peak; median of "
                                 f"{repeats} launches of {args.steps} iterations"}}
    line.update(extras)
    if not args.no_cpu_baseline:
        tf, dt, _ = cpu_sample(8)
        nrows = int(max(8, min(tokens, 12.0 / (dt / 8))))
        tf, dt, _ = cpu_sample(nrows)
        line["cpu_baseline"] = {"value": tf, "unit": UNIT, "cores": os.cpu_count() or 1, "kind": "port",
                                "sample": f"{nrows} of {tokens} token rows through the full-width FFN, {dt:.1f} s (OpenMP over rows)"}
    print(json.dumps(line))
    if world > 1:
        torch.distributed.destroy_process_group()
    if bad:
        sys.exit(3)


if __name__ == "__main__":
    main()
