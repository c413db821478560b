"""Benchmark of the loop-kernel engine on the tensor-parallel FFN block
(X[4096,8192] · W1[8192,32768/p] -> GeLU -> · W2[32768/p,8192], fp16, fp32
accumulate, partial outputs summed by the in-kernel all_reduce for p > 1).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One JSON line on stdout (rank 0). `value` is whole-job TFLOP/s with operands
resident in HBM; `e2e` goes through the public Executor API with host buffers
(H2D of X and D2H of Y inside the timed region, every step). `--impl reference`
times the CPU host-baseline port (the oracle) on a bounded sample.
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ark_b200")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-fused-all-reduce", action="store_true",
                    help="run the W2 matmul and the all_reduce as separate stages (two-shot) instead of fusing them")
    ap.add_argument("--no-e2e", action="store_true", help="skip the loop-mode end-to-end leg (profiler captures)")
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
    allgather = None
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

    ark.init()
    ark.set_rank(rank)
    ark.set_world_size(world)
    from ark_b200.ffn import build_ffn
    tx, t1, t2, ty = build_ffn(tokens, D_MODEL, D_FF, ark.fp16, rank, world, act="gelu", weights_nk=args.weights_nk,
                               fuse_all_reduce=not args.no_fused_all_reduce)
    plan = ark.Planner(local, num_sm=args.procs or None).plan()
    x, w1, w2 = synth(rank, world)
    x = x[:tokens]
    if args.weights_nk:
        w1, w2 = np.ascontiguousarray(w1.T), np.ascontiguousarray(w2.T)

    def barrier():
        if world > 1:
            torch.distributed.barrier(group=host_group)
        torch.cuda.synchronize()

    # ---- device-resident timing: one launch runs all K iterations of the stage program ----
    ex = ark.Executor(local, 0, "bench", str(plan), loop_mode=False, allgather=allgather)
    ex.compile()
    ex.tensor_from_numpy(tx, x)
    ex.tensor_from_numpy(t1, w1)
    ex.tensor_from_numpy(t2, w2)
    stream = torch.cuda.ExternalStream(ex.stream())
    ex.launch()
    ex.run(warm)
    ex.wait()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()  # before the barrier: every rank must enter the timed region together
    barrier()
    t_b = time.perf_counter()
    e0.record(stream)
    ex.run(args.steps)
    e1.record(stream)
    ex.wait()
    t_e = time.perf_counter()
    barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop(t_b, t_e) if rank == 0 else None
    st = ex.status()
    n_stages = st["n_stages"]
    ex.stop()

    # ---- end to end through the Executor API with host buffers (loop mode) ----
    if args.no_e2e:
        ex.destroy()
        value = flops / (ms / args.steps * 1e-3) / 1e12
        if rank == 0:
            print(json.dumps({"metric": METRIC, "value": value, "unit": UNIT, "ms_per_step": ms / args.steps,
                              "tokens": tokens, "clocks": clocks, "note": "device-timed leg only"}))
        if world > 1:
            torch.distributed.destroy_process_group()
        return
    hx = torch.from_numpy(x.copy()).pin_memory()
    hy = torch.empty((tokens, D_MODEL), dtype=torch.float16).pin_memory()
    nby = hx.numel() * 2
    from concurrent.futures import ThreadPoolExecutor
    pool = ThreadPoolExecutor(2)
    # End to end through the Executor API, host buffers in pinned memory: every step copies its X to the device and
    # reads its Y back (tensor_write / tensor_read block like the reference's), all inside the timed region.
    if world == 1:
        # Two executors over the same plan (each with its own arena, weights loaded once) take the steps in turn from
        # two host threads: while one computes, the other's result goes back and its next input comes in.
        exs, hys, streams = [], [hy, torch.empty_like(hy).pin_memory()], [torch.cuda.Stream(), torch.cuda.Stream()]
        for i in range(2):
            e = ark.Executor(local, 0, f"bench_e2e{i}", str(plan), loop_mode=False)
            e.compile()
            e.tensor_from_numpy(t1, w1)
            e.tensor_from_numpy(t2, w2)
            e.launch()
            exs.append(e)

        def lane(i, n):
            for _ in range(n):
                exs[i].tensor_write(tx, hx.data_ptr(), nby, streams[i].cuda_stream)
                exs[i].run(1)
                exs[i].wait()
                exs[i].tensor_read(ty, hys[i].data_ptr(), nby, streams[i].cuda_stream)

        def e2e_steps(n):
            jobs = [pool.submit(lane, 0, (n + 1) // 2), pool.submit(lane, 1, n // 2)]
            for j in jobs:
                j.result()

        def e2e_close():
            for e in exs:
                e.stop()
                e.destroy()
    else:
        # Tensor-parallel: one executor per rank (two would let the ranks pair up different kernels at the in-kernel
        # barriers). PCIe is full duplex, so the read of step i's Y and the write of step i+1's X are issued together
        # (two host threads, one stream each).
        ex2 = ark.Executor(local, 0, "bench_e2e", str(plan), loop_mode=True, allgather=allgather)
        ex2.compile()
        ex2.tensor_from_numpy(t1, w1)
        ex2.tensor_from_numpy(t2, w2)
        ex2.launch()
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()

        def e2e_steps(n):
            ex2.tensor_write(tx, hx.data_ptr(), nby, s_in.cuda_stream)
            for i in range(n):
                ex2.run(1)
                ex2.wait()
                rd = pool.submit(ex2.tensor_read, ty, hy.data_ptr(), nby, s_out.cuda_stream)
                if i + 1 < n:
                    wr = pool.submit(ex2.tensor_write, tx, hx.data_ptr(), nby, s_in.cuda_stream)
                    wr.result()
                rd.result()

        def e2e_close():
            ex2.stop()
            ex2.destroy()
    e2e_steps(warm)
    if world > 1:
        torch.distributed.barrier(group=host_group)
    t0 = time.perf_counter()
    e2e_steps(args.steps)
    e2e_s = time.perf_counter() - t0
    checksum = float(hy.float().abs().mean())
    e2e_close()
    ex.destroy()

    if world > 1:
        t = torch.tensor([ms, e2e_s], device="cuda", dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms, e2e_s = float(t[0]), float(t[1])
    if rank != 0:
        if world > 1:
            torch.distributed.destroy_process_group()
        return
    ms_step = ms / args.steps
    value = flops / (ms_step * 1e-3) / 1e12
    peaks, which = measured_peaks()
    timed_s = ms * 1e-3
    peak = peaks["bf16_tflops_sustained"] if timed_s >= 1.0 else peaks["bf16_tflops"]
    per_gpu = value / world
    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warm,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp16",
            "data": "synthetic",
            "config": {"workload": "tp_ffn_4096x8192x32768_gelu_fp16", "tokens": tokens, "d_model": D_MODEL, "d_ff": D_FF,
                       "parallelism": f"tp{world}", "l2": "operands (1.1 GiB of weights per step) exceed the 126 MB L2",
                       "stages": n_stages, "checksum_mean_abs": checksum},
            "clocks": clocks,
            "e2e": {"value": flops / (e2e_s / args.steps) / 1e12, "unit": UNIT, "h2d_bytes_per_step": nby,
                    "d2h_bytes_per_step": nby},
            "gpu_launches": 1,
            "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": peak, "unit": "TFLOP/s", "frac": per_gpu / peak,
                         "traffic": None,
                         "note": f"per-GPU tensor-core rate of the loop kernel (both GEMMs of the step), of {which} "
                                 f"{'sustained' if timed_s >= 1.0 else 'burst'} cuBLAS bf16 peak"}}
    if not args.no_cpu_baseline:
        tf, dt, _ = cpu_sample(8)
        rows = int(max(8, min(tokens, 12.0 / (dt / 8))))
        tf, dt, _ = cpu_sample(rows)
        line["cpu_baseline"] = {"value": tf, "unit": UNIT, "cores": os.cpu_count() or 1, "kind": "port",
                                "sample": f"{rows} of {tokens} token rows through the full-width FFN, {dt:.1f} s (OpenMP over rows)"}
    print(json.dumps(line))
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
