"""In-kernel all_reduce sweep (fp16 sum, 1 KiB .. 1 GiB, doubling) under
torch.distributed.run, one process per GPU:

  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
      --master-port P bench_allreduce.py [--max-bytes B] [--iters K] [--nccl]

Per size, rank 0 prints one JSON line: device time per all_reduce (max over
ranks, CUDA events around one launch of K iterations), algorithm bandwidth
S/t and bus bandwidth S*2(p-1)/p/t (the NCCL convention), the fraction of the
measured peer-copy bandwidth (770 GB/s per direction on this pool), and with
--nccl the same measurement for torch.distributed.all_reduce as an
out-of-kernel comparison. Inputs are zeros so that repeated in-place sums stay finite.
"""
import argparse
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
NVLINK_PEER_GBS = 770.0  # measured peer copy, per direction


def run_size(size, rank, world, local, ag, host_group, iters=20, nccl=False):
    """Times the in-kernel all_reduce of `size` bytes of fp16; returns the result line on rank 0, None elsewhere."""
    import torch
    import torch.distributed as dist
    import ark_b200 as ark
    n = size // 2
    ark.init()
    ark.set_rank(rank)
    ark.set_world_size(world)
    t = ark.tensor([n], ark.fp16)
    ark.all_reduce(t, rank, world, output=t)
    ex = ark.Executor(local, 0, "ar", str(ark.Planner(local).plan()), loop_mode=False, allgather=ag)
    ex.compile()
    ex.tensor_from_numpy(t, np.zeros(n, np.float16))
    stream = torch.cuda.ExternalStream(ex.stream())
    ex.launch()
    ex.barrier()
    ex.run(3)
    ex.wait()
    iters = iters if size <= (64 << 20) else max(3, iters // 4)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dist.barrier(group=host_group)
    torch.cuda.synchronize()
    e0.record(stream)
    ex.run(iters)
    e1.record(stream)
    ex.wait()
    ms = e0.elapsed_time(e1) / iters
    text = ex.program_dump()
    ex.barrier()
    ex.stop()
    ex.destroy()
    nccl_ms = None
    if nccl:
        buf = torch.zeros(n, dtype=torch.float16, device="cuda")
        for _ in range(3):
            dist.all_reduce(buf)
        torch.cuda.synchronize()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        for _ in range(iters):
            dist.all_reduce(buf)
        a1.record()
        torch.cuda.synchronize()
        nccl_ms = a0.elapsed_time(a1) / iters
    v = torch.tensor([ms, nccl_ms or 0.0], device="cuda", dtype=torch.float64)
    dist.all_reduce(v, op=dist.ReduceOp.MAX)
    ms, nccl_ms = float(v[0]), (float(v[1]) if nccl else None)
    if rank != 0:
        return None
    bus = size * 2 * (world - 1) / world / (ms * 1e-3) / 1e9
    line = {"bytes": size, "n_gpus": world, "us": ms * 1e3, "alg_GB/s": size / (ms * 1e-3) / 1e9, "bus_GB/s": bus,
            "frac_of_peer_copy": bus / NVLINK_PEER_GBS, "frac_of_nominal_900": bus / 900.0,
            "algo": "one-shot" if "one-shot" in text else "nvls" if "NVLS" in text else "two-shot"}
    if nccl_ms:
        line["nccl_us"] = nccl_ms * 1e3
        line["nccl_bus_GB/s"] = size * 2 * (world - 1) / world / (nccl_ms * 1e-3) / 1e9
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--min-bytes", type=int, default=1024)
    ap.add_argument("--max-bytes", type=int, default=1 << 30)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--nccl", action="store_true")
    args = ap.parse_args()
    import torch
    import torch.distributed as dist
    from ark_b200.executor import torch_allgather
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    host_group = dist.new_group(backend="gloo")  # host-side rendezvous without GPU kernels
    ag = torch_allgather(host_group)
    size = args.min_bytes
    while size <= args.max_bytes:
        line = run_size(size, rank, world, local, ag, host_group, args.iters, args.nccl)
        if line is not None:
            print(json.dumps(line), flush=True)
        size *= 2
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
