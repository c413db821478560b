"""Llama-2-shaped decoder layers, tensor-parallel over the ranks (heads and feed-forward width split as in the
reference's examples/llama/model.py:102-216, 316-444), prefill or one decode step against a K/V cache. Random
weights; prints the time of one step and a finiteness check.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29400 \
        examples/llama_tp.py --model 7b --phase decode
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import bench_llama  # noqa: E402  (the same builder the benchmark uses)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", choices=["7b", "70b"], default="7b")
    ap.add_argument("--phase", choices=["prefill", "decode"], default="decode")
    ap.add_argument("--layers", type=int, default=2)
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    ag = host_group = None
    if world > 1:
        import torch.distributed as dist
        from ark_b200.executor import torch_allgather
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        host_group = dist.new_group(backend="gloo")
        ag = torch_allgather(host_group)
    line = bench_llama.run_case(args.model, args.phase, rank, world, local, ag, host_group, layers=args.layers)
    if line is not None:
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist
        dist.barrier(group=host_group)
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
