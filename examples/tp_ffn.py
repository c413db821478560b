"""Tensor-parallel feed-forward block Y = GeLU(X W1) W2 (W1 split by columns, W2 by rows over the ranks), the
layout of the reference's examples/transformer/megatron_ark.py. The partial products are summed by ONE in-kernel
all_reduce planned into the second matmul's task; there is no host-side collective on the data path.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29400 examples/tp_ffn.py
"""
import argparse
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import ark_b200 as ark  # noqa: E402
from ark_b200.executor import torch_allgather  # noqa: E402
from ark_b200.ffn import build_ffn  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--d-model", type=int, default=1024)
    ap.add_argument("--d-ff", type=int, default=4096)
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    allgather = None
    if world > 1:
        dist.init_process_group("gloo")  # bootstrap and host rendezvous only
        allgather = torch_allgather()
    ark.init()
    ark.set_rank(rank)
    ark.set_world_size(world)
    x, w1, w2, y = build_ffn(args.tokens, args.d_model, args.d_ff, ark.fp16, rank, world)
    rng = np.random.default_rng(0)
    hx = rng.standard_normal((args.tokens, args.d_model)).astype(np.float16)
    hw1 = (rng.standard_normal((args.d_model, args.d_ff)) * 0.02).astype(np.float16)
    hw2 = (rng.standard_normal((args.d_ff, args.d_model)) * 0.02).astype(np.float16)
    shard = args.d_ff // world
    runtime = ark.Runtime()
    runtime.launch(device_id=local, allgather=allgather)
    x.from_numpy(hx)
    w1.from_numpy(np.ascontiguousarray(hw1[:, rank * shard:(rank + 1) * shard]))
    w2.from_numpy(np.ascontiguousarray(hw2[rank * shard:(rank + 1) * shard]))
    runtime.barrier()
    runtime.run()
    got = y.to_numpy().astype(np.float32)
    runtime.barrier()
    runtime.stop()
    runtime.reset()
    h = hx.astype(np.float32) @ hw1.astype(np.float32)
    h = (0.5 * h * (1 + np.tanh(0.7978845608 * (h + 0.044715 * h ** 3)))).astype(np.float16).astype(np.float32)
    want = h @ hw2.astype(np.float32)
    err = np.abs(got - want).mean()
    print(f"rank {rank}/{world}: tp ffn mean abs error {err:.2e}")
    assert err < 5e-3
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
