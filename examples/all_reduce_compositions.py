"""Three ways to sum a tensor over the ranks, each checked against the closed form sum(r + 1):
the reference's packet composition (SendPacket / RecvReduceSendPacket / RecvPacket), its plain-data composition
(Send / DeviceSync / RecvReduceSend), both as its tests build them (ark/ops/ops_all_reduce_test.cpp:52-187), and
the single collective `ark.all_reduce`.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 --master-port 29400 \
        examples/all_reduce_compositions.py
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import ark_b200 as ark  # noqa: E402
from ark_b200.executor import torch_allgather  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("gloo")
    ag = torch_allgather()
    n = 8192 * world
    for kind in ("packet", "plain", "collective"):
        ark.init()
        ark.set_rank(rank)
        ark.set_world_size(world)
        t = ark.tensor([n], ark.fp16)
        if kind == "packet":
            ark.all_reduce_packet(t, rank, world, 1, t)
        elif kind == "plain":
            ark.all_reduce_sm(t, rank, world)
        else:
            ark.all_reduce(t, rank, world, output=t)
        runtime = ark.Runtime()
        runtime.launch(device_id=local, allgather=ag)
        t.from_numpy(np.full(n, rank + 1, np.float16))
        runtime.barrier()
        runtime.run()
        runtime.barrier()
        got = t.to_numpy()
        runtime.barrier()
        runtime.stop()
        runtime.reset()
        assert np.all(got == np.float16(world * (world + 1) / 2)), kind
        print(f"rank {rank}: {kind} all_reduce ok")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
