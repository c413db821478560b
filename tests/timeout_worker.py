"""Worker of the bounded-wait test: two ranks, rank 1 maps its memory but never runs the step, so rank 0's
Recv waits for a flag that nothing sets. The wait runs out after the short limit, the kernel returns a status,
wait() raises GpuError, and the same GPU then runs another executor. Nothing here faults or hangs a GPU:
the only failure is a wait that gives up by itself.

ARKB_SAME_DEVICE=1 puts both ranks on GPU 0 (rank 1 never launches a kernel, so only one kernel is ever
resident); otherwise rank r uses GPU r and a first step in which both ranks run is checked too."""
import os
import sys
import time

import numpy as np
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import ark_b200 as ark  # noqa: E402
from ark_b200.executor import torch_allgather  # noqa: E402
from oracle import oracle as O  # noqa: E402

LIMIT_NS = 50_000_000  # 50 ms


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    assert world == 2
    same = os.environ.get("ARKB_SAME_DEVICE") == "1"
    dev = 0 if same else int(os.environ["LOCAL_RANK"])
    dist.init_process_group("gloo")
    ag = torch_allgather()
    ark.init()
    ark.set_rank(rank)
    ark.set_world_size(world)
    src = ark.tensor([4, 1024], ark.fp16)
    dstbuf = ark.tensor([4, 1024], ark.fp16)
    s = ark.send(src, 1 - rank, tag=11)
    ark.send_done(s)
    r = ark.recv(dstbuf, 1 - rank, tag=11)
    res = ark.add(r, 0.0)
    ex = ark.Executor(dev, 0, "timeout", str(ark.Planner(dev).plan()), True, allgather=ag)
    ex.set_wait_limit(LIMIT_NS)
    ex.compile()
    ex.tensor_from_numpy(src, np.full((4, 1024), rank + 1, np.float16))
    ex.barrier()
    if not same:
        # step 1: both ranks run; the exchange completes
        ex.launch()
        ex.run(1)
        ex.wait()
        assert np.all(ex.tensor_to_numpy(res) == np.float16(2 - rank))
        dist.barrier()
    if rank == 0:
        if same:
            ex.launch()
        t0 = time.perf_counter()
        ex.run(1)  # the peer never runs this step
        try:
            ex.wait()
            raise SystemExit("wait() returned although the peer never signalled")
        except ark.GpuError as e:
            msg = str(e)
        took = time.perf_counter() - t0
        st = ex.status()
        assert st["code"] == 3, st  # peer flag wait timed out
        assert "status 3" in msg, msg
        assert took < 5.0, took  # the limit, not the 10 s default, ended the wait
        assert 0 <= st["stage"] < st["n_stages"]
        try:
            ex.stop()
        except ark.GpuError:
            pass
        # the context is still usable: a fresh single-rank executor on the same GPU passes a parity case
        ark.init()
        ark.set_rank(0)
        ark.set_world_size(1)
        a = ark.tensor([128, 256], ark.fp16)
        b = ark.tensor([256, 128], ark.fp16)
        c = ark.matmul(a, b)
        rng = np.random.default_rng(3)
        xa = O.to_storage(rng.uniform(-0.1, 0.1, (128, 256)).astype(np.float32), "fp16")
        xb = O.to_storage(rng.uniform(-0.1, 0.1, (256, 128)).astype(np.float32), "fp16")
        e2 = ark.Executor(dev, 0, "after", str(ark.Planner(dev).plan()), True)
        e2.set_wait_limit(3_000_000_000)
        e2.compile()
        e2.tensor_from_numpy(a, xa)
        e2.tensor_from_numpy(b, xb)
        e2.launch()
        e2.run(1)
        e2.wait()
        got = e2.tensor_to_numpy(c)
        e2.stop()
        e2.destroy()
        want = O.matmul(xa, xb, "fp16")
        err = np.abs(got.astype(np.float32) - want.astype(np.float32))
        assert err.max() <= 1e-2, err.max()
    # rank 1 keeps its memory mapped until rank 0 is done, then both leave (no kernel in flight anywhere)
    dist.barrier()
    if rank == 1 and not same:
        ex.stop()
    ex.destroy()
    dist.barrier()
    dist.destroy_process_group()
    print(f"rank {rank}: bounded-wait checks passed")


if __name__ == "__main__":
    main()
