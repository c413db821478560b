"""Worker of the NVLS test: with ARKB_NVLS=1 the arena of every rank is a symmetric allocation bound to one
NVSwitch multicast object, the large all_reduce is lowered to multimem.ld_reduce + multimem.st, and the all_reduce
fused into a Matmul broadcasts its sums with one multimem.st. Results against the oracle; where the GPUs or the
driver offer no multicast the executor falls back to the plain arena and the worker says so."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
os.environ["ARKB_NVLS"] = "1"
import ark_b200 as ark  # noqa: E402
from ark_b200.executor import torch_allgather  # noqa: E402
from ark_b200.ffn import build_ffn  # noqa: E402
from oracle import oracle as O  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("gloo")
    ag = torch_allgather()

    def run(outputs, feeds, iters=1):
        ex = ark.Executor(local, 0, "nvls", str(ark.Planner(local).plan()), True, allgather=ag)
        ex.set_wait_limit(5_000_000_000)
        ex.compile()
        text = ex.program_dump()
        for t, a in feeds.items():
            ex.tensor_from_numpy(t, a)
        ex.barrier()
        ex.launch()
        ex.run(iters)
        ex.wait()
        ex.barrier()
        outs = [ex.tensor_to_numpy(t) for t in outputs]
        ex.barrier()
        ex.stop()
        ex.destroy()
        return outs, text

    def fresh():
        ark.init()
        ark.set_rank(rank)
        ark.set_world_size(world)

    used = None
    nvls_ok = [True]
    for n in (512 * 1024, 8 * 1024 * 1024):
        for dt, adt in (("fp16", ark.fp16), ("bf16", ark.bf16), ("fp32", ark.fp32)):
            for closed in (True, False):
                if closed:
                    ins = [O.to_storage(np.full(n, r + 1, np.float32), dt) for r in range(world)]
                else:
                    ins = [O.to_storage(np.random.default_rng(3000 + r).uniform(-1, 1, n).astype(np.float32), dt) for r in range(world)]
                fresh()
                t = ark.tensor([n], adt)
                with ark.PlannerContext(config={"Algo": "nvls"}) if nvls_ok[0] else ark.PlannerContext():
                    out = ark.all_reduce(t, rank, world, output=t)
                try:
                    (got,), text = run([out], {t: ins[rank]})
                except ark.UnsupportedError:
                    # no multicast on these GPUs (the executor said so and kept the plain arena): peer loads and stores
                    assert used is None
                    nvls_ok[0] = False
                    fresh()
                    t = ark.tensor([n], adt)
                    out = ark.all_reduce(t, rank, world, output=t)
                    (got,), text = run([out], {t: ins[rank]})
                if used is None:
                    used = "NVLS" in text
                    if not used:
                        print(f"rank {rank}: nvls unavailable, plain arena used")
                want = O.all_reduce(ins, dt)
                g, w = O.to_f32(got, dt), O.to_f32(want, dt)
                if closed:
                    assert np.array_equal(g, w), f"closed-form all_reduce {dt} n={n}"
                else:
                    # The switch accumulates in fp32 but does not round the way the oracle does (fp32 sum in rank order,
                    # then round to nearest even): measured on 2 ranks, where the fp32 sum is exact, 18 % of fp16
                    # results differ from the oracle in the last bit. One spacing of the storage type at the
                    # magnitude of the result is the bound; the default peer-load path is the bit-exact one.
                    tol = {"fp32": 1e-6, "fp16": 2.0 ** -10, "bf16": 2.0 ** -7}[dt] * np.maximum(1.0, np.abs(w))
                    assert bool((np.abs(g - w) <= tol).all()), (dt, n, float(np.abs(g - w).max()))
                assert ("NVLS" in text) == used
    # Matmul + all_reduce in one task: the sums leave through the multicast address
    tokens, d, f = 256 * world, 512, 2048
    rng = np.random.default_rng(5)
    x = O.to_storage(rng.normal(0, 1, (tokens, d)).astype(np.float32), "fp16")
    w1 = O.to_storage(rng.normal(0, 0.02, (d, f)).astype(np.float32), "fp16")
    w2 = O.to_storage(rng.normal(0, 0.02, (f, d)).astype(np.float32), "fp16")
    sh = f // world
    parts = [O.matmul(O.matmul(x, np.ascontiguousarray(w1[:, r * sh:(r + 1) * sh]), "fp16", act="gelu"),
                      np.ascontiguousarray(w2[r * sh:(r + 1) * sh, :]), "fp16") for r in range(world)]
    want = O.all_reduce(parts, "fp16")
    fresh()
    tx, t1, t2, ty = build_ffn(tokens, d, f, ark.fp16, rank, world, fuse_all_reduce=True)
    (got,), text = run([ty], {tx: x, t1: np.ascontiguousarray(w1[:, rank * sh:(rank + 1) * sh]),
                              t2: np.ascontiguousarray(w2[rank * sh:(rank + 1) * sh, :])}, iters=2)
    assert ("multicast store" in text) == used, text
    err = np.abs(got.astype(np.float32) - want.astype(np.float32))
    assert err.mean() <= 2e-3 and err.max() <= 5e-2, ("tp ffn over nvls", err.mean(), err.max())
    dist.barrier()
    dist.destroy_process_group()
    print(f"rank {rank}: nvls checks passed (multicast {'used' if used else 'not available'})")


if __name__ == "__main__":
    main()
