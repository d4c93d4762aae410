"""Child process of test_tp_gpu.py: stand-alone collectives against NCCL."""

import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from modular_b200 import ops
    from modular_b200.parallel.tp import TPContext

    coll = TPContext(device=dev).collectives(32 << 20)
    res = {"rank": rank, "multicast": bool(coll.multicast_ptr), "cases": []}
    algos = ["lamport", "one_shot", "two_shot", "auto"] + (["multimem"] if coll.multicast_ptr and os.environ.get("MB200_TEST_MULTIMEM") == "1" else [])
    for n in (8, 4096, 64 * 4096, 3 * 1000 * 1000 - 8 * 7):
        g = torch.Generator().manual_seed(n + rank)
        x = torch.randn(n, generator=g).to(torch.bfloat16).to(dev)
        want = x.float().clone()
        dist.all_reduce(want)
        for algo in algos:
            if algo == "lamport" and n > coll.lam_cap:
                continue
            got = coll.all_reduce(x, algo)
            torch.cuda.synchronize()
            err = float((got.float() - want).abs().max() / want.abs().max())
            # identical on every rank
            ref0 = got.clone()
            dist.broadcast(ref0, 0)
            res["cases"].append(["allreduce", algo, n, err, bool(torch.equal(ref0, got))])
    # barrier-free all-reduce + residual + RMSNorm, shrinking and growing row counts across calls
    for it, rows in enumerate((64, 7, 128, 64, 1)):
        g = torch.Generator().manual_seed(500 + it)
        xs = [torch.randn(rows, 1024, generator=g).to(torch.bfloat16) for _ in range(world)]
        h0 = torch.randn(rows, 1024, generator=g).to(torch.bfloat16).to(dev)
        gamma = (1 + 0.1 * torch.randn(1024, generator=g)).to(torch.bfloat16).to(dev)
        h = h0.clone()
        y, h = coll.all_reduce_add_rms_norm(xs[rank].to(dev), h, gamma, 1e-5)
        torch.cuda.synchronize()
        hs = (h0.float() + sum(t.float() for t in xs).to(dev)).to(torch.bfloat16)
        yr = (hs.float() * torch.rsqrt(hs.float().pow(2).mean(-1, keepdim=True) + 1e-5)).to(torch.bfloat16).float() * gamma.float()
        err = float((y.float() - yr).abs().max() / yr.abs().max())
        ref0 = y.clone()
        dist.broadcast(ref0, 0)
        res["cases"].append(["allreduce", "lamport+rmsnorm", rows * 1024, err, bool(torch.equal(ref0, y))])
    x = torch.randn(5, 24, generator=torch.Generator().manual_seed(rank)).to(torch.bfloat16).to(dev)
    got = coll.all_gather(x)
    want = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(want, x)
    res["cases"].append(["allgather", "", x.numel(), float((got - torch.cat(want)).abs().max()), True])
    y = torch.randn(1000, 8, generator=torch.Generator().manual_seed(100 + rank)).to(dev)
    got = coll.broadcast(y, root=world - 1)
    want = y.clone()
    dist.broadcast(want, world - 1)
    res["cases"].append(["broadcast", "", y.numel(), float((got - want).abs().max()), True])
    full = torch.randn(world, 33, 16, generator=torch.Generator().manual_seed(7)).to(dev)
    got = coll.scatter(full if rank == 1 % world else None, full[0], root=1 % world)
    res["cases"].append(["scatter", "", full[0].numel(), float((got - full[rank]).abs().max()), True])
    torch.cuda.synchronize()
    ops.check_device_error()
    gathered = [None] * world
    dist.all_gather_object(gathered, res)
    if rank == 0:
        print("COLL_RESULT " + json.dumps(gathered), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
