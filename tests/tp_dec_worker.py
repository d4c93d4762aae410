"""Child process of test_tp_gpu.py: one rank running the decode-step GEMM fused with the sentinel-polled
all-reduce, residual add and RMSNorm, several times in a row with changing token counts (so that every
receive-buffer generation is reused and shrinking / growing batches exercise the row clean-up).

Checked: every rank ends with bit-identical residual and normalised rows, and both match the fp32
computation on the gathered operands.
"""

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
    from modular_b200._native import lib
    from modular_b200.parallel.tp import TPContext

    L = lib()
    ctx = TPContext(device=dev)
    H, K_local, rows = 2048, 1536, 256
    sym = ctx.alloc_symmetric(L.gemm_dec_lamport_elems(world, rows, H), torch.bfloat16)
    sym.tensor.view(torch.int16).fill_(-32768)
    ctx.barrier()
    _, state = ops.decode_gemm_workspace(dev)
    tp = dict(world=world, rank=rank, lam=sym.peer_ptrs, lam_rows=rows, state=state)
    g = torch.Generator().manual_seed(11)
    w_full = (torch.randn(world, H, K_local, generator=g) * 0.04).to(torch.bfloat16).to(dev)
    gamma = (1 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16).to(dev)
    w = w_full[rank].contiguous()
    errs = []
    for it, T in enumerate((64, 64, 1, 130, 17, 256, 64, 8, 200, 64)):
        gx = torch.Generator().manual_seed(100 + it)
        x_full = torch.randn(world, T, K_local, generator=gx).to(torch.bfloat16).to(dev)
        # exact zeros and negative zeros in the operands must not be mistaken for "not arrived"
        x_full[:, :, : K_local // 2] = 0 if it % 3 == 1 else x_full[:, :, : K_local // 2]
        h0 = torch.randn(T, H, generator=gx).to(torch.bfloat16).to(dev)
        h = h0.clone()
        xn, h = ops.linear_decode(x_full[rank].contiguous(), w, mode="add_norm", h=h, gamma=gamma, tp=tp)
        torch.cuda.synchronize()
        parts = [(x_full[r].float() @ w_full[r].float().t()) for r in range(world)]
        hs = (h0.float() + sum(p.to(torch.bfloat16).float() for p in parts)).to(torch.bfloat16)
        xr = (hs.float() * torch.rsqrt(hs.float().pow(2).mean(-1, keepdim=True) + 1e-5)).to(torch.bfloat16).float() * gamma.float()
        e_h = float((h.float() - hs.float()).abs().max() / hs.float().abs().max())
        e_x = float((xn.float() - xr).abs().max() / xr.abs().max())
        # every rank must hold the same bits
        both = torch.cat([h.view(torch.int16).reshape(-1), xn.view(torch.int16).reshape(-1)]).to(torch.int64)
        digest = int((both * torch.arange(1, both.numel() + 1, device=dev) % 1000003).sum().item())
        errs.append([T, e_h, e_x, digest])
    ops.check_device_error()
    gathered = [None] * world
    dist.all_gather_object(gathered, {"rank": rank, "errs": errs})
    if rank == 0:
        print("TPD_RESULT " + json.dumps(gathered), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
