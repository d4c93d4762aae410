"""Child process of test_tp_gpu.py: one rank exercising the GEMM kernels fused with collectives.

Chain under test (what one tensor-parallel half-layer does):
    row-parallel GEMM with epilogue pushes to the row owners   (GEMM -> reduce-scatter)
    reduce + residual + RMSNorm + pushes of the normalised rows, closing with ready flags
    column-parallel GEMM whose tiles wait on the per-source flags (all-gather -> GEMM)
compared with an fp32 PyTorch computation on NCCL-gathered operands.
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
    H, K_local, N2, T_max = 1024, 2048, 768, 640
    partial_rows = T_max + world
    sym_partial = ctx.alloc_symmetric(partial_rows * H, torch.bfloat16)
    sym_xn = ctx.alloc_symmetric(T_max * H, torch.bfloat16)
    sym_flags = ctx.alloc_symmetric(L.tp_flag_ints(), torch.int32, zero=True)
    ctx.barrier()
    g = torch.Generator().manual_seed(7)            # same weights drawn on every rank
    w1_full = (torch.randn(world, H, K_local, generator=g) * 0.05).to(torch.bfloat16).to(dev)
    w2 = (torch.randn(N2 * 2, H, generator=g) * 0.05).to(torch.bfloat16).to(dev)   # [gate; up]
    gamma = (1 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16).to(dev)
    w1 = w1_full[rank].contiguous()
    errs = []
    for it, T in enumerate((64, 640, 1, 130, 333, 64)):
        rpr = (T + world - 1) // world
        gx = torch.Generator().manual_seed(1000 * it)
        x_full = (torch.randn(world, T, K_local, generator=gx)).to(torch.bfloat16).to(dev)
        h_full = (torch.randn(T, H, generator=gx)).to(torch.bfloat16).to(dev)
        x = x_full[rank].contiguous()
        row0 = rank * rpr
        n_mine = max(0, min(rpr, T - row0))
        h_local = torch.zeros(rpr, H, dtype=torch.bfloat16, device=dev)
        h_local[:n_mine] = h_full[row0:row0 + n_mine]
        max_slots = partial_rows // rpr
        expected, splits = L.gemm_bf16_comm(x, w1, None, T, False, False, True, 0, 0, world, rank, rpr,
                                            sym_flags.peer_ptrs, sym_partial.peer_ptrs, max_slots)
        L.tp_rs_norm_ag_ex(world, rank, sym_partial.peer_ptrs, sym_xn.peer_ptrs, sym_flags.peer_ptrs,
                           h_local, gamma, T, rpr, 1e-5, True, 3, world * splits, expected)
        xn_view = sym_xn.tensor[: T * H].view(T, H)
        y = torch.empty(T, N2, dtype=torch.bfloat16, device=dev)
        L.gemm_bf16_comm(xn_view, w2, y, T, True, True, False, 0, 1, world, rank, rpr,
                         sym_flags.peer_ptrs, [], 0)
        torch.cuda.synchronize()
        # reference in fp32
        part = sum(x_full[r].float() @ w1_full[r].float().t() for r in range(world))
        hs = (h_full.float() + part).to(torch.bfloat16).float()
        xn_ref = (hs * torch.rsqrt(hs.pow(2).mean(-1, keepdim=True) + 1e-5)).to(torch.bfloat16).float() * gamma.float()
        xn_ref = xn_ref.to(torch.bfloat16)
        gu = xn_ref.float() @ w2.float().t()
        y_ref = torch.nn.functional.silu(gu[:, :N2]) * gu[:, N2:]
        e_h = float((h_local[:n_mine].float() - hs[row0:row0 + n_mine]).abs().max()) if n_mine else 0.0
        e_xn = float((xn_view.float() - xn_ref.float()).abs().max() / xn_ref.float().abs().max())
        e_y = float((y.float() - y_ref).abs().max() / y_ref.abs().max())
        errs.append([T, splits, e_h, e_xn, e_y])
        dist.barrier()   # the test reuses buffers across iterations without the layer chain's ordering
    ops.check_device_error()
    gathered = [None] * world
    dist.all_gather_object(gathered, {"rank": rank, "errs": errs})
    if rank == 0:
        print("TPF_RESULT " + json.dumps(gathered), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
