"""Child process of test_ep.py: one rank of an expert-parallel MoE layer (launched by torchrun).

Backend ``gloo`` runs the host exchange on CPU; ``nccl`` runs the peer-memory kernels on one GPU
per rank. Every rank builds the same full MoE from a seed, keeps its expert slice, runs its own
token batch through the EP layer several times and compares with the full single-rank layer.
"""

import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    backend = sys.argv[1]
    fp8 = len(sys.argv) > 2 and sys.argv[2] in ("fp8", "fp8experts")
    fp8_experts = len(sys.argv) > 2 and sys.argv[2] == "fp8experts"
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    from modular_b200.nn.moe import MoE, MoEConfig
    from modular_b200.parallel.ep import EPContext, EPMoE, shard_moe

    if backend == "nccl":
        local = int(os.environ["LOCAL_RANK"])
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
        dist.init_process_group("nccl", device_id=dev)
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
    if len(sys.argv) > 2 and sys.argv[2] == "deepseek":
        return deepseek_model(rank, world, dev)
    if len(sys.argv) > 2 and sys.argv[2] == "engine":
        return deepseek_engine(rank, world, dev)
    cfg = MoEConfig(hidden_size=512, moe_intermediate_size=256, n_routed_experts=16, num_experts_per_tok=4,
                    n_shared_experts=1, n_group=4, topk_group=2, routed_scaling_factor=2.5)
    full = MoE.random_init(cfg, dev, torch.bfloat16, seed=3, std=0.05)
    if fp8_experts:
        # block-scaled fp8 expert weights: the dispatched rows stay quantised and feed the grouped fp8 GEMM
        from modular_b200.nn.moe import Fp8ExpertWeights
        full = MoE(cfg, full.gate, Fp8ExpertWeights.quantize(full.w_gate_up), Fp8ExpertWeights.quantize(full.w_down),
                   full.bias, full.shared_gate_up, full.shared_down)
    mine = shard_moe(full, rank, world)
    ep = None
    if backend == "nccl":
        from modular_b200.parallel.tp import TPContext
        ep = EPContext(TPContext(device=dev), cfg.hidden_size, cfg.n_routed_experts, cfg.num_experts_per_tok,
                       max_tokens=96, fp8_dispatch=fp8)
    layer = EPMoE(mine, ep)
    errs, drops = [], 0
    for it, T in enumerate((64, 96, 1, 33)):
        g = torch.Generator().manual_seed(100 * it + rank)
        x = (torch.randn(T, cfg.hidden_size, generator=g)).to(torch.bfloat16).to(dev)
        y = layer(x)
        ref = full(x)
        errs.append(float((y.float() - ref.float()).abs().max() / ref.float().abs().max()))
        drops += layer.dropped
    if backend == "nccl":
        torch.cuda.synchronize()
        from modular_b200 import ops
        ops.check_device_error()
    out = {"rank": rank, "errs": errs, "dropped": drops}
    gathered = [None] * world
    dist.all_gather_object(gathered, out)
    if rank == 0:
        print("EP_RESULT " + json.dumps(gathered), flush=True)
    dist.barrier()
    dist.destroy_process_group()


def deepseek_model(rank, world, dev):
    """A tiny DeepSeek-V3 with expert-parallel MoE layers (data-parallel attention: every rank runs
    its own sequence) against the same model with all experts local."""
    from modular_b200 import ops
    from modular_b200.models.deepseek_v3 import DeepseekV3Config, DeepseekV3Model, DeepseekV3Weights
    from modular_b200.parallel.ep import EPContext
    from modular_b200.parallel.tp import TPContext

    cfg = DeepseekV3Config.tiny(hidden_size=512, moe_intermediate_size=256, intermediate_size=1024,
                                kv_lora_rank=128, q_lora_rank=256, num_attention_heads=8)
    full = DeepseekV3Weights.random_init(cfg, dev, torch.bfloat16, seed=11, std=0.05)
    El = cfg.n_routed_experts // world
    mine = DeepseekV3Weights.random_init(cfg, dev, torch.bfloat16, seed=11, std=0.05,
                                         e_begin=rank * El, e_end=(rank + 1) * El)
    page, T = 16, 40 + 3 * rank
    ep = EPContext(TPContext(device=dev), cfg.hidden_size, cfg.n_routed_experts, cfg.num_experts_per_tok,
                   max_tokens=64, fp8_dispatch=False, host_group=dist.new_group(backend="gloo"))
    kv = lambda: torch.zeros(8, 1, cfg.num_hidden_layers, 1, page, cfg.latent_dim, dtype=torch.bfloat16, device=dev)
    m_ep, m_full = DeepseekV3Model(cfg, mine, kv(), ep=ep), DeepseekV3Model(cfg, full, kv())
    tok = torch.randint(0, cfg.vocab_size, (T,), generator=torch.Generator().manual_seed(rank)).to(dev)
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    slots = torch.arange(T, dtype=torch.long, device=dev) + page
    bt = torch.tensor([[1, 2, 3, 0]], dtype=torch.int32, device=dev)
    i32 = lambda v: torch.tensor([v], dtype=torch.int32, device=dev)
    args = (tok, pos, slots, bt, i32(0), i32(T), i32(T), torch.arange(T, dtype=torch.int32, device=dev))
    m_ep.capture_decode_graphs([4])          # every rank, same sizes: the warm-up run exchanges rows
    got, want = m_ep.forward_tensors(*args), m_full.forward_tensors(*args)
    torch.cuda.synchronize()
    ops.check_device_error()
    err = float((got - want).abs().max() / want.abs().max())
    # one decode step on top of the prefill: the EP model replays its captured graph (one real sequence, three
    # dummies), the reference model runs eagerly
    nxt = want[-1].argmax().view(1)
    dargs = (nxt, i32(T), torch.tensor([T + page], dtype=torch.long, device=dev), bt, i32(0), i32(1), i32(T + 1), i32(0))
    got_d, want_d = m_ep.forward_tensors(*dargs), m_full.forward_tensors(*dargs)
    torch.cuda.synchronize()
    ops.check_device_error()
    assert m_ep.graph_replays == 1, m_ep.graph_replays
    err_d = float((got_d - want_d).abs().max() / want_d.abs().max())
    gathered = [None] * world
    dist.all_gather_object(gathered, {"rank": rank, "errs": [err, err_d], "dropped": 0})
    if rank == 0:
        print("EP_RESULT " + json.dumps(gathered), flush=True)
    dist.barrier()
    dist.destroy_process_group()


def deepseek_engine(rank, world, dev):
    """The engine under expert parallelism with data-parallel attention: every rank serves its OWN requests
    (different counts and lengths, so the ranks' schedulers take different numbers of steps; ranks that run out of
    work keep taking idle steps), against the same requests on an engine that holds all experts."""
    from modular_b200 import ops
    from modular_b200.entrypoints.llm import LLM
    from modular_b200.models.deepseek_v3 import DeepseekV3Config, DeepseekV3Weights
    from modular_b200.pipelines.context import SamplingParams

    cfg = DeepseekV3Config.tiny(hidden_size=512, moe_intermediate_size=256, intermediate_size=1024,
                                kv_lora_rank=128, q_lora_rank=256, num_attention_heads=8)
    El = cfg.n_routed_experts // world
    mine = DeepseekV3Weights.random_init(cfg, dev, torch.bfloat16, seed=11, std=0.05, e_begin=rank * El, e_end=(rank + 1) * El)
    full = DeepseekV3Weights.random_init(cfg, dev, torch.bfloat16, seed=11, std=0.05)
    kw = dict(device=str(dev), dtype=torch.bfloat16, max_length=128, max_batch_size=4, max_batch_input_tokens=64,
              page_size=16, num_kv_pages=64, enable_prefix_caching=False, graph_batch_sizes=[4])
    ep_llm = LLM(cfg, mine, ep_size=world, ep_rank=rank, **kw)
    g = torch.Generator().manual_seed(50 + rank)
    prompts = [torch.randint(0, cfg.vocab_size, (int(n),), generator=g).tolist() for n in (9 + 20 * rank, 70, 5)[: 2 + rank]]
    sp = SamplingParams(temperature=0.0, max_new_tokens=6 + 5 * rank, ignore_eos=True)
    got = [list(r.tokens) for r in ep_llm.generate(prompts, sp)]
    torch.cuda.synchronize()
    ops.check_device_error()
    ref_llm = LLM(cfg, full, **kw)
    want = [list(r.tokens) for r in ref_llm.generate(prompts, sp)]
    same_first = sum(a[0] == b[0] for a, b in zip(got, want))
    ok = all(len(a) == 6 + 5 * rank for a in got) and same_first >= len(got) - 1 and ep_llm.model.graph_replays > 0
    gathered = [None] * world
    dist.all_gather_object(gathered, {"rank": rank, "errs": [0.0 if ok else 1.0], "dropped": 0,
                                      "detail": [got, want, ep_llm.model.graph_replays]})
    if rank == 0:
        print("EP_RESULT " + json.dumps(gathered), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
