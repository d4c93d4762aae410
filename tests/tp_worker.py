"""Child process of test_tp_gpu.py: one rank of a tensor-parallel run (launched by torchrun)."""

import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
    from modular_b200 import ops
    from modular_b200.entrypoints.llm import LLM
    from modular_b200.models.llama3 import Llama3Config, Llama3Weights
    from modular_b200.pipelines.context import SamplingParams

    cfg = Llama3Config(hidden_size=1024, intermediate_size=2816, num_hidden_layers=3, num_attention_heads=8,
                       num_key_value_heads=4, head_dim=128, vocab_size=4096, max_position_embeddings=2048)
    dev = f"cuda:{os.environ['LOCAL_RANK']}"
    w = Llama3Weights.random_init(cfg, dev, torch.bfloat16, seed=0, std=0.05)
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, cfg.vocab_size, size=n).tolist() for n in (200, 64, 17, 130, 64)]
    sp = SamplingParams(temperature=0.0, max_new_tokens=10, ignore_eos=True)
    args = dict(device=dev, dtype=torch.bfloat16, max_length=512, max_batch_size=8, max_batch_input_tokens=256,
                page_size=64, num_kv_pages=80, enable_in_flight_batching=True, graph_batch_sizes=[4, 8])
    tp = LLM(cfg, w, tp_size=world, tp_rank=rank, **args)
    got = tp.generate(prompts, sp, max_concurrency=4)
    torch.cuda.synchronize()
    ops.check_device_error()
    out = {"rank": rank, "tokens": [r.tokens for r in got], "graph_replays": tp.pipeline.stats.graph_replays}
    if rank == 0:
        ref = LLM(cfg, w, **args).generate(prompts, sp, max_concurrency=4)
        out["ref"] = [r.tokens for r in ref]
    gathered = [None] * world
    dist.all_gather_object(gathered, out)
    if rank == 0:
        print("TP_RESULT " + json.dumps(gathered), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
