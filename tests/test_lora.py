"""LoRA: batched multi-adapter deltas equal the merged-weight model; manager slot policy."""

import pytest
import torch

from modular_b200.models.llama3 import Llama3Config, Llama3Model, Llama3Weights
from modular_b200.pipelines.lora import LoRAAdapter, LoRABatch, LoRAManager, token_slots_for


def _adapter(cfg, name, seed, rank=8, alpha=16.0, modules=("q_proj", "v_proj", "o_proj", "gate_proj", "down_proj"),
             dtype=torch.float32, device="cpu"):
    g = torch.Generator().manual_seed(seed)
    dims = {"q_proj": (cfg.hidden_size, cfg.q_dim), "k_proj": (cfg.hidden_size, cfg.kv_dim),
            "v_proj": (cfg.hidden_size, cfg.kv_dim), "o_proj": (cfg.q_dim, cfg.hidden_size),
            "gate_proj": (cfg.hidden_size, cfg.intermediate_size), "up_proj": (cfg.hidden_size, cfg.intermediate_size),
            "down_proj": (cfg.intermediate_size, cfg.hidden_size)}
    sd = {}
    for i in range(cfg.num_hidden_layers):
        for m in modules:
            kind = "mlp" if m in ("gate_proj", "up_proj", "down_proj") else "self_attn"
            din, dout = dims[m]
            sd[f"base_model.model.model.layers.{i}.{kind}.{m}.lora_A.weight"] = torch.randn(rank, din, generator=g) * 0.05
            sd[f"base_model.model.model.layers.{i}.{kind}.{m}.lora_B.weight"] = torch.randn(dout, rank, generator=g) * 0.05
    return LoRAAdapter.from_state_dict(name, sd, alpha=alpha, dtype=dtype, device=device), sd


def _merged(cfg, w, sd, scale):
    hf = {k: v.clone() for k, v in w.to_hf_state_dict(cfg).items()}
    for k in sd:
        if "lora_A" in k:
            base = k.replace("base_model.model.", "").replace(".lora_A.weight", ".weight")
            hf[base] = hf[base] + scale * (sd[k.replace("lora_A", "lora_B")] @ sd[k])
    from modular_b200.models.llama3 import adapt_hf_state_dict
    return Llama3Weights.from_state_dict(cfg, adapt_hf_state_dict(hf), "cpu", torch.float32)


def _run(model, tok_lists, lora=None):
    page = 16
    lens = [len(t) for t in tok_lists]
    i32 = lambda a: torch.tensor(a, dtype=torch.int32)
    bt = torch.tensor([[1 + 2 * i, 2 + 2 * i] for i in range(len(lens))], dtype=torch.int32)
    slots = torch.cat([torch.arange(n) + (1 + 2 * i) * page for i, n in enumerate(lens)])
    pos = torch.cat([torch.arange(n) for n in lens]).int()
    qs = torch.cumsum(i32(lens), 0, dtype=torch.int32) - i32(lens)
    rows = (qs + i32(lens) - 1).int()
    toks = torch.tensor([t for tl in tok_lists for t in tl])
    return model.forward_tensors(toks, pos, slots, bt, qs, i32(lens), i32(lens), rows, lora=lora)


def test_mixed_adapter_batch_matches_merged_weights():
    cfg = Llama3Config.tiny()
    w = Llama3Weights.random_init(cfg, "cpu", torch.float32, seed=0, std=0.05)
    kv = lambda: torch.zeros(8, 2, cfg.num_hidden_layers, cfg.num_key_value_heads, 16, cfg.head_dim)
    a1, sd1 = _adapter(cfg, "a1", 1)
    a2, sd2 = _adapter(cfg, "a2", 2, rank=16, alpha=8.0, modules=("k_proj", "up_proj"))
    mgr = LoRAManager(max_loras=4)
    mgr.load(a1), mgr.load(a2)
    seqs = [[5, 6, 7, 8], [9, 10, 11], [12, 13, 14, 15, 16]]
    names = ["a1", None, "a2"]
    batch = LoRABatch(mgr, token_slots_for(mgr, [len(s) for s in seqs], names, "cpu"))
    got = _run(Llama3Model(cfg, w, kv()), seqs, batch)
    base = Llama3Model(cfg, w, kv())
    m1 = Llama3Model(cfg, _merged(cfg, w, sd1, a1.scale), kv())
    m2 = Llama3Model(cfg, _merged(cfg, w, sd2, a2.scale), kv())
    want = torch.stack([_run(m1, [seqs[0]])[0], _run(base, [seqs[1]])[0], _run(m2, [seqs[2]])[0]])
    assert torch.allclose(got, want, atol=2e-4), (got - want).abs().max()
    assert not torch.allclose(got[0], _run(base, [seqs[0]])[0], atol=1e-3)      # the adapter does change the output


def test_manager_slots_lru_and_pinning():
    cfg = Llama3Config.tiny()
    mgr = LoRAManager(max_loras=2)
    ads = [_adapter(cfg, f"x{i}", i, modules=("q_proj",))[0] for i in range(3)]
    s0, s1 = mgr.load(ads[0]), mgr.load(ads[1])
    assert {s0, s1} == {0, 1} and mgr.slot_of(None) == -1
    mgr.slot_of("x0")                  # x0 becomes most recently used
    mgr.pin("x0")
    s2 = mgr.load(ads[2])              # evicts x1
    assert s2 == s1 and mgr.names() == ["x0", "x2"]
    with pytest.raises(KeyError):
        mgr.slot_of("x1")
    with pytest.raises(RuntimeError):
        mgr.unload("x0")
    mgr.unpin("x0")
    assert mgr.unload("x0") and not mgr.unload("x0")
    bad, _ = _adapter(cfg, "bad", 9, rank=12, modules=("q_proj",))
    with pytest.raises(ValueError):
        mgr.load(bad)


@pytest.mark.gpu
def test_grouped_gemm_lora_path_matches_reference_on_gpu():
    cfg = Llama3Config.tiny()
    dev = torch.device("cuda")
    mgr = LoRAManager()
    a1, _ = _adapter(cfg, "a1", 1, rank=16, modules=("q_proj",), dtype=torch.bfloat16, device=dev)
    a2, _ = _adapter(cfg, "a2", 2, rank=16, modules=("q_proj",), dtype=torch.bfloat16, device=dev)
    mgr.load(a1), mgr.load(a2)
    slots = torch.tensor([0] * 70 + [-1] * 5 + [1] * 33 + [0] * 3, dtype=torch.int32, device=dev)
    x = (torch.randn(slots.numel(), cfg.hidden_size, generator=torch.Generator().manual_seed(0)) * 0.5).to(torch.bfloat16).to(dev)
    got = LoRABatch(mgr, slots).delta(0, "q_proj", x).float()
    want = torch.zeros_like(got)
    for s, a in ((0, a1), (1, a2)):
        A, B = a.weights[(0, "q_proj")]
        sel = slots == s
        want[sel] = (x[sel].float() @ A.float().t()) @ B.float().t() * a.scale
    assert (got - want).abs().max() < 0.03 * want.abs().max() + 1e-3
    assert got[70:75].abs().sum() == 0


def test_engine_applies_adapter_per_request():
    from modular_b200.entrypoints.llm import LLM
    from modular_b200.pipelines.context import SamplingParams

    cfg = Llama3Config.tiny()
    w = Llama3Weights.random_init(cfg, "cpu", torch.float32, seed=0, std=0.05)
    a1, sd1 = _adapter(cfg, "a1", 1, alpha=64.0)
    mk = lambda weights: LLM(cfg, weights, device="cpu", dtype=torch.float32, max_length=128, max_batch_size=4,
                             max_batch_input_tokens=64, page_size=16, num_kv_pages=32)
    sp = SamplingParams(temperature=0.0, max_new_tokens=8, ignore_eos=True)
    prompt = [5, 6, 7, 8, 9]
    llm = mk(w)
    llm.load_lora("a1", sd1, alpha=64.0)
    r_lora = llm.add_request(prompt, sp, lora_name="a1")
    r_base = llm.add_request(prompt, sp)
    done = {}
    while llm.has_unfinished():
        for rec in llm.step():
            done[rec.request_id] = rec.tokens
    merged = mk(_merged(cfg, w, sd1, a1.scale)).generate([prompt], sp)[0].tokens
    plain = mk(w).generate([prompt], sp)[0].tokens
    assert done[r_lora] == merged and done[r_base] == plain and merged != plain
    with pytest.raises(KeyError):
        llm.add_request(prompt, sp, lora_name="nope")


def test_prefix_cache_never_crosses_adapters():
    """A prompt of several pages run on the base model and then on an adapter (and the other way round, and
    after the adapter was loaded again under the same name) must not reuse the other run's KV pages: adapters
    change the k/v projections, so the page hashes carry the adapter identity."""
    from modular_b200.entrypoints.llm import LLM
    from modular_b200.pipelines.context import SamplingParams

    cfg = Llama3Config.tiny()
    w = Llama3Weights.random_init(cfg, "cpu", torch.float32, seed=0, std=0.05)
    a1, sd1 = _adapter(cfg, "a1", 1, alpha=64.0)
    a2, sd2 = _adapter(cfg, "a1", 2, alpha=64.0)       # different weights, same name
    mk = lambda weights: LLM(cfg, weights, device="cpu", dtype=torch.float32, max_length=128, max_batch_size=4,
                             max_batch_input_tokens=64, page_size=16, num_kv_pages=64)
    sp = SamplingParams(temperature=0.0, max_new_tokens=6, ignore_eos=True)
    prompt = [int(t) for t in torch.randint(0, cfg.vocab_size, (40,), generator=torch.Generator().manual_seed(1))]
    merged1 = mk(_merged(cfg, w, sd1, a1.scale)).generate([prompt], sp)[0].tokens
    merged2 = mk(_merged(cfg, w, sd2, a2.scale)).generate([prompt], sp)[0].tokens
    plain = mk(w).generate([prompt], sp)[0].tokens

    def run(llm, lora_name=None):
        rid = llm.add_request(prompt, sp, lora_name=lora_name)
        out = None
        while llm.has_unfinished():
            for rec in llm.step():
                if rec.request_id == rid:
                    out = rec.tokens
        return out

    llm = mk(w)
    llm.load_lora("a1", sd1, alpha=64.0)
    assert run(llm) == plain                       # base first: fills the prefix cache
    assert run(llm, "a1") == merged1               # adapter after base
    assert run(llm) == plain                       # base after adapter
    hits_before = llm.kv.stats.hit_tokens if hasattr(llm.kv, "stats") else None
    assert run(llm, "a1") == merged1               # same adapter again may hit its own pages
    llm.unload_lora("a1")
    llm.load_lora("a1", sd2, alpha=64.0)           # re-loaded under the same name with other weights
    assert run(llm, "a1") == merged2
    del hits_before
