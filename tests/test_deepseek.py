"""DeepSeek-V3: MLA (absorbed form) + MoE model against a dense fp32 oracle, and the MLA kernels.

Oracle: ``hf_reference_forward`` recomputes the model the textbook way (per-head K/V decompressed
from the latent, softmax attention, per-token expert loop) from an HF-named state dict.
"""

import pytest
import torch

from modular_b200 import ops
from modular_b200.models.deepseek_v3 import (DeepseekV3Config, DeepseekV3Model, DeepseekV3Weights, Fp8Weight,
                                             hf_reference_forward)

i32 = lambda *a, dev="cpu": torch.tensor(a, dtype=torch.int32, device=dev)


def _single_seq_inputs(T, page, dev="cpu"):
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    slots = torch.arange(T, dtype=torch.long, device=dev) + page          # pages 1, 2, ...
    n_pages = (T + page - 1) // page
    bt = torch.zeros(1, n_pages + 1, dtype=torch.int32, device=dev)
    bt[0, :n_pages] = torch.arange(1, n_pages + 1)
    return pos, slots, bt


def _new_kv(cfg, pages, page, dev="cpu", dtype=torch.float32):
    return torch.zeros(pages, 1, cfg.num_hidden_layers, 1, page, cfg.latent_dim, dtype=dtype, device=dev)


def test_model_matches_dense_oracle_and_roundtrips_state_dict():
    cfg = DeepseekV3Config.tiny()
    w = DeepseekV3Weights.random_init(cfg, "cpu", torch.float32, seed=1, std=0.05)
    sd = w.to_hf_state_dict()
    T, page = 37, 16
    tok = torch.randint(0, cfg.vocab_size, (T,), generator=torch.Generator().manual_seed(0))
    pos, slots, bt = _single_seq_inputs(T, page)
    m = DeepseekV3Model(cfg, w, _new_kv(cfg, 8, page))
    logits = m.forward_tensors(tok, pos, slots, bt, i32(0), i32(T), i32(T), torch.arange(T, dtype=torch.int32))
    ref = hf_reference_forward(cfg, sd, tok)
    assert (logits - ref).abs().max() < 1e-4
    w2 = DeepseekV3Weights.from_state_dict(cfg, sd, "cpu", torch.float32)
    m2 = DeepseekV3Model(cfg, w2, _new_kv(cfg, 8, page))
    l2 = m2.forward_tensors(tok, pos, slots, bt, i32(0), i32(T), i32(T), torch.arange(T, dtype=torch.int32))
    assert torch.equal(l2, logits)


def test_chunked_prefill_then_decode_matches_full_prefill():
    cfg = DeepseekV3Config.tiny(q_lora_rank=None)
    w = DeepseekV3Weights.random_init(cfg, "cpu", torch.float32, seed=2, std=0.05)
    T, page = 29, 8
    tok = torch.randint(0, cfg.vocab_size, (T,), generator=torch.Generator().manual_seed(1))
    pos, slots, bt = _single_seq_inputs(T, page)
    ref = hf_reference_forward(cfg, w.to_hf_state_dict(), tok)
    m = DeepseekV3Model(cfg, w, _new_kv(cfg, 8, page))
    outs = [m.forward_tensors(tok[:11], pos[:11], slots[:11], bt, i32(0), i32(11), i32(11), i32(10)),
            m.forward_tensors(tok[11:20], pos[11:20], slots[11:20], bt, i32(0), i32(9), i32(20), i32(8))]
    for t in range(20, T):
        outs.append(m.forward_tensors(tok[t:t + 1], pos[t:t + 1], slots[t:t + 1], bt, i32(0), i32(1), i32(t + 1), i32(0)))
    got = torch.cat(outs)
    want = torch.cat([ref[10:11], ref[19:20], ref[20:]])
    assert (got - want).abs().max() < 1e-4


def test_fp8_checkpoint_tensors_are_dequantised_consistently():
    cfg = DeepseekV3Config.tiny()
    w = DeepseekV3Weights.random_init(cfg, "cpu", torch.float32, seed=3, std=0.05)
    sd = w.to_hf_state_dict()
    # quantise the attention output projections the way fp8 checkpoints store them
    q8 = {}
    for k, v in sd.items():
        if k.endswith("o_proj.weight"):
            q, s = ops.reference.quant_fp8_weight_block128(v.float())
            q8[k] = q
            q8[k + "_scale_inv"] = s
        else:
            q8[k] = v
    w8 = DeepseekV3Weights.from_state_dict(cfg, q8, "cpu", torch.float32)
    assert isinstance(w8.layers[0].wo, Fp8Weight)
    assert (w8.layers[0].wo.dequant() - sd["model.layers.0.self_attn.o_proj.weight"]).abs().max() < 0.02
    T, page = 12, 16
    tok = torch.randint(0, cfg.vocab_size, (T,), generator=torch.Generator().manual_seed(2))
    pos, slots, bt = _single_seq_inputs(T, page)
    m = DeepseekV3Model(cfg, w8, _new_kv(cfg, 4, page))
    logits = m.forward_tensors(tok, pos, slots, bt, i32(0), i32(T), i32(T), i32(T - 1))
    # the oracle runs on the dequantised values, so only the code path differs, not the numbers
    sd_dq = dict(sd)
    for i in range(cfg.num_hidden_layers):
        k = f"model.layers.{i}.self_attn.o_proj.weight"
        sd_dq[k] = ops.reference.dequant_fp8_weight_block128(q8[k], q8[k + "_scale_inv"])
    ref = hf_reference_forward(cfg, sd_dq, tok)[-1:]
    assert (logits - ref).abs().max() < 1e-3


# ------------------------------------------------------------------------------------ GPU
def _ragged_case(dev, h, R, page, gen):
    """Two decode sequences, one chunked prefill with cached prefix, one fresh prefill."""
    q_lens, kv_lens = [1, 1, 37, 70], [130, 1, 90, 70]
    B, T = len(q_lens), sum(q_lens)
    n_pages_seq = [(k + page - 1) // page for k in kv_lens]
    total_pages = sum(n_pages_seq) + 1
    cache_full = torch.zeros(total_pages, 3, page, R + 64, dtype=torch.bfloat16, device=dev)   # 3 "layers"
    cache = cache_full[:, 1]                                                                      # strided view
    bt = torch.zeros(B, max(n_pages_seq), dtype=torch.int32, device=dev)
    nxt = 1
    for b, n in enumerate(n_pages_seq):
        bt[b, :n] = torch.arange(nxt, nxt + n)
        nxt += n
    cache[1:] = (torch.randn(total_pages - 1, page, R + 64, generator=gen) * 0.5).to(torch.bfloat16).to(dev)
    q_lat = (torch.randn(T, h, R, generator=gen) * 0.3).to(torch.bfloat16).to(dev)
    q_rope = (torch.randn(T, h, 64, generator=gen) * 0.3).to(torch.bfloat16).to(dev)
    q_start = torch.tensor([0, 1, 2, 39], dtype=torch.int32, device=dev)
    return (q_lat, q_rope, cache, bt, q_start, torch.tensor(q_lens, dtype=torch.int32, device=dev),
            torch.tensor(kv_lens, dtype=torch.int32, device=dev))


@pytest.mark.gpu
@pytest.mark.parametrize("h,R,page", [(128, 512, 64), (16, 512, 128), (4, 128, 16), (12, 256, 32)])
def test_mla_kernel_matches_reference(h, R, page):
    dev = torch.device("cuda")
    args = _ragged_case(dev, h, R, page, torch.Generator().manual_seed(h + R))
    scale = 0.11
    got = ops.mla_paged_attention(*args, scale)
    want = ops.reference.mla_paged_attention(*[a.float() if a.is_floating_point() else a for a in args], scale)
    err = (got.float() - want).abs().max() / want.abs().max()
    assert err < 2e-2, err
    ops.check_device_error()


@pytest.mark.gpu
def test_mla_kv_store_and_batched_linear():
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(5)
    T, R, page = 50, 512, 16
    cache_full = torch.zeros(6, 2, page, R + 64, dtype=torch.bfloat16, device=dev)
    cache, want = cache_full[:, 1], torch.zeros(6, page, R + 64, dtype=torch.bfloat16, device=dev)
    c_kv = torch.randn(T, R, generator=g).to(torch.bfloat16).to(dev)
    k_rope = torch.randn(T, 64, generator=g).to(torch.bfloat16).to(dev)
    slots = (torch.randperm(5 * page, generator=g)[:T] + page).to(dev)
    slots[3] = -1
    ops.mla_kv_store(c_kv, k_rope, slots, cache)
    ops.reference.mla_kv_store(c_kv, k_rope, slots, want)
    assert torch.equal(cache, want) and cache_full[:, 0].abs().sum() == 0
    x = (torch.randn(8, 33, 128, generator=g)).to(torch.bfloat16).to(dev)
    w = (torch.randn(8, 512, 128, generator=g) * 0.1).to(torch.bfloat16).to(dev)
    y = ops.batched_linear(x, w)
    ref = ops.reference.batched_linear(x.float(), w.float())
    assert (y.float() - ref).abs().max() / ref.abs().max() < 2e-2
    ops.check_device_error()


@pytest.mark.gpu
def test_model_on_gpu_matches_cpu_oracle():
    cfg = DeepseekV3Config.tiny(hidden_size=512, moe_intermediate_size=256, intermediate_size=1024,
                                kv_lora_rank=128, q_lora_rank=256, num_attention_heads=8)
    w32 = DeepseekV3Weights.random_init(cfg, "cpu", torch.float32, seed=4, std=0.05)
    sd = w32.to_hf_state_dict()
    dev = torch.device("cuda")
    w = DeepseekV3Weights.from_state_dict(cfg, sd, dev, torch.bfloat16)
    T, page = 45, 16
    tok = torch.randint(0, cfg.vocab_size, (T,), generator=torch.Generator().manual_seed(3))
    pos, slots, bt = _single_seq_inputs(T, page, dev)
    m = DeepseekV3Model(cfg, w, _new_kv(cfg, 8, page, dev, torch.bfloat16))
    d = lambda *a: i32(*a, dev=dev)
    got = torch.cat([m.forward_tensors(tok[:40].to(dev), pos[:40], slots[:40], bt, d(0), d(40), d(40), d(39))] +
                    [m.forward_tensors(tok[t:t + 1].to(dev), pos[t:t + 1], slots[t:t + 1], bt, d(0), d(1), d(t + 1), d(0))
                     for t in range(40, T)])
    ref = hf_reference_forward(cfg, {k: v.to(torch.bfloat16) for k, v in sd.items()}, tok)[39:]
    err = (got.cpu() - ref).abs().max() / ref.abs().max()
    assert err < 0.06, err
    ops.check_device_error()


def _engine_tokens(device, dtype, batch, budget, prompts, **kw):
    from modular_b200.entrypoints.llm import LLM
    from modular_b200.pipelines.context import SamplingParams

    cfg = DeepseekV3Config.tiny(**kw)
    llm = LLM(cfg, device=device, dtype=dtype, max_length=256, max_batch_size=batch, max_batch_input_tokens=budget,
              page_size=16, num_kv_pages=96, seed=5)
    sp = SamplingParams(temperature=0.0, max_new_tokens=6, ignore_eos=True)
    return [r.tokens for r in llm.generate(prompts, sp)]


def test_engine_serves_deepseek_with_chunked_prefill_on_cpu():
    import numpy as np
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, 512, size=n).tolist() for n in (30, 7, 70)]
    batched = _engine_tokens("cpu", torch.float32, 4, 64, prompts)       # 70-token prompt is chunked
    solo = [_engine_tokens("cpu", torch.float32, 1, 128, [p])[0] for p in prompts]
    assert batched == solo


@pytest.mark.gpu
def test_engine_serves_deepseek_on_gpu():
    import numpy as np
    rng = np.random.default_rng(1)
    prompts = [rng.integers(0, 512, size=n).tolist() for n in (30, 7, 70, 33)]
    kw = dict(hidden_size=512, moe_intermediate_size=256, intermediate_size=1024, kv_lora_rank=128,
              q_lora_rank=256, num_attention_heads=8)
    got = _engine_tokens("cuda", torch.bfloat16, 4, 64, prompts, **kw)
    assert all(len(t) == 6 for t in got)
    solo = [_engine_tokens("cuda", torch.bfloat16, 1, 128, [p], **kw)[0] for p in prompts]
    # bf16 batches of different shapes may flip a late near-tie; the first tokens must agree
    assert all(a[:2] == b[:2] for a, b in zip(got, solo))
    ops.check_device_error()


@pytest.mark.gpu
@pytest.mark.parametrize("h,page,kv_lens", [(128, 64, [1, 64, 65, 130, 700]), (256, 128, [1152, 33, 1280]),
                                            (128, 128, [3000]), (128, 64, [1100] * 32), (128, 128, [257, 4000, 64, 1]),
                                            (128, 64, [5000, 5000])])
def test_mla_decode_tcgen05_matches_reference(h, page, kv_lens):
    """Decode step (one query token per sequence) on the tcgen05 kernel, against the fp32 reference and the
    mma.sync kernel; queries scaled up so that the lazily rescaled accumulator path is exercised."""
    dev = torch.device("cuda")
    gen = torch.Generator().manual_seed(h + page)
    R, B = 512, len(kv_lens)
    n_pages_seq = [(k + page - 1) // page for k in kv_lens]
    total_pages = sum(n_pages_seq) + 1
    cache_full = torch.zeros(total_pages, 2, page, R + 64, dtype=torch.bfloat16, device=dev)
    cache = cache_full[:, 1]
    order = torch.randperm(total_pages - 1, generator=gen) + 1           # pages in random order
    bt = torch.zeros(B, max(n_pages_seq), dtype=torch.int32, device=dev)
    nxt = 0
    for b, n in enumerate(n_pages_seq):
        bt[b, :n] = order[nxt:nxt + n].to(torch.int32)
        nxt += n
    cache[1:] = (torch.randn(total_pages - 1, page, R + 64, generator=gen) * 0.5).to(torch.bfloat16).to(dev)
    q_lat = (torch.randn(B, h, R, generator=gen) * 1.5).to(torch.bfloat16).to(dev)
    q_rope = (torch.randn(B, h, 64, generator=gen) * 1.5).to(torch.bfloat16).to(dev)
    q_start = torch.arange(B, dtype=torch.int32, device=dev)
    q_len = torch.ones(B, dtype=torch.int32, device=dev)
    kv_len = torch.tensor(kv_lens, dtype=torch.int32, device=dev)
    args = (q_lat, q_rope, cache, bt, q_start, q_len, kv_len)
    scale = 0.07
    got = ops.mla_paged_attention(*args, scale)                          # T == B: tcgen05 kernel (KV split when few)
    torch.cuda.synchronize()
    ops.check_device_error()
    from modular_b200._native import lib
    lib().set_mla_split(0)
    try:
        unsplit = ops.mla_paged_attention(*args, scale)                  # one CTA pair per sequence
    finally:
        lib().set_mla_split(1)
    again = ops.mla_paged_attention(*args, scale)                        # counters were left at zero
    assert torch.equal(again, got)
    old = ops.mla_paged_attention(*args, scale, decode_only=False)       # mma.sync kernel
    want = ops.reference.mla_paged_attention(*[a.float() if a.is_floating_point() else a for a in args], scale)
    assert (old.float() - want).abs().max() / want.abs().max() < 2e-2
    assert (unsplit.float() - want).abs().max() / want.abs().max() < 2e-2
    err = (got.float() - want).abs().max() / want.abs().max()
    assert err < 2e-2, err
