"""State-space layers: chunked prefill + decode with carried state equals the one-shot result (CPU), and the
CUDA kernels match the fp32 PyTorch forms (GPU)."""

import pytest
import torch

from modular_b200.nn import state_space as ss


def _cu(lens, device="cpu"):
    return torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=device)


def test_mamba_mixer_chunked_matches_one_shot():
    torch.manual_seed(0)
    m = ss.MambaMixer(hidden=32, d_inner=64, d_state=16, d_conv=4)
    lens = [7, 12]
    h = torch.randn(sum(lens), 32)
    full = m(h, _cu(lens))
    # the same two sequences in two chunks each, then the rest token by token
    state = m.alloc_state(4)
    idx = torch.tensor([2, 0], dtype=torch.int32)
    seqs = [h[:7], h[7:]]
    first = [3, 5]
    out = [[], []]
    c1 = torch.cat([seqs[0][:3], seqs[1][:5]])
    y = m(c1, _cu(first), state, idx, torch.tensor([0, 0], dtype=torch.int32))
    out[0].append(y[:3]); out[1].append(y[3:])
    pos = list(first)
    while any(p < l for p, l in zip(pos, lens)):
        live = [i for i in range(2) if pos[i] < lens[i]]
        x = torch.cat([seqs[i][pos[i] : pos[i] + 1] for i in live])
        y = m(x, _cu([1] * len(live)), state, idx[live], torch.ones(len(live), dtype=torch.int32))
        for j, i in enumerate(live):
            out[i].append(y[j : j + 1]); pos[i] += 1
    got = torch.cat([torch.cat(out[0]), torch.cat(out[1])])
    assert torch.allclose(got, full, atol=1e-4, rtol=1e-4)


def test_mamba2_mixer_chunked_matches_one_shot():
    torch.manual_seed(1)
    m = ss.Mamba2Mixer(hidden=32, n_heads=4, head_dim=8, d_state=16, n_groups=2, d_conv=4)
    lens = [9, 4]
    h = torch.randn(sum(lens), 32)
    full = m(h, _cu(lens))
    state = m.alloc_state(2)
    idx = torch.tensor([1, 0], dtype=torch.int32)
    a = m(torch.cat([h[:5], h[9:11]]), _cu([5, 2]), state, idx, torch.zeros(2, dtype=torch.int32))
    b = m(torch.cat([h[5:9], h[11:13]]), _cu([4, 2]), state, idx, torch.ones(2, dtype=torch.int32))
    got = torch.cat([a[:5], b[:4], a[5:], b[4:]])
    assert torch.allclose(got, full, atol=1e-4, rtol=1e-4)


def _rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-6)).item()


@pytest.mark.gpu
@pytest.mark.parametrize("W", [2, 4])
def test_causal_conv1d_kernel(W):
    torch.manual_seed(2)
    dev = "cuda"
    lens = [1, 33, 7, 128]
    D = 200
    x = torch.randn(sum(lens), D, device=dev, dtype=torch.bfloat16)
    w = (torch.randn(D, W, device=dev) * 0.5).to(torch.bfloat16)
    b = torch.randn(D, device=dev, dtype=torch.bfloat16)
    idx = torch.tensor([3, -1, 0, 1], dtype=torch.int32, device=dev)
    init = torch.tensor([1, 0, 0, 1], dtype=torch.int32, device=dev)
    st = torch.randn(4, D, W - 1, device=dev)
    st_ref = st.clone()
    y = ss.causal_conv1d_varlen(x, w, b, _cu(lens, dev), st, idx, init, True)
    y_ref = ss.causal_conv1d_reference(x, w, b, _cu(lens), st_ref, idx.cpu(), init.cpu(), True)
    assert _rel(y, y_ref) < 1e-2
    assert torch.allclose(st, st_ref, atol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("N", [16, 32])
def test_selective_scan_kernel(N):
    torch.manual_seed(3)
    dev = "cuda"
    lens = [5, 1, 64]
    T, D = sum(lens), 192
    u = torch.randn(T, D, device=dev, dtype=torch.bfloat16)
    delta = (torch.randn(T, D, device=dev) * 0.5).to(torch.bfloat16)
    A = -torch.rand(D, N, device=dev) - 0.1
    B = torch.randn(T, N, device=dev, dtype=torch.bfloat16)
    C = torch.randn(T, N, device=dev, dtype=torch.bfloat16)
    Dk = torch.randn(D, device=dev)
    z = torch.randn(T, D, device=dev, dtype=torch.bfloat16)
    bias = torch.randn(D, device=dev) * 0.1
    idx = torch.tensor([1, 0, -1], dtype=torch.int32, device=dev)
    init = torch.tensor([0, 1, 0], dtype=torch.int32, device=dev)
    st = torch.randn(2, D, N, device=dev)
    st_ref = st.clone()
    y = ss.selective_scan_varlen(u, delta, A, B, C, Dk, z, bias, _cu(lens, dev), st, idx, init, True)
    y_ref = ss.selective_scan_reference(u, delta, A, B, C, Dk, z, bias, _cu(lens), st_ref, idx.cpu(), init.cpu(), True)
    assert _rel(y, y_ref) < 1e-2
    assert _rel(st, st_ref) < 1e-3


@pytest.mark.gpu
@pytest.mark.parametrize("H,P,N,G", [(4, 64, 128, 1), (6, 32, 64, 2), (2, 128, 16, 2)])
def test_ssd_scan_kernel(H, P, N, G):
    torch.manual_seed(4)
    dev = "cuda"
    lens = [3, 40, 1]
    T = sum(lens)
    x = torch.randn(T, H, P, device=dev, dtype=torch.bfloat16)
    dt = (torch.randn(T, H, device=dev) * 0.5).to(torch.bfloat16)
    A = -torch.rand(H, device=dev) - 0.1
    B = (torch.randn(T, G, N, device=dev) * 0.3).to(torch.bfloat16)
    C = (torch.randn(T, G, N, device=dev) * 0.3).to(torch.bfloat16)
    Dk = torch.randn(H, device=dev)
    bias = torch.randn(H, device=dev) * 0.1
    idx = torch.tensor([0, 2, 1], dtype=torch.int32, device=dev)
    init = torch.tensor([1, 0, 1], dtype=torch.int32, device=dev)
    st = torch.randn(3, H, P, N, device=dev) * 0.2
    st_ref = st.clone()
    y = ss.ssd_scan_varlen(x, dt, A, B, C, Dk, bias, _cu(lens, dev), st, idx, init, True)
    y_ref = ss.ssd_scan_reference(x, dt, A, B, C, Dk, bias, _cu(lens), st_ref, idx.cpu(), init.cpu(), True)
    assert _rel(y, y_ref) < 1e-2
    assert _rel(st, st_ref) < 1e-3
