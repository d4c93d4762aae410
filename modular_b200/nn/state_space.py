"""State-space layers for ragged batches: causal depthwise conv1d, the Mamba-1 selective scan and the
Mamba-2 SSD recurrence, plus ``MambaMixer`` / ``Mamba2Mixer`` blocks built from them.

Every function takes token-major tensors for a packed batch (``cu_seqlens`` int32 ``[n_seqs + 1]``) and
optional recurrent state: ``state`` tensors are indexed by ``state_idx[s]`` (one slot per live request,
-1 = stateless), read when ``has_init[s]`` is set and written back, so a chunked prefill followed by
single-token decode steps reproduces the one-shot result. On CUDA with bf16 inputs the kernels of
``csrc/kernels/state_space.cu`` run; otherwise the PyTorch fp32 forms below, which are also the test
oracles.

Reference: max/python/max/nn/state_space/ (varlen causal conv1d, selective scan and gated-delta wrappers)
over max/kernels/src/state_space/ (causal_conv1d.mojo, selective_scan.mojo, the Mamba-2 SSD kernels).
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from .._native import lib as _lib

__all__ = ["causal_conv1d_varlen", "selective_scan_varlen", "ssd_scan_varlen", "MambaMixer", "Mamba2Mixer",
           "causal_conv1d_reference", "selective_scan_reference", "ssd_scan_reference"]


def _opt_i32(t, device):
    return None if t is None else t.to(device=device, dtype=torch.int32).contiguous()


# ------------------------------------------------------------------------------------ references (fp32)
def causal_conv1d_reference(x, w, bias, cu_seqlens, conv_state=None, state_idx=None, has_init=None, silu=True):
    T, D = x.shape
    W = w.shape[1]
    y = torch.empty(T, D, dtype=torch.float32, device=x.device)
    xf, wf = x.float(), w.float()
    cs = cu_seqlens.tolist()
    for s in range(len(cs) - 1):
        t0, t1 = cs[s], cs[s + 1]
        slot = int(state_idx[s]) if state_idx is not None else -1
        hist = torch.zeros(W - 1, D, dtype=torch.float32, device=x.device)
        if slot >= 0 and conv_state is not None and has_init is not None and int(has_init[s]):
            hist = conv_state[slot].float().t().clone()            # [W-1, D]
        seq = torch.cat([hist, xf[t0:t1]], 0)                      # [W-1+L, D]
        out = torch.zeros(t1 - t0, D, dtype=torch.float32, device=x.device)
        for k in range(W):
            out += seq[k : k + (t1 - t0)] * wf[:, k]
        if bias is not None:
            out += bias.float()
        y[t0:t1] = F.silu(out) if silu else out
        if slot >= 0 and conv_state is not None:
            conv_state[slot] = seq[seq.shape[0] - (W - 1):].t().to(conv_state.dtype)
    return y.to(x.dtype)


def selective_scan_reference(u, delta, A, B, C, D=None, z=None, dt_bias=None, cu_seqlens=None, ssm_state=None,
                             state_idx=None, has_init=None, dt_softplus=True):
    T, Dm = u.shape
    N = A.shape[1]
    y = torch.empty(T, Dm, dtype=torch.float32, device=u.device)
    uf, df, Bf, Cf = u.float(), delta.float(), B.float(), C.float()
    cs = cu_seqlens.tolist()
    for s in range(len(cs) - 1):
        slot = int(state_idx[s]) if state_idx is not None else -1
        h = torch.zeros(Dm, N, dtype=torch.float32, device=u.device)
        if slot >= 0 and ssm_state is not None and has_init is not None and int(has_init[s]):
            h = ssm_state[slot].float().clone()
        for t in range(cs[s], cs[s + 1]):
            dt = df[t] + (dt_bias.float() if dt_bias is not None else 0.0)
            if dt_softplus:
                dt = F.softplus(dt)
            h = torch.exp(dt[:, None] * A.float()) * h + (dt * uf[t])[:, None] * Bf[t][None, :]
            out = (h * Cf[t][None, :]).sum(-1)
            if D is not None:
                out = out + D.float() * uf[t]
            if z is not None:
                out = out * F.silu(z[t].float())
            y[t] = out
        if slot >= 0 and ssm_state is not None:
            ssm_state[slot] = h.to(ssm_state.dtype)
    return y.to(u.dtype)


def ssd_scan_reference(x, dt, A, B, C, D=None, dt_bias=None, cu_seqlens=None, ssm_state=None, state_idx=None,
                       has_init=None, dt_softplus=True):
    T, H, P = x.shape
    G, N = B.shape[1], B.shape[2]
    rep = H // G
    y = torch.empty(T, H, P, dtype=torch.float32, device=x.device)
    xf, dtf, Bf, Cf = x.float(), dt.float(), B.float(), C.float()
    cs = cu_seqlens.tolist()
    for s in range(len(cs) - 1):
        slot = int(state_idx[s]) if state_idx is not None else -1
        S = torch.zeros(H, P, N, dtype=torch.float32, device=x.device)
        if slot >= 0 and ssm_state is not None and has_init is not None and int(has_init[s]):
            S = ssm_state[slot].float().clone()
        for t in range(cs[s], cs[s + 1]):
            d = dtf[t] + (dt_bias.float() if dt_bias is not None else 0.0)          # [H]
            if dt_softplus:
                d = F.softplus(d)
            Bt = Bf[t].repeat_interleave(rep, 0)                                      # [H, N]
            Ct = Cf[t].repeat_interleave(rep, 0)
            S = torch.exp(d * A.float())[:, None, None] * S + (d[:, None] * xf[t])[:, :, None] * Bt[:, None, :]
            out = (S * Ct[:, None, :]).sum(-1)
            if D is not None:
                out = out + D.float()[:, None] * xf[t]
            y[t] = out
        if slot >= 0 and ssm_state is not None:
            ssm_state[slot] = S.to(ssm_state.dtype)
    return y.to(x.dtype)


# ------------------------------------------------------------------------------------ dispatching ops
def _native_ok(t):
    return t.is_cuda and t.dtype == torch.bfloat16


def causal_conv1d_varlen(x, w, bias, cu_seqlens, conv_state=None, state_idx=None, has_init=None, silu=True):
    """x [T, D]; w [D, W]; conv_state fp32 [slots, D, W-1] holds the last W-1 inputs of each live sequence."""
    if not _native_ok(x) or w.shape[1] not in (2, 3, 4, 8):
        return causal_conv1d_reference(x, w, bias, cu_seqlens, conv_state, state_idx, has_init, silu)
    y = torch.empty_like(x)
    _lib().causal_conv1d_varlen(x, w.contiguous(), bias, y, conv_state, _opt_i32(cu_seqlens, x.device),
                                _opt_i32(state_idx, x.device), _opt_i32(has_init, x.device), silu)
    return y


def selective_scan_varlen(u, delta, A, B, C, D=None, z=None, dt_bias=None, cu_seqlens=None, ssm_state=None,
                          state_idx=None, has_init=None, dt_softplus=True):
    """u, delta, z [T, D]; A fp32 [D, N]; B, C [T, N]; ssm_state fp32 [slots, D, N]."""
    if not _native_ok(u) or A.shape[1] not in (8, 16, 32):
        return selective_scan_reference(u, delta, A, B, C, D, z, dt_bias, cu_seqlens, ssm_state, state_idx,
                                        has_init, dt_softplus)
    y = torch.empty_like(u)
    _lib().selective_scan_varlen(u.contiguous(), delta.contiguous(), A.float().contiguous(), B.contiguous(),
                                 C.contiguous(), None if D is None else D.float().contiguous(),
                                 None if z is None else z.contiguous(),
                                 None if dt_bias is None else dt_bias.float().contiguous(), y, ssm_state,
                                 _opt_i32(cu_seqlens, u.device), _opt_i32(state_idx, u.device),
                                 _opt_i32(has_init, u.device), dt_softplus)
    return y


def ssd_scan_varlen(x, dt, A, B, C, D=None, dt_bias=None, cu_seqlens=None, ssm_state=None, state_idx=None,
                    has_init=None, dt_softplus=True):
    """x [T, H, P]; dt [T, H]; A fp32 [H]; B, C [T, G, N]; ssm_state fp32 [slots, H, P, N]."""
    P = x.shape[2]
    if not _native_ok(x) or P & (P - 1) or P > 256 or B.shape[2] > 256:
        return ssd_scan_reference(x, dt, A, B, C, D, dt_bias, cu_seqlens, ssm_state, state_idx, has_init,
                                  dt_softplus)
    y = torch.empty_like(x)
    _lib().ssd_scan_varlen(x.contiguous(), dt.contiguous(), A.float().contiguous(), B.contiguous(), C.contiguous(),
                           None if D is None else D.float().contiguous(),
                           None if dt_bias is None else dt_bias.float().contiguous(), y, ssm_state,
                           _opt_i32(cu_seqlens, x.device), _opt_i32(state_idx, x.device),
                           _opt_i32(has_init, x.device), dt_softplus)
    return y


# ------------------------------------------------------------------------------------ blocks
class MambaMixer(torch.nn.Module):
    """Mamba-1 block: in_proj -> (x, z); causal conv + SiLU; x_proj -> (dt, B, C); dt_proj; selective scan gated
    by silu(z); out_proj. Weight names follow the Hugging Face ``MambaMixer``."""

    def __init__(self, hidden: int, d_inner: int, d_state: int = 16, d_conv: int = 4, dt_rank: Optional[int] = None,
                 dtype=torch.float32, device="cpu"):
        super().__init__()
        self.hidden, self.d_inner, self.d_state, self.d_conv = hidden, d_inner, d_state, d_conv
        self.dt_rank = dt_rank or (hidden + 15) // 16
        kw = dict(dtype=dtype, device=device)
        self.in_proj = torch.nn.Linear(hidden, 2 * d_inner, bias=False, **kw)
        self.conv_w = torch.nn.Parameter(torch.randn(d_inner, d_conv, **kw) * 0.2)
        self.conv_b = torch.nn.Parameter(torch.zeros(d_inner, **kw))
        self.x_proj = torch.nn.Linear(d_inner, self.dt_rank + 2 * d_state, bias=False, **kw)
        self.dt_proj = torch.nn.Linear(self.dt_rank, d_inner, bias=True, **kw)
        self.A_log = torch.nn.Parameter(torch.log(torch.arange(1, d_state + 1, dtype=torch.float32, device=device))
                                        .repeat(d_inner, 1))
        self.D = torch.nn.Parameter(torch.ones(d_inner, dtype=torch.float32, device=device))
        self.out_proj = torch.nn.Linear(d_inner, hidden, bias=False, **kw)

    def alloc_state(self, slots: int, device=None):
        device = device or self.conv_w.device
        return (torch.zeros(slots, self.d_inner, self.d_conv - 1, dtype=torch.float32, device=device),
                torch.zeros(slots, self.d_inner, self.d_state, dtype=torch.float32, device=device))

    @torch.no_grad()
    def forward(self, h, cu_seqlens, state=None, state_idx=None, has_init=None):
        conv_state, ssm_state = state if state is not None else (None, None)
        xz = self.in_proj(h)
        x, z = xz[:, : self.d_inner].contiguous(), xz[:, self.d_inner:].contiguous()
        x = causal_conv1d_varlen(x, self.conv_w, self.conv_b, cu_seqlens, conv_state, state_idx, has_init, True)
        dbc = self.x_proj(x)
        dt = self.dt_proj.weight @ dbc[:, : self.dt_rank].t()
        dt = dt.t().contiguous()
        B = dbc[:, self.dt_rank : self.dt_rank + self.d_state].contiguous()
        C = dbc[:, self.dt_rank + self.d_state:].contiguous()
        y = selective_scan_varlen(x, dt, -torch.exp(self.A_log.float()), B, C, self.D, z,
                                  self.dt_proj.bias.float(), cu_seqlens, ssm_state, state_idx, has_init, True)
        return self.out_proj(y)


class Mamba2Mixer(torch.nn.Module):
    """Mamba-2 block: in_proj -> (z, xBC, dt); causal conv + SiLU over xBC; SSD recurrence per head; gated
    RMSNorm; out_proj."""

    def __init__(self, hidden: int, n_heads: int, head_dim: int, d_state: int = 128, n_groups: int = 1,
                 d_conv: int = 4, eps: float = 1e-5, dtype=torch.float32, device="cpu"):
        super().__init__()
        self.hidden, self.H, self.P, self.N, self.G, self.d_conv, self.eps = (hidden, n_heads, head_dim, d_state,
                                                                             n_groups, d_conv, eps)
        self.d_inner = n_heads * head_dim
        self.conv_dim = self.d_inner + 2 * n_groups * d_state
        kw = dict(dtype=dtype, device=device)
        self.in_proj = torch.nn.Linear(hidden, self.d_inner + self.conv_dim + n_heads, bias=False, **kw)
        self.conv_w = torch.nn.Parameter(torch.randn(self.conv_dim, d_conv, **kw) * 0.2)
        self.conv_b = torch.nn.Parameter(torch.zeros(self.conv_dim, **kw))
        self.A_log = torch.nn.Parameter(torch.log(torch.arange(1, n_heads + 1, dtype=torch.float32, device=device)))
        self.D = torch.nn.Parameter(torch.ones(n_heads, dtype=torch.float32, device=device))
        self.dt_bias = torch.nn.Parameter(torch.zeros(n_heads, dtype=torch.float32, device=device))
        self.norm_w = torch.nn.Parameter(torch.ones(self.d_inner, **kw))
        self.out_proj = torch.nn.Linear(self.d_inner, hidden, bias=False, **kw)

    def alloc_state(self, slots: int, device=None):
        device = device or self.conv_w.device
        return (torch.zeros(slots, self.conv_dim, self.d_conv - 1, dtype=torch.float32, device=device),
                torch.zeros(slots, self.H, self.P, self.N, dtype=torch.float32, device=device))

    @torch.no_grad()
    def forward(self, h, cu_seqlens, state=None, state_idx=None, has_init=None):
        conv_state, ssm_state = state if state is not None else (None, None)
        proj = self.in_proj(h)
        z = proj[:, : self.d_inner]
        xbc = proj[:, self.d_inner : self.d_inner + self.conv_dim].contiguous()
        dt = proj[:, self.d_inner + self.conv_dim:].contiguous()
        xbc = causal_conv1d_varlen(xbc, self.conv_w, self.conv_b, cu_seqlens, conv_state, state_idx, has_init, True)
        T = h.shape[0]
        x = xbc[:, : self.d_inner].reshape(T, self.H, self.P).contiguous()
        gn = self.G * self.N
        B = xbc[:, self.d_inner : self.d_inner + gn].reshape(T, self.G, self.N).contiguous()
        C = xbc[:, self.d_inner + gn:].reshape(T, self.G, self.N).contiguous()
        y = ssd_scan_varlen(x, dt, -torch.exp(self.A_log.float()), B, C, self.D, self.dt_bias, cu_seqlens,
                            ssm_state, state_idx, has_init, True).reshape(T, self.d_inner)
        g = (y.float() * F.silu(z.float()))
        g = g * torch.rsqrt(g.pow(2).mean(-1, keepdim=True) + self.eps) * self.norm_w.float()
        return self.out_proj(g.to(h.dtype))
