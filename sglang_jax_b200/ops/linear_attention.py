"""Linear-attention primitives for the hybrid models (gated delta rule, short causal convolution).

Reference: `python/sgl_jax/srt/layers/attention/linear/{gdn_backend,short_convolution}.py` and
the `kernels/gdn` Pallas kernels.  Both phases are stated here in PyTorch:

* prefill — chunked form: inside a chunk of 64 tokens the recurrence is solved with a
  triangular system (all matmuls), chunks are chained through the `[Dk, Dv]` state, so the work
  is GEMM-shaped;
* decode — one recurrence step for a whole batch of sequences:
  `S <- exp(g) S;  d = beta (v - S^T k);  S <- S + k d^T;  o = S^T q`.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F


def l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return x * torch.rsqrt(x.pow(2).sum(-1, keepdim=True) + eps)


def causal_conv1d_prefill(x: torch.Tensor, weight: torch.Tensor, init_state: torch.Tensor | None, activation=True):
    """Depth-wise causal convolution over one sequence.  `x [T, C]`, `weight [C, K]`,
    `init_state [C, K-1]` (the last K-1 inputs of the previous chunk, zeros at a sequence start).
    Returns `(y [T, C], final_state [C, K-1])`."""
    T, C = x.shape
    K = weight.shape[1]
    xf = x.float().t()                                                   # [C, T]
    prev = init_state.float() if init_state is not None else xf.new_zeros(C, K - 1)
    full = torch.cat([prev, xf], dim=1)                                  # [C, K-1+T]
    y = F.conv1d(full.unsqueeze(0), weight.float().unsqueeze(1), groups=C).squeeze(0)     # [C, T]
    if activation:
        y = F.silu(y)
    return y.t().to(x.dtype), full[:, -(K - 1):].contiguous()


def causal_conv1d_update(x: torch.Tensor, state: torch.Tensor, weight: torch.Tensor, activation=True):
    """One token per sequence.  `x [B, C]`, `state [B, C, K-1]` (updated copy returned)."""
    full = torch.cat([state.float(), x.float().unsqueeze(-1)], dim=-1)   # [B, C, K]
    y = (full * weight.float().unsqueeze(0)).sum(-1)
    if activation:
        y = F.silu(y)
    return y.to(x.dtype), full[:, :, 1:].contiguous()


def chunk_gated_delta_rule(q, k, v, g, beta, initial_state=None, chunk_size: int = 64):
    """One sequence.  `q,k [T, H, Dk]`, `v [T, H, Dv]`, `g,beta [T, H]` (g = log decay <= 0),
    `initial_state [H, Dk, Dv]`.  q and k are L2-normalised here.  Returns `(o [T, H, Dv], state)`."""
    T, H, Dk = k.shape
    Dv = v.shape[-1]
    dt = v.dtype
    q = l2norm(q.float()).transpose(0, 1) * Dk ** -0.5                  # [H, T, Dk]
    k = l2norm(k.float()).transpose(0, 1)
    v = v.float().transpose(0, 1)
    g = g.float().transpose(0, 1)                                        # [H, T]
    beta = beta.float().transpose(0, 1)
    C = chunk_size
    pad = (C - T % C) % C
    if pad:
        q, k, v = (F.pad(t, (0, 0, 0, pad)) for t in (q, k, v))
        g, beta = F.pad(g, (0, pad)), F.pad(beta, (0, pad))
    n = (T + pad) // C
    q, k, v = (t.reshape(H, n, C, -1) for t in (q, k, v))
    g = g.reshape(H, n, C).cumsum(-1)
    beta = beta.reshape(H, n, C)
    k_beta, v_beta = k * beta[..., None], v * beta[..., None]
    decay = (g[..., :, None] - g[..., None, :]).tril().exp().tril()      # [H, n, C, C]
    upper = torch.triu(torch.ones(C, C, dtype=torch.bool, device=q.device), 0)
    A = -((k_beta @ k.transpose(-1, -2)) * decay).masked_fill(upper, 0)
    for i in range(1, C):                                                # forward substitution
        row = A[..., i, :i].clone()
        A[..., i, :i] = row + (row.unsqueeze(-1) * A[..., :i, :i].clone()).sum(-2)
    A = A + torch.eye(C, dtype=A.dtype, device=A.device)
    u = A @ v_beta                                                       # "pseudo values"
    w = A @ (k_beta * g.exp()[..., None])
    S = initial_state.float().clone() if initial_state is not None else q.new_zeros(H, Dk, Dv)
    out = torch.zeros(H, n, C, Dv, dtype=torch.float32, device=q.device)
    strict = torch.triu(torch.ones(C, C, dtype=torch.bool, device=q.device), 1)
    for i in range(n):
        qi, ki = q[:, i], k[:, i]
        attn = ((qi @ ki.transpose(-1, -2)) * decay[:, i]).masked_fill(strict, 0)
        v_new = u[:, i] - w[:, i] @ S
        out[:, i] = (qi * g[:, i, :, None].exp()) @ S + attn @ v_new
        S = S * g[:, i, -1, None, None].exp() + (ki * (g[:, i, -1, None] - g[:, i]).exp()[..., None]).transpose(-1, -2) @ v_new
    o = out.reshape(H, n * C, Dv)[:, :T].transpose(0, 1)
    return o.to(dt), S


def recurrent_gated_delta_rule_step(q, k, v, g, beta, state):
    """A batch of single steps.  `q,k [B, H, Dk]`, `v [B, H, Dv]`, `g,beta [B, H]`,
    `state [B, H, Dk, Dv]` fp32.  Returns `(o [B, H, Dv], new_state)`."""
    Dk = k.shape[-1]
    qf = l2norm(q.float()) * Dk ** -0.5
    kf = l2norm(k.float())
    S = state * g.float().exp()[..., None, None]
    kv = (S * kf[..., None]).sum(-2)                                     # [B, H, Dv]
    d = (v.float() - kv) * beta.float()[..., None]
    S = S + kf[..., None] * d[..., None, :]
    o = (S * qf[..., None]).sum(-2)
    return o.to(v.dtype), S


def kda_recurrent(q, k, v, g, beta, state):
    """Kimi Delta Attention for a batch of sequences stepped together.  `q,k [B, T, H, Dk]`,
    `v [B, T, H, Dv]`, `g [B, T, H, Dk]` (per-channel log decay), `beta [B, T, H]`,
    `state [B, H, Dk, Dv]` fp32.  Per step: `S <- diag(exp(g)) S;  S <- S + beta k (v - S^T k)^T;
    o = S^T (q / sqrt(Dk))`.  q and k are L2-normalised.  Returns `(o [B, T, H, Dv], state)`."""
    B, T, H, Dk = k.shape
    qf = l2norm(q.float()) * Dk ** -0.5
    kf = l2norm(k.float())
    vf, gf, bf = v.float(), g.float(), beta.float()
    S = state.float().clone()
    out = torch.empty(B, T, H, v.shape[-1], dtype=torch.float32, device=v.device)
    for t in range(T):
        S = S * gf[:, t].exp().unsqueeze(-1)
        resid = vf[:, t] - (S * kf[:, t].unsqueeze(-1)).sum(-2)
        S = S + (bf[:, t, :, None] * kf[:, t]).unsqueeze(-1) * resid.unsqueeze(-2)
        out[:, t] = (S * qf[:, t].unsqueeze(-1)).sum(-2)
    return out.to(v.dtype), S


def lightning_attention(q, k, v, slopes, state):
    """Lightning (linear attention with a fixed per-head decay).  `q,k [B, T, H, D]`, `v [B, T, H, Dv]`,
    `slopes [H]` (decay rate, gamma = exp(-slope)), `state [B, H, D, Dv]`:
    `S <- gamma S + k v^T;  o = S^T q`."""
    B, T, H, D = k.shape
    gamma = torch.exp(-slopes.float()).view(1, H, 1, 1)
    S = state.float().clone()
    out = torch.empty(B, T, H, v.shape[-1], dtype=torch.float32, device=v.device)
    qf, kf, vf = q.float(), k.float(), v.float()
    for t in range(T):
        S = S * gamma + kf[:, t].unsqueeze(-1) * vf[:, t].unsqueeze(-2)
        out[:, t] = (S * qf[:, t].unsqueeze(-1)).sum(-2)
    return out.to(v.dtype), S


def alibi_slopes(num_heads: int) -> torch.Tensor:
    """The geometric per-head slope sequence Lightning attention uses for its decay."""
    import math

    def pow2(n):
        start = 2 ** (-(2 ** -(math.log2(n) - 3)))
        return [start * start ** i for i in range(n)]

    if math.log2(num_heads).is_integer():
        return torch.tensor(pow2(num_heads))
    c = 2 ** math.floor(math.log2(num_heads))
    return torch.tensor(pow2(c) + pow2(2 * c)[0::2][: num_heads - c])
