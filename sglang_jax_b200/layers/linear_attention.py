"""Gated DeltaNet token mixer of the hybrid models (Qwen3-Next / Qwen3.5) over the recurrent
state pool (reference `python/sgl_jax/srt/layers/attention/linear/gdn_backend.py`,
`hybrid_linear_attn_backend.py:171`).

The state of a request lives in slot `row + 1` of the runner's `RecurrentStatePool` (one slot
per request row).  A prefill chunk that starts a sequence (`prefix_len == 0`) starts from zero
state; later chunks and decode steps continue from the stored state."""

from __future__ import annotations

import torch
from torch import nn

from ..ops import linear_attention as la
from .layernorm import GatedRMSNorm
from .linear import ReplicatedLinear


class GatedDeltaNet(nn.Module):
    def __init__(self, config, linear_layer_index: int, dtype):
        super().__init__()
        H = config.hidden_size
        self.nv, self.nk = config.linear_num_value_heads, config.linear_num_key_heads
        self.dk, self.dv = config.linear_key_head_dim, config.linear_value_head_dim
        self.key_dim, self.value_dim = self.dk * self.nk, self.dv * self.nv
        self.conv_kernel = config.linear_conv_kernel_dim
        self.conv_dim = 2 * self.key_dim + self.value_dim
        self.layer_index = linear_layer_index
        # projections are replicated across tensor ranks: the recurrent state is per head and the
        # layers are a small share of the model's FLOPs
        self.in_proj_qkvz = ReplicatedLinear(H, 2 * self.key_dim + 2 * self.value_dim, False, dtype)
        self.in_proj_ba = ReplicatedLinear(H, 2 * self.nv, False, dtype)
        self.conv1d_weight = nn.Parameter(torch.empty(self.conv_dim, self.conv_kernel, dtype=dtype), requires_grad=False)
        self.dt_bias = nn.Parameter(torch.ones(self.nv, dtype=torch.float32), requires_grad=False)
        self.A_log = nn.Parameter(torch.zeros(self.nv, dtype=torch.float32), requires_grad=False)
        self.norm = GatedRMSNorm(self.dv, config.rms_norm_eps, dtype)
        self.out_proj = ReplicatedLinear(self.value_dim, H, False, dtype)

    def weight_loader(self, param, w, shard_id=None):
        if w.dim() == 3:                 # depth-wise conv kernel stored [C, 1, K]
            w = w.squeeze(1)
        param.data.copy_(w.to(param.dtype))

    def _split(self, qkvz, ba):
        T = qkvz.shape[0]
        r = self.nv // self.nk
        qkvz = qkvz.view(T, self.nk, 2 * self.dk + 2 * r * self.dv)
        q, k, v, z = torch.split(qkvz, [self.dk, self.dk, r * self.dv, r * self.dv], dim=-1)
        ba = ba.view(T, self.nk, 2 * r)
        b, a = torch.split(ba, [r, r], dim=-1)
        return (q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1), z.reshape(T, self.nv, self.dv),
                b.reshape(T, self.nv), a.reshape(T, self.nv))

    def forward(self, x: torch.Tensor, forward_batch) -> torch.Tensor:
        fb = forward_batch
        pool = fb.extras["recurrent_pool"]
        conv_all, rec_all = pool.conv_state[self.layer_index], pool.recurrent_state[self.layer_index]
        q, k, v, z, b, a = self._split(self.in_proj_qkvz(x), self.in_proj_ba(x))
        mixed = torch.cat([q, k, v], dim=-1)                             # [T, conv_dim]
        beta = torch.sigmoid(b.float())
        g = -self.A_log.float().exp() * torch.nn.functional.softplus(a.float() + self.dt_bias)
        slots = fb.req_pool_indices.long() + 1
        r = self.nv // self.nk
        T = x.shape[0]

        def heads(m):
            qq, kk, vv = torch.split(m, [self.key_dim, self.key_dim, self.value_dim], dim=-1)
            qq = qq.reshape(-1, self.nk, self.dk)
            kk = kk.reshape(-1, self.nk, self.dk)
            if r > 1:
                qq, kk = qq.repeat_interleave(r, 1), kk.repeat_interleave(r, 1)
            return qq, kk, vv.reshape(-1, self.nv, self.dv)

        if fb.forward_mode.is_decode():
            y, new_conv = la.causal_conv1d_update(mixed, conv_all[slots], self.conv1d_weight)
            conv_all[slots] = new_conv.to(conv_all.dtype)
            qq, kk, vv = heads(y)
            o, S = la.recurrent_gated_delta_rule_step(qq, kk, vv, g, beta, rec_all[slots])
            rec_all[slots] = S
        else:
            o = torch.empty(T, self.nv, self.dv, dtype=x.dtype, device=x.device)
            cu = fb.cu_q_lens.tolist()
            pre = fb.extend_prefix_lens_cpu
            sl = slots.tolist()
            for i in range(fb.batch_size):
                a0, a1 = cu[i], cu[i + 1]
                if a1 == a0:
                    continue
                fresh = int(pre[i]) == 0
                y, new_conv = la.causal_conv1d_prefill(mixed[a0:a1], self.conv1d_weight,
                                                       None if fresh else conv_all[sl[i]])
                conv_all[sl[i]] = new_conv.to(conv_all.dtype)
                qq, kk, vv = heads(y)
                oi, S = la.chunk_gated_delta_rule(qq, kk, vv, g[a0:a1], beta[a0:a1],
                                                  None if fresh else rec_all[sl[i]])
                o[a0:a1] = oi
                rec_all[sl[i]] = S
        out = self.norm(o.reshape(-1, self.dv), z.reshape(-1, self.dv)).reshape(T, self.value_dim)
        return self.out_proj(out)
