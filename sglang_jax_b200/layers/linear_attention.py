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


def track_pieces(a0: int, a1: int, track):
    """Token ranges of one sequence's extend `[a0, a1)` and, per range, the snapshot slot that receives the
    recurrent state at its end: `track = (tokens before the checkpoint, slot)` splits the extend there."""
    if track is None:
        return [(a0, a1, None)]
    k, slot = track
    cut = a0 + k
    if cut <= a0 or cut > a1:
        return [(a0, a1, None)]
    if cut == a1:
        return [(a0, a1, slot)]
    return [(a0, cut, slot), (cut, a1, None)]


def recurrent_slots(fb) -> torch.Tensor:
    """State slot of every row of the batch: request row + 1 (slot 0 is scratch).  A captured decode step
    supplies them itself so that its padding rows land on the scratch slot."""
    slots = fb.extras.get("recurrent_slots")
    return slots if slots is not None else fb.req_pool_indices.long() + 1


def _native_step_ok(x, conv_all, rec_all, dk: int, dv: int) -> bool:
    """Whether a decode step can run the in-place CUDA kernels (`csrc/linear_attn.cu`)."""
    from .. import ops
    return (ops.use_native(x) and rec_all.dtype == torch.float32 and conv_all.dtype in (torch.bfloat16, torch.float32)
            and rec_all.is_contiguous() and conv_all.is_contiguous() and dk <= 256 and dv <= 256 and dv % 32 == 0
            and conv_all.shape[-1] + 1 <= 8)


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
        slots = recurrent_slots(fb)
        r = self.nv // self.nk
        T = x.shape[0]

        def heads(m):
            qq, kk, vv = torch.split(m, [self.key_dim, self.key_dim, self.value_dim], dim=-1)
            qq = qq.reshape(-1, self.nk, self.dk)
            kk = kk.reshape(-1, self.nk, self.dk)
            if r > 1:
                qq, kk = qq.repeat_interleave(r, 1), kk.repeat_interleave(r, 1)
            return qq, kk, vv.reshape(-1, self.nv, self.dv)

        if fb.forward_mode.is_decode() and _native_step_ok(x, conv_all, rec_all, self.dk, self.dv):
            # sm_100a path: the convolution window and the state matrix are updated in place in their pools
            from ..ops import native
            y = native.conv1d_update(mixed, conv_all, self.conv1d_weight, slots)
            qq, kk, vv = torch.split(y, [self.key_dim, self.key_dim, self.value_dim], dim=-1)
            o = native.delta_rule_step(qq.reshape(T, self.nk, self.dk), kk.reshape(T, self.nk, self.dk),
                                       vv.reshape(T, self.nv, self.dv), g, beta, rec_all, slots)
        elif fb.forward_mode.is_decode():
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
            tracks = fb.extras.get("recurrent_tracks") or {}
            for i in range(fb.batch_size):
                if cu[i + 1] == cu[i]:
                    continue
                fresh = int(pre[i]) == 0
                # a checkpoint inside the extend splits it: the state after the first piece also goes to the snapshot slot
                for a0, a1, snap in track_pieces(cu[i], cu[i + 1], tracks.get(i)):
                    y, new_conv = la.causal_conv1d_prefill(mixed[a0:a1], self.conv1d_weight,
                                                           None if fresh else conv_all[sl[i]])
                    conv_all[sl[i]] = new_conv.to(conv_all.dtype)
                    qq, kk, vv = heads(y)
                    oi, S = la.chunk_gated_delta_rule(qq, kk, vv, g[a0:a1], beta[a0:a1],
                                                      None if fresh else rec_all[sl[i]])
                    o[a0:a1] = oi
                    rec_all[sl[i]] = S
                    fresh = False
                    if snap is not None:
                        conv_all[snap] = conv_all[sl[i]]
                        rec_all[snap] = rec_all[sl[i]]
        out = self.norm(o.reshape(-1, self.dv), z.reshape(-1, self.dv)).reshape(T, self.value_dim)
        return self.out_proj(out)


class _RecurrentMixer(nn.Module):
    """Shared plumbing of the recurrent token mixers: per-request state lives in slot `row + 1` of the
    runner's `RecurrentStatePool`; sequences of an extend batch are stepped one after another, a decode
    batch in one go."""

    layer_index: int

    def _run(self, fb, T, per_seq, per_batch):
        pool = fb.extras["recurrent_pool"]
        conv_all, rec_all = pool.conv_state[self.layer_index], pool.recurrent_state[self.layer_index]
        slots = recurrent_slots(fb)
        if fb.forward_mode.is_decode():
            return per_batch(conv_all, rec_all, slots)
        cu = fb.cu_q_lens.tolist()
        pre = fb.extend_prefix_lens_cpu
        tracks = fb.extras.get("recurrent_tracks") or {}
        outs = []
        for i, s in enumerate(slots.tolist()):
            if cu[i + 1] > cu[i]:
                fresh = int(pre[i]) == 0
                for a0, a1, snap in track_pieces(cu[i], cu[i + 1], tracks.get(i)):
                    outs.append(per_seq(conv_all, rec_all, s, a0, a1, fresh))
                    fresh = False
                    if snap is not None:
                        conv_all[snap] = conv_all[s]
                        rec_all[snap] = rec_all[s]
        return torch.cat(outs, 0)


class KimiDeltaAttention(_RecurrentMixer):
    """KDA (reference `python/sgl_jax/srt/models/kimi_linear.py:74`, `layers/attention/linear/kda_backend.py`):
    q/k/v projections followed by short causal convolutions, a per-channel forget gate from a low-rank
    projection, a scalar write strength `beta`, the delta-rule recurrence and a low-rank output gate
    through a gated RMSNorm."""

    def __init__(self, config, linear_layer_index: int, dtype):
        super().__init__()
        lc = config.linear_attn_config
        H = config.hidden_size
        self.nh, self.hd = lc["num_heads"], lc["head_dim"]
        self.conv_kernel = lc["short_conv_kernel_size"]
        self.layer_index = linear_layer_index
        P = self.nh * self.hd
        self.conv_dim = 3 * P
        self.q_proj = ReplicatedLinear(H, P, False, dtype)
        self.k_proj = ReplicatedLinear(H, P, False, dtype)
        self.v_proj = ReplicatedLinear(H, P, False, dtype)
        self.q_conv1d_weight = nn.Parameter(torch.empty(P, self.conv_kernel, dtype=dtype), requires_grad=False)
        self.k_conv1d_weight = nn.Parameter(torch.empty(P, self.conv_kernel, dtype=dtype), requires_grad=False)
        self.v_conv1d_weight = nn.Parameter(torch.empty(P, self.conv_kernel, dtype=dtype), requires_grad=False)
        self.A_log = nn.Parameter(torch.zeros(self.nh, dtype=torch.float32), requires_grad=False)
        self.dt_bias = nn.Parameter(torch.zeros(P, dtype=torch.float32), requires_grad=False)
        self.f_a_proj = ReplicatedLinear(H, self.hd, False, dtype)
        self.f_b_proj = ReplicatedLinear(self.hd, P, False, dtype)
        self.b_proj = ReplicatedLinear(H, self.nh, False, dtype)
        self.g_a_proj = ReplicatedLinear(H, self.hd, False, dtype)
        self.g_b_proj = ReplicatedLinear(self.hd, P, False, dtype)
        self.o_norm = GatedRMSNorm(self.hd, config.rms_norm_eps, dtype)
        self.o_norm.gate_act = "sigmoid"
        self.o_proj = ReplicatedLinear(P, H, False, dtype)

    def weight_loader(self, param, w, shard_id=None):
        param.data.copy_((w.squeeze(1) if w.dim() == 3 else w).reshape(param.shape).to(param.dtype))

    def forward(self, x, fb):
        T = x.shape[0]
        nh, hd = self.nh, self.hd
        mixed = torch.cat([self.q_proj(x), self.k_proj(x), self.v_proj(x)], -1)
        w = torch.cat([self.q_conv1d_weight, self.k_conv1d_weight, self.v_conv1d_weight], 0)
        raw = self.f_b_proj(self.f_a_proj(x)).view(T, nh, hd).float() + self.dt_bias.view(nh, hd)
        g = -self.A_log.float().exp().view(1, nh, 1) * torch.nn.functional.softplus(raw)
        beta = torch.sigmoid(self.b_proj(x).float())

        def split(y):
            q, k, v = y.split(nh * hd, -1)
            return q.reshape(-1, nh, hd), k.reshape(-1, nh, hd), v.reshape(-1, nh, hd)

        def per_seq(conv_all, rec_all, s, a0, a1, fresh):
            y, cs = la.causal_conv1d_prefill(mixed[a0:a1], w, None if fresh else conv_all[s])
            conv_all[s] = cs.to(conv_all.dtype)
            q, k, v = split(y)
            init = torch.zeros_like(rec_all[s]) if fresh else rec_all[s]
            o, S = la.kda_recurrent(q[None], k[None], v[None], g[None, a0:a1], beta[None, a0:a1], init[None])
            rec_all[s] = S[0]
            return o[0]

        def per_batch(conv_all, rec_all, slots):
            if _native_step_ok(x, conv_all, rec_all, hd, hd):
                from ..ops import native
                q, k, v = split(native.conv1d_update(mixed, conv_all, w, slots))
                return native.delta_rule_step(q, k, v, g, beta, rec_all, slots, gate_per_channel=True)
            y, cs = la.causal_conv1d_update(mixed, conv_all[slots], w)
            conv_all[slots] = cs.to(conv_all.dtype)
            q, k, v = split(y)
            o, S = la.kda_recurrent(q[:, None], k[:, None], v[:, None], g[:, None], beta[:, None], rec_all[slots])
            rec_all[slots] = S
            return o[:, 0]

        o = self._run(fb, T, per_seq, per_batch)
        gate = self.g_b_proj(self.g_a_proj(x)).view(T, nh, hd)
        of = o.float()
        y = of * torch.rsqrt(of.pow(2).mean(-1, keepdim=True) + self.o_norm.eps) * self.o_norm.weight.float()
        y = (y * torch.sigmoid(gate.float())).to(x.dtype)
        return self.o_proj(y.reshape(T, nh * hd))


class LightningAttention(_RecurrentMixer):
    """Lightning linear attention (reference `layers/attention/linear/lightning_backend.py:86`): SiLU'd
    q/k/v from one fused projection, a fixed geometric per-head decay scaled by layer depth, RMS-normed
    output gated by `sigmoid(g_proj(x))`."""

    def __init__(self, config, linear_layer_index: int, layer_id: int, dtype):
        super().__init__()
        H = config.hidden_size
        self.nh = config.num_attention_heads
        self.hd = getattr(config, "head_dim", None) or H // self.nh
        self.layer_index = linear_layer_index
        self.conv_dim, self.conv_kernel = 1, 1
        P = self.nh * self.hd
        self.query_key_value = ReplicatedLinear(H, 3 * P, getattr(config, "use_qkv_bias", False), dtype)
        self.g_proj = ReplicatedLinear(H, P, False, dtype)
        self.g_norm = nn.Parameter(torch.ones(P, dtype=dtype), requires_grad=False)
        self.dense = ReplicatedLinear(P, H, getattr(config, "use_bias", False), dtype)
        n_layers = config.num_hidden_layers
        scale = 1.0 - layer_id / max(n_layers - 1, 1) + 1e-5
        self.register_buffer("slopes", la.alibi_slopes(self.nh) * scale, persistent=False)
        self.eps = config.rms_norm_eps

    def weight_loader(self, param, w, shard_id=None):
        param.data.copy_(w.reshape(param.shape).to(param.dtype))

    def forward(self, x, fb):
        T = x.shape[0]
        nh, hd = self.nh, self.hd
        qkv = torch.nn.functional.silu(self.query_key_value(x)).view(T, nh, 3 * hd)
        q, k, v = qkv.split(hd, -1)

        def per_seq(conv_all, rec_all, s, a0, a1, fresh):
            init = torch.zeros_like(rec_all[s]) if fresh else rec_all[s]
            o, S = la.lightning_attention(q[None, a0:a1], k[None, a0:a1], v[None, a0:a1], self.slopes, init[None])
            rec_all[s] = S[0]
            return o[0]

        def per_batch(conv_all, rec_all, slots):
            o, S = la.lightning_attention(q[:, None], k[:, None], v[:, None], self.slopes, rec_all[slots])
            rec_all[slots] = S
            return o[:, 0]

        o = self._run(fb, T, per_seq, per_batch).reshape(T, nh * hd).float()
        o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + self.eps) * self.g_norm.float()
        o = (o * torch.sigmoid(self.g_proj(x).float())).to(x.dtype)
        return self.dense(o)
