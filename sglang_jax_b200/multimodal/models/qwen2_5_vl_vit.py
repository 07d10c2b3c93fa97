"""Qwen2.5-VL vision transformer (reference `multimodal/models/qwen2_5VL`): patch embedding of
flattened (temporal x patch x patch) pixel blocks, 2-D rotary position (row, column), blocks that
alternate windowed and full attention over a window-major token order, RMSNorm + biased SwiGLU
MLP, and a 2x2 spatial merger that emits one LLM-width embedding per merged patch.

Attention runs over packed variable-length segments (whole images for the full-attention blocks,
windows otherwise): on the GPU through the varlen attention kernel, elsewhere as a block-diagonal
mask over the packed sequence."""

from __future__ import annotations

from typing import Iterable

import torch
import torch.nn.functional as F
from torch import nn

from ... import ops


def _rms(x, w, eps=1e-6):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


class Segments:
    """Contiguous attention segments of a packed sequence: lengths for the varlen kernel, and the
    block-diagonal mask (built on first use) for the PyTorch path."""

    def __init__(self, cu: torch.Tensor, n: int, device):
        self.cu, self.n, self.device = cu, n, device
        self.lens = (cu[1:] - cu[:-1]).tolist()
        self._mask = None

    def mask(self) -> torch.Tensor:
        if self._mask is None:
            seg = torch.bucketize(torch.arange(self.n), self.cu[1:], right=True)
            self._mask = (seg[:, None] == seg[None, :]).to(self.device)
        return self._mask

class _Lin(nn.Module):
    def __init__(self, i, o, dtype, bias=True):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(o, i, dtype=dtype), requires_grad=False)
        self.bias = nn.Parameter(torch.zeros(o, dtype=dtype), requires_grad=False) if bias else None

    def forward(self, x):
        return ops.linear(x, self.weight, self.bias)


class VisionBlock(nn.Module):
    def __init__(self, cfg, dtype):
        super().__init__()
        D = cfg.hidden_size
        self.heads = cfg.num_heads
        self.norm1 = nn.Parameter(torch.ones(D, dtype=dtype), requires_grad=False)
        self.norm2 = nn.Parameter(torch.ones(D, dtype=dtype), requires_grad=False)
        self.qkv = _Lin(D, 3 * D, dtype)
        self.proj = _Lin(D, D, dtype)
        self.gate_proj = _Lin(D, cfg.intermediate_size, dtype)
        self.up_proj = _Lin(D, cfg.intermediate_size, dtype)
        self.down_proj = _Lin(cfg.intermediate_size, D, dtype)

    def forward(self, x, seg_mask, cos, sin):
        N, D = x.shape
        H = self.heads
        qkv = self.qkv(_rms(x, self.norm1)).view(N, 3, H, D // H)
        q, k, v = qkv[:, 0], qkv[:, 1], qkv[:, 2]

        def rot(t):
            tf = t.float()
            half = tf.shape[-1] // 2
            rh = torch.cat([-tf[..., half:], tf[..., :half]], -1)
            return (tf * cos[:, None] + rh * sin[:, None]).to(t.dtype)

        if ops.use_native(x):
            # packed segments through the paged extend kernel with the causal rule off: no N x N mask
            a = ops.varlen_attention(rot(q), rot(k), v.contiguous(), seg_mask.lens, (D // H) ** -0.5).reshape(N, D)
        else:
            a = F.scaled_dot_product_attention(rot(q).transpose(0, 1)[None], rot(k).transpose(0, 1)[None],
                                               v.transpose(0, 1)[None], attn_mask=seg_mask.mask()[None, None])
            a = a[0].transpose(0, 1).reshape(N, D)
        x = x + self.proj(a)
        h = _rms(x, self.norm2)
        return x + self.down_proj(F.silu(self.gate_proj(h)) * self.up_proj(h))


class Qwen2_5_VisionTransformer(nn.Module):
    def __init__(self, config, dtype=torch.bfloat16, quant_config=None):
        super().__init__()
        c = config
        self.config = c
        self.merge = c.spatial_merge_size
        self.unit = self.merge ** 2
        pdim = c.in_channels * c.temporal_patch_size * c.patch_size * c.patch_size
        self.patch_embed = _Lin(pdim, c.hidden_size, dtype, bias=False)
        self.blocks = nn.ModuleList([VisionBlock(c, dtype) for _ in range(c.depth)])
        self.ln_q = nn.Parameter(torch.ones(c.hidden_size, dtype=dtype), requires_grad=False)
        self.merger_fc1 = _Lin(c.hidden_size * self.unit, c.hidden_size * self.unit, dtype)
        self.merger_fc2 = _Lin(c.hidden_size * self.unit, c.out_hidden_size, dtype)
        self.head_dim = c.hidden_size // c.num_heads

    # ------------------------------------------------------------------ index helpers
    def _rot_pos(self, grid_thw: torch.Tensor, device):
        m = self.merge
        pos = []
        for t, h, w in grid_thw.tolist():
            hp = torch.arange(h).unsqueeze(1).expand(-1, w).reshape(h // m, m, w // m, m).permute(0, 2, 1, 3).flatten()
            wp = torch.arange(w).unsqueeze(0).expand(h, -1).reshape(h // m, m, w // m, m).permute(0, 2, 1, 3).flatten()
            pos.append(torch.stack([hp, wp], -1).repeat(t, 1))
        pos = torch.cat(pos, 0)
        dim = self.head_dim // 2
        inv = 1.0 / (10000.0 ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
        freqs = torch.outer(torch.arange(int(grid_thw[:, 1:].max()), dtype=torch.float32), inv)
        return freqs[pos].flatten(1).to(device)                                  # [N, head_dim/2]

    def _windows(self, grid_thw: torch.Tensor):
        c = self.config
        ws = c.window_size // self.merge // c.patch_size
        index, cu, base = [], [0], 0
        for t, h, w in grid_thw.tolist():
            gh, gw = h // self.merge, w // self.merge
            idx = torch.arange(t * gh * gw).reshape(t, gh, gw)
            ph, pw = ws - gh % ws, ws - gw % ws
            nh, nw = (gh + ph) // ws, (gw + pw) // ws
            pad = F.pad(idx, (0, pw, 0, ph), value=-100).reshape(t, nh, ws, nw, ws).permute(0, 1, 3, 2, 4)
            pad = pad.reshape(t, nh * nw, ws, ws)
            lens = (pad != -100).sum([2, 3]).reshape(-1)
            flat = pad.reshape(-1)
            index.append(flat[flat != -100] + base)
            cu.extend((lens.cumsum(0) * self.unit + cu[-1]).tolist())
            base += t * gh * gw
        cu_t = torch.unique_consecutive(torch.tensor(cu))
        return torch.cat(index), cu_t

    @staticmethod
    def _segment_mask(cu: torch.Tensor, n: int, device) -> "Segments":
        return Segments(cu, n, device)

    # ------------------------------------------------------------------ forward
    @torch.inference_mode()
    def forward(self, pixel_values: torch.Tensor, grid_thw: torch.Tensor) -> torch.Tensor:
        """`pixel_values [N, C*tp*p*p]` (flattened patches of all images), `grid_thw [num_images, 3]`
        -> `[N / merge^2, out_hidden_size]` embeddings in the original patch order."""
        dev = self.patch_embed.weight.device
        x = self.patch_embed(pixel_values.to(dev, self.patch_embed.weight.dtype))
        N = x.shape[0]
        grid = grid_thw.cpu()
        rot = self._rot_pos(grid, dev)
        win_index, cu_win = self._windows(grid)
        win_index = win_index.to(dev)
        x = x.view(N // self.unit, self.unit, -1)[win_index].reshape(N, -1)
        rot = rot.view(N // self.unit, self.unit, -1)[win_index].reshape(N, -1)
        emb = torch.cat([rot, rot], -1)
        cos, sin = emb.cos(), emb.sin()
        cu_full = F.pad(torch.repeat_interleave(grid[:, 1] * grid[:, 2], grid[:, 0]).cumsum(0), (1, 0))
        m_full = self._segment_mask(cu_full, N, dev)
        m_win = self._segment_mask(cu_win, N, dev)
        full = set(self.config.fullatt_block_indexes)
        for i, blk in enumerate(self.blocks):
            x = blk(x, m_full if i in full else m_win, cos, sin)
        h = _rms(x, self.ln_q).view(-1, self.config.hidden_size * self.unit)
        h = self.merger_fc2(F.gelu(self.merger_fc1(h)))
        return h[torch.argsort(win_index)]

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]):
        params = dict(self.named_parameters())
        ren = [("visual.", ""), ("model.", ""), (".attn.qkv.", ".qkv."), (".attn.proj.", ".proj."), (".mlp.", "."),
               (".norm1.weight", ".norm1"), (".norm2.weight", ".norm2"), ("merger.ln_q.weight", "ln_q"),
               ("merger.0.", "merger_fc1."), ("merger.2.", "merger_fc2."), ("patch_embed.proj.weight", "patch_embed.weight")]
        loaded = set()
        for name, w in weights:
            if not (name.startswith("visual.") or name.startswith("model.visual.") or name.split(".")[0] in
                    ("blocks", "merger", "patch_embed")):
                continue
            for a, b in ren:
                name = name.replace(a, b) if not (a == ".mlp." and "merger" in name) else name
            name = name.replace("merger.mlp.0.", "merger_fc1.").replace("merger.mlp.2.", "merger_fc2.")
            if name not in params:
                continue
            p = params[name]
            p.data.copy_(w.reshape(p.shape).to(p.dtype))
            loaded.add(name)
        return loaded


EntryClass = [Qwen2_5_VisionTransformer]
