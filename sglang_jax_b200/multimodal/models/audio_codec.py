"""Audio tokenizer of the speech pipelines (reference `multimodal/models/mimo_audio` tokenizer:
waveform -> mel -> strided convolutions -> transformer -> residual vector quantiser; decoder:
codes -> embeddings -> transformer -> transposed-convolution vocoder)."""

from __future__ import annotations

import math
from typing import Iterable

import torch
import torch.nn.functional as F
from torch import nn


def mel_filterbank(n_mels: int, n_fft: int, rate: int, device=None) -> torch.Tensor:
    def hz2mel(f):
        return 2595.0 * math.log10(1.0 + f / 700.0)
    mels = torch.linspace(hz2mel(0.0), hz2mel(rate / 2), n_mels + 2)
    hz = 700.0 * (10 ** (mels / 2595.0) - 1.0)
    bins = torch.floor((n_fft + 1) * hz / rate).long()
    fb = torch.zeros(n_mels, n_fft // 2 + 1)
    for m in range(1, n_mels + 1):
        l, c, r = int(bins[m - 1]), int(bins[m]), int(bins[m + 1])
        for k in range(l, c):
            fb[m - 1, k] = (k - l) / max(c - l, 1)
        for k in range(c, r):
            fb[m - 1, k] = (r - k) / max(r - c, 1)
    return fb.to(device)


def log_mel(wave: torch.Tensor, rate=24000, n_fft=1024, hop=240, n_mels=80) -> torch.Tensor:
    """`wave [T]` -> `[frames, n_mels]`."""
    win = torch.hann_window(n_fft, device=wave.device)
    spec = torch.stft(wave.float(), n_fft, hop, window=win, return_complex=True).abs() ** 2     # [F, frames]
    mel = mel_filterbank(n_mels, n_fft, rate, wave.device) @ spec
    return torch.log(mel.clamp_min(1e-10)).t()


class _Block(nn.Module):
    def __init__(self, d, heads):
        super().__init__()
        self.attn = nn.MultiheadAttention(d, heads, batch_first=True)
        self.n1, self.n2 = nn.LayerNorm(d), nn.LayerNorm(d)
        self.ff = nn.Sequential(nn.Linear(d, 4 * d), nn.GELU(), nn.Linear(4 * d, d))

    def forward(self, x):
        h = self.n1(x)
        x = x + self.attn(h, h, h, need_weights=False)[0]
        return x + self.ff(self.n2(x))


class ResidualVQ(nn.Module):
    def __init__(self, num_q, codebook, dim):
        super().__init__()
        self.codebooks = nn.Parameter(torch.randn(num_q, codebook, dim) * 0.1, requires_grad=False)

    def encode(self, x):                       # [T, D] -> [T, Q]
        res, codes = x, []
        for cb in self.codebooks:
            idx = torch.cdist(res, cb).argmin(-1)
            codes.append(idx)
            res = res - cb[idx]
        return torch.stack(codes, -1)

    def decode(self, codes):                   # [T, Q] -> [T, D]
        return sum(self.codebooks[q][codes[:, q]] for q in range(codes.shape[1]))


class MiMoAudioTokenizer(nn.Module):
    """`config`: sample_rate, n_mels, d_model, heads, layers, num_quantizers, codebook_size, hop."""

    def __init__(self, config, dtype=torch.float32, quant_config=None):
        super().__init__()
        c = config
        self.config = c
        d = c.d_model
        self.conv1 = nn.Conv1d(c.n_mels, d, 3, padding=1)
        self.conv2 = nn.Conv1d(d, d, 3, stride=2, padding=1)
        self.enc = nn.ModuleList([_Block(d, c.heads) for _ in range(c.layers)])
        self.rvq = ResidualVQ(c.num_quantizers, c.codebook_size, d)
        self.dec = nn.ModuleList([_Block(d, c.heads) for _ in range(c.layers)])
        self.up = nn.ConvTranspose1d(d, d // 2, 2 * c.hop // 4, stride=c.hop // 2, padding=c.hop // 8 * 0)
        self.out = nn.ConvTranspose1d(d // 2, 1, 8, stride=4, padding=2)

    @torch.inference_mode()
    def encode(self, wave: torch.Tensor) -> torch.Tensor:
        c = self.config
        mel = log_mel(wave.to(self.conv1.weight.device), c.sample_rate, 4 * c.hop, c.hop, c.n_mels)
        x = F.gelu(self.conv1(mel.t()[None].to(self.conv1.weight.dtype)))
        x = F.gelu(self.conv2(x)).transpose(1, 2)
        for b in self.enc:
            x = b(x)
        return self.rvq.encode(x[0])

    @torch.inference_mode()
    def decode(self, codes: torch.Tensor) -> torch.Tensor:
        x = self.rvq.decode(codes.to(self.rvq.codebooks.device))[None]
        for b in self.dec:
            x = b(x)
        y = self.out(F.gelu(self.up(x.transpose(1, 2))))
        return torch.tanh(y)[0, 0]

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]):
        params = dict(self.named_parameters())
        loaded = set()
        for n, w in weights:
            if n in params:
                params[n].data.copy_(w.to(params[n].dtype))
                loaded.add(n)
        return loaded


EntryClass = [MiMoAudioTokenizer]
