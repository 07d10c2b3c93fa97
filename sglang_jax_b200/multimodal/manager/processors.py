"""Media preprocessing for the understanding pipelines (reference
`python/sgl_jax/srt/multimodal/manager/multimodal_tokenizer.py`, which delegates to the HF
processors): images / video frames -> flattened patch rows + `(t, h, w)` grids in the Qwen2-VL
layout, waveforms -> Whisper-style log-mel spectrograms, and expansion of the single
`<|image_pad|>` / `<|audio_pad|>` placeholders of a chat-templated prompt to one token per
encoder output."""

from __future__ import annotations

import base64
import io
import math

import numpy as np
import torch

OPENAI_CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
OPENAI_CLIP_STD = (0.26862954, 0.26130258, 0.27577711)


def smart_resize(height: int, width: int, factor: int = 28, min_pixels: int = 56 * 56,
                 max_pixels: int = 14 * 14 * 4 * 1280) -> tuple[int, int]:
    """Closest size whose sides are multiples of `factor`, with the pixel count inside
    [min_pixels, max_pixels] and the aspect ratio kept as far as possible."""
    if max(height, width) / min(height, width) > 200:
        raise ValueError("aspect ratio above 200 is not supported")
    h = max(factor, round(height / factor) * factor)
    w = max(factor, round(width / factor) * factor)
    if h * w > max_pixels:
        beta = math.sqrt(height * width / max_pixels)
        h = max(factor, math.floor(height / beta / factor) * factor)
        w = max(factor, math.floor(width / beta / factor) * factor)
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * beta / factor) * factor
        w = math.ceil(width * beta / factor) * factor
    return h, w


def load_image(src) -> "np.ndarray":
    """`src`: PIL image, `[H, W, 3]` uint8 array, raw bytes, a `data:` URI or base64 text -> RGB uint8 array."""
    from PIL import Image
    if isinstance(src, np.ndarray):
        return src
    if isinstance(src, str):
        if src.startswith("data:"):
            src = src.split(",", 1)[1]
        src = base64.b64decode(src)
    if isinstance(src, (bytes, bytearray)):
        src = Image.open(io.BytesIO(src))
    return np.asarray(src.convert("RGB"))


def frames_to_patches(frames: np.ndarray, patch_size: int = 14, merge_size: int = 2, temporal_patch_size: int = 2,
                      mean=OPENAI_CLIP_MEAN, std=OPENAI_CLIP_STD, min_pixels: int = 56 * 56,
                      max_pixels: int = 14 * 14 * 4 * 1280, resize: bool = True):
    """`frames [T, H, W, 3]` uint8 (T = 1 for an image) -> (`pixel_values [t*h*w, 3*tp*p*p]` float32,
    `grid (t, h, w)`); rows are ordered frame-group, then `merge x merge` blocks of patches, as the
    vision encoders expect."""
    from PIL import Image
    T, H, W, _ = frames.shape
    if resize:
        rh, rw = smart_resize(H, W, patch_size * merge_size, min_pixels, max_pixels)
        if (rh, rw) != (H, W):
            frames = np.stack([np.asarray(Image.fromarray(f).resize((rw, rh), Image.BICUBIC)) for f in frames])
            H, W = rh, rw
    x = frames.astype(np.float32) / 255.0
    x = (x - np.asarray(mean, np.float32)) / np.asarray(std, np.float32)
    x = x.transpose(0, 3, 1, 2)                                         # [T, C, H, W]
    if T % temporal_patch_size:
        x = np.concatenate([x, np.repeat(x[-1:], temporal_patch_size - T % temporal_patch_size, 0)])
    gt, gh, gw = x.shape[0] // temporal_patch_size, H // patch_size, W // patch_size
    m, p, tp = merge_size, patch_size, temporal_patch_size
    x = x.reshape(gt, tp, 3, gh // m, m, p, gw // m, m, p)
    x = x.transpose(0, 3, 6, 4, 7, 2, 1, 5, 8)                          # gt, gh/m, gw/m, m, m, C, tp, p, p
    return np.ascontiguousarray(x.reshape(gt * gh * gw, 3 * tp * p * p)), (gt, gh, gw)


def hz_to_mel(f):
    """Slaney scale (linear below 1 kHz, logarithmic above)."""
    f = np.asarray(f, np.float64)
    lin = f / (200.0 / 3)
    log = 15.0 + np.log(np.maximum(f, 1e-10) / 1000.0) / (np.log(6.4) / 27.0)
    return np.where(f >= 1000.0, log, lin)


def mel_to_hz(m):
    m = np.asarray(m, np.float64)
    lin = m * (200.0 / 3)
    log = 1000.0 * np.exp((np.log(6.4) / 27.0) * (m - 15.0))
    return np.where(m >= 15.0, log, lin)


def mel_filter_bank(n_freqs: int, n_mels: int, sr: int, fmin: float = 0.0, fmax: float | None = None) -> np.ndarray:
    """Slaney-normalised triangular filters `[n_freqs, n_mels]`."""
    fmax = fmax or sr / 2
    freqs = np.linspace(0, sr / 2, n_freqs)
    pts = mel_to_hz(np.linspace(hz_to_mel(fmin), hz_to_mel(fmax), n_mels + 2))
    d = np.diff(pts)
    slopes = pts[None, :] - freqs[:, None]
    down, up = -slopes[:, :-2] / d[:-1], slopes[:, 2:] / d[1:]
    fb = np.maximum(0, np.minimum(down, up))
    return fb * (2.0 / (pts[2:] - pts[:-2]))[None, :]


def log_mel_spectrogram(wave, sr: int = 16000, n_fft: int = 400, hop: int = 160, n_mels: int = 128) -> torch.Tensor:
    """Whisper-style features `[n_mels, frames]`: Hann STFT power, Slaney mel filters, log10, floor
    at 8 dB below the peak, affine to roughly [-1, 1]."""
    w = torch.as_tensor(np.asarray(wave), dtype=torch.float32)
    win = torch.hann_window(n_fft)
    st = torch.stft(w, n_fft, hop, window=win, return_complex=True)
    mag = st[..., :-1].abs() ** 2
    fb = torch.from_numpy(mel_filter_bank(n_fft // 2 + 1, n_mels, sr)).float()
    spec = torch.clamp(fb.T @ mag, min=1e-10).log10()
    spec = torch.maximum(spec, spec.max() - 8.0)
    return (spec + 4.0) / 4.0


def expand_placeholders(input_ids: list[int], token_id: int, counts: list[int]) -> list[int]:
    """Replace the i-th occurrence of `token_id` by `counts[i]` copies (one per encoder output)."""
    out, k = [], 0
    for t in input_ids:
        if t == token_id:
            if k >= len(counts):
                raise ValueError("more placeholder tokens than media items")
            out.extend([token_id] * counts[k])
            k += 1
        else:
            out.append(t)
    if k != len(counts):
        raise ValueError(f"{len(counts)} media items for {k} placeholder tokens")
    return out
