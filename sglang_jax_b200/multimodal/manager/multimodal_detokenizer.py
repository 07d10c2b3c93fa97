"""Turns the last stage's tensors into API payloads: PNG / raw frames for images and videos,
WAV for audio (reference `multimodal/manager/multimodal_detokenizer.py`)."""

from __future__ import annotations

import base64
import io
import struct
import zlib

import numpy as np


def encode_png(rgb: np.ndarray) -> bytes:
    """`rgb [H, W, 3]` uint8 -> PNG bytes (stored with zlib, no external imaging library)."""
    h, w, c = rgb.shape
    assert c == 3 and rgb.dtype == np.uint8
    raw = b"".join(b"\x00" + rgb[y].tobytes() for y in range(h))

    def chunk(tag: bytes, data: bytes) -> bytes:
        return struct.pack(">I", len(data)) + tag + data + struct.pack(">I", zlib.crc32(tag + data) & 0xFFFFFFFF)

    return (b"\x89PNG\r\n\x1a\n" + chunk(b"IHDR", struct.pack(">IIBBBBB", w, h, 8, 2, 0, 0, 0))
            + chunk(b"IDAT", zlib.compress(raw, 6)) + chunk(b"IEND", b""))


def encode_wav(samples: np.ndarray, rate: int = 24000) -> bytes:
    pcm = (np.clip(samples, -1, 1) * 32767).astype("<i2").tobytes()
    return (b"RIFF" + struct.pack("<I", 36 + len(pcm)) + b"WAVEfmt " + struct.pack("<IHHIIHH", 16, 1, 1, rate, rate * 2, 2, 16)
            + b"data" + struct.pack("<I", len(pcm)) + pcm)


class MultimodalDetokenizer:
    def image_payload(self, pixels, fmt: str = "b64_png") -> dict:
        """`pixels [C, T, H, W]` uint8 tensor."""
        arr = pixels.numpy()
        frames = [np.ascontiguousarray(arr[:3, t].transpose(1, 2, 0)) for t in range(arr.shape[1])]
        if fmt == "raw":
            return {"frames": [f.tolist() for f in frames]}
        return {"b64_png": [base64.b64encode(encode_png(f)).decode() for f in frames],
                "width": int(arr.shape[3]), "height": int(arr.shape[2]), "num_frames": len(frames)}

    def audio_payload(self, wave, rate: int = 24000) -> bytes:
        return encode_wav(np.asarray(wave, np.float32), rate)
