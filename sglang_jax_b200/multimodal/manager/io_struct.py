"""Messages of the multimodal pipeline (reference `multimodal/manager/io_struct.py`)."""

from __future__ import annotations

import dataclasses
import time
import uuid
from typing import Any


@dataclasses.dataclass
class GenerateMMReqInput:
    """Image / video generation request as it arrives at the HTTP layer."""
    prompt: str = ""
    negative_prompt: str | None = None
    height: int = 64
    width: int = 64
    num_frames: int = 1
    num_inference_steps: int = 8
    guidance_scale: float = 1.0
    seed: int = 0
    output_format: str = "b64_png"
    rid: str = dataclasses.field(default_factory=lambda: uuid.uuid4().hex)


@dataclasses.dataclass
class TokenizedGenerateMMReqInput:
    rid: str
    input_ids: list[int]
    negative_input_ids: list[int] | None
    height: int
    width: int
    num_frames: int
    num_inference_steps: int
    guidance_scale: float
    seed: int
    output_format: str = "b64_png"


@dataclasses.dataclass
class TokenizedGenerateOmniReqInput:
    """Vision-language / omni request: token ids with placeholder runs plus the media tensors."""
    rid: str
    input_ids: list[int]
    pixel_values: Any = None            # [num_patches, patch_dim]
    image_grid_thw: Any = None          # [num_images, 3]
    audio_features: Any = None          # log-mel spectrogram [num_mel_bins, frames]
    sampling_params: dict = dataclasses.field(default_factory=dict)
    audio_feature_lens: Any = None      # frames per clip when several clips are concatenated


@dataclasses.dataclass
class TokenizedGenerateAudioReqInput:
    rid: str
    input_ids: list[int] | None = None
    audio: Any = None                   # waveform (ASR) or None (TTS)
    task: str = "tts"                   # tts | asr
    sampling_params: dict = dataclasses.field(default_factory=dict)


@dataclasses.dataclass
class AbortMMReq:
    rid: str


@dataclasses.dataclass
class MMReq:
    """A request travelling through the stages; each stage reads and adds fields of `data`."""
    rid: str
    kind: str                           # image | video | omni | audio
    data: dict = dataclasses.field(default_factory=dict)
    created: float = dataclasses.field(default_factory=time.time)
    aborted: bool = False
    error: str | None = None
    stage_times: dict = dataclasses.field(default_factory=dict)


@dataclasses.dataclass
class MMOutput:
    rid: str
    kind: str
    result: Any = None                  # image/video tensor, token ids, waveform, text
    error: str | None = None
    meta: dict = dataclasses.field(default_factory=dict)
