"""Process-wide tunables read from the environment.

Same knobs as the reference's `python/sgl_jax/global_config.py:24-51`
(new-token-ratio schedule, retract step count), expressed as a frozen-at-import
dataclass so the scheduler can snapshot them.
"""

from __future__ import annotations

import os
from dataclasses import dataclass


def _f(name: str, default: float) -> float:
    return float(os.environ.get(name, default))


def _i(name: str, default: int) -> int:
    return int(os.environ.get(name, default))


@dataclass
class GlobalConfig:
    # Fraction of `max_new_tokens` each running request is assumed to still need
    # when the scheduler decides whether another prefill fits.
    default_init_new_token_ratio: float = _f("SGLANG_INIT_NEW_TOKEN_RATIO", 0.7)
    default_min_new_token_ratio_factor: float = _f("SGLANG_MIN_NEW_TOKEN_RATIO_FACTOR", 0.14)
    default_new_token_ratio_decay_steps: int = _i("SGLANG_NEW_TOKEN_RATIO_DECAY_STEPS", 600)
    # How many decode steps of head-room a retraction must free.
    retract_decode_steps: int = _i("SGLANG_RETRACT_DECODE_STEPS", 20)
    # Upper bound used when estimating how many tokens a request will still emit.
    clip_max_new_tokens_estimation: int = _i("SGLANG_CLIP_MAX_NEW_TOKENS_ESTIMATION", 4096)
    # Token rows below which a row-parallel output stays replicated instead of
    # being reduce-scattered over the tensor ranks.
    scatter_min_local_size: int = _i("SGLANG_SCATTER_MIN_LOCAL_SIZE", 128)
    # Streaming is forced at least every this many decode steps.
    default_force_stream_interval: int = 50
    # Detokenizer keeps at most this many per-request states.
    detokenizer_max_states: int = _i("SGLANG_DETOKENIZER_MAX_STATES", 1 << 16)


global_config = GlobalConfig()
