"""Small helpers shared by the speculative workers (reference
`python/sgl_jax/srt/speculative/spec_utils.py`)."""

from __future__ import annotations

import os


def simulated_accept_len() -> int | None:
    """`SGLANG_SIMULATE_ACC_LEN=<n>` forces every verification to accept `n` draft tokens,
    which lets throughput be measured for a given acceptance rate with an untrained draft
    head (the generated text is then meaningless)."""
    v = os.environ.get("SGLANG_SIMULATE_ACC_LEN")
    if v is None or v == "":
        return None
    n = int(float(v))
    return n if n >= 0 else None


def validate_spec_args(num_steps: int, topk: int, num_draft_tokens: int) -> None:
    if num_steps < 1 or topk < 1 or num_draft_tokens < 2:
        raise ValueError("speculative decoding needs num_steps >= 1, eagle_topk >= 1 and num_draft_tokens >= 2")
    if topk == 1 and num_draft_tokens != num_steps + 1:
        raise ValueError("with eagle_topk == 1 the tree is a chain: num_draft_tokens must be num_steps + 1")
    max_nodes = topk + (num_steps - 1) * topk * topk + 1
    if num_draft_tokens > max_nodes:
        raise ValueError(f"num_draft_tokens {num_draft_tokens} exceeds the {max_nodes} nodes the draft can propose")
