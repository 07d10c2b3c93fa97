"""Shared-secret authentication of the PD control plane (reference
`python/sgl_jax/srt/disaggregation/pd_auth.py`): HTTP endpoints take a bearer token derived
from the secret, side-channel messages carry an HMAC tag over their payload."""

from __future__ import annotations

import hashlib
import hmac
import os

ENV_SECRET = "SGLANG_PD_SHARED_SECRET"


def resolve_secret(explicit: str | None = None) -> str | None:
    return explicit or os.environ.get(ENV_SECRET) or None


def bearer_token(secret: str) -> str:
    return hmac.new(secret.encode(), b"sglang-pd-bearer", hashlib.sha256).hexdigest()


def auth_headers(secret: str | None) -> dict:
    return {"Authorization": f"Bearer {bearer_token(secret)}"} if secret else {}


def check_bearer(header_value: str | None, secret: str | None) -> bool:
    if not secret:
        return True
    if not header_value or not header_value.startswith("Bearer "):
        return False
    return hmac.compare_digest(header_value[len("Bearer "):], bearer_token(secret))


def sign(payload: bytes, secret: str | None) -> bytes:
    if not secret:
        return b""
    return hmac.new(secret.encode(), payload, hashlib.sha256).digest()


def verify(payload: bytes, tag: bytes, secret: str | None) -> bool:
    if not secret:
        return True
    return hmac.compare_digest(tag, sign(payload, secret))
