"""The address other engines should use to reach this one."""

from __future__ import annotations

import os
import socket


def get_host_ip(explicit: str | None = None) -> str:
    if explicit:
        return explicit
    env = os.environ.get("SGLANG_HOST_IP")
    if env:
        return env
    try:
        s = socket.socket(socket.AF_INET, socket.SOCK_DGRAM)
        try:
            s.connect(("10.255.255.255", 1))     # no packet is sent; picks the outbound interface
            return s.getsockname()[0]
        finally:
            s.close()
    except OSError:
        return "127.0.0.1"
