"""`python -m sglang_jax_b200.disaggregation.run_bootstrap --port 8998` starts the registry."""

from __future__ import annotations

import argparse

from . import pd_auth
from .bootstrap import DEFAULT_TTL, Registry, build_app


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--host", default="0.0.0.0")
    ap.add_argument("--port", type=int, default=8998)
    ap.add_argument("--ttl", type=float, default=DEFAULT_TTL)
    ap.add_argument("--shared-secret", default=None)
    ap.add_argument("--log-level", default="info")
    a = ap.parse_args(argv)
    import uvicorn
    uvicorn.run(build_app(Registry(a.ttl), pd_auth.resolve_secret(a.shared_secret)), host=a.host, port=a.port,
                log_level=a.log_level.lower())


if __name__ == "__main__":
    main()
