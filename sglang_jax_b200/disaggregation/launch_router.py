"""`python -m sglang_jax_b200.disaggregation.launch_router --decode http://d:30000 --bootstrap-url http://b:8998`"""

from __future__ import annotations

import argparse

from .mini_lb import build_router_app
from .router_args import RouterArgs


def main(argv=None):
    ap = argparse.ArgumentParser(description="PD disaggregation router")
    RouterArgs.add_cli_args(ap)
    args = RouterArgs.from_cli_args(ap.parse_args(argv))
    import uvicorn
    uvicorn.run(build_router_app(args), host=args.host, port=args.port, log_level="info")


if __name__ == "__main__":
    main()
