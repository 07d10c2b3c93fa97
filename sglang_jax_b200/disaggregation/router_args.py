"""Arguments of the PD router (reference `python/sgl_jax/srt/disaggregation/router_args.py`)."""

from __future__ import annotations

import argparse
import dataclasses


@dataclasses.dataclass
class RouterArgs:
    host: str = "0.0.0.0"
    port: int = 8000
    prefill_urls: list[str] = dataclasses.field(default_factory=list)
    decode_urls: list[str] = dataclasses.field(default_factory=list)
    bootstrap_url: str | None = None
    policy: str = "round_robin"            # round_robin | random | shortest_queue
    shared_secret: str | None = None
    request_timeout: float = 600.0
    health_check_interval: float = 5.0
    max_concurrent_requests: int = 0       # 0 = no limit; more wait at the router instead of piling up on the engines
    prefill_bootstrap_host: str | None = None   # host written into forwarded requests instead of the registered one

    @staticmethod
    def add_cli_args(p: argparse.ArgumentParser):
        p.add_argument("--host", default="0.0.0.0")
        p.add_argument("--port", type=int, default=8000)
        p.add_argument("--prefill", dest="prefill_urls", nargs="*", default=[], help="prefill engine URLs")
        p.add_argument("--decode", dest="decode_urls", nargs="+", required=True, help="decode engine URLs")
        p.add_argument("--bootstrap-url", default=None,
                       help="discover prefill engines from the bootstrap registry instead of --prefill")
        p.add_argument("--policy", default="round_robin", choices=["round_robin", "random", "shortest_queue"])
        p.add_argument("--shared-secret", default=None)
        p.add_argument("--request-timeout", "--request-timeout-secs", dest="request_timeout", type=float, default=600.0)
        p.add_argument("--max-concurrent-requests", type=int, default=0,
                       help="upper bound on requests running through the router at once (0: unlimited)")
        p.add_argument("--prefill-bootstrap-host", default=None,
                       help="override the host of the prefill engine's transfer address in forwarded requests "
                            "(engines registered under an address the decode side cannot reach)")
        # accepted for command lines written for the reference launcher: this router is always the mini
        # load balancer for PD pairs
        p.add_argument("--mini-lb", action="store_true")
        p.add_argument("--pd-disaggregation", action="store_true")
        p.add_argument("--test-external-dp-routing", action="store_true")
        p.add_argument("--health-check-interval", type=float, default=5.0)

    @classmethod
    def from_cli_args(cls, a: argparse.Namespace) -> "RouterArgs":
        return cls(**{f.name: getattr(a, f.name) for f in dataclasses.fields(cls)})
