"""Wiring of the PD pieces into a scheduler and their shutdown (reference
`python/sgl_jax/srt/disaggregation/runtime.py:18`, `:163`)."""

from __future__ import annotations

import logging
import os

from . import pd_auth
from .bootstrap import BootstrapClient, HeartbeatDaemon
from .common.core import CommonKVManager
from .host_ip import get_host_ip
from .factory import create_transfer_backend, pick_transfer_mode  # noqa: F401

logger = logging.getLogger(__name__)


def kv_layout_of(scheduler) -> dict:
    from ..mem_cache.host_kv_pool import _layer_views
    views = _layer_views(scheduler.token_to_kv_pool)
    return {"page_size": scheduler.page_size, "num_layers": len(views),
            "page_bytes_per_layer": [int(v.shape[1] * v.element_size()) for v in views],
            "dtype": str(views[0].dtype).replace("torch.", ""), "tp_size": scheduler.server_args.tp_size,
            "model": scheduler.model_config.architectures[0] if scheduler.model_config is not None else ""}


def build_kv_manager(scheduler, role: str, engine_id: str):
    sa = scheduler.server_args
    secret = pd_auth.resolve_secret(sa.disaggregation_shared_secret)
    host = get_host_ip(sa.disaggregation_host_ip) if sa.disaggregation_host_ip else "127.0.0.1"
    if os.environ.get("DISAGG_LAUNCH_BOOTSTRAP", "") == "1" and getattr(scheduler, "disagg_bootstrap_server", None) is None:
        # one engine of the deployment hosts the registry itself (reference `runtime.py:66`), on
        # `--disaggregation-bootstrap-port`
        from .bootstrap import BootstrapServer
        scheduler.disagg_bootstrap_server = BootstrapServer(host, sa.disaggregation_bootstrap_port, secret=secret).start()
        logger.info("embedded PD bootstrap server at %s", scheduler.disagg_bootstrap_server.url)
        if not sa.disaggregation_bootstrap_url:
            sa.disaggregation_bootstrap_url = scheduler.disagg_bootstrap_server.url
    layout = kv_layout_of(scheduler)
    backend = create_transfer_backend(scheduler.token_to_kv_pool, sa, local_host=host, role=role, shared_secret=secret,
                                      max_req_input_len=getattr(scheduler, "max_req_input_len", None))
    transfer_addr = backend.start() if role == "prefill" else None
    mirror = None
    worker = scheduler.tp_worker
    if getattr(worker, "tp_size", 1) > 1 and hasattr(worker, "send_control"):
        from .tp_mirror import RankMirror
        mirror = RankMirror(worker, role, host, secret, backend.mode, sa.disaggregation_pull_timeout_seconds, transfer_addr)
        if role == "prefill":
            backend.peer_addrs = mirror.addrs
    mgr = CommonKVManager(role, backend, sum(layout["page_bytes_per_layer"]), host,
                          sa.disaggregation_side_channel_port if role == "prefill" else 0, secret,
                          sa.disaggregation_channel_number, sa.disaggregation_pull_timeout_seconds,
                          sa.disaggregation_ack_timeout_seconds, sa.disaggregation_orphan_reaper_interval_seconds,
                          mirror=mirror)
    hb = None
    if role == "prefill":
        info = dict(layout, engine_id=engine_id, tp_rank=0, transfer_addr=transfer_addr, ack_addr=mgr.ack_addr,
                    transfer_addrs=backend.peer_addrs or [transfer_addr],
                    http_url=f"http://{sa.host}:{sa.port}", transfer_mode=backend.mode)
        client = BootstrapClient(sa.disaggregation_bootstrap_url, secret, sa.disaggregation_bootstrap_timeout_seconds)
        hb = HeartbeatDaemon(client, info).start()
        logger.info("PD prefill engine %s registered: transfer %s, ack %s (%s)", engine_id, transfer_addr,
                    mgr.ack_addr, backend.mode)
    return mgr, hb


def shutdown_disaggregation(scheduler, drain_timeout: float = 10.0):
    mgr = getattr(scheduler, "disagg_kv_manager", None)
    hb = getattr(scheduler, "disagg_heartbeat", None)
    wd = getattr(scheduler, "disagg_decode_watchdog", None)
    if wd is not None:
        wd.stop()
    if hb is not None:
        hb.stop()          # stop advertising first, then let running transfers finish
    if mgr is not None:
        if not mgr.drain(drain_timeout):
            logger.warning("PD shutdown: %d transfers still in flight", mgr.inflight())
        mgr.shutdown()
    srv = getattr(scheduler, "disagg_bootstrap_server", None)
    if srv is not None:
        srv.stop()
        scheduler.disagg_bootstrap_server = None
