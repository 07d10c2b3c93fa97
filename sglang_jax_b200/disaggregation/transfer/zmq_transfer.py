"""KV page transfer between engines.

The reference moves KV with `jax.experimental.transfer` (or the optional native
`tpu-raiden` extension): prefill registers gathered arrays under a transfer id, decode pulls
them (`disaggregation/jax_transfer/{wrapper,conn}.py`).  Same pull model here, two data paths
behind one control channel (a ZMQ ROUTER socket on the prefill side):

* `mode="tcp"`: the reply carries the bytes of the requested pages, layer by layer.  On a GPU
  the pages are gathered into pinned host memory by the page-copy kernel before they are sent
  and scattered from pinned memory after they are received.  Works across nodes and on CPU.
* `mode="cuda_ipc"`: both engines sit in one NVLink domain.  The reply carries CUDA IPC handles
  of the prefill engine's KV layer buffers (once per peer) and the page ids; the decode engine
  maps them, gathers the pages on the exporting GPU, moves them with one device-to-device copy
  per layer over NVLink and scatters them into its own pool — no host staging.
"""

from __future__ import annotations

import json
import logging
import threading
import time

import numpy as np
import torch

from .. import pd_auth
from ...mem_cache.host_kv_pool import _layer_views

logger = logging.getLogger(__name__)

NOT_READY = b"not_ready"


class TransferError(RuntimeError):
    pass


class ZmqTransferBackend:
    name = "zmq"

    def __init__(self, device_pool, host: str = "127.0.0.1", port: int = 0, mode: str = "tcp",
                 secret: str | None = None, pull_timeout: float = 30.0, staging_pages: int = 0):
        """`staging_pages` > 0 (host-staged mode on a GPU): a `QueueHostKVPool` of that many pinned pages that the
        transfer threads reserve from, instead of allocating pinned memory per transfer."""
        self.views = _layer_views(device_pool)
        self.staging = None
        if staging_pages > 0 and mode == "tcp" and self.views[0].is_cuda:
            from ...mem_cache.host_kv_pool import QueueHostKVPool
            self.staging = QueueHostKVPool(device_pool, staging_pages)
        self.on_gpu = self.views[0].is_cuda
        if mode == "cuda_ipc" and not self.on_gpu:
            raise ValueError("cuda_ipc transfer needs the KV pool on a GPU")
        self.mode = mode
        self.host, self.port = host, port
        self.secret = secret
        self.pull_timeout = pull_timeout
        self.registered: dict[str, tuple[np.ndarray, dict]] = {}
        self.lock = threading.Lock()
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None
        self._ctx = None
        self._ipc_cache: dict[str, list[torch.Tensor]] = {}
        self._ipc_handles = None
        self.bytes_sent = 0
        self.bytes_received = 0
        self.addr: str | None = None
        self.peer_addrs: list[str] | None = None       # set on rank 0 of a tensor-parallel prefill engine
        self._peers_cache: dict[str, list[str]] = {}

    # ------------------------------------------------------------------ prefill side
    def start(self) -> str:
        import zmq
        self._ctx = zmq.Context.instance()
        sock = self._ctx.socket(zmq.ROUTER)
        sock.setsockopt(zmq.LINGER, 0)
        if self.port:
            sock.bind(f"tcp://{self.host}:{self.port}")
        else:
            self.port = sock.bind_to_random_port(f"tcp://{self.host}")
        self.addr = f"{self.host}:{self.port}"
        self._sock = sock
        self._thread = threading.Thread(target=self._serve, daemon=True, name="pd-transfer")
        self._thread.start()
        return self.addr

    def register(self, transfer_id: str, pages: np.ndarray, meta: dict) -> None:
        if self.on_gpu:
            # the KV of these pages must be complete before a peer may read it
            torch.cuda.current_stream(self.views[0].device).synchronize()
        with self.lock:
            self.registered[transfer_id] = (np.asarray(pages, np.int64).copy(), dict(meta))

    def unregister(self, transfer_id: str) -> None:
        with self.lock:
            self.registered.pop(transfer_id, None)

    def _serve(self):
        import zmq
        poller = zmq.Poller()
        poller.register(self._sock, zmq.POLLIN)
        while not self._stop.is_set():
            if not poller.poll(100):
                continue
            try:
                ident, tag, body = self._sock.recv_multipart()
            except Exception:  # noqa: BLE001
                continue
            if not pd_auth.verify(body, tag, self.secret):
                self._sock.send_multipart([ident, b"error", b"unauthorized"])
                continue
            req = json.loads(body)
            if req.get("op") == "peers":
                # transfer address of every tensor rank of this engine, rank 0 (this server) first
                self._sock.send_multipart([ident, b"ok", json.dumps(self.peer_addrs or [self.addr]).encode()])
                continue
            with self.lock:
                ent = self.registered.get(req["transfer_id"])
            if ent is None:
                self._sock.send_multipart([ident, NOT_READY, b""])
                continue
            pages, meta = ent
            try:
                self._sock.send_multipart([ident, b"ok"] + self._payload(pages, meta, req))
            except Exception as e:  # noqa: BLE001
                logger.exception("transfer reply failed")
                self._sock.send_multipart([ident, b"error", str(e).encode()])

    def _device_guard(self):
        """Transfers run on helper threads, whose current CUDA device is device 0 unless set: kernels and streams
        must belong to the GPU that holds this engine's pool."""
        import contextlib
        return torch.cuda.device(self.views[0].device) if self.on_gpu else contextlib.nullcontext()

    def _payload(self, pages: np.ndarray, meta: dict, req: dict) -> list[bytes]:
        with self._device_guard():
            return self._payload_on_device(pages, meta, req)

    def _payload_on_device(self, pages: np.ndarray, meta: dict, req: dict) -> list[bytes]:
        head = dict(meta, num_pages=int(len(pages)), mode=self.mode)
        if self.mode == "cuda_ipc":
            head["pages"] = pages.tolist()
            if req.get("need_handles", True):
                head["ipc_handles"] = self._export_handles()
            return [json.dumps(head).encode()]
        idx = torch.as_tensor(pages)
        frames = [json.dumps(head).encode()]
        stage_pages = self.staging.reserve(len(pages), self.pull_timeout) if self.staging is not None else None
        if stage_pages is not None:
            # pinned staging slots of the queue pool: device -> host with the page-copy kernel, then one frame per layer
            try:
                self.staging.backup_from_device(pages, stage_pages)
                torch.cuda.current_stream().synchronize()
                for layer in range(len(self.views)):
                    frames.append(self.staging.host_bytes(layer, stage_pages))
            finally:
                self.staging.release(stage_pages)
        elif self.on_gpu:
            from ...ops import native
            dev_idx = idx.to(self.views[0].device)
            seq = torch.arange(len(pages), device=dev_idx.device)
            for v in self.views:
                stage = torch.empty((len(pages), v.shape[1]), dtype=v.dtype, pin_memory=True)
                native.kv_page_copy(stage, v, seq, dev_idx)
                torch.cuda.current_stream().synchronize()
                frames.append(memoryview(stage.view(torch.uint8).numpy()).tobytes())
        else:
            for v in self.views:
                frames.append(v[idx].contiguous().view(torch.uint8).numpy().tobytes())
        self.bytes_sent += sum(len(f) for f in frames[1:])
        return frames

    def _export_handles(self):
        if self._ipc_handles is None:
            hs = []
            for v in self.views:
                st = v.untyped_storage()
                hs.append({"handle": [h if not isinstance(h, bytes) else h.hex() for h in st._share_cuda_()],
                           "shape": list(v.shape), "dtype": str(v.dtype).replace("torch.", ""),
                           "offset": v.storage_offset()})
            self._ipc_handles = hs
        return self._ipc_handles

    # ------------------------------------------------------------------ decode side
    def pull(self, addr: str, transfer_id: str, dst_pages: np.ndarray) -> dict:
        import zmq
        ctx = self._ctx or zmq.Context.instance()
        sock = ctx.socket(zmq.DEALER)
        sock.setsockopt(zmq.LINGER, 0)
        sock.connect(f"tcp://{addr}")
        try:
            deadline = time.monotonic() + self.pull_timeout
            body = json.dumps({"transfer_id": transfer_id, "need_handles": addr not in self._ipc_cache}).encode()
            while True:
                sock.send_multipart([pd_auth.sign(body, self.secret), body])
                left = deadline - time.monotonic()
                if left <= 0 or not sock.poll(int(min(left, 5.0) * 1000)):
                    if time.monotonic() >= deadline:
                        raise TransferError(f"pull of {transfer_id} from {addr} timed out")
                    continue
                frames = sock.recv_multipart()
                status = frames[0]
                if status == NOT_READY:
                    time.sleep(0.005)
                    continue
                if status != b"ok":
                    raise TransferError(f"pull of {transfer_id} refused: {frames[1].decode(errors='replace')}")
                head = json.loads(frames[1])
                if head["num_pages"] != len(dst_pages):
                    raise TransferError(f"page count mismatch: peer has {head['num_pages']}, "
                                        f"reserved {len(dst_pages)}")
                self._scatter(addr, head, frames[2:], np.asarray(dst_pages, np.int64))
                return head
        finally:
            sock.close()

    def query_peers(self, addr: str) -> list[str]:
        """Transfer addresses of all tensor ranks of the prefill engine whose rank 0 listens at `addr`."""
        if addr in self._peers_cache:
            return self._peers_cache[addr]
        import zmq
        sock = (self._ctx or zmq.Context.instance()).socket(zmq.DEALER)
        sock.setsockopt(zmq.LINGER, 0)
        sock.connect(f"tcp://{addr}")
        try:
            body = json.dumps({"op": "peers"}).encode()
            sock.send_multipart([pd_auth.sign(body, self.secret), body])
            if not sock.poll(int(self.pull_timeout * 1000)):
                raise TransferError(f"{addr} did not answer the peer-address query")
            frames = sock.recv_multipart()
            if frames[0] != b"ok":
                raise TransferError(f"peer-address query refused: {frames[1].decode(errors='replace')}")
            self._peers_cache[addr] = json.loads(frames[1])
            return self._peers_cache[addr]
        finally:
            sock.close()

    def _scatter(self, addr: str, head: dict, frames: list[bytes], dst_pages: np.ndarray):
        with self._device_guard():
            self._scatter_on_device(addr, head, frames, dst_pages)

    def _scatter_on_device(self, addr: str, head: dict, frames: list[bytes], dst_pages: np.ndarray):
        if head.get("mode") == "cuda_ipc":
            if "ipc_handles" in head:
                self._ipc_cache[addr] = [self._open_handle(h) for h in head["ipc_handles"]]
            peer = self._ipc_cache[addr]
            dev = self.views[0].device
            # The mapping of the prefill engine's pool belongs to ITS GPU's context inside this process.  Pages are
            # gathered there (a kernel of that GPU reading its own memory), cross NVLink as one device-to-device copy
            # per layer (the copy engine, no kernel dereferences another GPU's memory), and are scattered into this
            # engine's pool by a kernel of this GPU.
            src_dev = peer[0].device
            s_idx = torch.as_tensor(np.asarray(head["pages"], np.int64)).to(src_dev)
            d_idx = torch.as_tensor(dst_pages).to(dev)
            for dv, sv in zip(self.views, peer):
                with torch.cuda.device(src_dev):
                    staged = sv.index_select(0, s_idx)
                dv.index_copy_(0, d_idx, staged.to(dev, non_blocking=True))
            torch.cuda.current_stream(src_dev).synchronize()
            torch.cuda.current_stream(dev).synchronize()
            self.bytes_received += sum(v.shape[1] * v.element_size() for v in self.views) * len(dst_pages)
            return
        if len(frames) != len(self.views):
            raise TransferError(f"peer sent {len(frames)} layers, this engine has {len(self.views)}")
        idx = torch.as_tensor(dst_pages)
        for v, raw in zip(self.views, frames):
            want = len(dst_pages) * v.shape[1] * v.element_size()
            if len(raw) != want:
                raise TransferError(f"layer payload is {len(raw)} bytes, expected {want}")
        stage_pages = self.staging.reserve(len(dst_pages), self.pull_timeout) if self.staging is not None else None
        if stage_pages is not None:
            try:
                for layer, raw in enumerate(frames):
                    self.staging.fill_host(layer, stage_pages, raw)
                    self.bytes_received += len(raw)
                self.staging.load_to_device(stage_pages, dst_pages)
                torch.cuda.current_stream().synchronize()
            finally:
                self.staging.release(stage_pages)
            return
        for v, raw in zip(self.views, frames):
            if self.on_gpu:
                from ...ops import native
                stage = torch.empty((len(dst_pages), v.shape[1]), dtype=v.dtype, pin_memory=True)
                stage.view(torch.uint8).view(-1).numpy()[:] = np.frombuffer(raw, np.uint8)
                seq = torch.arange(len(dst_pages), device=v.device)
                native.kv_page_copy(v, stage, idx.to(v.device), seq)
                torch.cuda.current_stream().synchronize()
            else:
                src = torch.frombuffer(bytearray(raw), dtype=torch.uint8).view(v.dtype).view(len(dst_pages), v.shape[1])
                v[idx] = src
            self.bytes_received += len(raw)

    @staticmethod
    def _open_handle(h: dict) -> torch.Tensor:
        args = [bytes.fromhex(x) if isinstance(x, str) else x for x in h["handle"]]
        st = torch.UntypedStorage._new_shared_cuda(*args)
        dtype = getattr(torch, h["dtype"])
        t = torch.empty(0, dtype=dtype, device=st.device).set_(st, h["offset"], h["shape"])
        return t

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
        try:
            self._sock.close()
        except Exception:  # noqa: BLE001
            pass
