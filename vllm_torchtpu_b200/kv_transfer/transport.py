"""Block transports (data plane) and side channels (control plane) of the KV connectors.

Data plane
  ``LocalTransport``  pools of engines living in one process (tests, single-process P/D);
                      CPU pools are copied with index ops, CUDA pools with the block-copy kernel.
  ``IpcTransport``    pools of other processes on the same node: the producer exports one CUDA IPC
                      handle per layer, the consumer maps them once and pulls blocks GPU→GPU over
                      NVLink with ONE kernel launch per transfer (all layers, all blocks).
Control plane
  ``InProcessChannel``  dictionary of endpoints (tests);
  ``TcpChannel``        length-prefixed, HMAC-signed JSON messages over TCP on 127.0.0.1 or the node
                        address; requests time out instead of blocking forever.

Replaces the reference's host-staged D2H → shm → ZMQ → H2D path and its native DMA engine
(reference: src/vllm_torchtpu/distributed/kv_transfer/zmq_shm_base.py:14-170, tpu_connector.py:4119-4235).
"""
from __future__ import annotations

import ctypes
import socket
import socketserver
import struct
import threading
from typing import Callable, Optional

import torch

from ..logger import init_logger
from .base import sign_message, verify_message

logger = init_logger(__name__)


class TransferError(RuntimeError):
    pass


# ------------------------------------------------------------------ data plane
class PoolInfo:
    def __init__(self, engine_id: str, layers: list):
        self.engine_id = engine_id
        self.layers = layers                       # list of tensors [num_blocks, ...]
        self.num_blocks = layers[0].shape[0]
        self.block_bytes = layers[0][0].numel() * layers[0].element_size()
        self._ptr_table = None

    def ptr_table(self) -> torch.Tensor:
        if self._ptr_table is None:
            self._ptr_table = torch.tensor([t.data_ptr() for t in self.layers], dtype=torch.int64,
                                           device=self.layers[0].device)
        return self._ptr_table


def copy_blocks(src: PoolInfo, dst: PoolInfo, src_ids: list, dst_ids: list) -> None:
    """dst[dst_ids[i]] <- src[src_ids[i]] for every layer."""
    if len(src_ids) != len(dst_ids):
        raise TransferError("block id lists differ in length")
    if not src_ids:
        return
    if src.block_bytes != dst.block_bytes or len(src.layers) != len(dst.layers):
        raise TransferError("source and destination pools have different geometry")
    if max(src_ids) >= src.num_blocks or max(dst_ids) >= dst.num_blocks or min(src_ids + dst_ids) < 0:
        raise TransferError("block id out of range")
    if dst.layers[0].is_cuda or src.layers[0].is_cuda:
        # one side may be pinned, device-mapped host memory (offload tier): the kernel reads or
        # writes it through unified addressing
        from ..ops import cuda
        dev = dst.layers[0].device if dst.layers[0].is_cuda else src.layers[0].device
        s = torch.tensor(src_ids, dtype=torch.int32, device=dev)
        d = torch.tensor(dst_ids, dtype=torch.int32, device=dev)
        ws = cuda.Workspace.get(dev)
        # both tables stay referenced until the launch is queued: a device copy of a host pool's table
        # is a temporary, and its block must not be handed to the other table's allocation
        src_tbl, dst_tbl = src.ptr_table().to(dev), dst.ptr_table().to(dev)
        cuda._check(cuda.lib().b200_kv_copy_blocks(
            cuda._p(src_tbl), cuda._p(dst_tbl), cuda._p(s), cuda._p(d),
            ctypes.c_int(len(src_ids)), ctypes.c_int(len(src.layers)), ctypes.c_size_t(src.block_bytes),
            ctypes.c_longlong(src.num_blocks), ctypes.c_longlong(dst.num_blocks), cuda._p(ws.status),
            cuda._stream()), "kv_copy_blocks")
        from ..ops import count_launch
        count_launch()
        return
    si, di = torch.tensor(src_ids), torch.tensor(dst_ids)
    for a, b in zip(src.layers, dst.layers):
        b[di] = a[si].to(b.dtype)


def copy_block_spans(src: PoolInfo, dst: PoolInfo, src_ids: list, dst_ids: list, span) -> None:
    """Part of every block (``reshard.Span``): pools of different block sizes, e.g. a head range of a
    tensor-parallel producer into the blocks of a consumer with another degree."""
    if len(src_ids) != len(dst_ids):
        raise TransferError("block id lists differ in length")
    if not src_ids:
        return
    if len(src.layers) != len(dst.layers):
        raise TransferError("source and destination pools have different layer counts")
    if max(src_ids) >= src.num_blocks or max(dst_ids) >= dst.num_blocks or min(src_ids + dst_ids) < 0:
        raise TransferError("block id out of range")
    last = (span.chunks - 1)
    if (span.src_off + last * span.src_stride + span.nbytes > src.block_bytes
            or span.dst_off + last * span.dst_stride + span.nbytes > dst.block_bytes):
        raise TransferError("span leaves the block")
    if dst.layers[0].is_cuda or src.layers[0].is_cuda:
        from ..ops import count_launch, cuda
        dev = dst.layers[0].device if dst.layers[0].is_cuda else src.layers[0].device
        s = torch.tensor(src_ids, dtype=torch.int32, device=dev)
        d = torch.tensor(dst_ids, dtype=torch.int32, device=dev)
        ws = cuda.Workspace.get(dev)
        src_tbl, dst_tbl = src.ptr_table().to(dev), dst.ptr_table().to(dev)
        z = ctypes.c_size_t
        cuda._check(cuda.lib().b200_kv_copy_block_spans(
            cuda._p(src_tbl), cuda._p(dst_tbl), cuda._p(s), cuda._p(d), ctypes.c_int(len(src_ids)),
            ctypes.c_int(len(src.layers)), z(src.block_bytes), z(dst.block_bytes), z(span.src_off), z(span.dst_off),
            z(span.nbytes), ctypes.c_int(span.chunks), z(span.src_stride), z(span.dst_stride),
            ctypes.c_longlong(src.num_blocks), ctypes.c_longlong(dst.num_blocks), cuda._p(ws.status),
            cuda._stream()), "kv_copy_block_spans")
        count_launch()
        return
    si, di = torch.tensor(src_ids), torch.tensor(dst_ids)
    for a, b in zip(src.layers, dst.layers):
        av = a.reshape(a.shape[0], -1).view(torch.uint8)
        bv = b.reshape(b.shape[0], -1).view(torch.uint8)
        for c in range(span.chunks):
            so, do = span.src_off + c * span.src_stride, span.dst_off + c * span.dst_stride
            bv[di, do:do + span.nbytes] = av[si, so:so + span.nbytes]


def nan_blocks(pool: PoolInfo, block_ids: list) -> list:
    """Which of ``block_ids`` hold a non-finite bf16 value in any layer.  Saves and transfers of such
    blocks are refused: a poisoned block would otherwise be served to later requests
    (reference: src/vllm_torchtpu/distributed/kv_transfer/kv_save_nan_check.py:14-163)."""
    if not block_ids:
        return []
    first = pool.layers[0]
    if getattr(first, "dtype", None) != torch.bfloat16:
        return []
    if first.is_cuda:
        from ..ops import count_launch, cuda
        dev = first.device
        ids = torch.tensor(block_ids, dtype=torch.int32, device=dev)
        flags = torch.zeros(len(block_ids), dtype=torch.int32, device=dev)
        cuda._check(cuda.lib().b200_kv_nan_check(
            cuda._p(pool.ptr_table().to(dev)), cuda._p(ids), ctypes.c_int(len(block_ids)),
            ctypes.c_int(len(pool.layers)), ctypes.c_size_t(pool.block_bytes), cuda._p(flags), cuda._stream()),
            "kv_nan_check")
        count_launch()
        bad = flags.cpu().tolist()
    else:
        idx = torch.tensor(block_ids)
        bad = [0] * len(block_ids)
        for t in pool.layers:
            nf = ~torch.isfinite(t[idx].float()).flatten(1).all(1)
            bad = [b | int(x) for b, x in zip(bad, nf.tolist())]
    return [b for b, f in zip(block_ids, bad) if f]


class LocalTransport:
    _pools: dict = {}

    def __init__(self, engine_id: str):
        self.engine_id = engine_id

    def register_pool(self, layers: list) -> None:
        LocalTransport._pools[self.engine_id] = PoolInfo(self.engine_id, layers)

    def export(self) -> dict:
        p = LocalTransport._pools[self.engine_id]
        return {"engine_id": self.engine_id, "num_blocks": p.num_blocks, "block_bytes": p.block_bytes,
                "num_layers": len(p.layers), "kind": "local"}

    def open_remote(self, info: dict) -> None:
        if info["engine_id"] not in LocalTransport._pools:
            raise TransferError(f"unknown engine {info['engine_id']}")

    def pull(self, remote_engine: str, remote_ids: list, local_ids: list, span=None) -> None:
        src = LocalTransport._pools.get(remote_engine)
        if src is None:
            raise TransferError(f"source engine {remote_engine} unreachable")
        if span is None:
            copy_blocks(src, LocalTransport._pools[self.engine_id], remote_ids, local_ids)
        else:
            copy_block_spans(src, LocalTransport._pools[self.engine_id], remote_ids, local_ids, span)


class _RawLayer:
    """Minimal tensor-like view of IPC-mapped remote memory for PoolInfo."""

    def __init__(self, ptr: int, num_blocks: int, block_bytes: int, device):
        self._ptr, self.shape, self._bb, self.device = ptr, (num_blocks,), block_bytes, device
        self.is_cuda = True

    def data_ptr(self):
        return self._ptr

    def element_size(self):
        return 1

    def __getitem__(self, i):
        class _B:
            def __init__(s, n):
                s._n = n

            def numel(s):
                return s._n
        return _B(self._bb)


class IpcTransport:
    """Pools in other processes of this node, mapped through CUDA IPC."""

    def __init__(self, engine_id: str):
        self.engine_id = engine_id
        self.local: Optional[PoolInfo] = None
        self.remotes: dict = {}
        self._handles: list = []

    def register_pool(self, layers: list) -> None:
        from ..ops import cuda
        self.local = PoolInfo(self.engine_id, layers)
        self._handles, self._offsets = [], []
        for t in layers:
            # the handle names the allocation that holds the tensor (a caching allocator's segment):
            # the consumer adds the tensor's offset to the address it gets from opening the handle
            base, size = ctypes.c_ulonglong(), ctypes.c_ulonglong()
            cuda._check(cuda.lib().b200_ipc_range(ctypes.c_void_p(t.data_ptr()), ctypes.byref(base),
                                                  ctypes.byref(size)), "ipc_range")
            h = (ctypes.c_ubyte * 64)()
            cuda._check(cuda.lib().b200_ipc_get_handle(ctypes.c_void_p(base.value), h), "ipc_get_handle")
            self._handles.append(bytes(h).hex())
            self._offsets.append(t.data_ptr() - base.value)

    def export(self) -> dict:
        p = self.local
        return {"engine_id": self.engine_id, "num_blocks": p.num_blocks, "block_bytes": p.block_bytes,
                "num_layers": len(p.layers), "kind": "ipc", "handles": self._handles, "offsets": self._offsets}

    def open_remote(self, info: dict) -> None:
        from ..ops import cuda
        if info["engine_id"] in self.remotes:
            return
        if info["num_layers"] != len(self.local.layers):
            raise TransferError("remote pool has another number of layers")
        layers = []
        opened: dict = {}                    # several layers may live in one exported allocation
        for hx, off in zip(info["handles"], info.get("offsets") or [0] * len(info["handles"])):
            if hx not in opened:
                buf = (ctypes.c_ubyte * 64).from_buffer_copy(bytes.fromhex(hx))
                p = ctypes.c_void_p()
                cuda._check(cuda.lib().b200_ipc_open(buf, ctypes.byref(p)), "ipc_open")
                opened[hx] = p.value
            layers.append(_RawLayer(opened[hx] + int(off), info["num_blocks"], info["block_bytes"],
                                    self.local.layers[0].device))
        pool = PoolInfo.__new__(PoolInfo)
        pool.engine_id, pool.layers = info["engine_id"], layers
        pool.num_blocks, pool.block_bytes, pool._ptr_table = info["num_blocks"], info["block_bytes"], None
        pool._ptr_table = torch.tensor([l.data_ptr() for l in layers], dtype=torch.int64,
                                       device=self.local.layers[0].device)
        self.remotes[info["engine_id"]] = pool

    def pull(self, remote_engine: str, remote_ids: list, local_ids: list, span=None) -> None:
        src = self.remotes.get(remote_engine)
        if src is None:
            raise TransferError(f"source engine {remote_engine} is not mapped")
        if span is None:
            copy_blocks(src, self.local, remote_ids, local_ids)
        else:
            copy_block_spans(src, self.local, remote_ids, local_ids, span)


# --------------------------------------------------------------- control plane
class InProcessChannel:
    _endpoints: dict = {}

    def __init__(self, name: str, handler: Callable[[dict], dict]):
        self.name = name
        InProcessChannel._endpoints[name] = handler
        self.dropped = 0
        self.drop_next = 0           # fault injection: drop this many requests

    def address(self):
        return ("inproc", self.name)

    def request(self, address, msg: dict, timeout_s: float = 5.0) -> dict:
        if self.drop_next > 0:
            self.drop_next -= 1
            self.dropped += 1
            raise TimeoutError("control message dropped")
        handler = InProcessChannel._endpoints.get(address[1])
        if handler is None:
            raise ConnectionError(f"no endpoint {address[1]}")
        return verify_message(sign_message(handler(verify_message(sign_message(msg)))))

    def close(self):
        InProcessChannel._endpoints.pop(self.name, None)


class TcpChannel:
    """Threaded TCP server for incoming requests plus a blocking client with a timeout."""

    def __init__(self, host: str, port: int, handler: Callable[[dict], dict]):
        outer = self

        class _H(socketserver.BaseRequestHandler):
            def handle(self):
                try:
                    raw = _recv_frame(self.request)
                    reply = handler(verify_message(raw))
                except PermissionError as e:
                    reply = {"ok": False, "error": str(e)}
                except Exception as e:                 # noqa: BLE001 - reported to the peer
                    reply = {"ok": False, "error": repr(e)}
                _send_frame(self.request, sign_message(reply))

        class _S(socketserver.ThreadingTCPServer):
            allow_reuse_address = True
            daemon_threads = True

        self.server = _S((host, port), _H)
        self.host, self.port = self.server.server_address
        self.thread = threading.Thread(target=self.server.serve_forever, name="KV:SideChannel", daemon=True)
        self.thread.start()

    def address(self):
        return (self.host, self.port)

    def request(self, address, msg: dict, timeout_s: float = 5.0) -> dict:
        with socket.create_connection(tuple(address), timeout=timeout_s) as s:
            s.settimeout(timeout_s)
            _send_frame(s, sign_message(msg))
            return verify_message(_recv_frame(s))

    def close(self):
        self.server.shutdown()
        self.server.server_close()


def _send_frame(sock, payload: bytes) -> None:
    sock.sendall(struct.pack("!I", len(payload)) + payload)


def _recv_frame(sock) -> bytes:
    hdr = _recv_exact(sock, 4)
    (n,) = struct.unpack("!I", hdr)
    if n > 64 * 2**20:
        raise ValueError("control frame too large")
    return _recv_exact(sock, n)


def _recv_exact(sock, n: int) -> bytes:
    buf = b""
    while len(buf) < n:
        chunk = sock.recv(n - len(buf))
        if not chunk:
            raise ConnectionError("peer closed the control connection")
        buf += chunk
    return buf
