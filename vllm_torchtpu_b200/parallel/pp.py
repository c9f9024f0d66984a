"""Pipeline parallelism: layer partition, validation and the stage hand-off.

Hand-off protocol (same contract as the reference's buffered point-to-point
hand-off, reference: src/vllm_torchtpu/distributed/pp_buffered.py:14-85,220-687):

* what travels is ``hidden + residual`` as ONE tensor in the model dtype (plus
  optional side tensors); the receiver starts from that sum and a zero residual;
* every stage runs the same sequence of forwards, so a per-process transfer
  counter numbers them alike everywhere and, with the tensor's place, gives the tag;
* receives are posted ahead of time by a posting thread (``begin_step`` queues one
  per forward of the step); at most ``max_posted`` receives may be outstanding;
* sends happen on a helper thread that first waits for the device fence recorded
  after the producing forward, so the compute stream never blocks on the link;
  at most ``depth`` forwards wait in the send queue (back-pressure on a stage
  that runs ahead);
* an error on a helper thread is captured and re-raised on the worker thread at
  its next call, and queued receives are cancelled;
* ``warmup`` sends a known pattern down the pipe and checks it on arrival.

On GPUs the transport is NCCL ``isend``/``irecv`` issued on a side stream so the
transfer overlaps the next forward.  Tests use a fake in-memory transport.
"""
from __future__ import annotations

import queue
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Optional

import torch

from .. import envs
from ..logger import init_logger

logger = init_logger(__name__)


def partition_layers(num_layers: int, pp_size: int) -> list:
    """Contiguous, as-even-as-possible layer ranges; later stages get the remainder
    (the last stage also owns the final norm and lm_head)."""
    base, rem = divmod(num_layers, pp_size)
    out, lo = [], 0
    for s in range(pp_size):
        n = base + (1 if s >= pp_size - rem else 0)
        out.append((lo, lo + n))
        lo += n
    return out


def validate_pipeline_parallel_config(cfg) -> None:
    """Every stage must hold at least one layer, and for hybrid models at least one
    full-attention layer (its KV blocks drive the scheduler's block accounting,
    reference: src/vllm_torchtpu/platforms/pp_validation.py:22-80)."""
    m, p = cfg.model, cfg.parallel
    pp = p.pipeline_parallel_size
    if pp > m.num_layers:
        raise ValueError(f"pipeline_parallel_size {pp} exceeds the {m.num_layers} layers")
    for lo, hi in partition_layers(m.num_layers, pp):
        if hi <= lo:
            raise ValueError("a pipeline stage would hold no layer")
        if m.is_hybrid_gdn and not any(m.layer_is_full_attention(i) for i in range(lo, hi)):
            raise ValueError(f"pipeline stage with layers [{lo},{hi}) holds no full-attention layer")
    if cfg.kv_transfer and cfg.kv_transfer.get("kv_connector") not in (
            "B200P2PConnector", "B200HostConnector", "B200MultiConnector", "B200OffloadingConnector"):
        raise ValueError("this KV connector is not supported under pipeline parallelism")


def buffered_steps_in_flight(pp_size: int) -> int:
    """The engine keeps ``stages + max(1, stages // 2)`` steps in flight
    (reference: src/vllm_torchtpu/distributed/pp_engine.py:44-56)."""
    return pp_size + max(1, pp_size // 2)


def check_buffered_receives(depth: int, pp_size: int, max_posted: int) -> None:
    if buffered_steps_in_flight(pp_size) + depth - 1 > max_posted + pp_size:
        raise ValueError(f"hand-off depth {depth} could hold more than {max_posted} posted receives")


class Transport:
    """isend/irecv with tags.  ``isend`` returns a handle whose ``wait()`` blocks until the
    data has left; ``irecv`` returns a handle whose ``wait()`` blocks until it has landed."""

    def isend(self, tensor: torch.Tensor, dst: int, tag: int):
        raise NotImplementedError

    def irecv(self, tensor: torch.Tensor, src: int, tag: int):
        raise NotImplementedError


class NcclTransport(Transport):
    """torch.distributed p2p on a dedicated CUDA stream."""

    def __init__(self, group=None):
        import torch.distributed as dist
        self.dist = dist
        self.group = group
        self.stream = torch.cuda.Stream() if torch.cuda.is_available() else None

    def isend(self, tensor, dst, tag):
        if self.stream is not None:
            with torch.cuda.stream(self.stream):
                return self.dist.isend(tensor, dst, group=self.group, tag=tag)
        return self.dist.isend(tensor, dst, group=self.group, tag=tag)

    def irecv(self, tensor, src, tag):
        if self.stream is not None:
            with torch.cuda.stream(self.stream):
                return self.dist.irecv(tensor, src, group=self.group, tag=tag)
        return self.dist.irecv(tensor, src, group=self.group, tag=tag)

    def drain(self) -> None:
        """Block the calling (helper) thread until the transfers issued so far have left: a NCCL
        handle's ``wait()`` only orders streams, and the payload is released right after."""
        if self.stream is not None:
            self.stream.synchronize()


@dataclass
class _PostedRecv:
    transfer: int
    tensors: list
    handles: list = field(default_factory=list)
    posted: threading.Event = field(default_factory=threading.Event)
    consumed: bool = False


class PPHandoff:
    TAG_STRIDE = 8          # tensors per transfer (main + side tensors)

    def __init__(self, transport: Transport, *, prev_rank: Optional[int], next_rank: Optional[int],
                 hidden_size: int, dtype: torch.dtype, device, depth: Optional[int] = None,
                 max_posted: Optional[int] = None, fence: Optional[Callable] = None,
                 side_widths: tuple = (), my_rank: int = 0):
        self.t = transport
        self.my_rank = my_rank
        self.prev_rank, self.next_rank = prev_rank, next_rank
        self.hidden_size, self.dtype, self.device = hidden_size, dtype, device
        self.depth = depth or envs.B200_PP_HANDOFF_DEPTH
        self.max_posted = max_posted or envs.B200_PP_MAX_POSTED_RECVS
        self.side_widths = tuple(side_widths)
        self._fence = fence or self._default_fence
        self._send_counter = 0
        self._recv_counter = 0
        self._error: Optional[BaseException] = None
        self._lock = threading.Lock()
        self._recv_queue: "queue.Queue" = queue.Queue()
        self._posted: dict = {}
        self._outstanding = 0
        self._outstanding_cv = threading.Condition()
        self._send_queue: "queue.Queue" = queue.Queue(maxsize=self.depth)
        self._stop = False
        self._zero_residual: dict = {}
        self._threads = []
        if prev_rank is not None:
            self._threads.append(threading.Thread(target=self._post_loop, name="PP:PostReceives", daemon=True))
        self._threads.append(threading.Thread(target=self._send_loop, name="PP:Send", daemon=True))
        for th in self._threads:
            th.start()

    # ---- helpers ---------------------------------------------------------------
    def _default_fence(self):
        if torch.cuda.is_available() and torch.device(self.device).type == "cuda":
            ev = torch.cuda.Event()
            ev.record()
            return ev.synchronize
        return lambda: None

    def _raise_pending(self):
        if self._error is not None:
            err, self._error = self._error, None
            raise RuntimeError(f"pipeline hand-off failed: {err!r}") from err

    def _fail(self, e: BaseException):
        with self._lock:
            if self._error is None:
                self._error = e
        # cancel receives nobody will post any more
        while True:
            try:
                pr = self._recv_queue.get_nowait()
                pr.posted.set()
            except queue.Empty:
                break
        with self._outstanding_cv:
            self._outstanding_cv.notify_all()

    def zero_residual(self, rows: int) -> torch.Tensor:
        """A fresh zero residual: the fused add + RMSNorm kernels update the residual in place, so a
        cached tensor would carry one forward's residual stream into the next."""
        return torch.zeros(rows, self.hidden_size, dtype=self.dtype, device=self.device)

    # ---- receiving side --------------------------------------------------------
    def begin_step(self, padded_rows_per_forward: list) -> None:
        """Queue one receive per forward of the coming step (no-op on the first stage)."""
        self._raise_pending()
        if self.prev_rank is None:
            return
        for rows in padded_rows_per_forward:
            self._queue_recv(rows)

    def _queue_recv(self, rows: int) -> _PostedRecv:
        self._recv_counter += 1
        tensors = [torch.empty(rows, self.hidden_size, dtype=self.dtype, device=self.device)]
        tensors += [torch.empty(rows, w, dtype=self.dtype, device=self.device) for w in self.side_widths]
        pr = _PostedRecv(self._recv_counter, tensors)
        self._posted[pr.transfer] = pr
        self._recv_queue.put(pr)
        return pr

    def _post_loop(self):
        while not self._stop:
            try:
                pr = self._recv_queue.get(timeout=0.05)
            except queue.Empty:
                continue
            try:
                with self._outstanding_cv:
                    # throttle: a receive posted beyond the cap would stall its sender silently
                    while self._outstanding >= self.max_posted and not self._stop and self._error is None:
                        self._outstanding_cv.wait(timeout=0.05)
                    self._outstanding += 1
                if self._error is not None:
                    pr.posted.set()
                    continue
                for i, t in enumerate(pr.tensors):
                    pr.handles.append(self.t.irecv(t, self.prev_rank, pr.transfer * self.TAG_STRIDE + i))
                pr.posted.set()
            except BaseException as e:           # noqa: BLE001 - forwarded to the worker thread
                pr.posted.set()
                self._fail(e)

    def start_forward(self, rows: int, timeout_s: float = 60.0):
        """Input of the next forward on this stage: (hidden_sum, zero_residual, side tensors).
        Returns None on the first stage."""
        self._raise_pending()
        if self.prev_rank is None:
            return None
        nxt = min(self._posted) if self._posted else None
        if nxt is None:
            pr = self._queue_recv(rows)          # a forward without begin_step (warm-up) posts its own
        else:
            pr = self._posted[nxt]
        if not pr.posted.wait(timeout_s):
            raise TimeoutError(f"receive {pr.transfer} was not posted within {timeout_s}s")
        self._raise_pending()
        for h in pr.handles:
            h.wait()
        del self._posted[pr.transfer]
        if pr.tensors[0].shape[0] != rows:
            raise RuntimeError(f"transfer {pr.transfer}: posted {pr.tensors[0].shape[0]} rows, forward has {rows}")
        with self._outstanding_cv:
            self._outstanding -= 1
            self._outstanding_cv.notify_all()
        return pr.tensors[0], self.zero_residual(rows), pr.tensors[1:]

    # ---- sending side ----------------------------------------------------------
    def end_forward(self, hidden: torch.Tensor, residual: Optional[torch.Tensor], side: tuple = ()) -> None:
        """Queue the hand-off of this forward's output; blocks while ``depth`` sends are queued."""
        self._raise_pending()
        self._send_counter += 1
        if self.next_rank is None:
            payload = None
        else:
            total = hidden if residual is None else (hidden.float() + residual.float()).to(hidden.dtype)
            payload = [total.contiguous()] + [s.contiguous() for s in side]
        item = (self._send_counter, payload, self._fence())
        while True:
            try:
                self._send_queue.put(item, timeout=0.05)
                break
            except queue.Full:
                self._raise_pending()

    def _send_loop(self):
        while not self._stop:
            try:
                transfer, payload, fence_wait = self._send_queue.get(timeout=0.05)
            except queue.Empty:
                continue
            try:
                fence_wait()
                if payload is not None:
                    hs = [self.t.isend(t, self.next_rank, transfer * self.TAG_STRIDE + i)
                          for i, t in enumerate(payload)]
                    for h in hs:
                        h.wait()
                    drain = getattr(self.t, "drain", None)
                    if drain is not None:
                        drain()
            except BaseException as e:           # noqa: BLE001
                self._fail(e)
            finally:
                self._send_queue.task_done()

    def flush(self, timeout_s: float = 60.0) -> None:
        t0 = time.monotonic()
        while self._send_queue.unfinished_tasks:
            self._raise_pending()
            if time.monotonic() - t0 > timeout_s:
                raise TimeoutError("pipeline sends did not drain")
            time.sleep(0.001)
        self._raise_pending()

    # ---- self test ---------------------------------------------------------------
    def warmup(self, rows: int = 8) -> None:
        """Send a rank-stamped pattern to the next stage and verify what arrives from the previous one."""
        got = self.start_forward(rows) if self.prev_rank is not None else None
        if got is not None:
            want = float(self.prev_rank + 1)
            if not torch.all(got[0].float() == want):
                raise RuntimeError(f"pipeline warm-up: expected bytes stamped {want} from rank {self.prev_rank}")
        if self.next_rank is not None:
            stamp = torch.full((rows, self.hidden_size), float(self.my_rank + 1), dtype=self.dtype,
                               device=self.device)
            self.end_forward(stamp, None, tuple(torch.zeros(rows, w, dtype=self.dtype, device=self.device)
                                                for w in self.side_widths))
        else:
            self.end_forward(torch.zeros(1, 1), None)
        self.flush()

    def close(self) -> None:
        self._stop = True
        for th in self._threads:
            th.join(timeout=1.0)
