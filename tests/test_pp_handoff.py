"""Pipeline hand-off protocol with threads and a fake in-memory transport: the
schedule must pair sends and receives or time out, errors on helper threads must
surface on the worker thread, and the posted-receive cap must hold."""
import threading
import time

import pytest
import torch

from vllm_torchtpu_b200.parallel.pp import (PPHandoff, Transport, buffered_steps_in_flight,
                                            partition_layers)


class _Handle:
    def __init__(self, ev, fail=None):
        self.ev, self.fail = ev, fail

    def wait(self, timeout=5.0):
        if self.fail:
            raise self.fail
        if not self.ev.wait(timeout):
            raise TimeoutError("fake transport: transfer never paired")


class FakeFabric:
    """Matches isend(dst, tag) with irecv(src, tag); the copy happens when both exist."""

    def __init__(self):
        self.lock = threading.Lock()
        self.sends, self.recvs = {}, {}
        self.max_posted_seen = 0
        self.posted_now = 0

    def endpoint(self, rank, fail_send=False, fail_recv=False):
        return _Endpoint(self, rank, fail_send, fail_recv)

    def _try_pair(self, key):
        if key in self.sends and key in self.recvs:
            src_t, sev = self.sends.pop(key)
            dst_t, rev = self.recvs.pop(key)
            dst_t.copy_(src_t)
            self.posted_now -= 1
            sev.set()
            rev.set()


class _Endpoint(Transport):
    def __init__(self, fabric, rank, fail_send, fail_recv):
        self.f, self.rank, self.fail_send, self.fail_recv = fabric, rank, fail_send, fail_recv

    def isend(self, tensor, dst, tag):
        if self.fail_send:
            return _Handle(None, RuntimeError("injected send failure"))
        ev = threading.Event()
        with self.f.lock:
            self.f.sends[(self.rank, dst, tag)] = (tensor, ev)
            self.f._try_pair((self.rank, dst, tag))
        return _Handle(ev)

    def irecv(self, tensor, src, tag):
        if self.fail_recv:
            raise RuntimeError("injected recv failure")
        ev = threading.Event()
        with self.f.lock:
            self.f.recvs[(src, self.rank, tag)] = (tensor, ev)
            self.f.posted_now += 1
            self.f.max_posted_seen = max(self.f.max_posted_seen, self.f.posted_now)
            self.f._try_pair((src, self.rank, tag))
        return _Handle(ev)


def _stage(fabric, rank, world, **kw):
    return PPHandoff(fabric.endpoint(rank, **{k: v for k, v in kw.items() if k.startswith("fail")}),
                     prev_rank=rank - 1 if rank > 0 else None, next_rank=rank + 1 if rank < world - 1 else None,
                     hidden_size=8, dtype=torch.float32, device="cpu", my_rank=rank,
                     depth=kw.get("depth", 2), max_posted=kw.get("max_posted", 7))


def test_partition_and_in_flight():
    assert partition_layers(32, 4) == [(0, 8), (8, 16), (16, 24), (24, 32)]
    assert partition_layers(61, 4) == [(0, 15), (15, 30), (30, 45), (45, 61)]
    assert buffered_steps_in_flight(4) == 6 and buffered_steps_in_flight(2) == 3


def test_three_stage_pipeline_passes_sum_and_zero_residual():
    fab = FakeFabric()
    stages = [_stage(fab, r, 3) for r in range(3)]
    results = {}

    def run(rank):
        st = stages[rank]
        st.warmup()
        for step in range(5):
            st.begin_step([4])
            got = st.start_forward(4)
            if got is None:
                h, res = torch.full((4, 8), float(step)), torch.ones(4, 8)
            else:
                h, res = got[0] + 1, got[1]
                assert torch.all(res == 0)
            st.end_forward(h, res)
            results[(rank, step)] = h.clone()
        st.flush()

    ths = [threading.Thread(target=run, args=(r,)) for r in range(3)]
    [t.start() for t in ths]
    [t.join(20) for t in ths]
    for step in range(5):
        # stage 0 sends step + 1 (hidden + residual); each later stage adds 1
        assert torch.all(results[(2, step)] == step + 1 + 2)
    [s.close() for s in stages]


def test_posted_receives_are_capped():
    fab = FakeFabric()
    recv = _stage(fab, 1, 2, max_posted=3)
    recv.begin_step([2] * 10)
    time.sleep(0.3)
    assert fab.max_posted_seen <= 3
    send = _stage(fab, 0, 2)
    for i in range(10):
        send.end_forward(torch.full((2, 8), float(i)), None)
        got = recv.start_forward(2)
        assert torch.all(got[0] == i)
        recv.end_forward(got[0], None)
    send.flush()
    assert fab.max_posted_seen <= 3
    send.close(), recv.close()


def test_send_failure_surfaces_on_worker_thread():
    fab = FakeFabric()
    st = _stage(fab, 0, 2, fail_send=True)
    st.end_forward(torch.zeros(2, 8), None)
    with pytest.raises(RuntimeError, match="hand-off failed"):
        for _ in range(100):
            time.sleep(0.01)
            st.end_forward(torch.zeros(2, 8), None)
    st.close()


def test_recv_failure_cancels_queued_receives():
    fab = FakeFabric()
    st = _stage(fab, 1, 2, fail_recv=True)
    st.begin_step([2, 2, 2])
    with pytest.raises(RuntimeError, match="hand-off failed"):
        st.start_forward(2, timeout_s=2.0)
    st.close()


def test_unpaired_schedule_times_out_rather_than_passing():
    fab = FakeFabric()
    st = _stage(fab, 1, 2)
    st.begin_step([2])
    with pytest.raises((TimeoutError, RuntimeError)):
        st.start_forward(2, timeout_s=0.5)
    st.close()
