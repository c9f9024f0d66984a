"""Symmetric heap: one cudaMalloc'd region per rank, IPC-mapped into every peer.

Offsets inside the heap are identical on all ranks, so a kernel addresses "peer
p's copy of buffer B" as ``peers[p] + offset(B)``.  Handles are exchanged once
over the group's CPU (gloo) process group.  Everything a fused
compute+collective kernel needs lives here: staging buffers for partial
results, the output buffers peers write into, arrival flags and the epoch word.

Stands in for the reference's per-op JAX meshes and remote-DMA buffers
(reference: src/vllm_torchtpu/distributed/sharded_jax_op.py:14-215,
kernels/collectives/util.py:33-58): with NVSwitch there is no topology to order,
only a table of peer pointers.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

from .. import envs
from ..logger import init_logger

logger = init_logger(__name__)

MAX_RANKS = 8
ALIGN = 1024


@dataclass
class HeapBuffer:
    offset: int
    nbytes: int
    tensor: torch.Tensor            # local view


class SymmetricHeap:
    def __init__(self, rank: int, world: int, nbytes: int, local_ptr: int, peer_ptrs: list,
                 device: torch.device):
        self.rank, self.world, self.nbytes = rank, world, nbytes
        self.local_ptr = local_ptr
        self.peer_ptrs = peer_ptrs
        self.device = device
        self._bump = 0
        self._named: dict = {}
        self.peers_c = (ctypes.c_void_p * world)(*peer_ptrs)
        # control words live in ordinary device memory of this rank
        self.ctrl = torch.zeros(16, dtype=torch.int32, device=device)
        self.flags = self.alloc("flags", 4096)          # arrival slots, tile flags
        self.spin_limit = int(envs.B200_SPIN_LIMIT)
        self.ar_stage_bytes = 32 * 2**20
        self.fused_tp = None
        self.ep_state = None             # fused expert-parallel plane (ops.cuda_moe.EpState)

    def configure_fused_tp(self, max_tokens: int, max_n: int) -> None:
        from ..ops import cuda
        if self.fused_tp is None:
            self.fused_tp = cuda.FusedTP(self, max_tokens, max_n)

    # ---- creation -------------------------------------------------------------
    @classmethod
    def create(cls, group, nbytes: int) -> "SymmetricHeap":
        from ..ops import cuda
        L = cuda.lib()
        dev = torch.device("cuda", torch.cuda.current_device())
        L.b200_set_device(ctypes.c_int(dev.index))
        ptr = ctypes.c_void_p()
        cuda._check(L.b200_ipc_alloc(ctypes.c_size_t(nbytes), ctypes.byref(ptr)), "ipc_alloc")
        handle = (ctypes.c_ubyte * 64)()
        cuda._check(L.b200_ipc_get_handle(ptr, handle), "ipc_get_handle")
        handles = [None] * group.size
        dist.all_gather_object(handles, bytes(handle), group=group.cpu_group)
        peers = []
        for i, h in enumerate(handles):
            if i == group.rank_in_group:
                peers.append(ptr.value)
                continue
            buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
            p = ctypes.c_void_p()
            cuda._check(L.b200_ipc_open(buf, ctypes.byref(p)), "ipc_open")
            peers.append(p.value)
        logger.info("symmetric heap: %d MiB on %d ranks (group %s)", nbytes >> 20, group.size, group.name)
        heap = cls(group.rank_in_group, group.size, nbytes, ptr.value, peers, dev)
        dist.barrier(group=group.cpu_group)
        return heap

    # ---- allocation -------------------------------------------------------------
    def alloc(self, name: str, nbytes: int) -> HeapBuffer:
        """Named bump allocation; every rank must allocate the same names in the same order."""
        if name in self._named:
            b = self._named[name]
            if b.nbytes < nbytes:
                raise RuntimeError(f"symmetric buffer {name!r} was allocated with {b.nbytes} < {nbytes} bytes")
            return b
        off = (self._bump + ALIGN - 1) // ALIGN * ALIGN
        if off + nbytes > self.nbytes:
            raise RuntimeError(f"symmetric heap exhausted: want {nbytes} bytes at {off} of {self.nbytes}; "
                               f"raise B200_SYMM_HEAP_MB")
        self._bump = off + nbytes
        t = self._view(off, nbytes)
        b = HeapBuffer(off, nbytes, t)
        self._named[name] = b
        return b

    def _view(self, offset: int, nbytes: int) -> torch.Tensor:
        """uint8 tensor aliasing local heap memory (the heap outlives every view)."""
        class _Holder:
            pass

        h = _Holder()
        h.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (self.local_ptr + offset, False), "version": 3,
            "strides": None}
        return torch.as_tensor(h, device=self.device)

    def tensor(self, buf: HeapBuffer, shape, dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        assert nbytes <= buf.nbytes
        return buf.tensor[:nbytes].view(dtype).view(*shape)

    def contains(self, t: torch.Tensor) -> Optional[int]:
        p = t.data_ptr()
        if self.local_ptr <= p < self.local_ptr + self.nbytes:
            return p - self.local_ptr
        return None
