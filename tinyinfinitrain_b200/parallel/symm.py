"""Peer-mapped (symmetric) device memory for the NVLink kernels.

Allocation and handle exchange use either ``torch.distributed._symmetric_memory`` (default) or this
package's own heap (``csrc/core/symm_heap.cc``, ``TITB200_SYMM_HEAP=native``).  Both create CUDA VMM
allocations, export them to every rank of the group and add an NVLS multicast mapping when the fabric
supports it; the kernels of ``csrc/kernels/comm.cu`` and the fused GEMM collectives then read and write
those addresses directly.  The reference has no counterpart: it is single-device
(infini_train/src/device.cc:11-17).
"""
from __future__ import annotations

import os
from typing import List, Optional

import torch
import torch.distributed as dist


_HEAPS = {}        # (id(group), device index) -> (heap, key) of the native backend
_NATIVE = os.environ.get("TITB200_SYMM_HEAP", "torch") == "native"


def use_multimem() -> bool:
    """Whether the NVLink kernels address NVSwitch multicast memory (``multimem.ld_reduce`` / ``multimem.st``) or use
    plain peer loads and stores.  Default: peer loads and stores -- measured on 2 B200s the fused ZeRO-1 step takes
    654 us that way against 1.75 ms through the multicast address (the switch pulls every rank's whole gradient, the
    peer path only the shard this rank owns), and the two-shot all-reduce is 1.7x faster.  ``TITB200_MULTIMEM=1``
    selects multicast; ``TITB200_NO_MULTIMEM=1`` (older switch) forces it off."""
    if os.environ.get("TITB200_NO_MULTIMEM"):
        return False
    return os.environ.get("TITB200_MULTIMEM", "0") == "1"


def _native_heap(group, device):
    """One heap (one listening socket) per process group and device, created collectively on first use."""
    from .._lib import C

    k = (id(group), torch.device(device).index)
    if k not in _HEAPS:
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        # a key every rank of the group agrees on: rank 0's pid and a counter, broadcast through the group
        box = [f"{os.getpid()}x{len(_HEAPS)}"] if rank == 0 else [None]
        dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0), group=group)
        heap = C.SymmHeap(rank, world, torch.device(device).index or 0, box[0], "cuda",
                          use_multimem())
        heap.listen()
        dist.barrier(group=group)          # every rank listens before anyone connects
        _HEAPS[k] = heap
    return _HEAPS[k]


class SymmetricBuffer:
    """A flat tensor that every rank of ``group`` can address on its own GPU.

    ``ptrs[r]`` is the address of rank r's copy as mapped on this GPU, ``mc_ptr`` the NVLS
    multicast address (0 unless multicast is available and selected with
    ``TITB200_MULTIMEM=1``, see :func:`use_multimem`), ``pad_ptrs[r]`` rank r's signal pad.

    Two back ends allocate and map the memory.  The default is PyTorch's symmetric-memory allocator.
    ``TITB200_SYMM_HEAP=native`` selects this package's own heap (``csrc/core/symm_heap.cc``: cuMemCreate,
    descriptor passing over unix sockets, cuMemMap of every peer, one cuMulticast object per allocation).
    """

    PAD_BYTES = 4096   # signal pad per rank: uint32 slots [channel][source rank]

    def __init__(self, numel: int, dtype: torch.dtype, device, group: Optional[dist.ProcessGroup] = None):
        self.group = group if group is not None else dist.group.WORLD
        if _NATIVE:
            self._init_native(numel, dtype, device)
            return
        import torch.distributed._symmetric_memory as symm_mem

        self.tensor = symm_mem.empty(numel, dtype=dtype, device=device)
        self.handle = symm_mem.rendezvous(self.tensor, self.group)
        self.rank = self.handle.rank
        self.world = self.handle.world_size
        self.ptrs: List[int] = [int(p) for p in self.handle.buffer_ptrs]
        self.pad_ptrs: List[int] = [int(p) for p in self.handle.signal_pad_ptrs]
        mc = 0
        if use_multimem():
            try:
                mc = int(self.handle.multicast_ptr or 0)
            except Exception:  # noqa: BLE001
                mc = 0
        self.mc_ptr = mc

    def _init_native(self, numel: int, dtype: torch.dtype, device) -> None:
        heap = self._heap = _native_heap(self.group, device)
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        dev = torch.device(device)
        nbytes = numel * torch.empty((), dtype=dtype).element_size()

        def collective_alloc(n: int):
            i = heap.exchange(n)
            # all devices must have joined the multicast object before any rank binds memory to it; the
            # all-reduce is both that barrier and the agreement on whether multicast is usable at all
            flag = torch.tensor([1 if heap.multicast_ready(i) else 0], device=dev, dtype=torch.int32)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
            info = heap.finish(i, bool(flag.item()))
            flag.fill_(1 if info["mc_ptr"] else 0)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
            if not flag.item():
                heap.drop_multicast(i)
                info = heap.get(i)
            return i, info

        self._id, info = collective_alloc(nbytes)
        self._pad_id, pad = collective_alloc(self.PAD_BYTES)
        heap.drop_multicast(self._pad_id)      # pads are addressed per peer only
        self.tensor = heap.tensor(self._id, self.rank, dtype, numel)
        self.ptrs = [int(p) for p in info["ptrs"]]
        self.pad_ptrs = [int(p) for p in pad["ptrs"]]
        self.mc_ptr = int(info["mc_ptr"])
        self.handle = None
        heap.tensor(self._pad_id, self.rank, torch.int32, self.PAD_BYTES // 4).zero_()
        torch.cuda.synchronize(dev)
        dist.barrier(group=self.group)         # every pad is zero before any barrier kernel runs

    def peer(self, r: int) -> torch.Tensor:
        """Rank r's buffer as a tensor on this device (peer-mapped view)."""
        if self.handle is None:
            return self._heap.tensor(self._id, r, self.tensor.dtype, self.tensor.numel())
        return self.handle.get_buffer(r, self.tensor.shape, self.tensor.dtype)


class DeviceBarrier:
    """Cross-GPU barrier executed by a kernel on the current stream (graph-capturable).

    Uses channel ``channel`` of the signal pads of ``buf``; the epoch counter lives in device
    memory and is advanced by the kernel.  A wait that exceeds ``timeout_s`` records a status
    code instead of hanging (read it with ``_lib.C.status_read``).
    """

    def __init__(self, buf: SymmetricBuffer, channel: int = 0, timeout_s: float = 2.0):
        self.buf, self.channel, self.timeout_s = buf, channel, timeout_s
        self.epoch = torch.zeros(1, dtype=torch.int32, device=buf.tensor.device)

    def __call__(self) -> None:
        from .._lib import C

        C.comm_barrier(self.buf.pad_ptrs, self.buf.rank, self.channel, self.epoch, self.timeout_s)
