"""Peer-mapped (symmetric) device memory for the NVLink kernels.

Allocation and handle exchange use ``torch.distributed._symmetric_memory`` (CUDA VMM
allocations exported to every rank of the group, plus an NVLS multicast mapping when
the fabric supports it); the kernels of ``csrc/kernels/comm.cu`` and the fused GEMM
collectives then read and write those addresses directly.  The reference has no
counterpart: it is single-device (infini_train/src/device.cc:11-17).
"""
from __future__ import annotations

import os
from typing import List, Optional

import torch
import torch.distributed as dist


class SymmetricBuffer:
    """A flat tensor that every rank of ``group`` can address on its own GPU.

    ``ptrs[r]`` is the address of rank r's copy as mapped on this GPU, ``mc_ptr`` the NVLS
    multicast address (0 when multicast is unavailable or disabled with
    ``TITB200_NO_MULTIMEM=1``), ``pad_ptrs[r]`` rank r's signal pad.
    """

    def __init__(self, numel: int, dtype: torch.dtype, device, group: Optional[dist.ProcessGroup] = None):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.tensor = symm_mem.empty(numel, dtype=dtype, device=device)
        self.handle = symm_mem.rendezvous(self.tensor, self.group)
        self.rank = self.handle.rank
        self.world = self.handle.world_size
        self.ptrs: List[int] = [int(p) for p in self.handle.buffer_ptrs]
        self.pad_ptrs: List[int] = [int(p) for p in self.handle.signal_pad_ptrs]
        mc = 0
        if not os.environ.get("TITB200_NO_MULTIMEM"):
            try:
                mc = int(self.handle.multicast_ptr or 0)
            except Exception:  # noqa: BLE001
                mc = 0
        self.mc_ptr = mc

    def peer(self, r: int) -> torch.Tensor:
        """Rank r's buffer as a tensor on this device (peer-mapped view)."""
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
