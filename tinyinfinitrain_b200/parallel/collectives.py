"""Standalone all-reduce / all-gather on symmetric memory (kernels in ``csrc/kernels/collectives.cu``).

The fused kernels cover the collectives that sit next to a GEMM or the optimizer.  What is left -- gradients of
parameters that tensor parallelism replicates, plain data parallelism without ZeRO, broadcasts of small state --
can go through NCCL, or through these two kernels when the data already lives in a :class:`SymmetricBuffer`:

* ``all_reduce_``: two-shot; each rank sums its 1/world slice of every rank's copy (``multimem.ld_reduce`` through
  NVSwitch when the buffer has a multicast mapping, peer loads otherwise) and writes the result into every copy,
* ``all_gather_``: each rank writes its slice into every copy.

Both are bracketed by the device barrier, run on the current stream and can be captured in a CUDA graph.  On CPU
tensors (gloo groups) the same calls fall back to ``torch.distributed`` so the callers can be tested without GPUs.
The reference has no communication layer (``infini_train/src/device.cc:11-17``).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .symm import DeviceBarrier, SymmetricBuffer


def padded_numel(numel: int, dtype: torch.dtype, world: int) -> int:
    """Smallest count >= numel whose byte size splits into ``world`` slices of whole 16-byte vectors."""
    per = 16 * world // torch.empty((), dtype=dtype).element_size()
    return (numel + per - 1) // per * per


class SymmCollective:
    """A symmetric staging buffer of ``numel`` elements plus the barrier that orders the kernels.

    ``tensor`` is this rank's copy; write the input there (or allocate the data there in the first place), call
    ``all_reduce_()`` / ``all_gather_()``, read the result from the same place."""

    def __init__(self, numel: int, dtype: torch.dtype, device, group: Optional[dist.ProcessGroup] = None, channel: int = 1,
                 timeout_s: float = 2.0):
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.dtype = dtype
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError("SymmCollective: fp32 or bf16")
        self.numel = padded_numel(numel, dtype, self.world)
        self.is_cuda = torch.device(device).type == "cuda"
        if self.is_cuda:
            self.buf = SymmetricBuffer(self.numel, dtype, device, self.group)
            self.tensor = self.buf.tensor
            self.tensor.zero_()
            self.barrier = DeviceBarrier(self.buf, channel=channel, timeout_s=timeout_s)
            torch.cuda.synchronize(device)
            dist.barrier(group=self.group)
        else:
            self.buf = self.barrier = None
            self.tensor = torch.zeros(self.numel, dtype=dtype, device=device)
        self.esize = self.tensor.element_size()

    def _range(self, numel: Optional[int], offset: int):
        n = self.numel - offset if numel is None else numel
        if offset < 0 or n < 0 or offset + n > self.numel:
            raise ValueError("SymmCollective: range outside of the buffer")
        if (offset * self.esize) % 16 or (n * self.esize) % (16 * self.world):
            raise ValueError("SymmCollective: offset must be 16-byte aligned and the size a multiple of 16 * world bytes "
                             "(see padded_numel)")
        return n

    @torch.no_grad()
    def all_reduce_(self, numel: Optional[int] = None, offset: int = 0, average: bool = False, max_blocks: int = 0) -> torch.Tensor:
        """Sum (or mean) over the ranks of ``tensor[offset:offset + numel]``, in place on every rank."""
        n = self._range(numel, offset)
        view = self.tensor[offset:offset + n]
        if n == 0:
            return view
        if not self.is_cuda:
            dist.all_reduce(view, group=self.group)
            if average:
                view.div_(self.world)
            return view
        from .._lib import C

        self.barrier()                                    # every rank's input is in its copy
        C.symm_allreduce(self.buf.ptrs, self.buf.mc_ptr, offset * self.esize, n * self.esize,
                         1 if self.dtype == torch.bfloat16 else 0, self.rank, (1.0 / self.world) if average else 1.0, max_blocks)
        self.barrier()                                    # every slice has landed in every copy
        return view

    @torch.no_grad()
    def all_gather_(self, numel: Optional[int] = None, offset: int = 0, max_blocks: int = 0) -> torch.Tensor:
        """``tensor[offset:offset + numel]`` is ``world`` equal slices; rank r's slice of its own copy is written into
        every rank's copy."""
        n = self._range(numel, offset)
        view = self.tensor[offset:offset + n]
        if n == 0:
            return view
        if not self.is_cuda:
            per = n // self.world
            mine = view[self.rank * per:(self.rank + 1) * per].clone()
            dist.all_gather_into_tensor(view, mine, group=self.group)
            return view
        from .._lib import C

        self.barrier()                                    # nobody still reads what is about to be overwritten
        C.symm_allgather(self.buf.ptrs, self.buf.mc_ptr, offset * self.esize, n * self.esize, self.rank, max_blocks)
        self.barrier()
        return view


class SymmFlag:
    """Point-to-point flags in the signal pads of a symmetric buffer: ``signal(peer)`` bumps this rank's counter for
    ``peer`` and publishes it in the peer's pad after all earlier work of the current stream; ``wait(peer)`` makes the
    current stream wait (at most ``timeout_s``; expiry sets the library status word, the stream carries on) until
    ``peer``'s next signal has arrived.  Slot layout: ``[channel][source rank]`` 32-bit words, the same pads the barrier
    uses, so give flags a channel of their own (the barrier of ``SymmCollective`` uses channel 1, ZeRO-1 channel 0)."""

    SLOTS_PER_CHANNEL = 16

    def __init__(self, buf: SymmetricBuffer, channel: int = 2, timeout_s: float = 2.0):
        if not 0 <= channel < 8:
            raise ValueError("SymmFlag: channel 0..7")
        self.buf, self.channel, self.timeout_s = buf, channel, timeout_s
        self.sent = [0] * buf.world
        self.seen = [0] * buf.world

    def _word(self, pad_owner: int, source: int) -> int:
        return self.buf.pad_ptrs[pad_owner] + 4 * (self.channel * self.SLOTS_PER_CHANNEL + source)

    def signal(self, peer: int) -> None:
        from .._lib import C

        self.sent[peer] += 1
        C.symm_signal(self._word(peer, self.buf.rank), self.sent[peer] & 0xFFFFFFFF)

    def wait(self, peer: int) -> None:
        from .._lib import C

        self.seen[peer] += 1
        C.symm_wait(self._word(self.buf.rank, peer), self.seen[peer] & 0xFFFFFFFF, self.timeout_s)
