"""Fused tensor-parallel collectives: all-gather -> GEMM and GEMM -> reduce-scatter in one kernel.

Buffers live in symmetric (peer-mapped) memory, allocated once per shape and reused.  Each fused
call is preceded by one device-side barrier, which both publishes the peers' inputs and proves
that every rank has finished reading what the previous call left in the shared buffers; a second
barrier is inserted only when a buffer would otherwise be rewritten with no barrier since it
was last read (first use in a step, or two consecutive calls on the same buffer).
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from .._lib import C
from ..ops import functional as F_
from .symm import DeviceBarrier, SymmetricBuffer


class FusedTP:
    AG_HELPERS = 0    # CTAs that pull peer shards over NVLink before they join the GEMM tiles; 0: the launcher sizes it
    RS_HELPERS = 8    # CTAs that reduce arriving partial tiles

    def __init__(self, comm):
        self.comm = comm
        self.world, self.rank, self.group = comm.world, comm.rank, comm.group
        self._ag: Dict[object, SymmetricBuffer] = {}
        self._rs: Dict[Tuple[int, int], Tuple[SymmetricBuffer, SymmetricBuffer]] = {}
        self._barrier = None
        self._nbar = 0
        self._last_read: Dict[object, int] = {}

    # ---- bookkeeping -----------------------------------------------------------------------
    def new_step(self) -> None:
        """Forget what is known about barriers since each buffer was last read (call at the start of
        a step: a captured graph replays from here, so the first use must assume nothing)."""
        self._last_read.clear()

    def _bar(self, dev) -> None:
        if self._barrier is None:
            anchor = SymmetricBuffer(1024, torch.float32, dev, self.group)
            self._barrier = DeviceBarrier(anchor, channel=1)
        self._barrier()
        self._nbar += 1

    def _ag_buf(self, numel: int, dev) -> SymmetricBuffer:
        b = self._ag.get(numel)
        if b is None:
            b = self._ag[numel] = SymmetricBuffer(numel, torch.bfloat16, dev, self.group)
        return b

    def _rs_buf(self, Ms: int, N: int, dev):
        key = (Ms, N)
        b = self._rs.get(key)
        if b is None:
            recv = SymmetricBuffer(self.world * Ms * N, torch.bfloat16, dev, self.group)
            cnt = SymmetricBuffer(max(128, Ms // 128 + 1), torch.int32, dev, self.group)
            cnt.tensor.zero_()
            torch.cuda.synchronize(dev)
            b = self._rs[key] = (recv, cnt)
        return b

    # ---- all-gather -> GEMM ---------------------------------------------------------------------
    def _ag_eligible(self, Ms: int, K: int) -> bool:
        return Ms % 128 == 0 and K % 8 == 0

    def ag_input(self, Ms: int, K: int, dev):
        """A [Ms, K] bf16 view of this rank's slot of the gather buffer, safe to overwrite: the kernel that produces
        the next :meth:`ag_gemm` operand (a norm) writes there directly, and :meth:`ag_gemm` recognises the
        address and skips its staging copy.  ``None`` for shapes the fused kernel does not take."""
        if not self._ag_eligible(Ms, K):
            return None
        buf = self._ag_buf(Ms * K, dev)
        key = ("ag", Ms * K)
        if self._last_read.get(key, 1 << 60) >= self._nbar:
            self._bar(dev)                       # peers may still be reading this buffer
            self._last_read[key] = -1            # nothing has read it since that barrier
        return buf.tensor.view(Ms, K)

    def ag_gemm(self, x_s, w, bias=None, gelu=False, b_mn=False):
        Ms, K = x_s.shape
        N = w.shape[1] if b_mn else w.shape[0]
        if not self._ag_eligible(Ms, K) or N % 8:
            X = self.comm.all_gather_rows(x_s)
            from .tp import _local_gemm

            return _local_gemm(X, w, bias, gelu, b_mn) + (X,)
        dev = x_s.device
        buf = self._ag_buf(Ms * K, dev)
        key = ("ag", Ms * K)
        if x_s.data_ptr() != buf.tensor.data_ptr():          # not produced in place through ag_input()
            if self._last_read.get(key, 1 << 60) >= self._nbar:
                self._bar(dev)                   # peers may still be reading this buffer
            buf.tensor.view(Ms, K).copy_(x_s)
        self._bar(dev)                           # every shard is written
        epi = F_.EPI_BIAS_GELU if gelu else (F_.EPI_BIAS if bias is not None else F_.EPI_NONE)
        out = C.gemm_ag(buf.ptrs, self.rank, Ms, K, w, b_mn, epi, bias, gelu, self.AG_HELPERS)
        self._last_read[key] = self._nbar
        return tuple(out)

    # ---- GEMM -> reduce-scatter ------------------------------------------------------------------
    def gemm_rs(self, y, w, b_mn=False, bias=None, residual_s=None):
        M, K = y.shape
        N = w.shape[1] if b_mn else w.shape[0]
        Ms = M // self.world
        if M % self.world or Ms % 128 or K % 8 or N % 8 or not y.is_contiguous():
            Z = C.gemm(y.contiguous(), w, False, b_mn)[0]
            z_s = self.comm.reduce_scatter_rows(Z)
            if bias is not None:
                z_s = z_s + bias
            if residual_s is not None:
                z_s = z_s + residual_s
            return z_s
        dev = y.device
        recv, cnt = self._rs_buf(Ms, N, dev)
        self._bar(dev)                           # every rank has consumed the previous contents of its receive buffer
        res = residual_s.contiguous() if residual_s is not None else None
        return C.gemm_rs(y, w, b_mn, recv.ptrs, cnt.ptrs, self.rank, bias, res, min(self.RS_HELPERS, Ms // 128))

    # ---- vocabulary-parallel embedding ------------------------------------------------------------
    def _emb_buf(self, Ms: int, Cd: int, dtype, dev) -> SymmetricBuffer:
        key = ("emb", Ms, Cd, dtype)
        b = self._ag.get(key)
        if b is None:
            b = self._ag[key] = SymmetricBuffer(Ms * Cd, dtype, dev, self.group)
        return b

    def embedding_push(self, idx, w, vocab_total: int):
        """Token shard [M / world, C] of the embedding of ``idx`` (M ids) from a table split by rows: every rank
        stores the rows it holds into the shard buffer of the rank that owns the token, then the shard is copied
        out of the shared buffer."""
        M, Ms, Cd = idx.numel(), idx.numel() // self.world, w.shape[1]
        buf = self._emb_buf(Ms, Cd, w.dtype, w.device)
        self._bar(w.device)                      # every rank has consumed the previous contents of its buffer
        C.embedding_vp_push(idx.reshape(-1), w, list(buf.ptrs), Ms, self.rank * w.shape[0], vocab_total, self.rank == 0)
        self._bar(w.device)                      # all rows have landed
        return buf.tensor.view(Ms, Cd).clone()

    def embedding_pull_bwd(self, idx, dx_s, dw) -> None:
        """dw (fp32, this rank's rows of the table) += gradient rows of the ids it holds, read from the token owners."""
        Ms, Cd = dx_s.shape
        buf = self._emb_buf(Ms, Cd, dx_s.dtype, dx_s.device)
        self._bar(dx_s.device)                   # nobody reads or writes the buffers any more
        buf.tensor.view(Ms, Cd).copy_(dx_s)
        self._bar(dx_s.device)                   # every shard is written
        C.embedding_vp_pull_bwd(idx.reshape(-1), list(buf.ptrs), dw, Ms, self.rank * dw.shape[0], dx_s)

    # ---- per-row statistics table of the vocabulary-parallel loss ----------------------------------
    def stats_table(self, rows: int, dev):
        """A [world, rows, 3] fp32 table in symmetric memory and the addresses of every rank's copy; rank r's
        kernel stores its triples into slot r of all of them.  Call :meth:`stats_publish` after that kernel."""
        key = ("vp", rows)
        buf = self._ag.get(key)
        if buf is None:
            buf = self._ag[key] = SymmetricBuffer(self.world * rows * 3, torch.float32, dev, self.group)
        if self._last_read.get(key, 1 << 60) >= self._nbar:
            self._bar(dev)                       # peers may still be reading the previous contents
        return buf.tensor.view(self.world, rows, 3), list(buf.ptrs)

    def stats_publish(self, rows: int, dev) -> None:
        self._bar(dev)                           # every rank's slot has landed everywhere
        self._last_read[("vp", rows)] = self._nbar
