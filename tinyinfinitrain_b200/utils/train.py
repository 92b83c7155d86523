"""Training-step driver: static buffers, optional CUDA-graph capture of the whole step.

``TrainStep`` is the public entry point a training loop (and ``bench.py``) calls:
one call copies a batch from pinned host memory, runs forward + backward + gradient
synchronisation + optimizer on the device, and returns the loss in pinned host memory.
With ``use_graph=True`` the device work of one step is captured once in a CUDA graph
and replayed, which removes every per-kernel launch cost from the loop; all
step-dependent scalars (Adam step count, learning rate) live in device memory so the
replayed graph stays correct.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch


class TrainStep:
    def __init__(self, model, optimizer, batch_size: int, seq_len: int, device, use_graph: bool = True,
                 grad_sync: Optional[Callable[[], None]] = None, loss_scale: float = 1.0):
        self.model, self.opt = model, optimizer
        self.device = torch.device(device)
        self.use_graph = use_graph and self.device.type == "cuda"
        self.grad_sync = grad_sync
        self.idx = torch.zeros(batch_size, seq_len, dtype=torch.int64, device=self.device)
        self.tgt = torch.zeros(batch_size, seq_len, dtype=torch.int64, device=self.device)
        self.loss = torch.zeros((), dtype=torch.float32, device=self.device)
        pin = self.device.type == "cuda"
        self.host_loss = torch.zeros((), dtype=torch.float32, pin_memory=pin)
        self.graph = None
        self.launches_per_step = 0

    def _device_step(self) -> None:
        self.opt.zero_grad()
        _, loss = self.model(self.idx, self.tgt, return_logits=False)
        loss.backward()
        if self.grad_sync is not None:
            self.grad_sync()
        self.opt.step()
        self.loss.copy_(loss.detach().float())

    def prepare(self, eager_warmup: int = 2) -> None:
        """Runs a few eager steps (first-use allocations, attribute set-up) and captures the graph."""
        from .._lib import C

        if self.device.type != "cuda":
            return
        s = torch.cuda.Stream(device=self.device)
        s.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(s):
            for i in range(max(1, eager_warmup)):
                before = C.launch_count()
                self._device_step()
                self.launches_per_step = C.launch_count() - before
        torch.cuda.current_stream(self.device).wait_stream(s)
        torch.cuda.synchronize(self.device)
        if self.use_graph:
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                self._device_step()
            torch.cuda.synchronize(self.device)

    def run_device(self) -> None:
        """Device work of one step on the current stream (inputs already in the static buffers)."""
        if self.graph is not None:
            self.graph.replay()
        else:
            self._device_step()

    def __call__(self, idx_host: torch.Tensor, tgt_host: torch.Tensor) -> torch.Tensor:
        """One end-to-end step; returns the pinned host scalar (valid after a stream sync)."""
        self.idx.copy_(idx_host, non_blocking=True)
        self.tgt.copy_(tgt_host, non_blocking=True)
        self.run_device()
        self.host_loss.copy_(self.loss, non_blocking=True)
        return self.host_loss


class ParallelTrainStep:
    """One training step of a tensor x pipeline x data parallel job (one process per GPU, process group initialised).

    Builds this rank's pipeline stage of the tensor-parallel model, the optimizer that matches the layout (ZeRO-1
    distributed optimizer when the data-parallel group has more than one rank and ``zero_stage == 1``, all-reduce +
    full Adam for ``zero_stage == 0``, plain mixed-precision Adam otherwise) and the 1F1B schedule.  ``__call__``
    takes ``num_microbatches`` pinned host batches, copies them to the device, runs the schedule, the
    sequence-parallel gradient sync and the optimizer, and returns the mean loss of this rank's replica in pinned host
    memory (valid after a stream sync; zero on ranks that are not the last pipeline stage).  ``run_device`` does the
    same from batches that are already resident.
    """

    def __init__(self, cfg, batch_size: int, seq_len: int, device, dtype=torch.bfloat16, tp: int = 1, pp: int = 1,
                 num_microbatches: int = 1, zero_stage: int = 1, comm: str = "fused", dp_buckets: int = 1,
                 lr: float = 1e-3, betas=(0.9, 0.999), weight_decay: float = 0.0, max_grad_norm: float = 0.0,
                 seed: Optional[int] = 42, exact_init_limit: int = 1 << 26, full_state_dict=None):
        """``full_state_dict``: unsharded tensors of the single-GPU model (may be memory-mapped views of a checkpoint
        file); every rank copies its own slices before the optimizer takes its master copy."""
        import tinyinfinitrain_b200 as tit
        from ..models.tp_models import TPTransformer
        from ..parallel import AllReduceOptimizer, DistributedOptimizer, PipelineStage, TPComm, init_mesh, partition_layers

        self.device = torch.device(device)
        cuda = self.device.type == "cuda"
        self.cfg, self.B, self.T, self.nm, self.tp, self.pp = cfg, batch_size, seq_len, max(1, num_microbatches), tp, pp
        assert (batch_size * seq_len) % tp == 0, "tokens of a micro-batch must divide over the tensor-parallel ranks"
        self.mesh = mesh = init_mesh(tp=tp, pp=pp)
        self.comm = TPComm(mesh.tp_group, comm if cuda else "nccl")
        layers = partition_layers(cfg.n_layer, pp)[mesh.pp_rank]
        self.model = TPTransformer(cfg, self.comm, device=self.device, dtype=dtype, seed=seed, layers=layers,
                                   first=mesh.is_first_stage, last=mesh.is_last_stage, exact_init_limit=exact_init_limit)
        if full_state_dict is not None:
            self.model.load_full_state_dict(full_state_dict)
        self.params = list(self.model.parameters())
        # GPT-2 ties the token embedding and the output projection.  With more than one pipeline stage the first
        # stage holds wte and the last stage its own copy: both start from the first stage's values, and their
        # gradients are summed over the two stages before every optimizer step, so the copies stay one parameter.
        self.tied = None
        if pp > 1 and not self.model.is_llama and mesh.embed_group is not None:
            import torch.distributed as dist

            self.tied = self.model.transformer["wte"].weight if mesh.is_first_stage else self.model.lm_head.weight
            with torch.no_grad():
                dist.broadcast(self.tied, src=mesh.pp_ranks[0], group=mesh.embed_group)
        kw = dict(lr=lr, betas=betas, weight_decay=weight_decay, max_grad_norm=max_grad_norm, mp_group=mesh.mp_group,
                  tp_world=tp)
        if mesh.dp > 1 and zero_stage == 1:
            self.opt = DistributedOptimizer(self.params, group=mesh.dp_group, comm=comm if cuda else "nccl",
                                            num_buckets=dp_buckets, overlap=dp_buckets > 1, **kw)
        elif mesh.dp > 1:
            import os

            self.opt = AllReduceOptimizer(self.params, group=mesh.dp_group,
                                          comm="symm" if os.environ.get("TITB200_SYMM_ALLREDUCE") == "1" else "nccl", **kw)
        else:
            self.opt = tit.optim.MixedPrecisionAdam(self.params, **kw)
        self.batches = [(torch.zeros(batch_size, seq_len, dtype=torch.int64, device=self.device),
                         torch.zeros(batch_size, seq_len, dtype=torch.int64, device=self.device)) for _ in range(self.nm)]

        def stage_fn(x_in, i):
            x, y = self.batches[i]
            if mesh.is_first_stage:
                return self.model(x, y if mesh.is_last_stage else None)
            return self.model(x_in, y if mesh.is_last_stage else None, B=batch_size, T=seq_len)

        self.stage = PipelineStage(stage_fn, mesh.pp_rank, pp, None if mesh.is_first_stage else mesh.prev_stage_rank(),
                                   None if mesh.is_last_stage else mesh.next_stage_rank(),
                                   (batch_size * seq_len // tp, cfg.n_embd), dtype, self.device)
        self.loss = torch.zeros((), dtype=torch.float32, device=self.device)
        self.host_loss = torch.zeros((), dtype=torch.float32, pin_memory=cuda)
        self.launches_per_step = 0
        self.graph = None

    @property
    def tokens_per_step(self) -> int:
        """Tokens the whole job consumes per step."""
        return self.B * self.T * self.nm * self.mesh.dp

    def run_device(self) -> None:
        from .._lib import C
        from ..parallel import sync_sequence_parallel_grads

        before = C.launch_count() if self.device.type == "cuda" else 0
        self.opt.zero_grad()
        loss = self.stage.run(self.nm)
        if self.tied is not None:
            import torch.distributed as dist

            self.opt.flat.finish_unwritten()      # gradients that came through plain autograd join the main buffer
            dist.all_reduce(self.tied.main_grad, group=self.mesh.embed_group)
        sync_sequence_parallel_grads(self.params, self.comm)
        self.opt.step()
        if loss is not None:
            self.loss.copy_(loss.detach().float())
        if self.device.type == "cuda":
            self.launches_per_step = C.launch_count() - before

    def __call__(self, host_batches) -> torch.Tensor:
        for (x, y), (hx, hy) in zip(self.batches, host_batches):
            x.copy_(hx, non_blocking=True)
            y.copy_(hy, non_blocking=True)
        self.run_device()
        self.host_loss.copy_(self.loss, non_blocking=True)
        return self.host_loss
