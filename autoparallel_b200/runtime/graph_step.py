"""A whole training step - forward, backward, optimizer - captured once in a CUDA graph and replayed.

The per-rank graphs this framework builds have static shapes and every node is one kernel launch, so
a step is a fixed sequence of several thousand launches.  Issued from Python that sequence is bound by
the host for the short kernels (normalisation, RoPE, residual adds): the GPU idles a few per cent of
the step between them.  ``GraphedTrainStep`` captures the sequence once (``torch.cuda.graph``) and
replays it with one launch; inputs are copied into static buffers, the loss is read from a static
tensor, and the optimizer's learning rate and bias corrections travel through a 12-byte device
buffer so that schedules keep working (``optim.AdamW.advance_for_replay``).

Collectives: NCCL collectives and the copy-engine all-gathers are capturable; the flag-protocol
kernels of ``runtime/symm.py`` and the copy-engine reduce-scatter carry host-side sequence numbers in
their launch arguments and are refused here (use the eager executor with them).

Reference counterpart: the reference relies on Inductor (``torch.compile``) to cut launch
overhead (autoparallel/compile.py:259-310); this framework has no tracing compiler on the hot path.
"""
from __future__ import annotations

from typing import Any, Callable, Optional

import torch


class GraphedTrainStep:
    """``step = GraphedTrainStep(module, optimizer, example_args, example_kwargs)``; then ``loss = step(*args, **kwargs)``.

    ``module(*args, **kwargs)`` must return the loss (or ``loss_of(output)`` must).  The tensors among the example
    arguments fix the shapes; every later call must pass tensors of the same shapes and dtypes.  Eager steps
    should have run before (``warmup_steps`` > 0 runs them here: they are real optimizer steps) so that lazy
    initialisation - library plans, scratch buffers, the optimizer state - is not part of the capture.
    The returned loss is a static tensor that the next call overwrites."""

    def __init__(self, module, optimizer, example_args=(), example_kwargs: Optional[dict] = None,
                 loss_of: Optional[Callable[[Any], torch.Tensor]] = None, warmup_steps: int = 0):
        from . import comm_ops

        if not hasattr(optimizer, "advance_for_replay"):
            raise TypeError("GraphedTrainStep needs an optimizer whose hyper-parameters live on the device "
                            "(autoparallel_b200.optim.AdamW)")
        if comm_ops._symm_backends and comm_ops._symm_standalone:
            raise RuntimeError("the symmetric-memory collectives keep epochs on the host and cannot be replayed from a graph")
        for be in comm_ops._dma_backends.values():
            if getattr(be, "reductions", False):
                raise RuntimeError("the copy-engine reduce-scatter keeps sequence numbers on the host and cannot be replayed; "
                                   "enable the copy-engine back-end with reductions=False")
        self.module, self.optimizer, self.loss_of = module, optimizer, loss_of
        example_kwargs = dict(example_kwargs or {})
        self._static_args = [a.clone() if isinstance(a, torch.Tensor) else a for a in example_args]
        self._static_kwargs = {k: (v.clone() if isinstance(v, torch.Tensor) else v) for k, v in example_kwargs.items()}
        for _ in range(warmup_steps):
            self._eager_step()
        from ..ops import cuda_impl

        optimizer.prepare_capture()
        torch.cuda.synchronize()
        # blocks cached by the eager steps would otherwise sit beside the graph's private pool
        torch.cuda.empty_cache()
        self.graph = torch.cuda.CUDAGraph()
        before = cuda_impl.launch_count
        with torch.cuda.graph(self.graph):
            self._static_loss = self._eager_step()
        #: kernels of this framework inside one replay (the launch counter only sees the capture)
        self.kernels_per_replay = cuda_impl.launch_count - before
        self.replays = 0

    def release(self) -> None:
        """Drop the captured graph and its memory pool.  Call before ``destroy_process_group`` when the step contains
        collectives: a communicator must not be torn down while a graph still holds its kernels."""
        torch.cuda.synchronize()
        if self.graph is not None:
            self.graph.reset()
        self.graph = None
        self._static_loss = None

    def _eager_step(self) -> torch.Tensor:
        out = self.module(*self._static_args, **self._static_kwargs)
        loss = self.loss_of(out) if self.loss_of is not None else out
        loss.backward()
        self.optimizer.step()
        self.optimizer.zero_grad(set_to_none=True)
        return loss.detach()

    def __call__(self, *args, **kwargs) -> torch.Tensor:
        if len(args) != len(self._static_args) or set(kwargs) != set(self._static_kwargs):
            raise ValueError("a graphed step must be called with the arguments it was captured with")
        for dst, src in zip(self._static_args, args):
            if isinstance(dst, torch.Tensor):
                dst.copy_(src, non_blocking=True)
        for k, dst in self._static_kwargs.items():
            if isinstance(dst, torch.Tensor):
                dst.copy_(kwargs[k], non_blocking=True)
        from ..ops import cuda_impl

        self.optimizer.advance_for_replay()
        self.graph.replay()
        self.replays += 1
        cuda_impl._count(self.kernels_per_replay)
        return self._static_loss
