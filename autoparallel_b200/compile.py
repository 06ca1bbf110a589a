"""``autoparallel_backend`` - a ``torch.compile`` backend for parallel modules.

The reference's backend hands the graph to Inductor with overlap scheduling, bucketing, its
activation-checkpointing joint pass and a partitioner that replays saved-tensor decisions
(autoparallel/compile.py:19-310).  This framework does not generate kernels with a tracing
compiler: the parallel module's forward is already a scheduled graph of hand-written kernels.  The
backend therefore keeps Dynamo from re-tracing that graph - it returns the captured FX module to
run eagerly (each node is one kernel launch) - and applies the options that still have a meaning:

* ``enable_ac`` / ``ac_stage_size_in_GiB``: every live parallel module that was built without
  activation checkpointing is re-partitioned under the "full" policy (recompute from stage
  boundaries chosen by least live memory, stages of the given size or, with ``"auto"``, of the square
  root of the recomputable memory) the first time the backend runs.  A module built with an explicit
  policy keeps it.
* ``overlap_scheduling`` / ``bucketing``: applied to a *user* graph that contains ``apb200_comm``
  collectives (code written against ``autoparallel_b200.collectives``).

``torch.compile(parallel, backend=autoparallel_backend(), fullgraph=True)`` works in training and
under ``no_grad``.
"""
from __future__ import annotations

import weakref
from typing import Callable, Optional, Union

import torch.fx as fx

_live_modules: "weakref.WeakSet" = weakref.WeakSet()


def register_parallel_module(module) -> None:
    """Called by ``AutoParallel.apply_placement`` for every parallel module it builds."""
    _live_modules.add(module)


def autoparallel_backend(enable_ac: bool = True, ac_stage_size_in_GiB: Optional[Union[float, str]] = "auto",
                         overlap_scheduling: bool = True, bucketing: bool = False) -> Callable:
    """Returns a Dynamo backend ``(gm, example_inputs) -> callable`` (defaults as in the reference:
    activation checkpointing on, stage size "auto")."""
    if ac_stage_size_in_GiB is not None and ac_stage_size_in_GiB != "auto" and not float(ac_stage_size_in_GiB) > 0:
        raise ValueError(f"ac_stage_size_in_GiB must be positive, 'auto' or None, got {ac_stage_size_in_GiB!r}")
    applied: list = []

    def backend(gm: fx.GraphModule, example_inputs):
        from .runtime import comm_ops

        if enable_ac:
            stage = None if ac_stage_size_in_GiB in (None, "auto") else float(ac_stage_size_in_GiB)
            for mod in list(_live_modules):
                if mod.__dict__.get("_apb200_ac_mode", "none") == "none" and "set_activation_checkpointing" in mod.__dict__:
                    applied.append(mod.__dict__["set_activation_checkpointing"]("full", stage))
        has_coll = any(n.op == "call_function" and n.target in comm_ops.COLLECTIVE_OPS for n in gm.graph.nodes)
        if has_coll and bucketing:
            from .parallel.passes.bucketing import bucket_collectives

            bucket_collectives(gm)
        if has_coll and overlap_scheduling:
            from .parallel.passes.overlap import schedule_for_streams

            gm = schedule_for_streams(gm)
        return gm.forward

    backend.enable_ac = enable_ac
    backend.ac_stage_size_in_GiB = ac_stage_size_in_GiB
    backend.reconfigured = applied  # what each re-partitioned module reported (mode, saved bytes)
    return backend
