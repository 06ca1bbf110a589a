"""``autoparallel_backend`` – a ``torch.compile`` backend for parallel modules.

The reference's backend hands the graph to Inductor with overlap scheduling, bucketing and a
partitioner that replays saved-tensor decisions (autoparallel/compile.py:19-310).  This framework
does not generate kernels with a tracing compiler: the parallel module's forward is already a
scheduled graph of hand-written kernels.  The backend therefore only has to keep Dynamo from
re-tracing that graph: it returns the captured FX module to run eagerly (each node is one kernel
launch), optionally after applying the activation-checkpointing, bucketing and overlap passes to
any *user* graph that reaches it.  ``torch.compile(parallel, backend=autoparallel_backend(),
fullgraph=True)`` works in training and under ``no_grad``.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch.fx as fx


def autoparallel_backend(enable_ac: bool = False, ac_stage_size_in_GiB: Optional[float] = None,
                         overlap_scheduling: bool = True, bucketing: bool = False) -> Callable:
    """Returns a Dynamo backend ``(gm, example_inputs) -> callable``.

    ``overlap_scheduling`` / ``bucketing`` apply this framework's passes when the graph handed over
    by Dynamo contains ``apb200_comm`` collectives (a user graph written against
    ``autoparallel_b200.collectives``); graphs without collectives are returned unchanged."""

    def backend(gm: fx.GraphModule, example_inputs):
        from .runtime import comm_ops

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
    return backend
