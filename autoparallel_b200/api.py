"""Public entry points: ``AutoParallel`` (context manager) and ``auto_parallel`` (one call).

    with AutoParallel(model, input_fn, mesh, mp_policy) as autop:
        autop.add_parameter_memory_constraint()            # FSDP knob
        autop.add_input_constraints([(Shard(0),), ...])
        placement = autop.optimize_placement()
        parallel = autop.apply_placement(placement)
    parallel.to_empty(device="cuda"); parallel.init_weights()
    loss = parallel(local_tokens, labels=local_labels); loss.backward()

``model`` lives on the meta device and ``input_fn`` returns *global* example inputs; the returned
module takes this rank's *local* shards, returns local tensors, and owns ``DTensor`` parameters
(so ``torch.distributed.checkpoint`` and ``torch.optim`` work on it unchanged).

Behavioural parity target: autoparallel/api.py:231-774.  What differs is everything under the
API: the ILP runs on HiGHS with node/edge variables, lowering builds the per-rank graph directly,
partitioning is tag-driven, and the per-rank graph is executed by this framework's runtime
(``runtime/executor.py``) on its own sm_100a kernels and collectives.
"""
from __future__ import annotations

import contextlib
import logging
import json
import time
from typing import Any, Callable, Optional, Sequence

import torch
import torch.nn as nn
from torch._subclasses import FakeTensorMode
from torch.distributed.tensor import DTensor
from torch.distributed.tensor.placement_types import Placement, Replicate, Shard
from torch.utils._pytree import tree_flatten, tree_unflatten

from .parallel.cost import comm as comm_cost
from .parallel.cost import device as device_cost
from .parallel.frontend import mp_cast
from .parallel.frontend.trace import ForwardInputs, JointGraph, build_joint_graph, clone_model_for_tracing, move_to_fake
from .parallel.lower import inputs as input_utils
from .parallel.lower.apply import LoweredGraph, lower_to_local_graph
from .parallel.lower.init_weights import wrap_init_weights
from .parallel.lower.module_build import make_parallel_module
from .parallel.lower.partition import extract_forward, partition_joint
from .parallel.passes.act_ckpt import apply_activation_checkpointing, apply_user_checkpoint_tags, mark_fsdp_recompute
from .parallel.solver.ilp import InfeasibleError, ShardingOptimizer

logger = logging.getLogger(__name__)


def _mesh_device(mesh) -> torch.device:
    if mesh.device_type == "cuda":
        return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    return torch.device(mesh.device_type)


def _artifact(name: str, encoding: str, payload_fn) -> None:
    """Structured-trace artifact (``TORCH_TRACE=<dir>`` + tlparse): the joint graph, the optimizer's log, the solution
    and the parallel graph are dumped under the names the reference uses (autoparallel/api.py:212-221, 409-418,
    430-437, 481-490), so existing tooling finds them.  The payload is only built when a trace is being written."""
    try:
        from torch._logging import trace_structured

        trace_structured("artifact", metadata_fn=lambda: {"name": name, "encoding": encoding}, payload_fn=payload_fn)
    except Exception as e:  # tracing must never break planning
        logger.debug("structured trace artifact %s not written: %s", name, e)


class AutoParallel:
    """Trace ``model``, search placements, and build the parallel module.

    Args:
        model: module on the meta device (it is deep-copied, never modified).
        input_fn: returns global example inputs – a tensor, a tuple, or ``ForwardInputs``.
        mesh: ``DeviceMesh`` whose dims are the axes placements refer to.
        mp_policy: object with ``param_dtype / reduce_dtype / output_dtype / cast_forward_inputs``.
        reshard_after_forward: re-gather FSDP parameters in backward instead of keeping them.
        cost_model: ``"auto"`` (NVLink-5 α–β model or CPU loopback by mesh device), ``"nccl"`` (NCCL's algorithm /
            protocol model, multi-node aware), ``"measured"`` / ``"measured:symm"`` (tables taken on B200), a
            ``comm.Topology``, or a path to a calibration table (JSON).
        repeated_subgraphs: share ILP variables between structurally identical layers.
        activation_checkpointing: ``"none" | "selective" | "full"``.
        uneven_sharding: allow shards of unequal size (extents that the mesh dim does not divide).
    """

    def __init__(
        self,
        model: nn.Module,
        input_fn: Callable,
        mesh,
        mp_policy: Any = None,
        reshard_after_forward: bool = True,
        dynamic: bool = False,
        cost_model: Any = "auto",
        repeated_subgraphs: bool = True,
        activation_checkpointing: str = "none",
        plan_device: Optional[str] = None,
        fuse_collectives: Any = None,
        bucket_collectives: Any = False,
        ordered_sharding: bool = True,
        uneven_sharding: bool = False,
        pattern_ops: bool = True,
    ):
        # pattern_ops=True: stock-PyTorch idioms of the model (nn.RMSNorm, F.silu(a) * b, rotary embedding by complex
        # multiplication, F.scaled_dot_product_attention) are rewritten to this framework's operators while tracing
        # (parallel/passes/pattern_ops.py); False keeps the traced ATen operators.
        self.pattern_ops = bool(pattern_ops)
        # uneven_sharding=True: a tensor dim may be sharded although the mesh dim does not divide it.  Shards are
        # ceil-sized chunks (the last one shorter; splits that would leave a rank empty are not offered); every rank lowers the graph with
        # its own shard shapes and collectives on such dims pad to the chunk size and cut the result.
        self.uneven_sharding = bool(uneven_sharding)
        # dynamic=True: graphs stay specialised to static shapes (every kernel launch has fixed extents), but the
        # parallel module accepts inputs of other shapes by building - once per shape - a new specialisation
        # that reuses the solved placements instead of solving again (see ``_specialize``).
        self.dynamic = bool(dynamic)
        self.fake_mode = FakeTensorMode()
        self.mp_policy = mp_cast.canonicalize_mp(mp_policy)
        self.mesh = mesh
        self.input_fn = input_fn
        self.reshard_after_forward = reshard_after_forward
        self.repeated_subgraphs = repeated_subgraphs
        self.cost_model = cost_model
        self.activation_checkpointing = activation_checkpointing
        #: "full" checkpointing: bytes of activations per recomputation stage (None = square-root rule)
        self.ac_stage_bytes: Optional[int] = None
        self.user_ac_stats: dict = {}
        self.ac_stats: dict = {}
        self.plan_device = plan_device
        self.fuse_collectives = fuse_collectives
        # False: every collective stays its own node; True: collectives below 4 MiB are merged up to fixed caps;
        # "auto": the bucket plan is made from priced collectives, a compute window and a memory headroom
        self.bucket_collectives = bucket_collectives
        #: "auto" bucketing: bytes a bucket may keep alive beyond what the separate collectives would
        self.bucket_headroom_bytes: int = 2 << 30
        self.ordered_sharding = ordered_sharding
        self.bucket_stats = {}
        self.fusion_stats = {}
        model = clone_model_for_tracing(model)
        if self.mp_policy is not None:
            mp_cast.apply_dtype_cast(model, self.mp_policy)
        # fake tensors live on CPU: planning never touches a device
        self.model = move_to_fake(model, self.fake_mode, "cpu")
        self.active: Optional[bool] = False
        self.input_constraints = None
        self.output_constraints = None
        self.timings: dict[str, float] = {}

    # ------------------------------------------------------------------ context management
    def __enter__(self):
        if self.active is not False:
            raise RuntimeError("AutoParallel is not re-entrant")
        self._stack = contextlib.ExitStack()
        try:
            self._prev_topology = comm_cost._topology
            self._prev_limit = device_cost._override
            self._install_cost_models()
            self._stack.enter_context(self.mesh)
            t0 = time.perf_counter()
            self.joint = build_joint_graph(self.model, self.input_fn, self.fake_mode, pattern_ops=self.pattern_ops)
            self.gm = self.joint.gm
            self.timings["trace"] = time.perf_counter() - t0
            _artifact("autoparallel_joint_graph", "string", lambda: self.gm.print_readable(print_output=False))
            t0 = time.perf_counter()
            self.sharding_optimizer = self._new_optimizer(self.joint)
            self.timings["build_optimizer"] = time.perf_counter() - t0
            self.active = True
        except BaseException:
            self._restore()
            self._stack.close()
            raise
        return self

    def _new_optimizer(self, joint) -> ShardingOptimizer:
        force_hp = (
            self.mp_policy is not None
            and self.mp_policy.reduce_dtype is not None
            and self.mp_policy.param_dtype is not None
            and self.mp_policy.reduce_dtype.itemsize > self.mp_policy.param_dtype.itemsize
        )
        return ShardingOptimizer(joint, self.mesh, force_grad_reduce_in_higher_precision=force_hp,
                                 repeated_subgraphs=self.repeated_subgraphs, even_only=not self.uneven_sharding)

    def _install_cost_models(self) -> None:
        # topology first, then the device table
        if isinstance(self.cost_model, comm_cost.Topology):
            comm_cost.set_topology(self.cost_model)
        else:
            topo = comm_cost.Topology.for_mesh(self.mesh)
            if self.plan_device is not None:
                topo = comm_cost.Topology([comm_cost.NVLINK5] * self.mesh.ndim)
            if self.cost_model == "nccl":
                # NCCL's own algorithm / protocol choice per collective; nodes of 8 GPUs unless the mesh is smaller
                from .parallel.cost import nccl_model

                name = self.plan_device or (torch.cuda.get_device_name(0) if torch.cuda.is_available() else "B200")
                cfg = nccl_model.detect_topology(self.mesh.size(), ranks_per_host=min(self.mesh.size(), 8), device_name=name)
                topo = comm_cost.NcclTopology(cfg, tuple(self.mesh.shape))
            if isinstance(self.cost_model, str) and self.cost_model not in ("auto", "nccl"):
                # "measured" / "measured:symm": the table taken on this device type that ships with the package
                if self.cost_model.startswith("measured"):
                    backend = self.cost_model.partition(":")[2] or "nccl"
                    path = comm_cost.Topology.measured_table_path(self.plan_device or "B200", backend)
                    if path is None:
                        raise ValueError(f"no measured collective table for {self.plan_device or 'B200'} / {backend}")
                    topo.load_table(path)
                else:
                    topo.load_table(self.cost_model)
            comm_cost.set_topology(topo)
        if self.plan_device is not None:
            device_cost.set_device_limit(device_cost.DEVICE_LIMITS[self.plan_device])

    def _restore(self):
        comm_cost.set_topology(self._prev_topology)
        device_cost.set_device_limit(self._prev_limit)

    def __exit__(self, exc_type, exc, tb):
        self._restore()
        self.active = None
        return self._stack.__exit__(exc_type, exc, tb)

    def _assert_entered(self):
        if self.active is False:
            raise RuntimeError("use AutoParallel as a context manager: `with AutoParallel(...) as autop:`")
        if self.active is None:
            raise RuntimeError("this AutoParallel context has exited; it is not re-entrant")

    # ------------------------------------------------------------------ constraints
    def add_parameter_memory_constraint(self, low: Optional[float] = None, high: Optional[float] = None, *,
                                        budget_bytes: Optional[float] = None, bytes_per_element: float = 16.0):
        """Bound how much of the parameters every rank holds.

        ``(low, high)`` is the reference's form (autoparallel/api.py: bounds on the mean per-parameter shard
        ratio; ``high`` defaults to ``1 / mesh.size()``, i.e. fully sharded).  ``budget_bytes`` states the bound in
        bytes instead: the per-rank bytes of parameter state, ``sum over parameters of (elements held locally x
        bytes_per_element)``, must not exceed it.  ``bytes_per_element`` is the state kept per parameter element -
        16 for an fp32 master copy, an fp32 gradient and two fp32 Adam moments, 18 with a bf16 copy on top - so
        "fit the optimizer state of a 70B model into 180 GB per GPU" is ``budget_bytes=180e9 - activations``."""
        self._assert_entered()
        if budget_bytes is not None:
            if low is not None or high is not None:
                raise ValueError("give either (low, high) or budget_bytes, not both")
            if budget_bytes <= 0 or bytes_per_element <= 0:
                raise ValueError("budget_bytes and bytes_per_element must be positive")
            return self.sharding_optimizer.add_parameter_bytes_constraint(float(budget_bytes), float(bytes_per_element))
        low = 0.0 if low is None else low
        high = 1.0 / self.mesh.size() if high is None else high
        if low > high:
            raise ValueError(f"low must be <= high, got low={low}, high={high}")
        return self.sharding_optimizer.add_parameter_memory_constraint(low, high)

    def add_input_constraints(self, constraints: Sequence[Optional[Sequence[Placement]]]):
        self._assert_entered()
        if self.input_constraints is not None:
            raise AssertionError("input constraints have already been set")
        self.sharding_optimizer.add_sharded_input_constraint(constraints)
        self.input_constraints = list(constraints)

    def add_output_constraints(self, constraints: Sequence[Optional[Sequence[Placement]]]):
        self._assert_entered()
        if self.output_constraints is not None:
            raise AssertionError("output constraints have already been set")
        self.sharding_optimizer.add_sharded_output_constraint(constraints)
        self.output_constraints = list(constraints)

    # ------------------------------------------------------------------ solve / apply
    def optimize_placement(self, verbose: bool = False):
        self._assert_entered()
        t0 = time.perf_counter()
        try:
            self.sharding_placement = self.sharding_optimizer.get_solution(verbose=False)
        except InfeasibleError as e:
            raise RuntimeError(
                "The sharding optimizer could not find a feasible solution. This usually means the constraints "
                "contradict each other or the mesh is too large for the tensors being sharded. " + str(e)
            ) from e
        self.timings["solve"] = time.perf_counter() - t0
        if verbose:
            logger.info(self.sharding_optimizer.get_log(verbose=True))
        _artifact("autoparallel_sharding_optimizer_log", "string", lambda: self.sharding_optimizer.get_log(verbose=True, colored=False))
        _artifact("autoparallel_solution", "json", lambda: json.dumps(self.sharding_optimizer.get_json()))
        return self.sharding_placement

    def lower(self, sharding_placement=None) -> LoweredGraph:
        self._assert_entered()
        sol = sharding_placement if sharding_placement is not None else self.sharding_placement
        t0 = time.perf_counter()
        lowered = self._lower(self.joint, sol)
        self.timings["lower"] = time.perf_counter() - t0
        self.lowered = lowered
        self.parallel_gm = lowered.gm
        _artifact("autoparallel_parallel_graph", "string", lambda: lowered.gm.print_readable(print_output=False))
        return lowered

    def _lower(self, joint: JointGraph, sol) -> LoweredGraph:
        """Solution -> per-rank graph with the graph passes applied (no state of this object is changed
        except the pass statistics)."""
        lowered = lower_to_local_graph(joint, sol, self.mesh, ordered_sharding=self.ordered_sharding)
        from .parallel.frontend.trace import index_joint_graph
        from .parallel.passes.fuse_collectives import fuse_collectives
        from .parallel.passes.peephole import fuse_cast_into_gemm

        changed = fuse_cast_into_gemm(lowered.gm)
        fuse = self.fuse_collectives
        if fuse is None:
            # A fused node is one kernel only where the mesh has symmetric-memory communicators; over
            # NCCL it would run gather-then-GEMM back to back and hide the gather from the overlap
            # scheduler, so the separate nodes are kept there.
            from .runtime import symm

            fuse = symm.enabled_for_mesh(self.mesh)
        if fuse:
            # "all" also fuses gathers along the contraction dim (kept apart by default: they cannot overlap tile by tile)
            # "reductions" rewrites GEMM -> reduce-scatter only (parameter gathers stay separate nodes)
            self.fusion_stats = fuse_collectives(lowered.gm, lowered.joint.tangent_nodes, self.reshard_after_forward,
                                                 fuse_contraction_gather=(fuse == "all"),
                                                 patterns=("mm_rs",) if fuse == "reductions" else ("ag_mm", "mm_rs"))
            changed += sum(self.fusion_stats.values())
        if self.bucket_collectives:
            from .parallel.passes.bucketing import bucket_collectives

            cost = None
            if self.bucket_collectives == "auto":
                # sizes decided by the priced collectives (a calibrated table when ``cost_model`` names one) and by the
                # memory left on the device next to parameters, gradients and optimizer state
                from .parallel.passes.bucketing import BucketCost

                cost = BucketCost.from_mesh(self.mesh, self.plan_device, headroom_bytes=self.bucket_headroom_bytes)
            self.bucket_stats = bucket_collectives(lowered.gm, cost=cost)
            changed += self.bucket_stats["members"]
        if changed:
            lowered.joint = index_joint_graph(lowered.gm, joint.traced_inputs, joint.out_spec)
        mark_fsdp_recompute(lowered.joint, self.reshard_after_forward)
        # regions the user wrapped in torch.utils.checkpoint (with or without a selective policy) come first;
        # the framework's own policy below never touches a node the user has tagged
        self.user_ac_stats = apply_user_checkpoint_tags(lowered.joint)
        if self.activation_checkpointing != "none":
            self.ac_stats = apply_activation_checkpointing(lowered.joint, self.activation_checkpointing,
                                                           stage_bytes=self.ac_stage_bytes)
        return lowered

    def _build_runtime(self, joint: JointGraph, lowered: LoweredGraph, executor, overlap_config):
        """(runtime, expected local inputs, traced inputs, pytree spec of the output) of one specialisation."""
        from .runtime.executor import build_runtime

        parts = partition_joint(lowered.joint)
        fwd_only = extract_forward(lowered.joint)
        runtime = build_runtime(lowered, parts, fwd_only, self.mesh, executor=executor, overlap_config=overlap_config)
        expected = input_utils.expected_local_inputs(joint.traced_inputs, lowered.input_placements, self.mesh)
        return runtime, expected, joint.traced_inputs, _user_out_spec(joint), parts

    def apply_placement(self, sharding_placement=None, *, executor: Optional[str] = None, overlap_config=None) -> nn.Module:
        """Build the parallel module.  ``executor``: ``None``/"graph" runs the generated FX code,
        "streams" runs it through the multi-stream overlap executor (``overlap_config``: an
        ``parallel.passes.overlap.OverlapConfig`` with the prefetch depth / bytes in flight / pending reductions)."""
        lowered = self.lower(sharding_placement)
        t0 = time.perf_counter()
        runtime, expected, traced, out_spec, parts = self._build_runtime(self.joint, lowered, executor, overlap_config)
        self.partitioned = parts
        sharded_params, sharded_buffers = _meta_state(self.model, lowered, self.mesh)
        param_names = list(lowered.joint.param_nodes)
        buffer_names = list(lowered.joint.buffer_nodes)
        updated_buffers = list(lowered.joint.buffer_updates)
        #: shape key -> specialisation; the planned shapes are the first entry
        specializations = {self._shape_key(expected): (runtime, expected, traced, out_spec)}
        solved = self.sharding_placement if sharding_placement is None else sharding_placement
        planner = self

        #: the specialisation of the planned shapes; replaced when activation checkpointing is reconfigured
        current = {"entry": (runtime, expected, traced, out_spec)}

        def forward(module, *args, **kwargs):
            flat = input_utils.flatten_call(traced, args, kwargs)
            entry = current["entry"]
            if planner.dynamic:
                key = planner._shape_key_of_call(flat, expected)
                entry = specializations.get(key)
                if entry is None:
                    entry = planner._specialize(flat, expected, lowered.input_placements, solved, executor, overlap_config)
                    specializations[key] = entry
            rt, exp, _, ospec = entry
            input_utils.check_forward_args(flat, exp)
            params = [_local(module.get_parameter(n)) for n in param_names]
            buffers = [_local(module.get_buffer(n)) for n in buffer_names]
            tensors = [a for a, e in zip(flat, exp) if e[0] == "tensor"]
            outs = rt(params, buffers, tensors, torch.is_grad_enabled())
            if updated_buffers:  # new values of the buffers the forward mutates ride behind the user's outputs
                outs, new_vals = outs[: len(outs) - len(updated_buffers)], outs[len(outs) - len(updated_buffers):]
                with torch.no_grad():
                    for name, val in zip(updated_buffers, new_vals):
                        _local(module.get_buffer(name)).copy_(val.detach())
            if ospec is not None:
                return tree_unflatten(list(outs), ospec)
            return outs[0] if len(outs) == 1 else tuple(outs)

        def set_activation_checkpointing(mode: str, stage_size_in_GiB: Optional[float] = None) -> dict:
            """Re-partition the lowered graph under another activation-checkpointing policy (same placements, same
            parameters): ``mode`` as in the constructor, ``stage_size_in_GiB`` the stage length of the "full" mode."""
            planner.activation_checkpointing = mode
            planner.ac_stage_bytes = None if stage_size_in_GiB is None else max(1, int(stage_size_in_GiB * 2**30))
            with planner.mesh:
                new_lowered = planner._lower(planner.joint, solved)
                rt, exp, tr, ospec, new_parts = planner._build_runtime(planner.joint, new_lowered, executor, overlap_config)
            planner.partitioned = new_parts
            current["entry"] = (rt, exp, tr, ospec)
            specializations.clear()
            specializations[planner._shape_key(exp)] = current["entry"]
            module.__dict__["_apb200_runtime"] = rt
            module.__dict__["_apb200_lowered"] = new_lowered
            module.__dict__["_apb200_ac_mode"] = mode
            return {"mode": mode, "saved_bytes": new_parts.saved_bytes, "num_saved": new_parts.num_saved}

        module = make_parallel_module(self.model, sharded_params, sharded_buffers, forward)
        module.__dict__["set_activation_checkpointing"] = set_activation_checkpointing
        module.__dict__["_apb200_ac_mode"] = self.activation_checkpointing
        from . import compile as _compile

        _compile.register_parallel_module(module)
        module.__dict__["_apb200_runtime"] = runtime
        module.__dict__["_apb200_lowered"] = lowered
        module.__dict__["_apb200_specializations"] = specializations
        wrap_init_weights(module)
        self.timings["apply"] = time.perf_counter() - t0
        return module

    # ------------------------------------------------------------------ shape specialisation (dynamic=True)
    @staticmethod
    def _shape_key(expected) -> tuple:
        return tuple(e[1] if e[0] == "tensor" else None for e in expected)

    @staticmethod
    def _shape_key_of_call(flat, expected) -> tuple:
        return tuple(tuple(a.shape) if e[0] == "tensor" and isinstance(a, torch.Tensor) else None for a, e in zip(flat, expected))

    def _specialize(self, flat, expected, input_placements, solved, executor, overlap_config):
        """A second (third, ...) specialisation of the parallel module for inputs of another shape: the model
        is traced again at the new global shapes and every node takes the placement it has in the solved
        plan - matched by node name and placement, not solved again.  Raises if the two graphs differ in
        structure (shape-dependent control flow) or a placement does not exist at the new shape (a dim that
        no longer divides by the mesh)."""
        flat_traced, spec = tree_flatten((self.joint.traced_inputs.args, self.joint.traced_inputs.kwargs))
        new_flat = []
        for a, e, pl, old in zip(flat, expected, list(input_placements) + [None] * len(flat), flat_traced):
            if e[0] != "tensor":
                new_flat.append(old)
                continue
            if not isinstance(a, torch.Tensor) or a.ndim != len(e[1]) or a.dtype != e[2]:
                input_utils.check_forward_args(flat, expected)  # reports rank / dtype mismatches in the usual words
            g = list(a.shape)
            for n, p in zip(self.mesh.shape, pl or ()):
                if isinstance(p, Shard):
                    g[p.dim] *= n
            new_flat.append(("global", tuple(g), a.dtype))

        def input_fn():
            vals = [torch.zeros(v[1], dtype=v[2]) if isinstance(v, tuple) and v and v[0] == "global" else v for v in new_flat]
            args, kwargs = tree_unflatten(vals, spec)
            return ForwardInputs(tuple(args), dict(kwargs))

        prev_topo, prev_limit = comm_cost._topology, device_cost._override
        try:
            self._install_cost_models()
            with self.mesh:
                joint = build_joint_graph(self.model, input_fn, self.fake_mode, pattern_ops=self.pattern_ops)
                opt = self._new_optimizer(joint)
                sol = _transfer_solution(solved, opt)
                lowered = self._lower(joint, sol)
                runtime, exp, traced, out_spec, _ = self._build_runtime(joint, lowered, executor, overlap_config)
        finally:
            comm_cost.set_topology(prev_topo)
            device_cost.set_device_limit(prev_limit)
        for (k, v), (k2, v2) in zip(lowered.param_placements.items(), self.lowered.param_placements.items()):
            if k != k2 or tuple(v or ()) != tuple(v2 or ()):
                raise RuntimeError(f"specialisation for new input shapes changed the placement of parameter {k}")
        got = self._shape_key_of_call(flat, exp)
        if got != self._shape_key(exp):
            raise ValueError(f"inputs of local shapes {got} do not correspond to whole shards of a global batch on this mesh")
        return runtime, exp, traced, out_spec


def _transfer_solution(solved: dict, opt) -> dict:
    """Solution for ``opt``'s graph that gives every node the placements it has in ``solved`` (a solution of a graph
    of the same structure traced at other shapes)."""
    from .parallel.solver.ilp import _out_placements

    def sig(spec):
        ins = tuple(tuple(i.placements) if i is not None else None for i in (spec.input_specs or ()))
        return (_out_placements(spec), ins)

    by_name = {n.name: sig(s) for n, s in solved.items()}
    sol, selected = {}, {}
    for n in opt.nodes:
        want = by_name.get(n.name)
        if want is None:
            raise RuntimeError(f"the graph traced at the new shapes has a node the plan does not know ({n.name}): "
                               "the model's structure depends on the input shape")
        idx = next((i for i, s in enumerate(opt.strats[n].strategies) if sig(s) == want), None)
        if idx is None:
            raise RuntimeError(f"placement {want[0]} of {n.name} is not available at the new input shape "
                               "(a sharded dim no longer divides by the mesh?)")
        selected[n] = idx
        sol[n] = opt.strats[n].strategies[idx]
    opt.selected, opt.solution = selected, sol
    opt._validate()
    return sol


def _local(t):
    return t.to_local() if isinstance(t, DTensor) else t


def _user_out_spec(joint: JointGraph):
    spec = joint.out_spec
    return spec


def _meta_state(model: nn.Module, lowered: LoweredGraph, mesh):
    """Meta-device DTensor parameters / buffers with the solved placements (the caller
    materialises them with ``to_empty`` + ``init_weights``)."""

    params, buffers = {}, {}

    def make(t: torch.Tensor, placements, requires_grad):
        placements = placements or (Replicate(),) * mesh.ndim
        from .parallel.strategies.dtensor_adapter import my_local_shape

        ls = my_local_shape(t.shape, mesh, placements)
        local = torch.empty(ls, dtype=t.dtype, device="meta")
        return DTensor.from_local(local, mesh, placements, run_check=False, shape=t.shape, stride=_contig_stride(t.shape))

    for fqn, p in model.named_parameters():
        dt = make(p, lowered.param_placements.get(fqn), p.requires_grad)
        params[fqn] = nn.Parameter(dt, requires_grad=p.requires_grad)
    for fqn, b in model.named_buffers():
        buffers[fqn] = make(b, lowered.buffer_placements.get(fqn), False)
    return params, buffers


def _contig_stride(shape):
    stride, acc = [], 1
    for s in reversed(shape):
        stride.append(acc)
        acc *= s
    return tuple(reversed(stride))


def auto_parallel(
    model: nn.Module,
    mesh,
    sample_inputs,
    *,
    sample_kwargs: Optional[dict] = None,
    out_shardings=None,
    mp_policy=None,
    parameter_memory: Optional[tuple] = (None, None),
    reshard_after_forward: bool = True,
    **kwargs,
) -> nn.Module:
    """One-call API: placements of DTensor sample inputs become input constraints, plain tensors are
    replicated, ``out_shardings`` (a placement tuple or a pytree of them) become output
    constraints, and the FSDP memory band is applied unless ``parameter_memory=None``.
    Reference: autoparallel/api.py:667-774."""
    if not isinstance(sample_inputs, tuple):
        sample_inputs = (sample_inputs,)
    input_fn, in_pl = input_utils.input_fn_from_samples(sample_inputs, sample_kwargs)
    with AutoParallel(model, input_fn, mesh, mp_policy=mp_policy, reshard_after_forward=reshard_after_forward, **kwargs) as ap:
        rep = (Replicate(),) * mesh.ndim
        cons = []
        for node, pl in zip(ap.joint.input_nodes, in_pl):
            cons.append(None if node is None else (pl if pl is not None else rep))
        ap.add_input_constraints(cons)
        if parameter_memory is not None:
            ap.add_parameter_memory_constraint(*parameter_memory)
        if out_shardings is not None:
            ap.add_output_constraints(
                input_utils.flatten_out_shardings(out_shardings, ap.joint.num_user_outputs or len(ap.joint.fwd_outputs), mesh)
            )
        ap.optimize_placement()
        return ap.apply_placement()
