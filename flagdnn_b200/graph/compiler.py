"""Capture -> optimise -> plan -> run, the user-facing half of the graph API.

Mirrors the call surface of the reference (src/flag_dnn/graph/capture.py:
109-208 ``graph`` / ``compile`` / ``CompiledGraph``; planner, kernel selector
and executor in src/flag_dnn/graph/{planner,kernel_selector,backend,executor,
plan,cache}.py) for graphs built from the ops this package registers.  The
keys of ``plan.debug_info`` that the reference's tests read ("fusion",
"kernel_candidates", "backend", "cache_hit", "cache_layer", "autotune",
"candidate_count") are kept.
"""
from __future__ import annotations

import functools
import hashlib
import json
import os
from dataclasses import dataclass, field
from typing import Any, Callable, Optional

import torch

from .ir import Graph
from .passes import apply_fusion_pass, eliminate_dead_nodes
from .memory import MemoryPlan, allocate_memory
from .registry import get_op_schema
from .spec import GraphTensor, TensorSpec, torch_dtype

_CAPTURE_STACK: list = []


def is_capturing() -> bool:
    return bool(_CAPTURE_STACK)


def current_capture() -> Optional["GraphCapture"]:
    return _CAPTURE_STACK[-1] if _CAPTURE_STACK else None


class GraphCapture:
    """Context in which op wrappers record nodes instead of running kernels."""

    def __init__(self, input_specs: list):
        self.graph = Graph()
        self.input_specs = input_specs
        self.graph_inputs: list = []

    def __enter__(self) -> "GraphCapture":
        _CAPTURE_STACK.append(self)
        for index, spec in enumerate(self.input_specs):
            self.graph_inputs.append(self.graph.add_input(spec if spec.name else spec.with_name(f"arg{index}")))
        return self

    def __exit__(self, exc_type, exc, tb) -> None:
        if _CAPTURE_STACK.pop() is not self:
            raise RuntimeError("graph capture stack is corrupted")

    def is_tensor_like(self, value: Any) -> bool:
        return isinstance(value, (GraphTensor, torch.Tensor))

    def as_value(self, value: Any, name_hint: str = "value") -> int:
        if isinstance(value, GraphTensor):
            if value.graph is not self.graph:
                raise RuntimeError("cannot mix GraphTensor values from graphs")
            return value.value_id
        if isinstance(value, (torch.Tensor, int, float, bool)):
            return self.graph.add_constant(value, name_hint=name_hint).value_id
        raise TypeError(f"unsupported graph operand type: {type(value)!r}")

    def add_op_call(self, op_type: str, args: tuple, kwargs: dict) -> GraphTensor:
        input_ids, attrs = get_op_schema(op_type).normalize(self, args, dict(kwargs))
        return self.graph.add_op(op_type, input_ids, attrs)

    def add_binary_op(self, op_type: str, left: Any, right: Any, reverse: bool = False) -> GraphTensor:
        attrs: dict = {}
        if reverse and self.is_tensor_like(right):
            ids = [self.as_value(right, "other"), self.as_value(left, "input")]
        else:
            ids = [self.as_value(left, "input")]
            if self.is_tensor_like(right):
                ids.append(self.as_value(right, "other"))
            else:
                attrs["other"] = right
                attrs["reverse"] = reverse
        return self.graph.add_op(op_type, ids, attrs)

    def finalize(self, outputs: Any) -> tuple:
        flat, structure = _flatten_outputs(outputs)
        self.graph.mark_outputs(flat)
        self.graph.lint()
        return self.graph, structure


def _flatten_outputs(outputs: Any) -> tuple:
    flat: list = []

    def visit(value: Any) -> Any:
        if isinstance(value, GraphTensor):
            flat.append(value.value_id)
            return ("leaf",)
        if isinstance(value, (tuple, list)):
            return ("tuple" if isinstance(value, tuple) else "list", [visit(v) for v in value])
        if isinstance(value, dict):
            return ("dict", [(k, visit(v)) for k, v in value.items()])
        raise TypeError(f"graph functions must return GraphTensor values, got {type(value)!r}")

    return flat, visit(outputs)


def _rebuild_outputs(structure: Any, flat: list) -> Any:
    it = iter(flat)

    def build(node: Any) -> Any:
        kind = node[0]
        if kind == "leaf":
            return next(it)
        if kind == "tuple":
            return tuple(build(c) for c in node[1])
        if kind == "list":
            return [build(c) for c in node[1]]
        return {k: build(c) for k, c in node[1]}

    return build(structure)


class GraphFunction:
    def __init__(self, fn: Callable, **options: Any) -> None:
        self.fn = fn
        self.options = dict(options)
        functools.update_wrapper(self, fn)

    def __call__(self, *args: Any, **kwargs: Any) -> Any:
        return self.fn(*args, **kwargs)


def graph(fn: Optional[Callable] = None, **options: Any):
    """Decorator marking a function for ``compile`` (src/flag_dnn/graph/capture.py:121)."""
    if fn is None:
        return lambda inner: GraphFunction(inner, **options)
    return GraphFunction(fn, **options)


# ------------------------------------------------------------------ planning
@dataclass
class ExecutionStep:
    op_type: str
    inputs: list
    outputs: list
    attrs: dict = field(default_factory=dict)
    backend: str = "sm100"
    kernel_name: Optional[str] = None
    workspace: int = 0


@dataclass
class ExecutionPlan:
    graph_hash: str
    plan_id: str
    graph: Graph
    steps: list
    input_specs: list
    output_specs: list
    workspace_size: int = 0
    memory_plan: Optional[MemoryPlan] = None
    tuned: bool = False
    debug_info: dict = field(default_factory=dict)

    def run(self, *inputs: Any) -> Any:
        return execute_plan(self, inputs)


def _candidates_for(node, graph: Graph) -> list:
    """Kernel candidates of a node, best first (cf. backend.py:109-151 of the reference)."""
    if node.op_type == "fused_conv2d_bias_relu":
        return [
            {"name": "fused_conv2d_bias_relu.sm100_igemm", "backend": "sm100", "op_type": node.op_type,
             "implementation": "sm100_fused", "priority": 0,
             "configs": [{"tile_m": 128, "tile_k_bytes": 128, "accumulators": 2}]},
            {"name": "fused_conv2d_bias_relu.sm100_direct", "backend": "sm100", "op_type": node.op_type,
             "implementation": "sm100_direct", "priority": 50, "configs": []},
        ]
    if node.op_type == "fused_conv2d_bias_gelu":
        return [{"name": "fused_conv2d_bias_gelu.sm100_igemm", "backend": "sm100", "op_type": node.op_type,
                 "implementation": "sm100_fused", "priority": 0,
                 "configs": [{"tile_m": 128, "tile_k_bytes": 128, "accumulators": 2}]}]
    if node.op_type == "fused_conv2d_bias_add_relu":
        return [{"name": "fused_conv2d_bias_add_relu.sm100_igemm", "backend": "sm100", "op_type": node.op_type,
                 "implementation": "sm100_fused_residual", "priority": 0,
                 "configs": [{"tile_m": 128, "tile_k_bytes": 128, "accumulators": 2}]}]
    if node.op_type == "conv2d":
        return [{"name": "conv2d.sm100", "backend": "sm100", "op_type": node.op_type,
                 "implementation": "sm100", "priority": 0, "configs": []}]
    return [{"name": node.op_type, "backend": "torch", "op_type": node.op_type,
             "implementation": "default", "priority": 100, "configs": []}]


def _build_plan(graph_obj: Graph, specs: list, output_structure: Any, options: dict) -> ExecutionPlan:
    steps, chosen, total_candidates = [], [], 1
    for node in graph_obj.topological_nodes():
        cands = _candidates_for(node, graph_obj)
        total_candidates *= len(cands)
        best = cands[0]
        attrs = dict(node.attrs)
        attrs["_implementation"] = best["implementation"]
        attrs["_kernel_candidate"] = best["name"]
        if best["configs"]:
            attrs["_kernel_config"] = dict(best["configs"][0])
        steps.append(ExecutionStep(node.op_type, list(node.inputs), list(node.outputs), attrs,
                                   backend=best["backend"], kernel_name=best["name"]))
        chosen.append(best)
    # Intermediate values get a place in one workspace (first-fit reuse of dead blocks); with
    # options={"workspace": True} the executor hands those places to the nodes as their outputs.
    memory_plan = allocate_memory(graph_obj)
    ghash = graph_obj.graph_hash()
    autotune = bool(options.get("autotune", False)) or str(os.getenv("FLAGDNN_AUTOTUNE", "0")).lower() in ("1", "true", "yes")
    debug = {
        "backend": "sm100",
        "requested_backend": str(options.get("backend", "auto")),
        "cache_hit": False,
        "output_structure": output_structure,
        "num_steps": len(steps),
        "fusion": dict(graph_obj.attrs.get("fusion", {})),
        "kernel_candidates": chosen,
        "candidate_count": min(total_candidates, int(options.get("max_plan_candidates", 8))),
        "memory": memory_plan.to_dict(),
        "selector": "static_priority",
        # Tile selection happens inside the native library from the problem
        # geometry (fdnn_conv2d_query); there is nothing to time at plan level.
        "autotune": {"enabled": autotune, "results": [], "selected": chosen[0]["name"] if chosen else None},
    }
    return ExecutionPlan(
        graph_hash=ghash,
        plan_id=hashlib.sha256((ghash + json.dumps([c["name"] for c in chosen])).encode()).hexdigest()[:16],
        graph=graph_obj, steps=steps, input_specs=specs,
        output_specs=[graph_obj.values[v].spec for v in graph_obj.outputs],
        workspace_size=memory_plan.workspace_size, memory_plan=memory_plan, tuned=False, debug_info=debug)


class PlanCache:
    """In-memory plan cache (the reference's also persists JSON; src/flag_dnn/graph/cache.py:62-130)."""

    def __init__(self, enable_disk: bool = False, max_entries: int = 128):
        self.enable_disk = False  # plans hold live graphs; only the memory layer is implemented
        self.max_entries = max_entries
        self._plans: dict = {}

    def get(self, key: str) -> Optional[ExecutionPlan]:
        return self._plans.get(key)

    def put(self, key: str, plan: ExecutionPlan) -> None:
        if len(self._plans) >= self.max_entries:
            self._plans.pop(next(iter(self._plans)))
        self._plans[key] = plan


_DEFAULT_CACHE = PlanCache()


def get_default_plan_cache() -> PlanCache:
    return _DEFAULT_CACHE


def _cache_key(graph_obj: Graph, specs: list, backend: str) -> str:
    payload = {"graph": graph_obj.graph_hash(), "backend": backend,
               "specs": [dict(s.signature(), name=s.name) for s in specs]}
    return hashlib.sha256(json.dumps(payload, sort_keys=True, default=str).encode()).hexdigest()


class CompiledGraph:
    """A planned graph.  With ``options={"workspace": True}`` the intermediates live in one buffer laid out by
    the memory plan (graph/memory.py) instead of coming from the allocator at every step.
    With ``options={"cuda_graph": True}`` the whole plan is captured into one
    CUDA graph on its first run with CUDA tensors and replayed afterwards: inputs are copied into
    static buffers (skipped for tensors that already are those buffers, see ``static_inputs``) and
    the returned tensors are static too — consume them before the next ``run``.  Multi-step plans
    (a bottleneck block, a whole conv stack) then cost one launch of host time instead of one per
    node; the reference executes such plans node by node from Python
    (src/flag_dnn/graph/executor.py:68-106)."""

    def __init__(self, plan: ExecutionPlan, cuda_graph: bool = False, workspace: bool = False):
        self.plan = plan
        self.graph = plan.graph
        self._use_cuda_graph = bool(cuda_graph)
        self._use_workspace = bool(workspace)
        self._workspaces: dict = {}
        self._captured = None
        self.static_inputs: Optional[list] = None
        self._static_outputs: Any = None

    def _workspace_for(self, inputs: tuple) -> Optional[torch.Tensor]:
        """One buffer of plan.workspace_size bytes per device, allocated at the first run and reused: the
        intermediates of consecutive runs then live at fixed addresses and nothing is allocated per step."""
        if not self._use_workspace or self.plan.workspace_size <= 0:
            return None
        device = next((t.device for t in inputs if isinstance(t, torch.Tensor)), None)
        if device is None or device.type != "cuda":
            return None
        if device not in self._workspaces:
            self._workspaces[device] = torch.empty(self.plan.workspace_size, dtype=torch.uint8, device=device)
        return self._workspaces[device]

    def _execute(self, inputs: tuple) -> Any:
        return execute_plan(self.plan, inputs, self._workspace_for(inputs))

    def run(self, *inputs: Any) -> Any:
        if not self._use_cuda_graph or not any(isinstance(t, torch.Tensor) and t.is_cuda for t in inputs):
            return self._execute(inputs)
        if len(inputs) != len(self.plan.input_specs):
            raise RuntimeError(f"graph expects {len(self.plan.input_specs)} inputs, got {len(inputs)}")
        for index, (spec, tensor) in enumerate(zip(self.plan.input_specs, inputs)):
            _validate_input(spec, tensor, index)
        if self._captured is None:
            self.static_inputs = [torch.empty_strided(t.shape, t.stride(), dtype=t.dtype, device=t.device).copy_(t)
                                  for t in inputs]
            self._execute(tuple(self.static_inputs))  # warm-up: packs filters, sets kernel attributes
            torch.cuda.synchronize()
            captured = torch.cuda.CUDAGraph()
            with torch.cuda.graph(captured):
                self._static_outputs = self._execute(tuple(self.static_inputs))
            self._captured = captured
        for static, given in zip(self.static_inputs, inputs):
            if static.data_ptr() != given.data_ptr():
                static.copy_(given, non_blocking=True)
        self._captured.replay()
        return self._static_outputs

    def __call__(self, *inputs: Any) -> Any:
        return self.run(*inputs)


def _fusion_enabled(options: dict) -> bool:
    if str(os.getenv("FLAGDNN_GRAPH_FUSION", "1")).lower() in ("0", "false", "no"):
        return False
    return bool(options.get("fusion", True))


def _dump_graph(graph_obj: Graph, stage: str) -> None:
    if str(os.getenv("FLAGDNN_DUMP_GRAPH", "0")).lower() in ("0", "false", "no"):
        return
    dump_dir = os.getenv("FLAGDNN_DUMP_GRAPH_DIR", "/tmp/flagdnn_graphs")
    try:
        os.makedirs(dump_dir, exist_ok=True)
        stem = os.path.join(dump_dir, f"{stage}_{graph_obj.graph_hash()[:12]}")
        with open(stem + ".json", "w", encoding="utf-8") as fh:
            json.dump(graph_obj.to_dict(), fh, indent=2, default=str)
        with open(stem + ".txt", "w", encoding="utf-8") as fh:
            fh.write(graph_obj.dump_text())
    except OSError:
        return


def compile(fn: Callable, inputs: Optional[list] = None, input_specs: Optional[list] = None,
            options: Optional[dict] = None) -> CompiledGraph:
    """Capture ``fn`` on symbolic inputs, fuse, and plan it (src/flag_dnn/graph/capture.py:127)."""
    opts: dict = {}
    if isinstance(fn, GraphFunction):
        opts.update(fn.options)
        fn = fn.fn
    if options:
        opts.update(options)
    values = input_specs if input_specs is not None else inputs
    specs = []
    for index, value in enumerate(values or []):
        if isinstance(value, TensorSpec):
            spec = value
        elif isinstance(value, torch.Tensor):
            spec = TensorSpec.from_tensor(value)
        else:
            raise TypeError(f"compile inputs must be TensorSpec or torch.Tensor values, got {type(value)!r}")
        specs.append(spec if spec.name else spec.with_name(f"arg{index}"))
    if not specs:
        raise ValueError("compile requires input TensorSpec values or tensors")

    with GraphCapture(specs) as ctx:
        outputs = fn(*ctx.graph_inputs)
    captured, structure = ctx.finalize(outputs)
    _dump_graph(captured, "capture")
    eliminate_dead_nodes(captured)
    if _fusion_enabled(opts):
        apply_fusion_pass(captured)
        eliminate_dead_nodes(captured)
    captured.lint()
    _dump_graph(captured, "optimized")

    cache = opts.get("cache", get_default_plan_cache())
    key = _cache_key(captured, specs, str(opts.get("backend", "auto")))
    plan = cache.get(key) if cache is not None else None
    if plan is None:
        plan = _build_plan(captured, specs, structure, opts)
        if cache is not None:
            cache.put(key, plan)
    else:
        plan.debug_info["cache_hit"] = True
        plan.debug_info["cache_layer"] = "memory"
        plan.debug_info["output_structure"] = structure
    return CompiledGraph(plan, cuda_graph=bool(opts.get("cuda_graph", False)),
                         workspace=bool(opts.get("workspace", False)))


# ----------------------------------------------------------------- execution
def _validate_input(spec: TensorSpec, tensor: Any, index: int) -> None:
    """Shape, dtype, exact strides and device must match what was compiled
    (src/flag_dnn/graph/executor.py:235-262)."""
    if not isinstance(tensor, torch.Tensor):
        raise TypeError(f"graph input {index} ({spec.name}) must be a tensor")
    if tuple(tensor.shape) != tuple(spec.shape):
        raise RuntimeError(f"graph input {index} ({spec.name}) shape {tuple(tensor.shape)} != compiled {spec.shape}")
    if tensor.dtype != torch_dtype(spec.dtype):
        raise RuntimeError(f"graph input {index} ({spec.name}) dtype {tensor.dtype} != compiled {spec.dtype}")
    if spec.stride is not None and tuple(tensor.stride()) != tuple(spec.stride):
        raise RuntimeError(f"graph input {index} ({spec.name}) stride {tuple(tensor.stride())} != compiled {spec.stride}")
    if spec.device is not None and torch.device(spec.device).type != tensor.device.type:
        raise RuntimeError(f"graph input {index} ({spec.name}) device {tensor.device} != compiled {spec.device}")


def _workspace_view(workspace: torch.Tensor, alloc, spec: TensorSpec, like: Any) -> Optional[torch.Tensor]:
    """The planned slice of the workspace as a tensor of the value's shape and dtype; channels-last strides
    when the node's first operand is channels-last (the rule the kernels use for their own outputs)."""
    dtype = torch_dtype(spec.dtype)
    shape = tuple(int(v) for v in spec.shape)
    numel = 1
    for v in shape:
        numel *= v
    nbytes = numel * torch.empty((), dtype=dtype).element_size()
    if numel == 0 or alloc.offset + nbytes > workspace.numel():
        return None
    flat = workspace[alloc.offset: alloc.offset + nbytes].view(dtype)
    channels_last = (len(shape) == 4 and shape[1] > 1 and isinstance(like, torch.Tensor) and like.dim() == 4
                     and like.stride(1) == 1 and dtype != torch.float64)
    if channels_last:
        n, c, h, w = shape
        return flat.as_strided(shape, (h * w * c, 1, w * c, c))
    return flat.view(shape)


def execute_plan(plan: ExecutionPlan, inputs: tuple, workspace: Optional[torch.Tensor] = None) -> Any:
    """Runs the plan's steps.  With ``workspace`` (a uint8 tensor of at least plan.workspace_size bytes on the
    inputs' device) every intermediate value the memory plan placed is written straight into its slice."""
    graph_obj = plan.graph
    if len(inputs) != len(graph_obj.inputs):
        raise RuntimeError(f"graph expects {len(graph_obj.inputs)} inputs, got {len(inputs)}")
    checks = getattr(plan, "_input_checks", None)
    if checks is None:
        # what _validate_input compares, precomputed once per plan
        checks = [(tuple(spec.shape), torch_dtype(spec.dtype), None if spec.stride is None else tuple(spec.stride),
                   None if spec.device is None else torch.device(spec.device).type) for spec in plan.input_specs]
        plan._input_checks = checks
    for index, (tensor, (shape, dtype, stride, dev_type)) in enumerate(zip(inputs, checks)):
        if not (isinstance(tensor, torch.Tensor) and tensor.shape == shape and tensor.dtype == dtype
                and (stride is None or tensor.stride() == stride)
                and (dev_type is None or tensor.device.type == dev_type)):
            _validate_input(plan.input_specs[index], tensor, index)   # raises with the precise message
    if len(plan.steps) == 1:  # single fused node: skip the environment bookkeeping
        single = getattr(plan, "_single_step", None)
        if single is None:
            step = plan.steps[0]
            if all(v in graph_obj.inputs for v in step.inputs) and graph_obj.outputs == step.outputs:
                single = (get_op_schema(step.op_type).run, [graph_obj.inputs.index(v) for v in step.inputs],
                          step.attrs, plan.debug_info.get("output_structure") or ("leaf",))
            else:
                single = False
            plan._single_step = single
        if single:
            run, arg_index, attrs, structure = single
            out = run([inputs[i] for i in arg_index], attrs)
            return out if structure == ("leaf",) else _rebuild_outputs(structure, [out])
    env: dict = dict(zip(graph_obj.inputs, inputs))
    for value in graph_obj.values.values():
        if value.is_constant:
            env[value.id] = value.const_value
    allocations = plan.memory_plan.allocations if (workspace is not None and plan.memory_plan is not None) else {}
    for step in plan.steps:
        args = [env[v] for v in step.inputs]
        attrs = step.attrs
        alloc = allocations.get(step.outputs[0])
        if alloc is not None:
            view = _workspace_view(workspace, alloc, graph_obj.values[step.outputs[0]].spec, args[0] if args else None)
            if view is not None:
                attrs = dict(attrs)
                attrs["_out"] = view
        env[step.outputs[0]] = get_op_schema(step.op_type).run(args, attrs)
    flat = [env[v] for v in graph_obj.outputs]
    return _rebuild_outputs(plan.debug_info.get("output_structure") or ("leaf",), flat)
