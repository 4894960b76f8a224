"""Graph API for the convolution path: capture, conv -> bias -> ReLU fusion,
planning and execution (counterpart of src/flag_dnn/graph/)."""
from .compiler import (  # noqa: F401
    CompiledGraph,
    ExecutionPlan,
    GraphFunction,
    PlanCache,
    compile,
    current_capture,
    get_default_plan_cache,
    graph,
    is_capturing,
)
from .ir import Graph, GraphValue, OpNode  # noqa: F401
from .passes import apply_fusion_pass, eliminate_dead_nodes  # noqa: F401
from .registry import OpSchema, get_op_schema, register_op  # noqa: F401
from .spec import GraphTensor, TensorSpec  # noqa: F401
