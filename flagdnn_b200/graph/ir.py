"""Graph IR: values, op nodes and the rewrite helpers the passes use
(counterpart of src/flag_dnn/graph/graph.py and node.py)."""
from __future__ import annotations

import hashlib
import json
from dataclasses import dataclass, field
from typing import Any, Optional

import torch

from .spec import GraphTensor, TensorSpec


@dataclass
class GraphValue:
    id: int
    spec: TensorSpec
    producer: Optional[int] = None
    const_value: Any = None
    is_constant: bool = False


@dataclass
class OpNode:
    id: int
    op_type: str
    inputs: list
    outputs: list
    attrs: dict = field(default_factory=dict)
    name: Optional[str] = None

    def to_dict(self) -> dict:
        return {"id": self.id, "op_type": self.op_type, "inputs": list(self.inputs),
                "outputs": list(self.outputs), "attrs": _plain(self.attrs), "name": self.name}


def _plain(value: Any) -> Any:
    if isinstance(value, dict):
        return {str(k): _plain(v) for k, v in value.items()}
    if isinstance(value, (list, tuple)):
        return [_plain(v) for v in value]
    if isinstance(value, (str, int, float, bool)) or value is None:
        return value
    return str(value)


class Graph:
    def __init__(self) -> None:
        self.values: dict[int, GraphValue] = {}
        self.nodes: list[OpNode] = []
        self.inputs: list[int] = []
        self.outputs: list[int] = []
        self.attrs: dict[str, Any] = {}
        self._next_value = 0
        self._next_node = 0

    # ---- construction
    def _new_value(self, spec: TensorSpec, **kw: Any) -> GraphValue:
        value = GraphValue(id=self._next_value, spec=spec, **kw)
        self.values[value.id] = value
        self._next_value += 1
        return value

    def new_node_id(self) -> int:
        nid = self._next_node
        self._next_node += 1
        return nid

    def add_input(self, spec: TensorSpec) -> GraphTensor:
        value = self._new_value(spec.as_input())
        self.inputs.append(value.id)
        return GraphTensor(value.id, self)

    def add_constant(self, const: Any, name_hint: str = "const") -> GraphTensor:
        if isinstance(const, torch.Tensor):
            spec = TensorSpec.from_tensor(const, f"{name_hint}_{self._next_value}")
        else:
            spec = TensorSpec(f"{name_hint}_{self._next_value}", (), "float32")
        value = self._new_value(spec, const_value=const, is_constant=True)
        return GraphTensor(value.id, self)

    def add_op(self, op_type: str, input_ids: list, attrs: dict) -> GraphTensor:
        from .registry import get_op_schema

        schema = get_op_schema(op_type)
        out_spec = schema.infer([self.values[i].spec for i in input_ids], attrs)
        node_id = self.new_node_id()
        out = self._new_value(out_spec.with_name(f"{op_type}_{node_id}"), producer=node_id)
        self.nodes.append(OpNode(id=node_id, op_type=op_type, inputs=list(input_ids), outputs=[out.id],
                                 attrs=dict(attrs), name=attrs.get("name") or op_type))
        return GraphTensor(out.id, self)

    def mark_outputs(self, value_ids: list) -> None:
        self.outputs = list(value_ids)
        for vid in value_ids:
            self.values[vid].spec = self.values[vid].spec.as_output()

    # ---- queries
    def node_by_id(self, node_id: int) -> Optional[OpNode]:
        for node in self.nodes:
            if node.id == node_id:
                return node
        return None

    def producer(self, value_id: int) -> Optional[OpNode]:
        pid = self.values[value_id].producer
        return None if pid is None else self.node_by_id(pid)

    def users(self, value_id: int) -> list:
        return [node for node in self.nodes if value_id in node.inputs]

    def num_users(self, value_id: int) -> int:
        count = sum(node.inputs.count(value_id) for node in self.nodes)
        return count + self.outputs.count(value_id)

    def topological_nodes(self) -> list:
        ready = set(self.inputs) | {v.id for v in self.values.values() if v.is_constant}
        pending, ordered = list(self.nodes), []
        while pending:
            progressed = False
            for node in list(pending):
                if all(i in ready for i in node.inputs):
                    ordered.append(node)
                    ready.update(node.outputs)
                    pending.remove(node)
                    progressed = True
            if not progressed:
                raise RuntimeError("graph has a cycle or a dangling input")
        return ordered

    # ---- rewrites
    def remove_nodes(self, node_ids: list) -> None:
        doomed = set(node_ids)
        self.nodes = [n for n in self.nodes if n.id not in doomed]
        live = set(self.inputs) | set(self.outputs)
        for node in self.nodes:
            live.update(node.inputs)
            live.update(node.outputs)
        for vid in list(self.values):
            if vid not in live:
                del self.values[vid]

    def replace_nodes_with(self, node_ids: list, new_node: OpNode) -> None:
        """Put ``new_node`` where the first of ``node_ids`` stood and drop the rest."""
        doomed = set(node_ids)
        position = min(i for i, n in enumerate(self.nodes) if n.id in doomed)
        self.nodes.insert(position, new_node)
        for vid in new_node.outputs:
            self.values[vid].producer = new_node.id
        self.remove_nodes(list(doomed))

    def lint(self) -> None:
        known = set(self.inputs) | {v.id for v in self.values.values() if v.is_constant}
        for node in self.topological_nodes():
            for vid in node.inputs:
                if vid not in known:
                    raise RuntimeError(f"node {node.id} ({node.op_type}) reads undefined value {vid}")
            known.update(node.outputs)
        for vid in self.outputs:
            if vid not in known:
                raise RuntimeError(f"graph output {vid} is never produced")

    # ---- serialisation
    def to_dict(self) -> dict:
        return {
            "inputs": list(self.inputs), "outputs": list(self.outputs),
            "nodes": [n.to_dict() for n in self.nodes],
            "values": {str(v.id): {"spec": _plain(v.spec.signature()), "name": v.spec.name,
                                   "producer": v.producer, "is_constant": v.is_constant}
                       for v in self.values.values()},
            "attrs": _plain(self.attrs),
        }

    def graph_hash(self) -> str:
        payload = json.dumps(self.to_dict(), sort_keys=True, default=str)
        return hashlib.sha256(payload.encode()).hexdigest()

    def dump_text(self) -> str:
        lines = [f"inputs: {self.inputs}"]
        for node in self.nodes:
            lines.append(f"  %{node.outputs} = {node.op_type}({node.inputs}) {_plain(node.attrs)}")
        lines.append(f"outputs: {self.outputs}")
        return "\n".join(lines)
