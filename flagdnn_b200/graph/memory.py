"""Lifetimes of a graph's intermediate values and their placement in one workspace.

Same planning rule and the same ``to_dict`` keys as the reference
(src/flag_dnn/graph/memory.py:125-171, 174-199): every value that is neither a
graph input, a graph output nor a constant lives from the node that produces it
to its last user; values are placed in birth order into the first block that is
large enough and already dead, else into a new 256-byte aligned block at the
end.  Unlike the reference, whose run functions never look at the plan
(src/flag_dnn/graph/executor.py:216-228 allocates the workspace and drops it),
the executor here hands each planned value its slice of the workspace as the
``out`` tensor of the node that produces it (``options={"workspace": True}``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Tuple

from .ir import Graph


@dataclass(frozen=True)
class TensorLifetime:
    value_id: int
    birth: int
    last_use: int
    size_bytes: int


@dataclass(frozen=True)
class BufferBlock:
    id: int
    offset: int
    size_bytes: int
    alignment: int = 256


@dataclass(frozen=True)
class TensorAllocation:
    value_id: int
    buffer_id: int
    offset: int
    size_bytes: int


@dataclass
class MemoryPlan:
    workspace_size: int = 0
    lifetimes: Tuple[TensorLifetime, ...] = ()
    blocks: Tuple[BufferBlock, ...] = ()
    allocations: Dict[int, TensorAllocation] = field(default_factory=dict)
    buffers: Dict[str, int] = field(default_factory=dict)   # value id -> bytes, every intermediate

    @property
    def reusable_value_ids(self) -> Tuple[int, ...]:
        return tuple(item.value_id for item in self.lifetimes)

    def to_dict(self) -> dict:
        return {
            "workspace_size": self.workspace_size,
            "lifetimes": [{"value_id": t.value_id, "birth": t.birth, "last_use": t.last_use,
                           "size_bytes": t.size_bytes} for t in self.lifetimes],
            "reusable_value_ids": list(self.reusable_value_ids),
            "blocks": [{"id": b.id, "offset": b.offset, "size_bytes": b.size_bytes, "alignment": b.alignment}
                       for b in self.blocks],
            "allocations": {str(a.value_id): {"buffer_id": a.buffer_id, "offset": a.offset,
                                              "size_bytes": a.size_bytes} for a in self.allocations.values()},
            "buffers": dict(self.buffers),
        }


def _align(value: int, alignment: int) -> int:
    return value if alignment <= 1 else (value + alignment - 1) // alignment * alignment


def compute_lifetimes(graph: Graph) -> List[TensorLifetime]:
    order = {node.id: index for index, node in enumerate(graph.topological_nodes())}
    skip = set(graph.inputs) | set(graph.outputs)
    lifetimes = []
    for value_id, value in graph.values.items():
        if value_id in skip or value.is_constant or value.producer is None or value.producer not in order:
            continue
        birth = order[value.producer]
        last_use = max([birth] + [order[user.id] for user in graph.users(value_id) if user.id in order])
        lifetimes.append(TensorLifetime(value_id, birth, last_use, int(value.spec.nbytes() or 0)))
    return lifetimes


def allocate_memory(graph: Graph, alignment: int = 256) -> MemoryPlan:
    lifetimes = sorted(compute_lifetimes(graph), key=lambda item: (item.birth, item.value_id))
    blocks: List[BufferBlock] = []
    block_busy_until: Dict[int, int] = {}
    allocations: Dict[int, TensorAllocation] = {}
    workspace_size = 0
    for item in lifetimes:
        if item.size_bytes <= 0:
            continue
        chosen = None
        for block in blocks:   # first fit: large enough and its tenant is dead before this value is born
            if block.size_bytes >= item.size_bytes and block_busy_until.get(block.id, -1) < item.birth:
                chosen = block
                break
        if chosen is None:
            offset = _align(workspace_size, alignment)
            chosen = BufferBlock(len(blocks), offset, _align(item.size_bytes, alignment), alignment)
            blocks.append(chosen)
            workspace_size = chosen.offset + chosen.size_bytes
        block_busy_until[chosen.id] = item.last_use
        allocations[item.value_id] = TensorAllocation(item.value_id, chosen.id, chosen.offset, item.size_bytes)
    ordered = tuple(sorted(lifetimes, key=lambda item: item.value_id))
    return MemoryPlan(workspace_size=workspace_size, lifetimes=ordered, blocks=tuple(blocks),
                      allocations=allocations, buffers={str(t.value_id): t.size_bytes for t in ordered})
