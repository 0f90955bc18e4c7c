"""Minimal host-side mirror of the altius graph IR.

Only what the session boundary needs: values with optional names and static
shapes, nodes with an operator name and its attributes, initializers, graph
inputs and outputs. Field and attribute names follow the reference structs so
that a graph built here reads like one built with `altius_core`:

* `Model{graph, opset_version}`      crates/core/src/model.rs:13-17
* `Graph{nodes, values, inits, inputs, outputs}`  crates/core/src/graph.rs:10-16
* `Node{op, name, inputs, outputs}`  crates/core/src/node.rs:8-14
* operator names and attribute fields  crates/core/src/op.rs:8-217
* element types `Bool, F32, I32, I64`  crates/core/src/tensor.rs:47-53

Tensors are contiguous row-major numpy arrays.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np

# Element types, numbered as the C ABI numbers them.
BOOL, F32, I32, I64 = 0, 1, 2, 3
_NP_OF = {BOOL: np.bool_, F32: np.float32, I32: np.int32, I64: np.int64}


def elem_type_of(dtype) -> int:
    dtype = np.dtype(dtype)
    for k, v in _NP_OF.items():
        if np.dtype(v) == dtype:
            return k
    raise TypeError(f"unsupported element type {dtype}")


def numpy_type_of(elem_ty: int):
    return _NP_OF[elem_ty]


# Operator names exactly as `Op::name()` prints them (crates/core/src/op.rs:333-385).
OP_NAMES = (
    "Identity", "Conv2d", "Add", "Sub", "Mul", "Div", "Pow", "Greater", "Sqrt", "ReLU", "Gelu",
    "LeakyReLU", "Sigmoid", "Erf", "Tanh", "Clip", "Where", "Softmax", "Cast", "MaxPool",
    "GlobalAveragePool", "Reshape", "Flatten", "Resize", "Concat", "Transpose", "Squeeze",
    "Unsqueeze", "ReduceMin", "ReduceMax", "ReduceMean", "Round", "Exp", "Expand", "Range", "Loop",
    "Tile", "Split", "Slice", "Gather", "Shape", "NonMaxSuppression", "MatMul", "Gemm",
    "BatchNormalization", "LayerNormalization", "HardSigmoid", "Constant", "FusedElemwise",
)
OP_CODE = {name: i for i, name in enumerate(OP_NAMES)}


@dataclass
class Value:
    name: Optional[str] = None
    shape: Optional[Tuple[int, ...]] = None  # static dims, if known
    elem_ty: int = F32


@dataclass
class Node:
    op: str
    inputs: List[int] = field(default_factory=list)
    outputs: List[int] = field(default_factory=list)
    attrs: Dict[str, Any] = field(default_factory=dict)
    name: Optional[str] = None

    def __post_init__(self):
        if self.op not in OP_CODE:
            raise ValueError(f"unknown operator {self.op!r}")


@dataclass
class Graph:
    nodes: List[Node] = field(default_factory=list)
    values: List[Value] = field(default_factory=list)
    inits: Dict[int, np.ndarray] = field(default_factory=dict)
    inputs: List[int] = field(default_factory=list)
    outputs: List[int] = field(default_factory=list)

    # -- construction helpers ------------------------------------------------
    def new_val(self, name: Optional[str] = None, shape: Optional[Sequence[int]] = None,
                elem_ty: int = F32) -> int:
        self.values.append(Value(name, None if shape is None else tuple(int(d) for d in shape),
                                 elem_ty))
        return len(self.values) - 1

    def new_init(self, array: np.ndarray, name: Optional[str] = None) -> int:
        array = np.ascontiguousarray(array)
        vid = self.new_val(name, array.shape, elem_type_of(array.dtype))
        self.inits[vid] = array
        return vid

    def add_input(self, name: str, shape: Sequence[int], elem_ty: int = F32) -> int:
        vid = self.new_val(name, shape, elem_ty)
        self.inputs.append(vid)
        return vid

    def add_node(self, op: str, inputs: Sequence[int], n_outputs: int = 1, name: Optional[str] = None,
                 **attrs) -> List[int]:
        outs = [self.new_val() for _ in range(n_outputs)]
        self.nodes.append(Node(op, list(inputs), outs, dict(attrs), name))
        return outs

    def op(self, op: str, *inputs: int, **attrs) -> int:
        """Add a single-output node and return its output value id."""
        return self.add_node(op, inputs, 1, **attrs)[0]


@dataclass
class Model:
    graph: Graph = field(default_factory=Graph)
    opset_version: int = 13

    def lookup_named_value(self, name: str) -> Optional[int]:
        for i, v in enumerate(self.graph.values):
            if v.name == name:
                return i
        return None

    def topo_sort_nodes(self) -> List[int]:
        """Node order as `Model::topo_sort_nodes` produces it
        (crates/core/src/model.rs:61-102): a LIFO work list seeded, in arena
        order, with the nodes whose non-constant inputs are all available."""
        g = self.graph
        users: Dict[int, List[int]] = {}
        parents: Dict[int, int] = {}
        for nid, node in enumerate(g.nodes):
            for i in node.inputs:
                if i >= 0 and nid not in users.setdefault(i, []):
                    users[i].append(nid)
            for o in node.outputs:
                parents[o] = nid
        consts = set(g.inputs) | set(g.inits.keys())
        pending: Dict[int, int] = {}
        work: List[int] = []
        for nid, node in enumerate(g.nodes):
            ins = {i for i in node.inputs if i >= 0 and i not in consts and i in parents}
            pending[nid] = len(ins)
            if not ins:
                work.append(nid)
        order: List[int] = []
        while work:
            nid = work.pop()
            order.append(nid)
            for o in g.nodes[nid].outputs:
                for u in users.get(o, ()):
                    pending[u] -= 1
                    if pending[u] == 0:
                        work.append(u)
        return order


def broadcast_shapes(*shapes: Sequence[int]) -> Optional[Tuple[int, ...]]:
    """`fixed_dim::broadcast` (crates/core/src/fixed_dim.rs:108-133): None when
    the shapes do not broadcast."""
    if not shapes:
        return None
    max_len = max(len(s) for s in shapes)
    out = []
    for i in range(max_len):
        size = 1
        for s in shapes:
            dim = s[len(s) - i - 1] if i < len(s) else 1
            if dim == 1:
                continue
            if size != 1 and dim != size:
                return None
            size = dim
        out.append(size)
    return tuple(reversed(out))
