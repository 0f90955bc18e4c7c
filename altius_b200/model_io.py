"""Loading `.onnx` files and running the graph passes, through the library's C ABI.

    model = model_io.load("vit.onnx")          # altius_py.load (crates/altius_py/src/lib.rs:32-43)
    model = model_io.optimize(model)           # the passes altius_py.session applies (:54-62)

Both happen in native code (`altius_model_*` of include/altius_session_cuda.h: a protobuf
wire decoder restating crates/core/src/onnx/load.rs, and the four graph rewrites of
crates/core/src/optimize/); this module only converts between the library's model handle
and the `ir.Model` the sessions and the tests work with.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import numpy as np

from . import ir
from .session import (AcGraphDesc, SessionError, attrs_from_arrays, graph_desc, load_library)

PASSES = ("fuse_layer_norm", "fuse_gelu", "fuse_fast_gelu", "eliminate_identity")


def _check(lib, rc: int, what: str):
    if rc != 0:
        msg = lib.altius_cuda_last_error(None)
        raise SessionError(rc, msg.decode() if msg else what)


def _to_ir(lib, handle) -> ir.Model:
    """`ir.Model` copy of a model handle."""
    desc = AcGraphDesc()
    _check(lib, lib.altius_model_graph(handle, ctypes.byref(desc)), "altius_model_graph failed")
    g = ir.Graph()
    for i in range(desc.n_values):
        d = desc.values[i]
        name = lib.altius_model_value_name(handle, i)
        shape = None if d.rank < 0 else tuple(int(d.dims[k]) for k in range(d.rank))
        g.values.append(ir.Value(name.decode() if name else None, shape, int(d.elem_ty)))
    for i in range(desc.n_nodes):
        d = desc.nodes[i]
        op = ir.OP_NAMES[d.op]
        ints = [int(d.ints[k]) for k in range(d.n_ints)]
        floats = [float(d.floats[k]) for k in range(d.n_floats)]
        g.nodes.append(ir.Node(op, [int(d.inputs[k]) for k in range(d.n_inputs)],
                               [int(d.outputs[k]) for k in range(d.n_outputs)],
                               attrs_from_arrays(op, ints, floats), d.name.decode() if d.name else None))
    for i in range(desc.n_inits):
        d = desc.inits[i]
        v = g.values[d.value]
        dt = np.dtype(ir.numpy_type_of(v.elem_ty))
        raw = ctypes.string_at(d.data, d.bytes) if d.bytes else b""
        g.inits[int(d.value)] = np.frombuffer(raw, dtype=dt).reshape(v.shape).copy()
    g.inputs = [int(desc.inputs[i]) for i in range(desc.n_inputs)]
    g.outputs = [int(desc.outputs[i]) for i in range(desc.n_outputs)]
    return ir.Model(g, int(desc.opset_version))


def load(path: str) -> ir.Model:
    """`altius_core::onnx::load_onnx` (crates/core/src/onnx/load.rs:55-58)."""
    lib = load_library()
    h = ctypes.c_void_p()
    _check(lib, lib.altius_model_load_onnx(str(path).encode(), ctypes.byref(h)), "Failed to load a ONNX model")
    try:
        return _to_ir(lib, h)
    finally:
        lib.altius_model_destroy(h)


def load_from_buffer(buf: bytes) -> ir.Model:
    """`load_onnx_from_buffer` (crates/core/src/onnx/load.rs:60-63)."""
    lib = load_library()
    h = ctypes.c_void_p()
    _check(lib, lib.altius_model_load_onnx_buffer(buf, len(buf), ctypes.byref(h)), "Failed to load a ONNX model")
    try:
        return _to_ir(lib, h)
    finally:
        lib.altius_model_destroy(h)


def optimize(model: ir.Model, passes: Optional[tuple] = None, counts: Optional[dict] = None) -> ir.Model:
    """The graph passes of `altius_py.session`, in its order: fuse_layer_norm, fuse_gelu,
    fuse_fast_gelu, eliminate_identity (crates/altius_py/src/lib.rs:54-62). `passes` selects
    a subset by name; `counts` (a dict) receives the number of rewrites per pass."""
    lib = load_library()
    desc, keep, _ = graph_desc(model)
    # Every graph input stays an input: graph_desc lists the run-time inputs only.
    h = ctypes.c_void_p()
    _check(lib, lib.altius_model_from_graph(ctypes.byref(desc), ctypes.byref(h)), "altius_model_from_graph failed")
    try:
        for name in (passes or PASSES):
            n = ctypes.c_int32(0)
            _check(lib, lib.altius_model_run_pass(h, PASSES.index(name), ctypes.byref(n)), name + " failed")
            if counts is not None:
                counts[name] = int(n.value)
        out = _to_ir(lib, h)
    finally:
        lib.altius_model_destroy(h)
    # Value names are not part of a graph description; carry them over by id.
    for i, v in enumerate(model.graph.values):
        if i < len(out.graph.values):
            out.graph.values[i].name = v.name
    return out
