"""Host-side mirror of the altius session API over the CUDA backend's C ABI.

    sess = CudaSessionBuilder(model).with_device(0).with_profiling_enabled(False).build()
    outputs = sess.run([x])                      # list of numpy arrays in, list out

mirrors `InterpreterSessionBuilder::{new, with_profiling_enabled, build}` and
`InterpreterSession::{model, run}` (crates/session_interpreter/src/builder.rs:18-65,
session.rs:61-66), and

    InferenceSession(model, backend="cuda").run(None, {"input": x})

mirrors `altius_py.InferenceSession` (crates/altius_py/altius_py/__init__.py:4-27),
so switching backends is the one-word change of the `backend` argument.

Everything here goes through `libaltius_session_cuda.so` (ctypes); there is no
CPU fallback: if the library is missing or no sm_100 GPU is visible, building a
session raises `SessionError`.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, List, Optional, Sequence

import numpy as np

from . import ir

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libaltius_session_cuda.so")
AC_MAX_RANK = 8


class SessionError(RuntimeError):
    """Counterpart of `altius_session::SessionError` (crates/session/src/lib.rs:14-34)."""

    KINDS = {1: "Invalid", 2: "Shape", 3: "Unsupported", 4: "Cuda", 5: "NoDevice"}

    def __init__(self, status: int, message: str):
        super().__init__(f"{self.KINDS.get(status, status)}: {message}")
        self.status = status


class AcValueDesc(ctypes.Structure):
    _fields_ = [("elem_ty", ctypes.c_int32), ("rank", ctypes.c_int32),
                ("dims", ctypes.c_int64 * AC_MAX_RANK)]


class AcNodeDesc(ctypes.Structure):
    _fields_ = [("op", ctypes.c_int32), ("n_inputs", ctypes.c_int32),
                ("inputs", ctypes.POINTER(ctypes.c_int32)), ("n_outputs", ctypes.c_int32),
                ("outputs", ctypes.POINTER(ctypes.c_int32)), ("n_ints", ctypes.c_int32),
                ("ints", ctypes.POINTER(ctypes.c_int64)), ("n_floats", ctypes.c_int32),
                ("floats", ctypes.POINTER(ctypes.c_float)), ("name", ctypes.c_char_p)]


class AcInitDesc(ctypes.Structure):
    _fields_ = [("value", ctypes.c_int32), ("location", ctypes.c_int32),
                ("data", ctypes.c_void_p), ("bytes", ctypes.c_uint64)]


class AcGraphDesc(ctypes.Structure):
    _fields_ = [("opset_version", ctypes.c_int64), ("n_values", ctypes.c_int32),
                ("values", ctypes.POINTER(AcValueDesc)), ("n_nodes", ctypes.c_int32),
                ("nodes", ctypes.POINTER(AcNodeDesc)), ("n_inits", ctypes.c_int32),
                ("inits", ctypes.POINTER(AcInitDesc)), ("n_inputs", ctypes.c_int32),
                ("inputs", ctypes.POINTER(ctypes.c_int32)), ("n_outputs", ctypes.c_int32),
                ("outputs", ctypes.POINTER(ctypes.c_int32))]


class AcOptions(ctypes.Structure):
    _fields_ = [("device", ctypes.c_int32), ("enable_profiling", ctypes.c_int32),
                ("disable_cuda_graph", ctypes.c_int32), ("disable_fusion", ctypes.c_int32),
                ("gemm_mode", ctypes.c_int32), ("plan_only", ctypes.c_int32),
                ("gemm_pairs", ctypes.c_int32), ("reserved", ctypes.c_int32)]


class AcProfileEntry(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char * 48), ("launches", ctypes.c_uint64),
                ("total_ms", ctypes.c_double), ("bytes", ctypes.c_double),
                ("flops", ctypes.c_double)]


# Every symbol include/altius_session_cuda.h declares.
ABI_SYMBOLS = (
    "altius_cuda_create", "altius_cuda_run", "altius_cuda_run_device", "altius_cuda_run_batches",
    "altius_cuda_time_device_runs", "altius_cuda_num_inputs",
    "altius_cuda_num_outputs", "altius_cuda_input_value", "altius_cuda_output_value",
    "altius_cuda_value_info", "altius_cuda_launches_per_run", "altius_cuda_arena_bytes",
    "altius_cuda_schedule", "altius_cuda_profile", "altius_cuda_profile_reset", "altius_cuda_last_error",
    "altius_cuda_destroy", "altius_cuda_host_alloc", "altius_cuda_host_free",
    "altius_cuda_device_count", "altius_cuda_reduce_max_noalloc",
    "altius_model_load_onnx", "altius_model_load_onnx_buffer", "altius_model_from_graph",
    "altius_model_run_pass", "altius_model_optimize", "altius_model_graph", "altius_model_value_name",
    "altius_model_lookup_named_value", "altius_model_destroy", "altius_cuda_create_from_onnx",
)

_lib = None


def load_library() -> ctypes.CDLL:
    """Loads the session library; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise SessionError(5, f"{LIB_PATH} is missing: run `python -m altius_b200.build` "
                              "(this backend has no CPU fallback)")
    lib = ctypes.CDLL(LIB_PATH)
    P = ctypes.c_void_p
    lib.altius_cuda_create.argtypes = [ctypes.POINTER(AcGraphDesc), ctypes.POINTER(AcOptions),
                                       ctypes.POINTER(P)]
    lib.altius_cuda_run.argtypes = [P, ctypes.POINTER(P), ctypes.POINTER(P)]
    lib.altius_cuda_run_device.argtypes = [P, ctypes.POINTER(P), ctypes.POINTER(P)]
    lib.altius_cuda_run_batches.argtypes = [P, ctypes.c_int32, ctypes.POINTER(P), ctypes.POINTER(P)]
    lib.altius_cuda_time_device_runs.argtypes = [P, ctypes.POINTER(P), ctypes.POINTER(P),
                                                 ctypes.c_int32, ctypes.POINTER(ctypes.c_float)]
    for name in ("altius_cuda_num_inputs", "altius_cuda_num_outputs"):
        getattr(lib, name).argtypes = [P]
    lib.altius_cuda_input_value.argtypes = [P, ctypes.c_int32]
    lib.altius_cuda_output_value.argtypes = [P, ctypes.c_int32]
    lib.altius_cuda_value_info.argtypes = [P, ctypes.c_int32, ctypes.POINTER(AcValueDesc)]
    lib.altius_cuda_launches_per_run.argtypes = [P]
    lib.altius_cuda_launches_per_run.restype = ctypes.c_int64
    lib.altius_cuda_arena_bytes.argtypes = [P]
    lib.altius_cuda_arena_bytes.restype = ctypes.c_uint64
    lib.altius_cuda_profile.argtypes = [P, ctypes.POINTER(AcProfileEntry),
                                        ctypes.POINTER(ctypes.c_size_t)]
    lib.altius_cuda_schedule.argtypes = [P, ctypes.POINTER(AcProfileEntry),
                                         ctypes.POINTER(ctypes.c_size_t)]
    lib.altius_cuda_profile_reset.argtypes = [P]
    lib.altius_cuda_last_error.argtypes = [P]
    lib.altius_cuda_last_error.restype = ctypes.c_char_p
    lib.altius_cuda_destroy.argtypes = [P]
    lib.altius_cuda_destroy.restype = None
    lib.altius_cuda_host_alloc.argtypes = [ctypes.c_size_t, ctypes.POINTER(P)]
    lib.altius_cuda_host_free.argtypes = [P]
    lib.altius_cuda_reduce_max_noalloc.argtypes = [P, ctypes.c_int64, P, P]
    lib.altius_model_load_onnx.argtypes = [ctypes.c_char_p, ctypes.POINTER(P)]
    lib.altius_model_load_onnx_buffer.argtypes = [ctypes.c_char_p, ctypes.c_size_t, ctypes.POINTER(P)]
    lib.altius_model_from_graph.argtypes = [ctypes.POINTER(AcGraphDesc), ctypes.POINTER(P)]
    lib.altius_model_run_pass.argtypes = [P, ctypes.c_int32, ctypes.POINTER(ctypes.c_int32)]
    lib.altius_model_optimize.argtypes = [P]
    lib.altius_model_graph.argtypes = [P, ctypes.POINTER(AcGraphDesc)]
    lib.altius_model_value_name.argtypes = [P, ctypes.c_int32]
    lib.altius_model_value_name.restype = ctypes.c_char_p
    lib.altius_model_lookup_named_value.argtypes = [P, ctypes.c_char_p]
    lib.altius_model_lookup_named_value.restype = ctypes.c_int32
    lib.altius_model_destroy.argtypes = [P]
    lib.altius_model_destroy.restype = None
    lib.altius_cuda_create_from_onnx.argtypes = [ctypes.c_char_p, ctypes.POINTER(AcOptions), ctypes.POINTER(P)]
    _lib = lib
    return lib


def _attr_arrays(node: ir.Node):
    """Flattens a node's attributes into the (ints, floats) layout of the C ABI."""
    a, op = node.attrs, node.op
    ints: List[int] = []
    floats: List[float] = []
    if op == "Conv2d":
        k = list(a["kernel_shape"])
        st = list(a.get("strides", [1, 1]))
        d = list(a.get("dilations", [1, 1]))
        auto = 1 if a.get("auto_pad", "") not in ("", "NOTSET") else 0
        if auto and a["auto_pad"] != "SAME_UPPER":
            raise SessionError(3, f"Conv2d: auto_pad {a['auto_pad']} is not supported")
        act = a.get("activation")
        act_code = 0 if act is None else (1 if act == "Relu" else 2)
        pads = list(a.get("padding", []))
        if not auto and not pads:
            pads = [0, 0, 0, 0]
        ints = k + st + d + [a.get("group", 1), auto, act_code, len(pads)] + pads
        floats = [a.get("activation_alpha", 0.2), a.get("activation_beta", 0.5)]
    elif op == "MaxPool":
        auto = 1 if a.get("auto_pad", "") not in ("", "NOTSET") else 0
        pads = list(a.get("padding", [0, 0, 0, 0]))
        ints = list(a["kernel_shape"]) + list(a.get("strides", [1, 1])) + [auto, len(pads)] + pads
    elif op == "HardSigmoid":
        floats = [a.get("alpha", 0.2), a.get("beta", 0.5)]
    elif op == "LeakyReLU":
        floats = [a.get("alpha", 0.01)]
    elif op == "Resize":
        ints = [0 if a.get("mode", "nearest") == "nearest" else 1,
                0 if a.get("coordinate_transformation_mode", "half_pixel") == "asymmetric" else 1,
                0 if a.get("nearest_mode", "round_prefer_floor") == "floor" else 1]
    elif op in ("Softmax",):
        ints = [a.get("axis", -1)]
    elif op == "Flatten":
        ints = [a.get("axis", 1)]
    elif op == "Cast":
        ints = [a["to"]]
    elif op in ("Concat", "Gather"):
        ints = [a.get("axis", 0)]
    elif op == "Transpose":
        ints = list(a["perm"])
    elif op in ("Squeeze", "Unsqueeze"):
        ints = list(a.get("axes", []))
    elif op in ("ReduceMax", "ReduceMean", "ReduceMin"):
        ints = [1 if a.get("keep_dims", True) else 0] + list(a.get("axes", []))
    elif op == "Split":
        ints = [a.get("axis", 0)] + list(a.get("split", []))
    elif op == "Gemm":
        ints = [1 if a.get("trans_a", False) else 0, 1 if a.get("trans_b", False) else 0]
        floats = [a.get("alpha", 1.0), a.get("beta", 1.0)]
    elif op == "BatchNormalization":
        floats = [a.get("epsilon", 1e-5)]
    elif op == "LayerNormalization":
        ints = [a.get("axis", -1), a.get("stash_type", 1)]
        floats = [a.get("epsilon", 1e-5)]
    elif op == "Shape":
        end = a.get("end")
        ints = [a.get("start", 0), 0 if end is None else 1, 0 if end is None else end]
    return ints, floats


def attrs_from_arrays(op: str, ints: Sequence[int], floats: Sequence[float]) -> dict:
    """Inverse of `_attr_arrays`: the attribute dictionary of an `ir.Node` from the flattened
    arrays of the C ABI (a graph that comes back from the loader or from the passes)."""
    ints, floats = list(ints), list(floats)
    if op == "Conv2d":
        npads = ints[9]
        act = {0: None, 1: "Relu", 2: "HardSigmoid"}[ints[8]]
        return dict(kernel_shape=ints[0:2], strides=ints[2:4], dilations=ints[4:6], group=ints[6],
                    auto_pad="SAME_UPPER" if ints[7] else "NOTSET", activation=act,
                    padding=ints[10:10 + npads], activation_alpha=floats[0], activation_beta=floats[1])
    if op == "MaxPool":
        npads = ints[5]
        return dict(kernel_shape=ints[0:2], strides=ints[2:4], auto_pad="SAME_UPPER" if ints[4] else "NOTSET",
                    padding=ints[6:6 + npads])
    if op == "HardSigmoid":
        return dict(alpha=floats[0], beta=floats[1])
    if op == "LeakyReLU":
        return dict(alpha=floats[0])
    if op == "Resize":
        return dict(mode="nearest" if ints[0] == 0 else "linear",
                    coordinate_transformation_mode="asymmetric" if ints[1] == 0 else "half_pixel",
                    nearest_mode="floor" if ints[2] == 0 else "round_prefer_floor")
    if op in ("Softmax", "Flatten", "Concat", "Gather"):
        return dict(axis=ints[0])
    if op == "Cast":
        return dict(to=ints[0])
    if op == "Transpose":
        return dict(perm=ints)
    if op in ("Squeeze", "Unsqueeze"):
        return dict(axes=ints) if ints else {}
    if op in ("ReduceMax", "ReduceMean", "ReduceMin"):
        return dict(keep_dims=bool(ints[0]), axes=ints[1:])
    if op == "Split":
        return dict(axis=ints[0], split=ints[1:])
    if op == "Gemm":
        return dict(trans_a=bool(ints[0]), trans_b=bool(ints[1]), alpha=floats[0], beta=floats[1])
    if op == "BatchNormalization":
        return dict(epsilon=floats[0])
    if op == "LayerNormalization":
        return dict(axis=ints[0], stash_type=ints[1], epsilon=floats[0])
    if op == "Shape":
        return dict(start=ints[0] if ints else 0, end=ints[2] if len(ints) > 2 and ints[1] else None)
    return {}


def graph_desc(model: ir.Model, device_inits: Optional[Dict[int, int]] = None):
    """`AcGraphDesc` of an `ir.Model` plus the ctypes buffers that must outlive its use."""
    g = model.graph
    keep = []
    values = (AcValueDesc * max(1, len(g.values)))()
    for i, v in enumerate(g.values):
        values[i].elem_ty = v.elem_ty
        if v.shape is None:
            values[i].rank = -1
        else:
            if len(v.shape) > AC_MAX_RANK:
                raise SessionError(2, "rank above 8 is not supported")
            values[i].rank = len(v.shape)
            for k, d in enumerate(v.shape):
                values[i].dims[k] = d
    nodes = (AcNodeDesc * max(1, len(g.nodes)))()
    for i, n in enumerate(g.nodes):
        ints, floats = _attr_arrays(n)
        ins = (ctypes.c_int32 * max(1, len(n.inputs)))(*n.inputs)
        outs = (ctypes.c_int32 * max(1, len(n.outputs)))(*n.outputs)
        ia = (ctypes.c_int64 * max(1, len(ints)))(*[int(x) for x in ints])
        fa = (ctypes.c_float * max(1, len(floats)))(*[float(x) for x in floats])
        keep += [ins, outs, ia, fa]
        nodes[i].op = ir.OP_CODE[n.op]
        nodes[i].n_inputs, nodes[i].inputs = len(n.inputs), ins
        nodes[i].n_outputs, nodes[i].outputs = len(n.outputs), outs
        nodes[i].n_ints, nodes[i].ints = len(ints), ia
        nodes[i].n_floats, nodes[i].floats = len(floats), fa
        nodes[i].name = n.name.encode() if n.name else None
    inits = (AcInitDesc * max(1, len(g.inits)))()
    for i, (vid, arr) in enumerate(g.inits.items()):
        arr = np.ascontiguousarray(arr)
        keep.append(arr)
        inits[i].value = vid
        if device_inits and vid in device_inits:
            inits[i].location, inits[i].data = 1, device_inits[vid]
        else:
            inits[i].location, inits[i].data = 0, arr.ctypes.data
        inits[i].bytes = arr.nbytes
    run_inputs = [i for i in g.inputs if i not in g.inits]
    gin = (ctypes.c_int32 * max(1, len(run_inputs)))(*run_inputs)
    gout = (ctypes.c_int32 * max(1, len(g.outputs)))(*g.outputs)
    desc = AcGraphDesc(model.opset_version, len(g.values), values, len(g.nodes), nodes,
                       len(g.inits), inits, len(run_inputs), gin, len(g.outputs), gout)
    keep += [values, nodes, inits, gin, gout]
    return desc, keep, run_inputs


class CudaSession:
    """One session = one device, one stream, one arena. The run calls of one session are
    serialised by a lock inside the library; distinct sessions run concurrently."""

    def __init__(self, model: ir.Model, device: int, enable_profiling: bool, use_cuda_graph: bool,
                 fuse: bool, gemm_mode: int, device_inits: Optional[Dict[int, int]] = None,
                 plan_only: bool = False, gemm_pairs: bool = False):
        self._model = model
        self._lib = load_library()
        self._handle = ctypes.c_void_p()
        g = model.graph
        desc, keep, run_inputs = graph_desc(model, device_inits)
        opt = AcOptions()
        opt.device = device
        opt.enable_profiling = int(enable_profiling)
        opt.disable_cuda_graph = int(not use_cuda_graph)
        opt.disable_fusion = int(not fuse)
        opt.gemm_mode = gemm_mode
        opt.plan_only = int(plan_only)
        opt.gemm_pairs = int(gemm_pairs)
        rc = self._lib.altius_cuda_create(ctypes.byref(desc), ctypes.byref(opt),
                                          ctypes.byref(self._handle))
        if rc != 0:
            msg = self._lib.altius_cuda_last_error(None)
            raise SessionError(rc, msg.decode() if msg else "create failed")
        self.input_ids = run_inputs
        self.output_ids = list(g.outputs)
        self.input_info = [self.value_info(v) for v in self.input_ids]
        self.output_info = [self.value_info(v) for v in self.output_ids]

    # -- facts ---------------------------------------------------------------
    def model(self) -> ir.Model:
        return self._model

    def value_info(self, value: int):
        d = AcValueDesc()
        rc = self._lib.altius_cuda_value_info(self._handle, value, ctypes.byref(d))
        if rc != 0:
            raise SessionError(rc, "bad value id")
        return tuple(d.dims[i] for i in range(d.rank)), ir.numpy_type_of(d.elem_ty)

    @property
    def launches_per_run(self) -> int:
        return int(self._lib.altius_cuda_launches_per_run(self._handle))

    @property
    def arena_bytes(self) -> int:
        return int(self._lib.altius_cuda_arena_bytes(self._handle))

    def _check(self, rc: int):
        if rc != 0:
            msg = self._lib.altius_cuda_last_error(self._handle)
            raise SessionError(rc, msg.decode() if msg else "run failed")

    def _check_outputs(self, outputs):
        """Caller-supplied output arrays are written by the library through raw pointers:
        they must be what it expects (C-contiguous, writable, right dtype and shape)."""
        if len(outputs) != len(self.output_ids):
            raise SessionError(1, f"expected {len(self.output_ids)} outputs, got {len(outputs)}")
        for o, (shape, dt) in zip(outputs, self.output_info):
            if not isinstance(o, np.ndarray) or o.dtype != np.dtype(dt) or tuple(o.shape) != tuple(shape) \
                    or not o.flags["C_CONTIGUOUS"] or not o.flags["WRITEABLE"]:
                raise SessionError(2, f"output array must be a writable C-contiguous {np.dtype(dt).name} "
                                      f"array of shape {tuple(shape)}")

    # -- run -------------------------------------------------------------------
    def run(self, inputs: Sequence[np.ndarray], outputs: Optional[List[np.ndarray]] = None
            ) -> List[np.ndarray]:
        """Positional inputs in `graph.inputs` order (initializers excluded), as
        `InterpreterSession::run` takes them. `outputs` may supply preallocated
        (e.g. page-locked) arrays to fill."""
        if len(inputs) != len(self.input_ids):
            raise SessionError(1, f"expected {len(self.input_ids)} inputs, got {len(inputs)}")
        arrs = []
        for a, (shape, dt) in zip(inputs, self.input_info):
            a = np.ascontiguousarray(a, dtype=dt)
            if tuple(a.shape) != tuple(shape):
                raise SessionError(2, f"input shape {a.shape} does not match {shape}")
            arrs.append(a)
        if outputs is None:
            outputs = [np.empty(shape, dt) for shape, dt in self.output_info]
        else:
            self._check_outputs(outputs)
        ins = (ctypes.c_void_p * max(1, len(arrs)))(*[a.ctypes.data for a in arrs])
        outs = (ctypes.c_void_p * max(1, len(outputs)))(*[o.ctypes.data for o in outputs])
        self._check(self._lib.altius_cuda_run(self._handle, ins, outs))
        return outputs

    def run_batches(self, batches: Sequence[Sequence[np.ndarray]],
                    outputs: Optional[List[List[np.ndarray]]] = None) -> List[List[np.ndarray]]:
        """`run` for a queue of batches, pipelined: the inputs of batch b+1 are copied to the
        device while batch b computes. Pass page-locked arrays (`alloc_pinned`) for the copies
        to overlap. Returns one output list per batch."""
        checked = []
        for inputs in batches:
            if len(inputs) != len(self.input_ids):
                raise SessionError(1, f"expected {len(self.input_ids)} inputs, got {len(inputs)}")
            row = []
            for a, (shape, dt) in zip(inputs, self.input_info):
                a = np.ascontiguousarray(a, dtype=dt)
                if tuple(a.shape) != tuple(shape):
                    raise SessionError(2, f"input shape {a.shape} does not match {shape}")
                row.append(a)
            checked.append(row)
        if outputs is None:
            outputs = [[np.empty(shape, dt) for shape, dt in self.output_info] for _ in checked]
        else:
            if len(outputs) != len(checked):
                raise SessionError(1, f"expected {len(checked)} output lists, got {len(outputs)}")
            for row in outputs:
                self._check_outputs(row)
        n = len(checked)
        flat_in = [a.ctypes.data for row in checked for a in row]
        flat_out = [o.ctypes.data for row in outputs for o in row]
        ins = (ctypes.c_void_p * max(1, len(flat_in)))(*flat_in)
        outs = (ctypes.c_void_p * max(1, len(flat_out)))(*flat_out)
        self._check(self._lib.altius_cuda_run_batches(self._handle, n, ins, outs))
        return outputs

    def run_device(self, in_ptrs: Sequence[int], out_ptrs: Sequence[int]) -> None:
        """Inputs and outputs are device addresses on the session's device."""
        ins = (ctypes.c_void_p * max(1, len(in_ptrs)))(*in_ptrs)
        outs = (ctypes.c_void_p * max(1, len(out_ptrs)))(*out_ptrs)
        self._check(self._lib.altius_cuda_run_device(self._handle, ins, outs))

    def time_device_runs(self, in_ptrs: Sequence[int], out_ptrs: Sequence[int], iters: int) -> float:
        """`iters` back-to-back runs on device buffers; returns the elapsed
        milliseconds between CUDA events on the session's stream."""
        ins = (ctypes.c_void_p * max(1, len(in_ptrs)))(*in_ptrs)
        outs = (ctypes.c_void_p * max(1, len(out_ptrs)))(*out_ptrs)
        ms = ctypes.c_float()
        self._check(self._lib.altius_cuda_time_device_runs(self._handle, ins, outs, iters,
                                                           ctypes.byref(ms)))
        return float(ms.value)

    # -- profiling ---------------------------------------------------------------
    def profile(self) -> Dict[str, dict]:
        n = ctypes.c_size_t(256)
        entries = (AcProfileEntry * 256)()
        self._check(self._lib.altius_cuda_profile(self._handle, entries, ctypes.byref(n)))
        return {entries[i].name.decode(): dict(launches=int(entries[i].launches),
                                               total_ms=entries[i].total_ms,
                                               bytes=entries[i].bytes, flops=entries[i].flops)
                for i in range(min(n.value, 256))}

    def schedule(self) -> List[dict]:
        """The static kernel schedule: one dict per step, in launch order."""
        n = ctypes.c_size_t(0)
        self._check(self._lib.altius_cuda_schedule(self._handle, None, ctypes.byref(n)))
        entries = (AcProfileEntry * max(1, n.value))()
        n = ctypes.c_size_t(len(entries))
        self._check(self._lib.altius_cuda_schedule(self._handle, entries, ctypes.byref(n)))
        return [dict(kind=entries[i].name.decode(), launches=int(entries[i].launches),
                     bytes=entries[i].bytes, flops=entries[i].flops) for i in range(n.value)]

    def profile_reset(self) -> None:
        self._check(self._lib.altius_cuda_profile_reset(self._handle))

    def close(self) -> None:
        if self._handle:
            self._lib.altius_cuda_destroy(self._handle)
            self._handle = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class CudaSessionBuilder:
    """Builder with the reference's shape (builder.rs:18-65); options that only
    make sense on a CPU (`with_intra_op_num_threads`) are accepted and ignored."""

    def __init__(self, model: ir.Model):
        self.model = model
        self.device = 0
        self.enable_profiling = False
        self.use_cuda_graph = True
        self.fuse = True
        self.gemm_mode = 0
        self.device_inits: Optional[Dict[int, int]] = None
        self.plan_only = False
        self.gemm_pairs = False

    def with_plan_only(self, b: bool):
        """Shapes, schedule and arena plan only; no GPU is touched and `run` fails."""
        self.plan_only = b
        return self

    def with_device(self, device: int):
        self.device = device
        return self

    def with_intra_op_num_threads(self, _n: int):
        return self

    def with_profiling_enabled(self, b: bool, cold_l2: bool = False):
        """`cold_l2`: additionally sweep L2 before every kernel, so that each one is timed
        from a cold cache without dirty lines (kernel-level HBM measurements)."""
        self.enable_profiling = 2 if (b and cold_l2) else b
        return self

    def with_cuda_graph(self, b: bool):
        self.use_cuda_graph = b
        return self

    def with_fusion(self, b: bool):
        self.fuse = b
        return self

    def with_gemm_mode(self, mode: int):
        self.gemm_mode = mode
        return self

    def with_gemm_pairs(self, b: int):
        """fp16-split GEMMs on clusters of two CTAs (AcOptions.gemm_pairs: 0 / 2 the default
        pre-split pairs, 1 register-staged pairs, 3 the one-CTA kernel only)."""
        self.gemm_pairs = b
        return self

    def with_device_initializers(self, ptrs: Dict[int, int]):
        """value id -> device address of an initializer already resident on the
        session's device (the landing buffer of a weight broadcast)."""
        self.device_inits = ptrs
        return self

    def build(self) -> CudaSession:
        return CudaSession(self.model, self.device, self.enable_profiling, self.use_cuda_graph,
                           self.fuse, self.gemm_mode, self.device_inits, self.plan_only, self.gemm_pairs)


class InferenceSession:
    """`altius_py.InferenceSession` look-alike (crates/altius_py/altius_py/__init__.py:4-27):
    `InferenceSession("model.onnx", backend="cuda")` loads the file, applies the graph passes
    altius_py applies (crates/altius_py/src/lib.rs:54-62) and builds the session. `model` may
    also be an `ir.Model`; it goes through the same passes."""

    def __init__(self, model, enable_profile: bool = False, intra_op_num_threads: int = 1,
                 backend: str = "cuda", device: int = 0):
        if backend != "cuda":
            # altius_py raises PyRuntimeError for an unknown backend string
            # (crates/altius_py/src/lib.rs:64-88).
            raise RuntimeError(f"Unknown backend: {backend}")
        from . import model_io
        if isinstance(model, (str, os.PathLike)):
            model = model_io.load(os.fspath(model))
        elif not isinstance(model, ir.Model):
            raise TypeError("model must be a path to an .onnx file or an altius_b200.ir.Model")
        model = model_io.optimize(model)
        self.model = model
        self.session = (CudaSessionBuilder(model).with_device(device)
                        .with_intra_op_num_threads(intra_op_num_threads)
                        .with_profiling_enabled(enable_profile).build())

    def run(self, output, input: Dict[str, np.ndarray]) -> List[np.ndarray]:
        assert output is None
        g = self.model.graph
        ordered = []
        for vid in self.session.input_ids:
            name = g.values[vid].name
            if name not in input:
                raise RuntimeError(f"Input not found: {name}")
            ordered.append(input[name])
        return self.session.run(ordered)


def reduce_max_noalloc(x_ptr: int, n: int, out_ptr: int, stream: int = 0) -> None:
    """Whole-tensor maximum of `n` device floats at `x_ptr` into the device float at
    `out_ptr`, for callers that may not allocate device memory (see the header):
    fixed scratch inside the library, at most 67,108,864 elements, calls on one GPU
    must not overlap. Raises SessionError on refusal."""
    lib = load_library()
    rc = lib.altius_cuda_reduce_max_noalloc(x_ptr, n, out_ptr, stream or None)
    if rc != 0:
        msg = lib.altius_cuda_last_error(None)
        raise SessionError(rc, msg.decode() if msg else "reduce_max_noalloc failed")


def alloc_pinned(shape, dtype=np.float32) -> np.ndarray:
    """A numpy array backed by page-locked host memory from the session library."""
    lib = load_library()
    nbytes = int(np.prod(shape, dtype=np.int64)) * np.dtype(dtype).itemsize
    p = ctypes.c_void_p()
    rc = lib.altius_cuda_host_alloc(nbytes, ctypes.byref(p))
    if rc != 0:
        raise SessionError(rc, "host_alloc failed")
    buf = (ctypes.c_char * max(nbytes, 1)).from_address(p.value)
    arr = np.frombuffer(buf, dtype=dtype, count=int(np.prod(shape, dtype=np.int64))).reshape(shape)
    return arr
