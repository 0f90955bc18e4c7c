"""CPU oracle session: a restatement of the altius reference interpreter.

THIS IS TEST INFRASTRUCTURE. Only the tests, the smoke check and the
benchmark's CPU-baseline leg may import it; the CUDA session never does.

It walks a graph exactly as `InterpreterSession::run` does
(crates/session_interpreter/src/session.rs:66-134): initializers and inputs go
into a value map, nodes run in `create_execution_plan` order
(crates/session/src/plan.rs:14-58) and dead values are dropped after their
last user. Kernels are the C++ restatements in `oracle.cpp` (called through
ctypes); pure data movement (Concat, Slice, Split, Gather) is numpy.

Shape rules restate `Model::compute_output_shapes`
(crates/core/src/analysis/shape.rs:23-654) for the operators supported here.

Parity is UNPINNED for MatMul/Gemm/Conv2d beyond the reference tests'
tolerances (BLIS summation order is unspecified) and for Erf (un-vendored
fastapprox); see the header of `oracle.cpp`. Operators marked EXTENSION below
accept shapes the reference interpreter asserts against; their results follow
the ONNX operator definitions.
"""
from __future__ import annotations

import ctypes
import math
import os
import time
from typing import Dict, List, Optional, Sequence

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

c_f32p = ctypes.POINTER(ctypes.c_float)
c_i64p = ctypes.POINTER(ctypes.c_int64)
c_u8p = ctypes.POINTER(ctypes.c_uint8)


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path):
            from . import build as _build
            _build.build_oracle()
        _LIB = ctypes.CDLL(path)
        I, L64, F, P = ctypes.c_int, ctypes.c_int64, ctypes.c_float, ctypes.c_void_p
        sigs = {
            "or_binary": [I, P, P, I, P, P, I, P, P, I, I],
            "or_pow": [P, P, P, L64, I],
            "or_sqrt": [P, P, L64], "or_relu": [P, P, L64], "or_erf": [P, P, L64],
            "or_tanh": [P, P, L64],
            "or_hard_sigmoid": [P, P, L64, F, F], "or_leaky_relu": [P, P, L64, F],
            "or_gelu": [P, P, L64, I], "or_sigmoid": [P, P, L64, I],
            "or_greater_scalar": [P, F, P, L64],
            "or_where": [I, P, P, P, P, L64, L64],
            "or_softmax": [P, P, L64, L64, I],
            "or_layer_norm": [P, P, P, P, L64, L64, F, I],
            "or_reduce_mean_last": [P, P, L64, L64], "or_reduce_max_last": [P, P, L64, L64],
            "or_reduce_max_all": [P, P, L64],
            "or_gavg_pool": [P, P, L64, L64],
            "or_max_pool": [P, P] + [L64] * 11,
            "or_resize": [P, P] + [L64] * 5 + [ctypes.c_int],
            "or_batch_norm": [P, P, P, P, P, P, L64, L64, L64, F],
            "or_sgemm": [I, I, L64, L64, L64, F, P, L64, P, L64, F, P, L64, I],
            "or_sgemm_batched": [L64, L64, L64, L64, P, P, P, I],
            "or_conv2d": [P, P, P, P] + [L64] * 16 + [I],
            "or_transpose": [P, P, P, P, I],
        }
        for name, argtypes in sigs.items():
            fn = getattr(_LIB, name)
            fn.argtypes = argtypes
            fn.restype = I if name in ("or_binary", "or_pow") else None
        _LIB.or_max_threads.restype = ctypes.c_int
    return _LIB


def _fp(a: np.ndarray):
    return a.ctypes.data_as(c_f32p)


def _dims(shape: Sequence[int]):
    return (ctypes.c_int64 * max(1, len(shape)))(*[int(d) for d in shape])


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def is_scalar(shape) -> bool:
    """crates/core/src/fixed_dim.rs:26-28"""
    return len(shape) == 0 or (len(shape) == 1 and shape[0] in (0, 1))


def broadcast(x, y):
    """crates/core/src/fixed_dim.rs:108-133"""
    shapes = [tuple(x), tuple(y)]
    max_len = max(len(s) for s in shapes)
    out = []
    for i in range(max_len):
        size = 1
        for s in shapes:
            dim = s[len(s) - i - 1] if i < len(s) else 1
            if dim == 1:
                continue
            if size != 1 and dim != size:
                raise ValueError(f"shapes {x} and {y} do not broadcast")
            size = dim
        out.append(size)
    return tuple(reversed(out))


def _same_upper(in_hw, kernel, stride):
    """crates/core/src/analysis/shape.rs:50-61 (SAME_UPPER padding)."""
    out0 = math.ceil(in_hw[0] / stride[0])
    out1 = math.ceil(in_hw[1] / stride[1])
    pad0 = max((out0 - 1) * stride[0] + kernel[0] - in_hw[0], 0)
    pad1 = max((out1 - 1) * stride[1] + kernel[1] - in_hw[1], 0)
    return [pad0 // 2, pad1 // 2, pad0 - pad0 // 2, pad1 - pad1 // 2]


def resolve_padding(attrs, in_hw, dil=(1, 1)):
    kernel, stride = attrs["kernel_shape"], attrs.get("strides", [1, 1])
    auto_pad = attrs.get("auto_pad", "")
    padding = list(attrs.get("padding", [0, 0, 0, 0]))
    if auto_pad and auto_pad != "NOTSET":
        assert auto_pad == "SAME_UPPER"
        return _same_upper(in_hw, kernel, stride)
    if len(padding) == 2:
        return [padding[0], padding[1], padding[0], padding[1]]
    if len(padding) == 4:
        return padding
    raise ValueError(f"Conv2d: Unknown padding pattern: {padding}")


class InterpreterSession:
    def __init__(self, model, intra_op_num_threads: int, enable_profiling: bool, sgemm: str):
        self._model = model
        self.threads = intra_op_num_threads
        self.enable_profiling = enable_profiling
        self.sgemm = sgemm
        self.profile: Dict[str, float] = {}
        order = model.topo_sort_nodes()
        # crates/session/src/plan.rs:14-58: free each produced value after its last user.
        pos = {nid: i for i, nid in enumerate(order)}
        users: Dict[int, List[int]] = {}
        for nid in order:
            for i in model.graph.nodes[nid].inputs:
                if i >= 0:
                    users.setdefault(i, []).append(nid)
        free_after: Dict[int, List[int]] = {}
        for nid in order:
            for o in model.graph.nodes[nid].outputs:
                if o in users:
                    last = max(users[o], key=lambda n: pos[n])
                    free_after.setdefault(last, []).append(o)
        self.plan = [(nid, free_after.get(nid, [])) for nid in order]

    def model(self):
        return self._model

    # -- the forward pass ---------------------------------------------------
    def run(self, inputs: Sequence[np.ndarray]) -> List[np.ndarray]:
        g = self._model.graph
        values: Dict[int, np.ndarray] = dict(g.inits)
        non_init_inputs = [i for i in g.inputs if i not in g.inits]
        for vid, t in zip(non_init_inputs, inputs):
            values[vid] = np.ascontiguousarray(t)
        self.profile = {}
        for nid, free_vals in self.plan:
            node = g.nodes[nid]
            ins = [values[i] if i >= 0 else None for i in node.inputs]
            t0 = time.perf_counter()
            outs = self._run_node(node, ins)
            if self.enable_profiling:
                self.profile[node.op] = self.profile.get(node.op, 0.0) + time.perf_counter() - t0
            for o, t in zip(node.outputs, outs):
                values[o] = t
            for v in free_vals:
                if v not in g.outputs:
                    values.pop(v, None)
        return [values[o] for o in g.outputs]

    # -- kernels ---------------------------------------------------------------
    def _sgemm(self, ta, tb, m, k, n, alpha, a, lda, b, ldb, beta, c, ldc):
        if self.sgemm == "openblas":
            # Stand-in for the reference's BLIS cblas_sgemm: numpy's bundled
            # OpenBLAS. C = alpha*op(A)*op(B) + beta*C.
            A = a.reshape(-1)[: (k if ta else m) * lda].reshape(-1, lda)[:, : (m if ta else k)]
            B = b.reshape(-1)[: (n if tb else k) * ldb].reshape(-1, ldb)[:, : (k if tb else n)]
            A = A.T if ta else A
            B = B.T if tb else B
            prod = A @ B
            C = c.reshape(-1, ldc)[:m, :n]
            if alpha != 1.0:
                prod = np.float32(alpha) * prod
            if beta == 0.0:
                C[...] = prod
            else:
                C[...] = np.float32(beta) * C + prod
            return
        lib().or_sgemm(int(ta), int(tb), m, k, n, ctypes.c_float(alpha), _fp(a), lda, _fp(b), ldb,
                       ctypes.c_float(beta), _fp(c), ldc, self.threads)

    def _run_node(self, node, ins):
        op, at = node.op, node.attrs
        L = lib()
        thr = self.threads
        if op in ("Identity", "Flatten", "Squeeze", "Unsqueeze", "Reshape"):
            # session.rs:530-535, 1280-1290, 1610-1620: share the data, new dims.
            x = ins[0]
            if op == "Reshape":
                # shape.rs:173-196
                spec = [int(v) for v in ins[1]]
                other = 1
                for v in spec:
                    if v != -1:
                        other *= v
                shape = [x.size // other if v == -1 else v for v in spec]
            elif op == "Flatten":
                axis = at.get("axis", 1)
                assert axis >= 0
                shape = [int(np.prod(x.shape[:axis], dtype=np.int64)),
                         int(np.prod(x.shape[axis:], dtype=np.int64))]
            elif op == "Squeeze":
                axes = at["axes"] if self._model.opset_version < 12 and "axes" in at else \
                    [int(v) for v in ins[1]]
                shape = [d for i, d in enumerate(x.shape) if i not in axes]
            elif op == "Unsqueeze":
                axes = [int(v) for v in ins[1]] if self._model.opset_version >= 13 and len(ins) > 1 \
                    else at["axes"]
                shape = list(x.shape)
                for a in axes:
                    shape.insert(a, 1)
            else:
                shape = list(x.shape)
            return [x.reshape(shape)]
        if op in ("Add", "Sub", "Mul", "Div"):
            a, b = _f32(ins[0]), _f32(ins[1])
            oshape = broadcast(a.shape, b.shape)
            out = np.empty(oshape, np.float32)
            rc = L.or_binary(("Add", "Sub", "Mul", "Div").index(op), _fp(a), _dims(a.shape), a.ndim,
                             _fp(b), _dims(b.shape), b.ndim, _fp(out), _dims(oshape), len(oshape),
                             thr)
            if rc != 0:
                raise ValueError(f"{op}: cannot broadcast {a.shape} with {b.shape}")
            return [out]
        if op == "Pow":
            a, b = _f32(ins[0]), _f32(ins[1])
            out = np.empty(broadcast(a.shape, b.shape), np.float32)
            if a.shape == b.shape:
                L.or_pow(_fp(a), _fp(b), _fp(out), a.size, 0)
            elif is_scalar(b.shape):
                L.or_pow(_fp(a), _fp(b), _fp(out), a.size, 1)
            else:
                raise NotImplementedError(f"Pow: A shape {a.shape}, B shape {b.shape}")  # session.rs:601
            return [out]
        if op in ("Sqrt", "ReLU", "Erf", "Tanh"):
            x = _f32(ins[0])
            out = np.empty_like(x)
            {"Sqrt": L.or_sqrt, "ReLU": L.or_relu, "Erf": L.or_erf, "Tanh": L.or_tanh}[op](
                _fp(x), _fp(out), x.size)
            return [out]
        if op in ("Gelu", "Sigmoid"):
            x = _f32(ins[0])
            out = np.empty_like(x)
            (L.or_gelu if op == "Gelu" else L.or_sigmoid)(_fp(x), _fp(out), x.size, thr)
            return [out]
        if op == "HardSigmoid":
            x = _f32(ins[0])
            out = np.empty_like(x)
            L.or_hard_sigmoid(_fp(x), _fp(out), x.size, ctypes.c_float(at.get("alpha", 0.2)),
                              ctypes.c_float(at.get("beta", 0.5)))
            return [out]
        if op == "LeakyReLU":
            x = _f32(ins[0])
            out = np.empty_like(x)
            L.or_leaky_relu(_fp(x), _fp(out), x.size, ctypes.c_float(at.get("alpha", 0.01)))
            return [out]
        if op == "Greater":
            x, y = _f32(ins[0]), _f32(ins[1])
            if not is_scalar(y.shape):
                # session.rs:559 stops here. EXTENSION: ONNX Greater with NumPy broadcasting
                # (a comparison: exact).
                return [np.ascontiguousarray(np.greater(x, y))]
            out = np.empty(x.shape, np.uint8)
            L.or_greater_scalar(_fp(x), ctypes.c_float(float(y.reshape(-1)[0])),
                                out.ctypes.data_as(c_u8p), x.size)
            return [out.view(np.bool_)]
        if op == "Where":
            cond = np.ascontiguousarray(ins[0]).view(np.uint8)
            x, y = _f32(ins[1]), _f32(ins[2])
            oshape = broadcast(x.shape, y.shape)
            out = np.empty(oshape, np.float32)
            if tuple(cond.shape) == tuple(y.shape) and is_scalar(x.shape):
                L.or_where(0, cond.ctypes.data_as(c_u8p), _fp(x), _fp(y), _fp(out), out.size, 0)
            elif is_scalar(y.shape) and x.ndim == 4 and cond.ndim == 4 and \
                    cond.shape[0] == 1 and cond.shape[1] == 1 and cond.shape[2:] == tuple(oshape[2:]):  # session.rs:958-964
                L.or_where(1, cond.ctypes.data_as(c_u8p), _fp(x), _fp(y), _fp(out), out.size,
                           oshape[2] * oshape[3])
            else:
                # EXTENSION beyond the reference's two patterns: ONNX Where with NumPy
                # broadcasting of all three operands (a selection: exact).
                return [np.ascontiguousarray(np.where(cond.view(np.bool_), x, y).astype(np.float32))]
            return [out]
        if op == "Cast":
            # session.rs:1350-1378: i32->f32, i64->i32, i64->f32, f32->bool
            x, to = ins[0], at["to"]
            table = {(np.dtype(np.int32), 1): np.float32, (np.dtype(np.int64), 2): np.int32,
                     (np.dtype(np.int64), 1): np.float32}
            if (x.dtype, to) in table:
                return [x.astype(table[(x.dtype, to)])]
            if x.dtype == np.float32 and to == 0:
                return [x != 0.0]
            # EXTENSION: the other pairs of bool / f32 / i32 / i64, converted as C does
            # (towards zero for float -> integer; anything non-zero -> true).
            target = {0: np.bool_, 1: np.float32, 2: np.int32, 3: np.int64}[to]
            if to == 0:
                return [x != 0]
            if x.dtype == np.float32 and target in (np.int32, np.int64):
                return [np.trunc(x).astype(target)]
            return [x.astype(target)]
        if op == "Softmax":
            x = _f32(ins[0])
            axis = at.get("axis", -1)
            assert axis == -1 or axis == x.ndim - 1  # session.rs:999
            out = np.empty_like(x)
            L.or_softmax(_fp(x), _fp(out), x.size // x.shape[-1], x.shape[-1], thr)
            return [out]
        if op == "LayerNormalization":
            x = _f32(ins[0])
            scale, bias = _f32(ins[1]).reshape(-1), _f32(ins[2]).reshape(-1)
            assert at.get("axis", -1) in (-1, x.ndim - 1) and at.get("stash_type", 1) == 1
            out = np.empty_like(x)
            L.or_layer_norm(_fp(x), _fp(scale), _fp(bias), _fp(out), x.size // x.shape[-1],
                            x.shape[-1], ctypes.c_float(at.get("epsilon", 1e-5)), thr)
            return [out]
        if op == "ReduceMean":
            x = _f32(ins[0])
            axes = [a + x.ndim if a < 0 else a for a in at["axes"]]
            keep = bool(at.get("keep_dims", True))
            # session.rs:1321-1326 accepts rank 3, axis 2, keepdims only; other
            # ranks with the last axis are an EXTENSION using the same row kernel.
            assert axes == [x.ndim - 1], "ReduceMean: last axis only"
            out = np.empty(x.shape[:-1] + ((1,) if keep else ()), np.float32)
            L.or_reduce_mean_last(_fp(x), _fp(out), x.size // x.shape[-1], x.shape[-1])
            return [out]
        if op == "ReduceMax":
            x = _f32(ins[0])
            axes = [a + x.ndim if a < 0 else a for a in at.get("axes", [])]
            keep = bool(at.get("keep_dims", True))
            if not axes:
                assert not keep  # session.rs:1295-1296
                out = np.empty((1,), np.float32)
                L.or_reduce_max_all(_fp(x), _fp(out), x.size)
                return [out]
            assert axes == [x.ndim - 1], "ReduceMax: all axes, or the last axis (EXTENSION)"
            out = np.empty(x.shape[:-1] + ((1,) if keep else ()), np.float32)
            L.or_reduce_max_last(_fp(x), _fp(out), x.size // x.shape[-1], x.shape[-1])
            return [out]
        if op == "GlobalAveragePool":
            x = _f32(ins[0])
            assert x.ndim == 4
            out = np.empty((x.shape[0], x.shape[1], 1, 1), np.float32)
            L.or_gavg_pool(_fp(x), _fp(out), x.shape[0] * x.shape[1], x.shape[2] * x.shape[3])
            return [out]
        if op == "MaxPool":
            x = _f32(ins[0])
            k, s = at["kernel_shape"], at.get("strides", [1, 1])
            pad = resolve_padding(at, x.shape[2:])
            oh = (x.shape[2] + pad[0] + pad[2] - (k[0] - 1) - 1) // s[0] + 1  # shape.rs:128-133
            ow = (x.shape[3] + pad[1] + pad[3] - (k[1] - 1) - 1) // s[1] + 1
            out = np.empty((x.shape[0], x.shape[1], oh, ow), np.float32)
            L.or_max_pool(_fp(x), _fp(out), x.shape[0] * x.shape[1], x.shape[2], x.shape[3], oh, ow,
                          k[0], k[1], s[0], s[1], pad[0], pad[1])
            return [out]
        if op == "Resize":
            # shape.rs:209-254 (sizes, or floor(dims * scales) for asymmetric / nearest / floor),
            # session.rs:1057-1132
            x = _f32(ins[0])
            if len(ins) == 4:
                oshape = tuple(int(v) for v in np.asarray(ins[3]).reshape(-1))
            elif len(ins) == 3:
                assert at.get("coordinate_transformation_mode", "half_pixel") == "asymmetric"
                assert at.get("mode", "nearest") == "nearest" and at.get("nearest_mode") == "floor"
                sc = np.asarray(ins[2], np.float32).reshape(-1)
                oshape = tuple(int(np.floor(np.float32(d) * s)) for d, s in zip(x.shape, sc))
            else:
                raise NotImplementedError("Resize: Unsupported pattern")
            assert len(oshape) == 4 and oshape[:2] == x.shape[:2]
            out = np.empty(oshape, np.float32)
            L.or_resize(_fp(x), _fp(out), x.shape[0] * x.shape[1], x.shape[2], x.shape[3], oshape[2], oshape[3],
                        0 if at.get("mode", "nearest") == "nearest" else 1)
            return [out]
        if op == "Expand":
            # shape.rs:148-160 takes the shape input as the output shape; session.rs:299-323
            # tiles an i64 row. Restated as a broadcast of any tensor to that shape.
            shape = tuple(int(v) for v in np.asarray(ins[1]).reshape(-1))
            return [np.ascontiguousarray(np.broadcast_to(ins[0], shape))]
        if op == "BatchNormalization":
            x = _f32(ins[0])
            out = np.empty_like(x)
            L.or_batch_norm(_fp(x), _fp(_f32(ins[1])), _fp(_f32(ins[2])), _fp(_f32(ins[3])),
                            _fp(_f32(ins[4])), _fp(out), x.shape[0], x.shape[1],
                            x.shape[2] * x.shape[3], ctypes.c_float(at.get("epsilon", 1e-5)))
            return [out]
        if op == "Conv2d":
            x, w = _f32(ins[0]), _f32(ins[1])
            bias = _f32(ins[2]) if len(ins) > 2 and ins[2] is not None else None
            k, s = at["kernel_shape"], at.get("strides", [1, 1])
            d = at.get("dilations", [1, 1])
            group = at.get("group", 1)
            pad = resolve_padding(at, x.shape[2:])
            oh = (x.shape[2] + pad[0] + pad[2] - d[0] * (k[0] - 1) - 1) // s[0] + 1  # shape.rs:79-84
            ow = (x.shape[3] + pad[1] + pad[3] - d[1] * (k[1] - 1) - 1) // s[1] + 1
            out = np.empty((x.shape[0], w.shape[0], oh, ow), np.float32)
            if self.sgemm == "openblas":
                self._conv_openblas(x, w, bias, out, k, s, d, pad, group)
            else:
                L.or_conv2d(_fp(x), _fp(w), _fp(bias) if bias is not None else None, _fp(out),
                            x.shape[0], x.shape[1], x.shape[2], x.shape[3], w.shape[0], oh, ow,
                            k[0], k[1], s[0], s[1], d[0], d[1], pad[0], pad[1], group, thr)
            return [out]
        if op == "MatMul":
            a, b = _f32(ins[0]), _f32(ins[1])
            ad, bd = a.shape, b.shape
            # session.rs:629-639
            assert (len(ad) == 2 and len(bd) == 2 and ad[1] == bd[0]) \
                or (len(ad) == 3 and len(bd) == 2 and ad[2] == bd[0]) \
                or (len(ad) == 3 and len(bd) == 3 and ad[0] == bd[0] and ad[2] == bd[1]) \
                or (len(ad) == 4 and len(bd) == 4 and ad[0] == 1 and bd[0] == 1 and ad[1] == bd[1]), \
                f"A shape: {ad}, B shape: {bd}"
            if len(bd) == 2:
                m = int(np.prod(ad[:-1]))
                k, n = bd
                out = np.empty(tuple(ad[:-1]) + (n,), np.float32)
                self._sgemm(False, False, m, k, n, 1.0, a, k, b, n, 0.0, out, n)
            else:
                batch = int(np.prod(ad[:-2]))
                m, k, n = ad[-2], ad[-1], bd[-1]
                out = np.empty(tuple(ad[:-1]) + (n,), np.float32)
                if self.sgemm == "openblas":
                    np.matmul(a, b, out=out)
                else:
                    L.or_sgemm_batched(batch, m, k, n, _fp(a), _fp(b), _fp(out), thr)
            return [out]
        if op == "Gemm":
            a, b = _f32(ins[0]), _f32(ins[1])
            ta, tb = bool(at.get("trans_a", False)), bool(at.get("trans_b", False))
            alpha, beta = float(at.get("alpha", 1.0)), float(at.get("beta", 1.0))
            m, k = (a.shape[1], a.shape[0]) if ta else a.shape
            n = b.shape[0] if tb else b.shape[1]
            out = np.empty((m, n), np.float32)
            # session.rs:702-717: C is pre-filled with the bias (or zeros)
            if len(ins) > 2 and ins[2] is not None:
                cin = _f32(ins[2])
                if cin.ndim == 1:
                    out[...] = cin[None, :]
                else:
                    assert cin.shape == (m, n)
                    out[...] = cin
            else:
                out.fill(0.0)
            self._sgemm(ta, tb, m, k, n, alpha, a, m if ta else k, b, k if tb else n, beta, out, n)
            return [out]
        if op == "Transpose":
            x = _f32(ins[0])
            perm = [int(p) for p in at["perm"]]
            out = np.empty([x.shape[p] for p in perm], np.float32)
            L.or_transpose(_fp(x), _fp(out), _dims(x.shape), _dims(perm), x.ndim)
            return [out]
        if op == "Concat":
            # session.rs:1134-1177 (ndarray::concatenate): a pure copy
            return [np.ascontiguousarray(np.concatenate(ins, axis=at["axis"]))]
        if op == "Split":
            # session.rs:1488-1512 (last axis)
            x = ins[0]
            axis = at.get("axis", 0)
            axis = axis + x.ndim if axis < 0 else axis
            sizes = [int(v) for v in ins[1]] if self._model.opset_version >= 13 and len(ins) > 1 \
                else at["split"]
            outs, s = [], 0
            for sz in sizes:
                idx = [slice(None)] * x.ndim
                idx[axis] = slice(s, s + sz)
                outs.append(np.ascontiguousarray(x[tuple(idx)]))
                s += sz
            return outs
        if op == "Slice":
            # session.rs:1514-1563 accepts rank 3, one axis == 2; other ranks/axes
            # are an EXTENSION with the same meaning (ONNX Slice, non-negative
            # starts/ends/steps).
            x = ins[0]
            starts, ends, axes = ins[1], ins[2], ins[3]
            steps = ins[4] if len(ins) > 4 and ins[4] is not None else np.ones(len(axes), np.int64)
            idx = [slice(None)] * x.ndim
            for st, en, ax, sp in zip(starts, ends, axes, steps):
                ax = int(ax) + x.ndim if ax < 0 else int(ax)
                idx[ax] = slice(int(st), min(int(en), x.shape[ax]), int(sp))
            return [np.ascontiguousarray(x[tuple(idx)])]
        if op == "Gather":
            # session.rs:1565-1598. Scalar index: the reference requires the
            # dims before `axis` to be 1; larger leading dims are an EXTENSION
            # (ONNX Gather with a scalar index = take along the axis).
            x, idx = ins[0], ins[1]
            axis = at.get("axis", 0)
            assert axis >= 0
            if is_scalar(idx.shape):
                return [np.ascontiguousarray(np.take(x, int(idx.reshape(-1)[0]), axis=axis))]
            assert idx.ndim == 2 and idx.shape[0] == 1 and axis == 0
            return [np.ascontiguousarray(x[idx.reshape(-1)][None])]
        if op == "Shape":
            return [np.array(ins[0].shape, np.int64)]
        raise NotImplementedError(f"{op}: Kernel not implemented")

    def _conv_openblas(self, x, w, bias, out, k, s, d, pad, group):
        """Same steps as `or_conv2d` (bias pre-fill, im2col, per-(batch, group)
        GEMM accumulated onto the bias) with numpy's OpenBLAS as the sgemm."""
        n, c, ih, iw = x.shape
        oc, oh, ow = out.shape[1], out.shape[2], out.shape[3]
        xp = np.zeros((n, c, ih + pad[0] + pad[2], iw + pad[1] + pad[3]), np.float32)
        xp[:, :, pad[0]:pad[0] + ih, pad[1]:pad[1] + iw] = x
        col = np.empty((n, c, k[0], k[1], oh, ow), np.float32)
        for fy in range(k[0]):
            for fx in range(k[1]):
                col[:, :, fy, fx] = xp[:, :, fy * d[0]:fy * d[0] + (oh - 1) * s[0] + 1:s[0],
                                       fx * d[1]:fx * d[1] + (ow - 1) * s[1] + 1:s[1]]
        icg, ocg = c // group, oc // group
        col = col.reshape(n, group, icg * k[0] * k[1], oh * ow)
        wg = w.reshape(group, ocg, icg * k[0] * k[1])
        res = np.matmul(wg[None], col).reshape(n, oc, oh, ow)
        if bias is not None:
            out[...] = bias.reshape(1, oc, 1, 1) + res
        else:
            out[...] = res


class InterpreterSessionBuilder:
    """Same builder shape as the reference's
    (crates/session_interpreter/src/builder.rs:18-65). `with_sgemm` is this
    oracle's own switch: "own" = the documented-order kernel in oracle.cpp,
    "openblas" = numpy's bundled OpenBLAS as the stand-in for BLIS."""

    def __init__(self, model):
        self.model = model
        self.intra_op_num_threads = 1
        self.enable_profiling = False
        self.sgemm = "own"

    def with_intra_op_num_threads(self, n: int):
        self.intra_op_num_threads = n
        return self

    def with_profiling_enabled(self, b: bool):
        self.enable_profiling = b
        return self

    def with_sgemm(self, which: str):
        assert which in ("own", "openblas")
        self.sgemm = which
        return self

    def build(self) -> InterpreterSession:
        return InterpreterSession(self.model, self.intra_op_num_threads, self.enable_profiling,
                                  self.sgemm)
