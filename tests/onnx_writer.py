"""A minimal ONNX serialiser for the loader tests (the `onnx` package is not installed).

Writes the protobuf wire format by hand from the field numbers of the ONNX schema
(ModelProto.graph = 7, .opset_import = 8; GraphProto.node = 1, .initializer = 5, .input = 11,
.output = 12; NodeProto.input = 1, .output = 2, .name = 3, .op_type = 4, .attribute = 5;
AttributeProto.name = 1, .f = 2, .i = 3, .s = 4, .t = 5, .floats = 7, .ints = 8, .type = 20;
TensorProto.dims = 1, .data_type = 2, .float_data = 4, .int32_data = 5, .int64_data = 7,
.name = 8, .raw_data = 9; ValueInfoProto.name = 1, .type = 2; TypeProto.tensor_type = 1;
TypeProto.Tensor.elem_type = 1, .shape = 2; TensorShapeProto.dim = 1; Dimension.dim_value = 1,
.dim_param = 2; OperatorSetIdProto.domain = 1, .version = 2). Test infrastructure only.
"""
import struct

import numpy as np

from altius_b200 import ir

DT = {np.dtype(np.float32): 1, np.dtype(np.int32): 6, np.dtype(np.int64): 7, np.dtype(np.bool_): 9}
DT_OF_ELEM = {ir.F32: 1, ir.I32: 6, ir.I64: 7, ir.BOOL: 9}


def varint(v: int) -> bytes:
    v &= (1 << 64) - 1
    out = bytearray()
    while True:
        b = v & 0x7F
        v >>= 7
        out.append(b | (0x80 if v else 0))
        if not v:
            return bytes(out)


def key(field: int, wire: int) -> bytes:
    return varint((field << 3) | wire)


def f_varint(field, v):
    return key(field, 0) + varint(int(v))


def f_bytes(field, b):
    if isinstance(b, str):
        b = b.encode()
    return key(field, 2) + varint(len(b)) + b


def f_float(field, v):
    return key(field, 5) + struct.pack("<f", float(v))


def tensor(name, array, raw=True, packed=True):
    """TensorProto; raw=False writes the typed arrays (float_data / int32_data / int64_data),
    packed or one key per element."""
    array = np.ascontiguousarray(array)
    out = b"".join(f_varint(1, d) for d in array.shape) + f_varint(2, DT[array.dtype])
    if raw or array.dtype == np.bool_:
        out += f_bytes(9, array.tobytes())
    elif array.dtype == np.float32:
        if packed:
            out += f_bytes(4, array.tobytes())
        else:
            out += b"".join(f_float(4, v) for v in array.reshape(-1))
    else:
        field = 5 if array.dtype == np.int32 else 7
        vals = [int(v) for v in array.reshape(-1)]
        if packed:
            out += f_bytes(field, b"".join(varint(v) for v in vals))
        else:
            out += b"".join(f_varint(field, v) for v in vals)
    if name is not None:
        out += f_bytes(8, name)
    return out


def attribute(name, value):
    out = f_bytes(1, name)
    if isinstance(value, bool):
        out += f_varint(3, int(value)) + f_varint(20, 2)
    elif isinstance(value, int):
        out += f_varint(3, value) + f_varint(20, 2)
    elif isinstance(value, float):
        out += f_float(2, value) + f_varint(20, 1)
    elif isinstance(value, str):
        out += f_bytes(4, value) + f_varint(20, 3)
    elif isinstance(value, np.ndarray):
        out += f_bytes(5, tensor(None, value)) + f_varint(20, 4)
    elif isinstance(value, (list, tuple)) and all(isinstance(v, float) for v in value) and value:
        out += f_bytes(7, b"".join(struct.pack("<f", v) for v in value)) + f_varint(20, 6)
    elif isinstance(value, (list, tuple)):
        out += f_bytes(8, b"".join(varint(int(v)) for v in value)) + f_varint(20, 7)
    else:
        raise TypeError(type(value))
    return out


def node(op_type, inputs, outputs, name="", **attrs):
    out = b"".join(f_bytes(1, i) for i in inputs) + b"".join(f_bytes(2, o) for o in outputs)
    if name:
        out += f_bytes(3, name)
    out += f_bytes(4, op_type)
    out += b"".join(f_bytes(5, attribute(k, v)) for k, v in attrs.items())
    return out


def value_info(name, elem_type, shape, typed=True, shaped=True):
    """shape entries: int (dim_value) or str (dim_param)."""
    dims = b""
    for d in shape:
        dims += f_bytes(1, f_bytes(2, d) if isinstance(d, str) else f_varint(1, d))
    tt = f_varint(1, elem_type) + (f_bytes(2, dims) if shaped else b"")
    return f_bytes(1, name) + (f_bytes(2, f_bytes(1, tt)) if typed else b"")


def model(nodes, initializers, inputs, outputs, opsets=(("", 13),)):
    g = b"".join(f_bytes(1, n) for n in nodes) + b"".join(f_bytes(5, t) for t in initializers)
    g += b"".join(f_bytes(11, v) for v in inputs) + b"".join(f_bytes(12, v) for v in outputs)
    out = f_varint(1, 8)                          # ir_version
    out += f_bytes(7, g)
    for domain, version in opsets:
        out += f_bytes(8, (f_bytes(1, domain) if domain else b"") + f_varint(2, version))
    return out


# ---- an ir.Model as an .onnx file: the inverse of the loader's operator table -----------------
_ONNX_NAME = {"ReLU": "Relu", "LeakyReLU": "LeakyRelu", "Conv2d": "Conv"}


def _onnx_attrs(n: ir.Node):
    a, op = n.attrs, n.op
    if op == "Conv2d":
        out = dict(kernel_shape=list(a["kernel_shape"]), strides=list(a.get("strides", [1, 1])),
                   dilations=list(a.get("dilations", [1, 1])), group=int(a.get("group", 1)))
        if a.get("auto_pad", "") not in ("", "NOTSET"):
            out["auto_pad"] = a["auto_pad"]
        if a.get("padding"):
            out["pads"] = list(a["padding"])
        return out
    if op == "MaxPool":
        out = dict(kernel_shape=list(a["kernel_shape"]), strides=list(a.get("strides", [1, 1])))
        if a.get("auto_pad", "") not in ("", "NOTSET"):
            out["auto_pad"] = a["auto_pad"]
        if a.get("padding"):
            out["pads"] = list(a["padding"])
        return out
    if op in ("HardSigmoid",):
        return dict(alpha=float(a.get("alpha", 0.2)), beta=float(a.get("beta", 0.5)))
    if op == "LeakyReLU":
        return dict(alpha=float(a.get("alpha", 0.01)))
    if op in ("Softmax", "Flatten", "Concat", "Gather"):
        return dict(axis=int(a["axis"])) if "axis" in a else {}
    if op == "Transpose":
        return dict(perm=list(a["perm"]))
    if op in ("ReduceMax", "ReduceMean", "ReduceMin"):
        out = dict(keepdims=int(bool(a.get("keep_dims", True))))
        if a.get("axes"):
            out["axes"] = list(a["axes"])
        return out
    if op == "Split":
        out = dict(axis=int(a.get("axis", 0)))
        if a.get("split"):
            out["split"] = list(a["split"])
        return out
    if op == "Gemm":
        return dict(alpha=float(a.get("alpha", 1.0)), beta=float(a.get("beta", 1.0)),
                    transA=int(bool(a.get("trans_a", False))), transB=int(bool(a.get("trans_b", False))))
    if op == "BatchNormalization":
        return dict(epsilon=float(a.get("epsilon", 1e-5)))
    if op == "LayerNormalization":
        return dict(axis=int(a.get("axis", -1)), epsilon=float(a.get("epsilon", 1e-5)),
                    stash_type=int(a.get("stash_type", 1)))
    if op == "Cast":
        return dict(to=DT_OF_ELEM[a["to"]])
    if op in ("Squeeze", "Unsqueeze"):
        return dict(axes=list(a["axes"])) if a.get("axes") else {}
    if op == "Resize":
        return {k: a[k] for k in ("mode", "coordinate_transformation_mode", "nearest_mode") if k in a}
    return {}


def serialize(m: ir.Model, raw=True, inits_as_inputs=False) -> bytes:
    g = m.graph
    names = [v.name or f"v{i}" for i, v in enumerate(g.values)]
    nodes = [node(_ONNX_NAME.get(n.op, n.op), [names[i] if i >= 0 else "" for i in n.inputs],
                  [names[o] for o in n.outputs], n.name or "", **_onnx_attrs(n)) for n in g.nodes]
    inits = [tensor(names[v], arr, raw=raw) for v, arr in g.inits.items()]
    ins = [value_info(names[v], DT_OF_ELEM[g.values[v].elem_ty], g.values[v].shape) for v in g.inputs]
    if inits_as_inputs:   # older exporters list every initializer among the graph inputs
        ins += [value_info(names[v], DT[arr.dtype], arr.shape) for v, arr in g.inits.items()]
    out_shapes = {v: g.values[v].shape for v in g.outputs}
    if any(sh is None for sh in out_shapes.values()):
        # A real export carries the shapes of its outputs: take them from shape inference.
        from altius_b200.session import CudaSessionBuilder
        planned = CudaSessionBuilder(m).with_plan_only(True).build()
        out_shapes = {v: planned.value_info(v)[0] for v in g.outputs}
    outs = [value_info(names[v], DT_OF_ELEM[g.values[v].elem_ty], out_shapes[v]) for v in g.outputs]
    return model(nodes, inits, ins, outs, opsets=(("", m.opset_version),))
