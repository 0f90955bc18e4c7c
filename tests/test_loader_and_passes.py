"""The ONNX loader and the graph passes (host code; the GPU tests at the end run what they
produce). Files are written by tests/onnx_writer.py; what the loader must do with them is
what the reference loader does (crates/core/src/onnx/load.rs:55-445) and what the passes
must find is what the reference passes find (crates/core/src/optimize/)."""
import numpy as np
import pytest

import onnx_writer as ow
from altius_b200 import configs, ir, model_io
from altius_b200.session import CudaSessionBuilder, InferenceSession, SessionError
from helpers import assert_bit_exact, run_oracle

RNG = np.random.default_rng(7)


def _graphs_equal(a: ir.Model, b: ir.Model):
    """Same operators, attributes and wiring up to value numbering; same initializer bytes."""
    assert a.opset_version == b.opset_version and len(a.graph.nodes) == len(b.graph.nodes)
    amap = {}
    def same(va, vb):
        if va < 0 or vb < 0:
            return va == vb
        if va in amap:
            return amap[va] == vb
        amap[va] = vb
        if va in a.graph.inits:
            assert vb in b.graph.inits
            x, y = a.graph.inits[va], b.graph.inits[vb]
            assert x.dtype == y.dtype and x.shape == y.shape and x.tobytes() == y.tobytes()
        return True
    for x, y in zip(a.graph.inputs, b.graph.inputs):
        assert same(x, y)
    for na, nb in zip(a.graph.nodes, b.graph.nodes):
        assert na.op == nb.op
        assert all(same(x, y) for x, y in zip(na.inputs, nb.inputs)) and len(na.inputs) == len(nb.inputs)
        assert all(same(x, y) for x, y in zip(na.outputs, nb.outputs))
    for x, y in zip(a.graph.outputs, b.graph.outputs):
        assert same(x, y)


def test_mnist_round_trip_through_the_loader(tmp_path):
    """The MNIST-structured graph (crates/core/src/model.rs:187-350) written as an .onnx file
    and loaded back: same nodes, weights and input list; the oracle computes the same bits."""
    m, feeds = configs.mnist_cnn()
    path = tmp_path / "mnist.onnx"
    path.write_bytes(ow.serialize(m, inits_as_inputs=True))
    loaded = model_io.load(str(path))
    _graphs_equal(m, loaded)
    assert [loaded.graph.values[v].name for v in loaded.graph.inputs] == ["Input3"]   # initializers removed, load.rs:143-148
    assert loaded.graph.values[loaded.graph.outputs[0]].name == "Plus214_Output_0"
    conv = loaded.graph.nodes[0]
    assert conv.op == "Conv2d" and conv.attrs["auto_pad"] == "SAME_UPPER" and conv.attrs["padding"] == [0, 0] \
        and conv.attrs["group"] == 1 and conv.attrs["kernel_shape"] == [5, 5]
    x = list(feeds.values())
    assert_bit_exact(run_oracle(loaded, x)[0], run_oracle(m, x)[0])
    planned = CudaSessionBuilder(loaded).with_plan_only(True).build()      # the loaded graph lowers
    assert planned.output_info[0][0] == (1, 10) and len(planned.schedule()) > 0


@pytest.mark.parametrize("raw,packed", [(True, True), (False, True), (False, False)])
def test_initializer_encodings(raw, packed):
    """raw_data, packed typed arrays and one-key-per-element typed arrays (load.rs:389-432)."""
    arrs = {"f": RNG.standard_normal((3, 5)).astype(np.float32), "l": np.array([[-5, 2 ** 40, 7]], np.int64),
            "i": np.array([-3, 9, 2 ** 30], np.int32), "b": np.array([True, False, True])}
    inits = [ow.tensor(k, v, raw=raw, packed=packed) for k, v in arrs.items()]
    nodes = [ow.node("Identity", ["f"], ["y"])]
    buf = ow.model(nodes, inits, [], [ow.value_info("y", 1, (3, 5))])
    m = model_io.load_from_buffer(buf)
    got = {m.graph.values[v].name: a for v, a in m.graph.inits.items()}
    for k, v in arrs.items():
        assert got[k].dtype == v.dtype and got[k].shape == v.shape and got[k].tobytes() == v.tobytes()


def test_attribute_defaults():
    """Every default of load.rs:170-361 that differs from "absent"."""
    def one(op_type, n_in=1, **attrs):
        ins = [f"x{i}" for i in range(n_in)]
        buf = ow.model([ow.node(op_type, ins, ["y"], **attrs)], [],
                       [ow.value_info(i, 1, (2, 3, 4, 4)) for i in ins], [ow.value_info("y", 1, (2, 3, 4, 4))])
        return model_io.load_from_buffer(buf).graph.nodes[0]
    assert one("Softmax").attrs == {"axis": -1}
    assert one("Flatten").attrs == {"axis": 1}
    assert one("Gather", 2).attrs == {"axis": 0}
    assert one("Split").attrs == {"axis": 0, "split": []}
    assert one("LeakyRelu").attrs["alpha"] == pytest.approx(0.01)
    hs = one("HardSigmoid").attrs
    assert hs["alpha"] == pytest.approx(0.2) and hs["beta"] == 0.5
    gm = one("Gemm", 3).attrs
    assert gm == {"trans_a": False, "trans_b": False, "alpha": 1.0, "beta": 1.0}
    assert one("Gemm", 3, transB=1, alpha=0.5).attrs["trans_b"] is True
    ln = one("LayerNormalization", 3).attrs
    assert ln["axis"] == -1 and ln["stash_type"] == 1 and ln["epsilon"] == pytest.approx(1e-5)
    assert one("BatchNormalization", 5).attrs["epsilon"] == pytest.approx(1e-5)
    cv = one("Conv", 2, kernel_shape=[3, 3]).attrs
    assert cv["strides"] == [1, 1] and cv["dilations"] == [1, 1] and cv["padding"] == [0, 0] \
        and cv["group"] == 1 and cv["auto_pad"] == "NOTSET" and cv["activation"] is None
    mp = one("MaxPool", kernel_shape=[2, 2], strides=[2, 2]).attrs
    assert mp["padding"] == [0, 0] and mp["auto_pad"] == "NOTSET"
    rz = one("Resize", 3).attrs
    assert rz == {"mode": "nearest", "coordinate_transformation_mode": "half_pixel",
                  "nearest_mode": "round_prefer_floor"}
    assert one("ReduceMax").attrs == {"keep_dims": True, "axes": []}
    assert one("ReduceMean", axes=[-1], keepdims=0).attrs == {"keep_dims": False, "axes": [-1]}
    assert one("Unsqueeze", 2).attrs == {}
    assert one("Relu").op == "ReLU" and one("LeakyRelu").op == "LeakyReLU" and one("Conv", 2, kernel_shape=[1, 1]).op == "Conv2d"
    assert one("Cast", to=7).attrs == {"to": ir.I64}


def test_squeeze_axes_depend_on_the_opset():
    def sq(opset, **attrs):
        buf = ow.model([ow.node("Squeeze", ["x"], ["y"], **attrs)], [], [ow.value_info("x", 1, (1, 3))],
                       [ow.value_info("y", 1, (3,))], opsets=(("", opset),))
        return model_io.load_from_buffer(buf).graph.nodes[0]
    assert sq(11, axes=[0]).attrs == {"axes": [0]}
    assert sq(13).attrs == {}
    with pytest.raises(SessionError, match="Attribute 'axes' is not specified"):
        sq(11)


def test_loader_errors():
    vi = [ow.value_info("x", 1, (1, 4))]
    ok_node = [ow.node("Relu", ["x"], ["y"])]
    out = [ow.value_info("y", 1, (1, 4))]
    with pytest.raises(SessionError, match="does not contain any graph"):
        model_io.load_from_buffer(ow.f_varint(1, 8) + ow.f_bytes(8, ow.f_varint(2, 13)))
    with pytest.raises(SessionError, match="duplicated opsets"):
        model_io.load_from_buffer(ow.model(ok_node, [], vi, out, opsets=(("", 13), ("ai.onnx", 12))))
    with pytest.raises(SessionError, match="duplicated opsets"):     # the reference's message for "no opset"
        model_io.load_from_buffer(ow.model(ok_node, [], vi, out, opsets=()))
    with pytest.raises(SessionError, match=r"Custom domain \('com.microsoft'\) not supported"):
        model_io.load_from_buffer(ow.model(ok_node, [], vi, out, opsets=(("", 13), ("com.microsoft", 1))))
    with pytest.raises(SessionError, match="Unsupported op: Einsum"):
        model_io.load_from_buffer(ow.model([ow.node("Einsum", ["x"], ["y"])], [], vi, out))
    with pytest.raises(SessionError, match="Attribute 'axis' is not specified"):
        model_io.load_from_buffer(ow.model([ow.node("Concat", ["x", "x"], ["y"])], [], vi, out))
    with pytest.raises(SessionError, match="Value type is not specified"):
        model_io.load_from_buffer(ow.model(ok_node, [], [ow.value_info("x", 1, (1, 4), typed=False)], out))
    with pytest.raises(SessionError, match="Value shape is not specified"):
        model_io.load_from_buffer(ow.model(ok_node, [], [ow.value_info("x", 1, (1, 4), shaped=False)], out))
    with pytest.raises(SessionError, match="Unsupported tensor element type"):
        model_io.load_from_buffer(ow.model(ok_node, [], [ow.value_info("x", 11, (1, 4))], out))   # DOUBLE
    with pytest.raises(SessionError):
        model_io.load_from_buffer(b"\x3a\xff\xff\xff\xff\x0f")        # a length that runs past the buffer
    with pytest.raises(SessionError, match="cannot open"):
        model_io.load("/nonexistent/model.onnx")


def test_dynamic_dimension_is_loaded_and_refused_at_build():
    buf = ow.model([ow.node("Relu", ["x"], ["y"])], [], [ow.value_info("x", 1, ("batch", 4))],
                   [ow.value_info("y", 1, ("batch", 4))])
    m = model_io.load_from_buffer(buf)
    assert m.graph.values[m.graph.inputs[0]].shape == (-1, 4)
    with pytest.raises(SessionError, match="Must be fixed dimension"):       # shape.rs:675
        CudaSessionBuilder(m).with_plan_only(True).build()


def test_constant_node_becomes_an_initializer():
    c = np.arange(4, dtype=np.float32).reshape(1, 4)
    buf = ow.model([ow.node("Constant", [], ["c"], value=c), ow.node("Add", ["x", "c"], ["y"])], [],
                   [ow.value_info("x", 1, (1, 4))], [ow.value_info("y", 1, (1, 4))])
    m = model_io.load_from_buffer(buf)
    assert [n.op for n in m.graph.nodes] == ["Add"]
    (vid, arr), = m.graph.inits.items()
    assert m.graph.values[vid].name == "c" and np.array_equal(arr, c)
    x = RNG.standard_normal((1, 4)).astype(np.float32)
    assert_bit_exact(run_oracle(m, [x])[0], x + c)


# ---- passes ---------------------------------------------------------------------------------
@pytest.mark.parametrize("form,which", [("erf", "fuse_gelu"), ("tanh", "fuse_fast_gelu")])
def test_passes_restore_the_fused_vit(form, which):
    """A ViT slice with every LayerNorm spelled as nine nodes and every Gelu as five (or
    eight): after the passes the graph is the pre-fused one, and lowers to the same schedule."""
    raw, _ = configs.vit_base_16(batch=2, depth=2, fused=False, gelu_form=form)
    fused, _ = configs.vit_base_16(batch=2, depth=2)
    counts = {}
    opt = model_io.optimize(raw, counts=counts)
    assert counts["fuse_layer_norm"] == 5 and counts[which] == 2 and sum(counts.values()) == 7
    assert sorted(n.op for n in opt.graph.nodes) == sorted(n.op for n in fused.graph.nodes)
    ln = [n for n in opt.graph.nodes if n.op == "LayerNormalization"][0]
    assert ln.attrs["axis"] == -1 and ln.attrs["stash_type"] == 1 and ln.attrs["epsilon"] == pytest.approx(1e-6)
    sched = lambda m: [e["kind"] for e in CudaSessionBuilder(m).with_plan_only(True).build().schedule()]
    assert sched(opt) == sched(fused)
    assert len(sched(raw)) > len(sched(fused))      # the raw graph lowers too, node by node


def test_passes_leave_near_misses_alone():
    def gelu_graph(sqrt2, one, half):
        g = ir.Graph()
        x = g.add_input("x", (4, 8))
        f = lambda v: g.new_init(np.array(v, np.float32))
        e = g.op("Erf", g.op("Div", x, f(sqrt2)))
        y = g.op("Mul", g.op("Mul", x, g.op("Add", e, f(one))), f(half))
        g.outputs.append(y)
        return ir.Model(g, 13)
    count = lambda m: [n.op for n in model_io.optimize(m).graph.nodes].count("Gelu")
    assert count(gelu_graph(1.41421356, 1.0, 0.5)) == 1
    assert count(gelu_graph(1.4142099618911743, 1.0, 0.5)) == 1      # the constant the reference matches
    assert count(gelu_graph(1.4143, 1.0, 0.5)) == 0                  # outside atol 1e-5
    assert count(gelu_graph(1.41421356, 1.0001, 0.5)) == 0           # the 1 and the 0.5 must be exact
    assert count(gelu_graph(1.41421356, 1.0, 0.4999)) == 0


def test_eliminate_identity():
    g = ir.Graph()
    x = g.add_input("x", (2, 3))
    a = g.op("Identity", x)
    b = g.op("Identity", a)
    r = g.op("ReLU", b)
    out = g.op("Identity", r)            # feeds the graph output: kept (identity_elim.rs:29-36)
    g.outputs.append(out)
    m = model_io.optimize(ir.Model(g, 13), passes=("eliminate_identity",))
    assert [n.op for n in m.graph.nodes] == ["ReLU", "Identity"]
    assert m.graph.nodes[0].inputs == [x]
    xv = RNG.standard_normal((2, 3)).astype(np.float32)
    assert_bit_exact(run_oracle(m, [xv])[0], np.maximum(xv, 0))


def test_layer_norm_fusion_rewires_a_graph_output():
    g = ir.Graph()
    x = g.add_input("x", (2, 5, 16))
    w = configs._W(3, 0.02)
    y = configs._ln(g, w, x, 16, 1e-5, fused=False)
    g.outputs.append(y)
    m = model_io.optimize(ir.Model(g, 13))
    assert [n.op for n in m.graph.nodes] == ["LayerNormalization"] and m.graph.outputs == m.graph.nodes[0].outputs


# ---- on the GPU -----------------------------------------------------------------------------
@pytest.mark.gpu
def test_inference_session_from_a_file(cuda_lib, tmp_path):
    """`InferenceSession("model.onnx", backend="cuda")`: load, passes, build, run."""
    m, feeds = configs.mnist_cnn()
    path = tmp_path / "mnist.onnx"
    path.write_bytes(ow.serialize(m, raw=False))
    sess = InferenceSession(str(path), backend="cuda")
    got = sess.run(None, feeds)[0]
    want = run_oracle(m, list(feeds.values()))[0]
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-5)
    sess.session.close()
    with pytest.raises(RuntimeError, match="Unknown backend"):
        InferenceSession(str(path), backend="tpu")


@pytest.mark.gpu
@pytest.mark.parametrize("form", ["erf", "tanh"])
def test_raw_vit_export_through_loader_and_passes(cuda_lib, tmp_path, form):
    """An un-fused ViT slice as an .onnx file: after the loader and the passes the session's
    output is bit-identical to the session built from the pre-fused graph, and matches the
    oracle run on the fused graph."""
    raw, feeds = configs.vit_base_16(batch=2, depth=2, fused=False, gelu_form=form)
    fused, _ = configs.vit_base_16(batch=2, depth=2)
    path = tmp_path / "vit_slice.onnx"
    path.write_bytes(ow.serialize(raw))
    sess = InferenceSession(str(path), backend="cuda")
    got = sess.run(None, feeds)[0]
    sess.session.close()
    ref = CudaSessionBuilder(fused).build()
    x = list(feeds.values())
    same = ref.run(x)[0]
    ref.close()
    assert_bit_exact(got, same)
    want = run_oracle(fused, x, sgemm="openblas")[0]
    assert np.abs(got - want).max() <= 1e-3 and (got.argmax(-1) == want.argmax(-1)).all()


@pytest.mark.gpu
def test_raw_graph_runs_without_the_passes(cuda_lib):
    """The nine-node LayerNorm and the five-node Gelu as they are (ReduceMean, Sub, Pow, Sqrt,
    Div, Erf ... kernels), against the oracle on the same raw graph."""
    raw, feeds = configs.vit_base_16(batch=2, depth=1, fused=False)
    x = list(feeds.values())
    sess = CudaSessionBuilder(raw).build()
    got = sess.run(x)[0]
    sess.close()
    want = run_oracle(raw, x, sgemm="openblas")[0]
    assert np.abs(got - want).max() <= 1e-3 and (got.argmax(-1) == want.argmax(-1)).all()
