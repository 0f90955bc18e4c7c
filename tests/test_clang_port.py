"""The restatement of the reference's generated-C backend (oracle/clang_port.py, a timed CPU
baseline) against the interpreter oracle: both restate the same reference on the same graphs,
so their outputs must agree within the tolerance for transcendentals and reductions."""
import numpy as np
import pytest

from altius_b200 import configs, ir
from oracle import InterpreterSessionBuilder
from oracle.clang_port import ClangPortSession, _Regions, translate


def _both(model, feeds, threads=2):
    x = list(feeds.values())
    ref = InterpreterSessionBuilder(model).with_intra_op_num_threads(threads).with_sgemm("openblas").build().run(x)
    got = ClangPortSession(model, threads).run(x)
    return ref, got


def test_micrograph_matches_the_interpreter():
    model, feeds = configs.micrograph(batch=2)
    ref, got = _both(model, feeds)
    assert len(ref) == len(got) == 4
    for r, g in zip(ref, got):
        assert r.shape == g.shape
        np.testing.assert_allclose(g, r, rtol=1e-5, atol=2e-6)


def test_vision_transformer_matches_the_interpreter():
    model, feeds = configs.vit_base_16(batch=2, depth=2)
    ref, got = _both(model, feeds)
    assert got[0].shape == (2, 1000)
    assert np.abs(got[0] - ref[0]).max() < 1e-4
    assert (got[0].argmax(-1) == ref[0].argmax(-1)).all()


def test_broadcast_binary_ops_follow_numpy():
    rng = np.random.default_rng(3)
    for op, fn in (("Add", np.add), ("Sub", np.subtract), ("Mul", np.multiply), ("Div", np.divide)):
        for sa, sb in (((3, 1, 5), (4, 1)), ((7,), (7,)), ((2, 3, 4), (1,)), ((1, 6), (5, 1))):
            g = ir.Graph()
            a = g.add_input("a", sa)
            b = g.add_input("b", sb)
            g.outputs = [g.op(op, a, b)]
            xa = rng.standard_normal(sa, dtype=np.float32)
            xb = rng.standard_normal(sb, dtype=np.float32) + np.float32(3.0)
            got = ClangPortSession(ir.Model(g, 13), 1).run([xa, xb])[0]
            np.testing.assert_array_equal(got, fn(xa, xb))


def test_the_arena_reuses_freed_ranges_and_never_overlaps_live_ones():
    r = _Regions()
    a = r.alloc("a", 100)
    b = r.alloc("b", 1000)
    r.release("a")
    c = r.alloc("c", 64)
    assert c == a                        # first fit into the freed range
    d = r.alloc("d", 64)
    live = sorted(r.live.values())
    for (s0, l0), (s1, _) in zip(live, live[1:]):
        assert s0 + l0 <= s1
    assert b == 128 and d == 64 and r.top == 128 + 1024


def test_translation_is_one_function_per_node_with_reshape_as_an_alias():
    model, _ = configs.vit_base_16(batch=1, depth=1)
    text, inits, shapes = translate(model, 2)
    kinds = [n.op for n in model.graph.nodes]
    assert text.count("static void node_") == sum(k != "Reshape" for k in kinds)
    assert "cblas_sgemm(CblasRowMajor, CblasNoTrans, CblasTrans" in text      # the classifier Gemm
    assert "#pragma omp parallel for num_threads(2)" in text
    assert len(inits) == len(model.graph.inits)
    assert shapes[model.graph.outputs[0]] == [1, 1000]


def test_unsupported_operator_is_refused():
    g = ir.Graph()
    a = g.add_input("a", (4,))
    g.outputs = [g.op("Tanh", a)]
    with pytest.raises(NotImplementedError):
        translate(ir.Model(g, 13), 1)
