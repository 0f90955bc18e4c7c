"""Pins the CPU oracle against what the reference's own tests hold for the hot
path, and against exact mathematics where the reference only has differential
tests (its oracle, ONNX Runtime, is not available offline).

Pins taken from the reference:
  * broadcast shape cases 1-7          crates/core/src/fixed_dim.rs:192-245
  * MNIST graph topological order      crates/core/src/snapshots/altius_core__model__mnist_model.snap
  * Add known-answer vector [4,2]      crates/session/tests/ort.rs:11-26
  * Add/Sub/Mul/Div == the IEEE operator on shapes [1,2], [3,1,10], [128,3,224,224]
                                       crates/session_interpreter/tests/op_bin.rs:44-90
  * the tolerances of the Python op tests (np.allclose defaults; LayerNorm
    rtol 1e-4 atol 1e-5)               crates/altius_py/tests/test_ops_*.py
"""
import numpy as np
import pytest
import scipy.special

from altius_b200 import configs, ir
from helpers import run_oracle, single_op_model, assert_bit_exact


def test_broadcast_shape_cases():
    b = ir.broadcast_shapes
    assert b([1]) == (1,)
    assert b([1], [4, 1]) == (4, 1)
    assert b([4, 1], [1]) == (4, 1)
    assert b([10, 20, 30], [10, 20]) is None          # broadcast_4 should_panic
    assert b([1, 3, 3], [5, 1, 3, 3]) == (5, 1, 3, 3)
    assert b([1, 3, 1], [5, 3, 10]) == (5, 3, 10)
    assert b([1, 3, 4, 4], [3, 1, 1]) == (1, 3, 4, 4)


def test_mnist_topological_order_snapshot():
    model, _ = configs.mnist_cnn()
    assert model.topo_sort_nodes() == [9, 0, 1, 2, 3, 4, 5, 6, 7, 8, 10, 11]


def test_add_known_answer():
    x = np.array([1, 3, 5, 7, 9, 11, 13, 15], np.float32).reshape(4, 2)
    y = np.array([2, 4, 6, 8, 10, 12, 14, 16], np.float32).reshape(4, 2)
    out = run_oracle(single_op_model("Add", [x, y]), [x, y])[0]
    assert out.shape == (4, 2)
    assert out.reshape(-1).tolist() == [3.0, 7.0, 11.0, 15.0, 19.0, 23.0, 27.0, 31.0]


@pytest.mark.parametrize("shape", [(1, 2), (3, 1, 10), (128, 3, 224, 224)])
@pytest.mark.parametrize("op,fn", [("Add", np.add), ("Sub", np.subtract), ("Mul", np.multiply),
                                   ("Div", np.divide)])
def test_binary_ops_are_the_ieee_operator(op, fn, shape):
    rng = np.random.default_rng(42)
    x = rng.random(shape, dtype=np.float32)
    y = rng.random(shape, dtype=np.float32) + np.float32(0.01)
    out = run_oracle(single_op_model(op, [x, y]), [x, y])[0]
    assert_bit_exact(out, fn(x, y))


@pytest.mark.parametrize("ashape,bshape", [
    ((1, 3, 28, 28), (3, 1, 1)), ((1, 12, 9, 9), (1, 1, 1, 9)), ((4, 1, 2), (3, 1)),
    ((3, 28, 28), (3, 28, 1)), ((3, 15, 15), (15,)), ((3, 15, 15), (1,)), ((1,), (3, 4)),
    ((1, 2, 3, 4, 5, 6, 7), (1, 2, 3, 4, 5, 6, 7))])
def test_binary_broadcast_matches_numpy(ashape, bshape):
    # shapes of crates/altius_py/tests/test_ops_bin.py:11-140
    rng = np.random.default_rng(0)
    a = rng.standard_normal(ashape).astype(np.float32)
    b = (rng.random(bshape, dtype=np.float32) + np.float32(0.5))
    for op, fn in (("Add", np.add), ("Sub", np.subtract), ("Mul", np.multiply), ("Div", np.divide)):
        out = run_oracle(single_op_model(op, [a, b]), [a, b])[0]
        assert_bit_exact(out, fn(a, b))


def test_invalid_broadcast_is_rejected():
    a = np.zeros((1, 3, 28, 28), np.float32)
    b = np.zeros((3, 1, 2), np.float32)               # test_add_5 (xfail in the reference)
    with pytest.raises(ValueError):
        run_oracle(single_op_model("Add", [a, b]), [a, b])


def test_softmax_close_to_exact():
    rng = np.random.default_rng(1)
    for shape in ((1, 2, 3), (3, 28, 28), (16, 197, 197)):   # test_ops_elemwise.py:109-126
        x = (rng.standard_normal(shape) * 3).astype(np.float32)
        out = run_oracle(single_op_model("Softmax", [x], axis=-1), [x])[0]
        ref = scipy.special.softmax(x.astype(np.float64), axis=-1)
        np.testing.assert_allclose(out, ref, rtol=1e-5, atol=1e-8)   # np.allclose defaults


def test_softmax_ignores_nothing_but_handles_extremes():
    x = np.array([[1000.0, 0.0, -1000.0, 1000.0]], np.float32)
    out = run_oracle(single_op_model("Softmax", [x], axis=-1), [x])[0]
    np.testing.assert_allclose(out, [[0.5, 0.0, 0.0, 0.5]], atol=1e-7)


def test_gelu_is_the_tanh_form():
    x = np.linspace(-12, 12, 4801, dtype=np.float32)
    out = run_oracle(single_op_model("Gelu", [x]), [x])[0]
    xd = x.astype(np.float64)
    ref = 0.5 * xd * (1 + np.tanh(0.7978845608028654 * (xd + 0.044715 * xd ** 3)))
    np.testing.assert_allclose(out, ref, rtol=0, atol=2e-6)
    # and within the reference's own acceptance of the erf form (atol 1e-1)
    erf_form = 0.5 * xd * (1 + scipy.special.erf(xd / np.sqrt(2)))
    np.testing.assert_allclose(out, erf_form, atol=1e-1)


def test_sigmoid_tanh_close_to_exact():
    x = np.concatenate([np.linspace(-30, 30, 2001), [-200.0, 200.0, 0.0]]).astype(np.float32)
    sig = run_oracle(single_op_model("Sigmoid", [x]), [x])[0]
    np.testing.assert_allclose(sig, scipy.special.expit(x.astype(np.float64)), rtol=2e-6, atol=1e-30)
    x7 = x[:7].reshape(1, 7)                           # tail shorter than 8 lanes
    sig7 = run_oracle(single_op_model("Sigmoid", [x7]), [x7])[0]
    assert_bit_exact(sig7.reshape(-1), sig[:7])
    th = run_oracle(single_op_model("Tanh", [x]), [x])[0]
    np.testing.assert_allclose(th, np.tanh(x.astype(np.float64)), rtol=0, atol=2e-6)


def test_layer_norm_close_to_exact():
    rng = np.random.default_rng(2)
    for shape in ((1, 20, 10), (5, 197, 768), (3, 7, 384)):  # test_ops_norm.py:58-64
        x = rng.standard_normal(shape).astype(np.float32)
        g = (1 + 0.02 * rng.standard_normal(shape[-1])).astype(np.float32)
        b = (0.02 * rng.standard_normal(shape[-1])).astype(np.float32)
        m = single_op_model("LayerNormalization", [x], [g.reshape(1, 1, -1), b.reshape(1, 1, -1)],
                            axis=-1, epsilon=1e-5, stash_type=1)
        out = run_oracle(m, [x])[0]
        xd = x.astype(np.float64)
        ref = (xd - xd.mean(-1, keepdims=True)) / np.sqrt(xd.var(-1, keepdims=True) + 1e-5) * g + b
        np.testing.assert_allclose(out, ref, rtol=1e-4, atol=1e-5)


def test_relu_hardsigmoid_leaky_maxpool_exact():
    rng = np.random.default_rng(3)
    x = rng.standard_normal((3, 1, 28, 28)).astype(np.float32)
    assert_bit_exact(run_oracle(single_op_model("ReLU", [x]), [x])[0], np.maximum(x, 0))
    hs = run_oracle(single_op_model("HardSigmoid", [x], alpha=0.2, beta=0.5), [x])[0]
    np.testing.assert_allclose(hs, np.clip(0.2 * x.astype(np.float64) + 0.5, 0, 1), rtol=0, atol=1e-7)
    lk = run_oracle(single_op_model("LeakyReLU", [x], alpha=0.1), [x])[0]
    assert_bit_exact(lk, np.where(x < 0, np.float32(0.1) * x, x))
    mp = run_oracle(single_op_model("MaxPool", [x], kernel_shape=[2, 2], strides=[2, 2],
                                    padding=[0, 0, 0, 0]), [x])[0]
    assert_bit_exact(mp, x.reshape(3, 1, 14, 2, 14, 2).max(axis=(3, 5)))
    # 5x5 s1 p2 (test_ops_pool.py): padded positions never win, shape is kept
    mp5 = run_oracle(single_op_model("MaxPool", [x], kernel_shape=[5, 5], strides=[1, 1],
                                     padding=[2, 2, 2, 2]), [x])[0]
    xp = np.full((3, 1, 32, 32), -np.inf, np.float32)
    xp[:, :, 2:30, 2:30] = x
    win = np.lib.stride_tricks.sliding_window_view(xp, (5, 5), axis=(2, 3)).max(axis=(-1, -2))
    assert_bit_exact(mp5, win)


def test_reductions():
    rng = np.random.default_rng(4)
    x = rng.standard_normal((1, 50, 70)).astype(np.float32)        # test_ops_reduce.py:10-41
    mean = run_oracle(single_op_model("ReduceMean", [x], axes=[-1], keep_dims=True), [x])[0]
    assert mean.shape == (1, 50, 1)
    np.testing.assert_allclose(mean, x.astype(np.float64).mean(-1, keepdims=True), rtol=1e-5, atol=1e-7)
    mx = run_oracle(single_op_model("ReduceMax", [x], axes=[], keep_dims=False), [x])[0]
    assert mx.shape == (1,) and mx[0] == x.max()
    mxl = run_oracle(single_op_model("ReduceMax", [x], axes=[-1], keep_dims=True), [x])[0]
    assert_bit_exact(mxl, x.max(-1, keepdims=True))
    y = rng.standard_normal((2, 5, 7, 7)).astype(np.float32)
    gap = run_oracle(single_op_model("GlobalAveragePool", [y]), [y])[0]
    np.testing.assert_allclose(gap, y.astype(np.float64).mean((2, 3), keepdims=True), rtol=1e-5, atol=1e-7)


def test_matmul_gemm_conv_against_float64():
    rng = np.random.default_rng(5)
    for ash, bsh in (((4, 8), (8, 3)), ((2, 5, 8), (8, 3)), ((3, 5, 8), (3, 8, 6)),
                     ((1, 2, 5, 8), (1, 2, 8, 6))):                  # test_ops_matmul.py
        a = rng.standard_normal(ash).astype(np.float32)
        b = rng.standard_normal(bsh).astype(np.float32)
        for sg in ("own", "openblas"):
            out = run_oracle(single_op_model("MatMul", [a, b]), [a, b], sgemm=sg)[0]
            np.testing.assert_allclose(out, a.astype(np.float64) @ b.astype(np.float64), rtol=1e-5, atol=1e-5)
    a = rng.standard_normal((7, 9)).astype(np.float32)
    for tb, bsh in ((False, (9, 5)), (True, (5, 9))):                # test_ops_gemm.py
        b = rng.standard_normal(bsh).astype(np.float32)
        for c in (rng.standard_normal(5).astype(np.float32), rng.standard_normal((7, 5)).astype(np.float32), None):
            m = single_op_model("Gemm", [a, b] + ([c] if c is not None else []), alpha=0.5, beta=2.0,
                                trans_a=False, trans_b=tb)
            out = run_oracle(m, [a, b] + ([c] if c is not None else []))[0]
            ref = 0.5 * (a.astype(np.float64) @ (b.T if tb else b)) + (2.0 * c if c is not None else 0)
            np.testing.assert_allclose(out, ref, rtol=1e-5, atol=1e-5)
    import torch
    import torch.nn.functional as F
    for (n, c, h, oc, k, s, p, g) in ((1, 1, 28, 8, 5, 1, 2, 1), (2, 4, 15, 6, 3, 2, 1, 1),
                                      (2, 16, 9, 16, 3, 1, 1, 16), (1, 3, 32, 8, 16, 16, 0, 1)):
        x = rng.standard_normal((n, c, h, h)).astype(np.float32)
        w = rng.standard_normal((oc, c // g, k, k)).astype(np.float32)
        b = rng.standard_normal(oc).astype(np.float32)
        m = single_op_model("Conv2d", [x], [w, b], kernel_shape=[k, k], strides=[s, s],
                            padding=[p, p, p, p], dilations=[1, 1], group=g, auto_pad="")
        ref = F.conv2d(torch.from_numpy(x).double(), torch.from_numpy(w).double(),
                       torch.from_numpy(b).double(), stride=s, padding=p, groups=g).numpy()
        for sg in ("own", "openblas"):
            out = run_oracle(m, [x], sgemm=sg)[0]
            np.testing.assert_allclose(out, ref, rtol=1e-5, atol=1e-5)  # ops_conv.rs:41-43 uses 1e-5


def test_data_movement():
    rng = np.random.default_rng(6)
    x = rng.standard_normal((2, 3, 4, 5)).astype(np.float32)
    for perm in ([1, 2, 0, 3], [0, 1, 3, 2], [2, 1, 0, 3], [0, 1, 2, 3], [3, 2, 1, 0]):
        out = run_oracle(single_op_model("Transpose", [x], perm=perm), [x])[0]
        assert_bit_exact(out, np.ascontiguousarray(x.transpose(perm)))
    y = rng.standard_normal((2, 7, 4, 5)).astype(np.float32)
    out = run_oracle(single_op_model("Concat", [x, y], axis=1), [x, y])[0]
    assert_bit_exact(out, np.concatenate([x, y], 1))
    z = rng.standard_normal((2, 3, 12)).astype(np.float32)
    outs = run_oracle(single_op_model("Split", [z], [np.array([4, 4, 4], np.int64)], n_outputs=3, axis=2), [z])
    for i, o in enumerate(outs):
        assert_bit_exact(o, z[:, :, 4 * i:4 * i + 4])
    sl = run_oracle(single_op_model("Slice", [z], [np.array([2], np.int64), np.array([9], np.int64),
                                                   np.array([2], np.int64)]), [z])[0]
    assert_bit_exact(sl, z[:, :, 2:9])
    ga = run_oracle(single_op_model("Gather", [z], [np.array(1, np.int64)], axis=1), [z])[0]
    assert_bit_exact(ga, z[:, 1, :])


def test_models_own_vs_openblas_sgemm_agree():
    for fn, kw in ((configs.mnist_cnn, {}), (configs.vit_base_16, dict(batch=2, depth=2)),
                   (configs.mobilenet_v3_large, dict(batch=1))):
        model, feeds = fn(**kw)
        a = run_oracle(model, feeds.values(), threads=8, sgemm="own")[0]
        b = run_oracle(model, feeds.values(), threads=8, sgemm="openblas")[0]
        assert np.abs(a - b).max() < 1e-4
        assert (a.argmax(-1) == b.argmax(-1)).all()


def test_resize_known_answers():
    """compute_resize (session.rs:1057-1132): nearest with an integer scale replicates pixels;
    the bilinear branch reproduces a constant image and blends rows / columns half a pixel
    off (its source coordinate is max(dst / scale - 0.5, 0))."""
    from helpers import run_oracle, single_op_model
    rng = np.random.default_rng(3)
    x = rng.standard_normal((1, 2, 5, 5)).astype(np.float32)
    none = np.zeros(0, np.float32)
    m = single_op_model("Resize", [x], [none, none, np.array([1, 2, 15, 15], np.int64)], mode="nearest")
    np.testing.assert_array_equal(run_oracle(m, [x])[0], x.repeat(3, axis=2).repeat(3, axis=3))
    c = np.full((1, 1, 4, 4), 2.5, np.float32)
    m = single_op_model("Resize", [c], [none, none, np.array([1, 1, 9, 9], np.int64)], mode="linear")
    np.testing.assert_array_equal(run_oracle(m, [c])[0], np.full((1, 1, 9, 9), 2.5, np.float32))
    r = np.arange(16, dtype=np.float32).reshape(1, 1, 4, 4)
    m = single_op_model("Resize", [r], [none, none, np.array([1, 1, 4, 4], np.int64)], mode="linear")
    out = run_oracle(m, [r])[0][0, 0]
    assert out[0, 0] == 0.0 and out[1, 0] == 2.0 and out[0, 1] == 0.5 and out[3, 3] == 12.5   # half a pixel off


def test_expand_is_a_broadcast_to_the_shape_input():
    from helpers import run_oracle, single_op_model
    x = np.arange(6, dtype=np.int64).reshape(1, 1, 1, 6)
    m = single_op_model("Expand", [x], [np.array([1, 1, 4, 6], np.int64)])
    out = run_oracle(m, [x])[0]
    assert out.dtype == np.int64 and out.shape == (1, 1, 4, 6) and (out == x).all()
