"""Parity of every CUDA kernel with the CPU oracle, one node at a time, through
the C ABI. Shapes are those of the reference's own op tests
(crates/altius_py/tests/test_ops_*.py, crates/session_interpreter/tests/op_bin.rs)
plus the benchmark configurations' shapes.

Bars: bit-exact for Add/Sub/Mul/Div, ReLU, LeakyReLU, HardSigmoid, Gelu,
Sigmoid, Tanh, Sqrt (per-element formulas restated operation by operation),
MaxPool and all data movement; max relative error 1e-5 for reductions and
softmax (tree summation order differs from the oracle's 8-lane partial sums);
rtol 1e-5 + atol 1e-5 for contractions (summation order is unspecified in the
reference's BLIS)."""
import os

import numpy as np
import pytest

from helpers import assert_bit_exact, max_rel_err, run_cuda, run_oracle, single_op_model

pytestmark = pytest.mark.gpu
RNG = np.random.default_rng(1234)


def both(model, inputs, **opts):
    return run_cuda(model, inputs, **opts), run_oracle(model, inputs)


BIN_SHAPES = [((1, 2), (1, 2)), ((3, 1, 10), (3, 1, 10)), ((1, 2, 3, 4, 5, 6, 7), (1, 2, 3, 4, 5, 6, 7)),
              ((1, 3, 28, 28), (3, 1, 1)), ((1, 12, 9, 9), (1, 1, 1, 9)), ((4, 1, 2), (3, 1)),
              ((3, 28, 28), (3, 28, 1)), ((3, 15, 15), (15,)), ((3, 15, 15), (1,)), ((1,), (5, 7)),
              ((8, 197, 768), (768,)), ((4, 16, 14, 14), (4, 16, 1, 1)), ((2, 197, 768), (1, 197, 768)),
              ((5, 33), (5, 33)), ((128, 3, 224, 224), (128, 3, 224, 224))]


@pytest.mark.parametrize("ashape,bshape", BIN_SHAPES)
def test_binary_bit_exact(cuda_lib, ashape, bshape):
    a = RNG.standard_normal(ashape).astype(np.float32)
    b = (RNG.random(bshape, dtype=np.float32) + np.float32(0.25))
    for op in ("Add", "Sub", "Mul", "Div"):
        got, want = both(single_op_model(op, [a, b]), [a, b])
        assert_bit_exact(got[0], want[0])


def test_binary_with_constant_operand_and_specials(cuda_lib):
    a = RNG.standard_normal((6, 10)).astype(np.float32)
    a[0, :4] = [np.inf, -np.inf, np.nan, 0.0]
    c = np.array([0.0, 1.0, -2.0, np.inf, 3.0, 1e-38, 1e38, -0.0, 5.0, 7.0], np.float32)
    for op in ("Add", "Sub", "Mul", "Div"):
        got, want = both(single_op_model(op, [a], [c]), [a])
        assert_bit_exact(got[0], want[0])
        got, want = both(single_op_model(op, [a], [c], const_first=True), [a])
        assert_bit_exact(got[0], want[0])


def test_pow(cuda_lib):
    a = (RNG.random((3, 17), dtype=np.float32) + np.float32(0.1))
    b = RNG.standard_normal((3, 17)).astype(np.float32)
    got, want = both(single_op_model("Pow", [a, b]), [a, b])
    assert max_rel_err(got[0], want[0]) < 1e-5
    got, want = both(single_op_model("Pow", [a], [np.array([2.0], np.float32)]), [a])
    assert_bit_exact(got[0], want[0])
    got, want = both(single_op_model("Pow", [a], [np.array([1.7], np.float32)]), [a])
    assert max_rel_err(got[0], want[0]) < 1e-5


@pytest.mark.parametrize("op,attrs", [("ReLU", {}), ("Gelu", {}), ("Sigmoid", {}), ("Tanh", {}),
                                      ("HardSigmoid", dict(alpha=0.2, beta=0.5)),
                                      ("HardSigmoid", dict(alpha=1.0 / 6.0, beta=0.5)),
                                      ("LeakyReLU", dict(alpha=0.1)), ("Sqrt", {})])
@pytest.mark.parametrize("shape", [(1, 2), (3, 1, 28, 28), (3, 1, 7, 7), (4, 197, 3072)])
def test_unary_bit_exact(cuda_lib, op, attrs, shape):
    x = (RNG.standard_normal(shape) * 4).astype(np.float32)
    if op == "Sqrt":
        x = np.abs(x)
    flat = x.reshape(-1)
    flat[: min(6, flat.size)] = [0.0, 100.0, -100.0, 9.5, -9.5, 1e-20][: min(6, flat.size)]
    got, want = both(single_op_model(op, [x], **attrs), [x])
    assert_bit_exact(got[0], want[0])


def test_erf_unpinned_tolerance(cuda_lib):
    # The reference's Erf lives in an un-vendored crate and is tested to atol 1e-1 only.
    x = RNG.standard_normal((3, 1, 28, 28)).astype(np.float32)
    got, want = both(single_op_model("Erf", [x]), [x])
    np.testing.assert_allclose(got[0], want[0], atol=1e-6)


@pytest.mark.parametrize("shape", [(1, 2, 3), (3, 28, 28), (16, 512, 512), (4, 12, 197, 197), (2, 3, 1500)])
def test_softmax(cuda_lib, shape):
    x = (RNG.standard_normal(shape) * 3).astype(np.float32)
    got, want = both(single_op_model("Softmax", [x], axis=-1), [x])
    assert max_rel_err(got[0], want[0]) < 1e-5


def test_softmax_extremes(cuda_lib):
    x = np.array([[1000.0, 0.0, -1000.0, 1000.0], [-np.inf, 0.0, 1.0, 2.0]], np.float32)
    got, want = both(single_op_model("Softmax", [x], axis=-1), [x])
    np.testing.assert_allclose(got[0], want[0], rtol=1e-5, atol=1e-30)


@pytest.mark.parametrize("shape", [(1, 20, 10), (6, 197, 768), (3, 198, 384), (5, 7, 1000), (2, 3, 5000)])
def test_layer_norm(cuda_lib, shape):
    x = RNG.standard_normal(shape).astype(np.float32)
    g = (1 + 0.02 * RNG.standard_normal(shape[-1])).astype(np.float32)
    b = (0.02 * RNG.standard_normal(shape[-1])).astype(np.float32)
    m = single_op_model("LayerNormalization", [x], [g.reshape(1, 1, -1), b.reshape(1, 1, -1)],
                        axis=-1, epsilon=1e-6, stash_type=1)
    got, want = both(m, [x])
    np.testing.assert_allclose(got[0], want[0], rtol=1e-5, atol=1e-6)


def test_reductions(cuda_lib):
    for shape in ((1, 50, 70), (4, 197, 768), (3, 5, 33)):
        x = RNG.standard_normal(shape).astype(np.float32)
        got, want = both(single_op_model("ReduceMean", [x], axes=[-1], keep_dims=True), [x])
        np.testing.assert_allclose(got[0], want[0], rtol=1e-5, atol=1e-7)
        got, want = both(single_op_model("ReduceMax", [x], axes=[-1], keep_dims=True), [x])
        assert_bit_exact(got[0], want[0])
        got, want = both(single_op_model("ReduceMax", [x], axes=[], keep_dims=False), [x])
        assert_bit_exact(got[0], want[0])
    for shape in ((2, 5, 7, 7), (4, 960, 7, 7), (2, 16, 56, 56)):
        y = RNG.standard_normal(shape).astype(np.float32)
        got, want = both(single_op_model("GlobalAveragePool", [y]), [y])
        np.testing.assert_allclose(got[0], want[0], rtol=1e-5, atol=1e-7)


def test_max_pool_bit_exact(cuda_lib):
    x = RNG.standard_normal((3, 4, 28, 28)).astype(np.float32)
    for k, s, p in ((2, 2, 0), (3, 3, 0), (5, 1, 2), (3, 2, 1)):
        m = single_op_model("MaxPool", [x], kernel_shape=[k, k], strides=[s, s], padding=[p, p, p, p])
        got, want = both(m, [x])
        assert_bit_exact(got[0], want[0])


def test_data_movement_bit_exact(cuda_lib):
    x = RNG.standard_normal((2, 3, 4, 5)).astype(np.float32)
    for perm in ([1, 2, 0, 3], [0, 1, 3, 2], [2, 1, 0, 3], [0, 1, 2, 3], [3, 2, 1, 0], [0, 2, 1, 3]):
        got, want = both(single_op_model("Transpose", [x], perm=perm), [x])
        assert_bit_exact(got[0], want[0])
    big = RNG.standard_normal((4, 197, 12, 64)).astype(np.float32)
    got, want = both(single_op_model("Transpose", [big], perm=[0, 2, 1, 3]), [big])
    assert_bit_exact(got[0], want[0])
    kt = RNG.standard_normal((48, 197, 64)).astype(np.float32)
    got, want = both(single_op_model("Transpose", [kt], perm=[0, 2, 1]), [kt])
    assert_bit_exact(got[0], want[0])
    y = RNG.standard_normal((2, 7, 4, 5)).astype(np.float32)
    got, want = both(single_op_model("Concat", [x, y], axis=1), [x, y])
    assert_bit_exact(got[0], want[0])
    z = RNG.standard_normal((2, 3, 12)).astype(np.float32)
    m = single_op_model("Split", [z], [np.array([4, 5, 3], np.int64)], n_outputs=3, axis=2)
    got, want = both(m, [z])
    for g_, w_ in zip(got, want):
        assert_bit_exact(g_, w_)
    m = single_op_model("Slice", [z], [np.array([2], np.int64), np.array([9], np.int64),
                                       np.array([2], np.int64)])
    got, want = both(m, [z])
    assert_bit_exact(got[0], want[0])
    for axis, idx in ((1, np.array(1, np.int64)), (0, np.array([[1, 0, 1]], np.int64))):
        got, want = both(single_op_model("Gather", [z], [idx], axis=axis), [z])
        assert_bit_exact(got[0], want[0])
    got, want = both(single_op_model("Reshape", [z], [np.array([6, -1], np.int64)]), [z])
    assert_bit_exact(got[0], want[0])
    got, want = both(single_op_model("Flatten", [x], axis=1), [x])
    assert_bit_exact(got[0], want[0])


def test_where_greater_cast(cuda_lib):
    x = RNG.standard_normal((1, 128, 10, 10)).astype(np.float32)
    got, want = both(single_op_model("Greater", [x], [np.array([0.1], np.float32)]), [x])
    assert_bit_exact(got[0], want[0])
    cond = RNG.random((1, 1, 10, 10)) > 0.5
    m = single_op_model("Where", [cond, x], [np.array([-1.0], np.float32)])
    got, want = both(m, [cond, x])
    assert_bit_exact(got[0], want[0])
    y = RNG.standard_normal((1, 1, 10, 10)).astype(np.float32)
    m = single_op_model("Where", [cond], [np.array([2.0], np.float32), y])
    got, want = both(m, [cond])
    assert_bit_exact(got[0], want[0])
    i64 = RNG.integers(-1000, 1000, (3, 9)).astype(np.int64)
    for to in (1, 2):
        got, want = both(single_op_model("Cast", [i64], to=to), [i64])
        assert_bit_exact(got[0], want[0])
    got, want = both(single_op_model("Cast", [x], to=0), [x])
    assert_bit_exact(got[0], want[0])


def test_batch_norm(cuda_lib):
    x = RNG.standard_normal((2, 6, 9, 9)).astype(np.float32)
    sc, b, mu = (RNG.standard_normal(6).astype(np.float32) for _ in range(3))
    var = RNG.random(6, dtype=np.float32) + np.float32(0.5)
    m = single_op_model("BatchNormalization", [x], [sc, b, mu, var], epsilon=1e-5)
    got, want = both(m, [x])
    assert_bit_exact(got[0], want[0])


MATMUL_SHAPES = [((4, 8), (8, 3)), ((2, 5, 8), (8, 3)), ((3, 5, 8), (3, 8, 6)), ((1, 2, 5, 8), (1, 2, 8, 6)),
                 ((1, 256), (256, 10)), ((2, 197, 768), (768, 2304)), ((24, 197, 64), (24, 64, 197)),
                 ((24, 197, 197), (24, 197, 64)), ((394, 3072), (3072, 768)), ((130, 70), (70, 129))]


@pytest.mark.parametrize("ashape,bshape", MATMUL_SHAPES)
@pytest.mark.parametrize("gemm_mode", [0, 1, 3])
def test_matmul(cuda_lib, ashape, bshape, gemm_mode):
    a = RNG.standard_normal(ashape).astype(np.float32)
    b = RNG.standard_normal(bshape).astype(np.float32)
    got, want = both(single_op_model("MatMul", [a, b]), [a, b], gemm_mode=gemm_mode)
    k = ashape[-1]
    np.testing.assert_allclose(got[0], want[0], rtol=1e-5, atol=1e-5 * np.sqrt(k))


@pytest.mark.parametrize("gemm_mode", [0, 1, 3])
def test_gemm(cuda_lib, gemm_mode):
    a = RNG.standard_normal((7, 9)).astype(np.float32)
    for ta, ash in ((False, (7, 9)), (True, (9, 7))):
        a = RNG.standard_normal(ash).astype(np.float32)
        for tb, bsh in ((False, (9, 5)), (True, (5, 9))):
            b = RNG.standard_normal(bsh).astype(np.float32)
            for c in (RNG.standard_normal(5).astype(np.float32),
                      RNG.standard_normal((7, 5)).astype(np.float32), None):
                ins = [a, b] + ([c] if c is not None else [])
                for alpha, beta in ((1.0, 1.0), (0.5, 2.0)):
                    m = single_op_model("Gemm", ins, alpha=alpha, beta=beta, trans_a=ta, trans_b=tb)
                    got, want = both(m, ins, gemm_mode=gemm_mode)
                    np.testing.assert_allclose(got[0], want[0], rtol=1e-5, atol=2e-5)
    a = RNG.standard_normal((32, 768)).astype(np.float32)
    w = (0.02 * RNG.standard_normal((1000, 768))).astype(np.float32)
    c = RNG.standard_normal(1000).astype(np.float32)
    m = single_op_model("Gemm", [a], [w, c], alpha=1.0, beta=1.0, trans_a=False, trans_b=True)
    got, want = both(m, [a], gemm_mode=gemm_mode)
    np.testing.assert_allclose(got[0], want[0], rtol=1e-5, atol=2e-5)


CONV_CASES = [(1, 1, 28, 8, 5, 1, 2, 1, True), (2, 4, 15, 6, 3, 2, 1, 1, True), (2, 16, 9, 16, 3, 1, 1, 16, True),
              (2, 16, 9, 16, 3, 1, 1, 16, False), (1, 3, 32, 8, 16, 16, 0, 1, True), (2, 24, 14, 40, 1, 1, 0, 1, True),
              (2, 32, 14, 32, 5, 2, 2, 32, True), (2, 3, 64, 16, 3, 2, 1, 1, False),
              (4, 24, 1, 8, 1, 1, 0, 1, True), (32, 960, 1, 240, 1, 1, 0, 1, True)]   # 1 x 1 planes (squeeze-excite)


@pytest.mark.parametrize("n,c,h,oc,k,s,p,g,with_bias", CONV_CASES)
@pytest.mark.parametrize("gemm_mode", [0, 1, 3])
def test_conv2d(cuda_lib, n, c, h, oc, k, s, p, g, with_bias, gemm_mode):
    x = RNG.standard_normal((n, c, h, h)).astype(np.float32)
    w = RNG.standard_normal((oc, c // g, k, k)).astype(np.float32)
    consts = [w] + ([RNG.standard_normal(oc).astype(np.float32)] if with_bias else [])
    m = single_op_model("Conv2d", [x], consts, kernel_shape=[k, k], strides=[s, s],
                        padding=[p, p, p, p], dilations=[1, 1], group=g, auto_pad="")
    got, want = both(m, [x], gemm_mode=gemm_mode)
    np.testing.assert_allclose(got[0], want[0], rtol=1e-5, atol=1e-5 * np.sqrt(c // g * k * k) * 4)


# Convolutions and batched products whose rhs is stored [K, N]: MN-major tiles in the
# tensor-core kernel. Edges: HW not a multiple of the 32-column box or of the tile width, fewer
# output channels than one 128-row tile, K not a multiple of the 16-float stage, batch-shared A.
MN_CONV_CASES = [(4, 64, 56, 96, 1, 1, 0, "relu"), (3, 40, 28, 72, 1, 1, 0, None), (2, 16, 30, 24, 3, 1, 1, None),
                 (2, 24, 16, 200, 3, 2, 1, "relu"), (16, 72, 14, 24, 1, 1, 0, None), (8, 160, 7, 320, 1, 1, 0, "relu"), (16, 3, 64, 16, 3, 2, 1, "relu")]


@pytest.mark.parametrize("n,c,h,oc,k,s,p,act", MN_CONV_CASES)
def test_conv2d_on_the_tensor_cores(cuda_lib, n, c, h, oc, k, s, p, act):
    from altius_b200.session import CudaSessionBuilder
    x = RNG.standard_normal((n, c, h, h)).astype(np.float32)
    w = (RNG.standard_normal((oc, c, k, k)) / np.sqrt(c * k * k)).astype(np.float32)
    bias = RNG.standard_normal(oc).astype(np.float32)

    def build(g):
        y = g.op("Conv2d", g.add_input("x", x.shape), g.new_init(w), g.new_init(bias), kernel_shape=[k, k],
                 strides=[s, s], padding=[p, p, p, p], dilations=[1, 1], group=1, auto_pad="")
        return [g.op("ReLU", y) if act == "relu" else y]
    m = _chain_model(build)
    sess = CudaSessionBuilder(m).build()
    try:
        assert "gemm_tf32x3_tcgen05" in [e["kind"] for e in sess.schedule()]
        got = sess.run([x])[0]
    finally:
        sess.close()
    want = run_oracle(m, [x])[0]
    xa, wa = np.abs(x), np.abs(w)
    import torch
    bound = torch.nn.functional.conv2d(torch.from_numpy(xa), torch.from_numpy(wa), torch.from_numpy(np.abs(bias)),
                                       stride=s, padding=p).numpy()
    assert got.shape == want.shape
    assert (np.abs(got - want) <= 1e-5 * np.abs(want) + 5e-6 * bound).all()


@pytest.mark.parametrize("ashape,bshape", [((8, 200, 72), (8, 72, 136)), ((24, 197, 200), (24, 200, 64)),
                                           ((1, 3, 130, 48), (1, 3, 48, 260))])
def test_batched_matmul_of_two_activations_on_the_tensor_cores(cuda_lib, ashape, bshape):
    from altius_b200.session import CudaSessionBuilder
    a = RNG.standard_normal(ashape).astype(np.float32)
    b = RNG.standard_normal(bshape).astype(np.float32)
    m = single_op_model("MatMul", [a, b])
    sess = CudaSessionBuilder(m).build()
    try:
        assert [e["kind"] for e in sess.schedule()] == ["gemm_tf32x3_tcgen05"]
        got = sess.run([a, b])[0]
    finally:
        sess.close()
    want = run_oracle(m, [a, b])[0]
    assert (np.abs(got - want) <= 1e-5 * np.abs(want) + 5e-6 * (np.abs(a) @ np.abs(b))).all()


def test_conv2d_same_upper(cuda_lib):
    x = RNG.standard_normal((1, 1, 28, 28)).astype(np.float32)
    w = RNG.standard_normal((8, 1, 5, 5)).astype(np.float32)
    m = single_op_model("Conv2d", [x], [w], kernel_shape=[5, 5], strides=[1, 1], padding=[],
                        dilations=[1, 1], group=1, auto_pad="SAME_UPPER")
    got, want = both(m, [x])
    assert got[0].shape == (1, 8, 28, 28)
    np.testing.assert_allclose(got[0], want[0], rtol=1e-5, atol=1e-5)   # ops_conv.rs:41-43


# ---- tensor-core (tcgen05, 3xTF32) path: needs a K-major rhs -------------------------
TC_SHAPES = [((2, 197, 768), (768, 2304)), ((394, 3072), (3072, 768)), ((1000, 768), (768, 768)),
             ((3, 130, 100), (100, 72)), ((257, 36), (36, 513)), ((128, 32), (32, 64)), ((640, 8), (8, 256))]


@pytest.mark.parametrize("ashape,bshape", TC_SHAPES)
@pytest.mark.parametrize("gemm_mode", [0, 1, 3])
def test_matmul_constant_weight(cuda_lib, ashape, bshape, gemm_mode):
    a = RNG.standard_normal(ashape).astype(np.float32)
    w = RNG.standard_normal(bshape).astype(np.float32)
    m = single_op_model("MatMul", [a], [w])
    got, want = both(m, [a], gemm_mode=gemm_mode)
    # 3xTF32 on the tensor cores: the fp32 accumulator in tensor memory truncates
    # after every MMA step, so the error is bounded relative to sum |a||b| (measured
    # rms 6e-7, max 3e-6 at K = 3072) rather than to the result.
    bound = 1e-5 * np.abs(want[0]) + 5e-6 * (np.abs(a).reshape(-1, ashape[-1]) @ np.abs(w)).reshape(want[0].shape)
    assert (np.abs(got[0] - want[0]) <= bound).all()


def test_fp16_split_falls_back_to_tf32_when_an_activation_is_out_of_range(cuda_lib):
    """gemm_mode 0 multiplies constant weights with fp16-split operands; an activation
    beyond 65504 is detected on the device and the session switches, for good, to a
    second plan on the 3xTF32 path and repeats the run there."""
    from altius_b200.session import CudaSessionBuilder
    a = RNG.standard_normal((128, 256)).astype(np.float32)
    w = RNG.standard_normal((256, 256)).astype(np.float32)
    m = single_op_model("MatMul", [a], [w])
    sess = CudaSessionBuilder(m).build()
    try:
        kinds = lambda: [e["kind"] for e in sess.schedule()]
        assert kinds() == ["gemm_f16x3_tcgen05"]
        big = np.where(np.arange(a.size).reshape(a.shape) == 901, 1e6, a).astype(np.float32)
        # in range, out of range (switches), in range again (the switch is permanent)
        for x, kind_after in ((a, "gemm_f16x3_tcgen05"), (big, "gemm_tf32x3_tcgen05"), (a, "gemm_tf32x3_tcgen05")):
            want = run_oracle(m, [x])[0]
            got = sess.run([x])[0]
            bound = 1e-5 * np.abs(want) + 5e-6 * (np.abs(x) @ np.abs(w))
            assert (np.abs(got - want) <= bound).all()
            assert kinds() == [kind_after]
    finally:
        sess.close()


@pytest.mark.parametrize("wscale", [1e5, 1.0, 1e-5, 1e-7, 1e-9, 1e-20])
def test_fp16_split_scales_weights_of_any_magnitude(cuda_lib, wscale):
    """Constant weights are split after scaling by a power of two that brings their largest
    magnitude to about 2^13, and the epilogue undoes it: weights far outside the fp16 range
    (either way) lose nothing. Infinite weights are the one case left for the 3xTF32 plan."""
    from altius_b200.session import CudaSessionBuilder
    a = RNG.standard_normal((128, 256)).astype(np.float32)
    w = (wscale * RNG.standard_normal((256, 256))).astype(np.float32)
    m = single_op_model("MatMul", [a], [w])
    sess = CudaSessionBuilder(m).build()
    try:
        assert [e["kind"] for e in sess.schedule()] == ["gemm_f16x3_tcgen05"]
        want = run_oracle(m, [a])[0]
        got = sess.run([a])[0]
        assert (np.abs(got - want) <= 1e-5 * np.abs(want) + 5e-6 * (np.abs(a) @ np.abs(w))).all()
    finally:
        sess.close()
    w[5, 17] = np.inf
    m = single_op_model("MatMul", [a], [w])
    sess = CudaSessionBuilder(m).build()
    try:
        assert [e["kind"] for e in sess.schedule()] == ["gemm_tf32x3_tcgen05"]
    finally:
        sess.close()


@pytest.mark.parametrize("ascale", [1e-5, 1e-7, 1e-9])
def test_fp16_split_falls_back_when_the_activations_are_all_tiny(cuda_lib, ascale):
    """Below 2^-14 the fp16 split of an activation loses relative precision (absolute floor
    2^-36). A region of non-zero activations none of which reaches 2^-14 is reported like an
    overflow, and the session repeats the run on its 3xTF32 plan."""
    from altius_b200.session import CudaSessionBuilder
    a = (ascale * RNG.standard_normal((512, 256))).astype(np.float32)
    w = RNG.standard_normal((256, 256)).astype(np.float32)
    m = single_op_model("MatMul", [a], [w])
    sess = CudaSessionBuilder(m).build()
    try:
        want = run_oracle(m, [a])[0]
        got = sess.run([a])[0]
        assert (np.abs(got - want) <= 1e-5 * np.abs(want) + 5e-6 * (np.abs(a) @ np.abs(w))).all()
        assert [e["kind"] for e in sess.schedule()] == ["gemm_tf32x3_tcgen05"]
    finally:
        sess.close()


@pytest.mark.parametrize("case", ["unit", "up_to_200", "small_1e-2", "rows_of_mixed_size", "one_beyond_255", "all_tiny"])
def test_presplit_gemm_on_the_fixed_scale(cuda_lib, case):
    """The CTA-pair kernel takes A as fp16 halves on the fixed scale 2^8 (full precision for
    |a| in [2^-11, 255]) and keeps one accumulator. In range: the usual bound. An element beyond
    255, or a tile of A with nothing as large as 2^-11, is reported by the kernel that writes
    the halves and the run is repeated on the 3xTF32 plan."""
    from altius_b200.session import CudaSessionBuilder
    rng = np.random.default_rng(99)
    a = rng.standard_normal((6304, 768)).astype(np.float32)
    if case == "up_to_200":
        a = (a * (200.0 / np.abs(a).max())).astype(np.float32)
    elif case == "small_1e-2":
        a = (a * 1e-2).astype(np.float32)
    elif case == "rows_of_mixed_size":
        a = (a * np.exp2(-(np.arange(6304) % 10)).astype(np.float32)[:, None]).astype(np.float32)   # rows down to 2^-9
    elif case == "one_beyond_255":
        a[4000, 17] = 300.0
    elif case == "all_tiny":
        a = (a * 1e-5).astype(np.float32)
    w = (0.05 * rng.standard_normal((768, 768))).astype(np.float32)
    b = rng.standard_normal(768).astype(np.float32) * np.float32(1e-3 if case in ("small_1e-2", "all_tiny") else 1.0)

    def build(g):
        return [g.op("Add", g.op("MatMul", g.add_input("a", a.shape), g.new_init(w)), g.new_init(b))]
    m = _chain_model(build)
    sess = CudaSessionBuilder(m).build()
    try:
        assert [e["kind"] for e in sess.schedule()] == ["act_f16_split", "gemm_f16x3_pair_tcgen05"]
        got = sess.run([a])[0]
        falls_back = case in ("one_beyond_255", "all_tiny")
        kinds = [e["kind"] for e in sess.schedule()]
        assert ("gemm_tf32x3_tcgen05" in kinds) == falls_back, kinds
    finally:
        sess.close()
    want = run_oracle(m, [a], sgemm="openblas")[0]
    bound = 1e-5 * np.abs(want) + 5e-6 * (np.abs(a) @ np.abs(w) + np.abs(b))
    assert (np.abs(got - want) <= bound).all(), float((np.abs(got - want) / bound).max())


@pytest.mark.parametrize("ashape,bshape", [((2, 197, 768), (768, 2304)), ((394, 3072), (3072, 768)), ((1000, 768), (768, 768)),
                                            ((300, 100), (100, 72)), ((257, 36), (36, 513)), ((5000, 64), (64, 256)),
                                            ((6304, 768), (768, 768))])
@pytest.mark.parametrize("pairs", [1, 2])
def test_matmul_on_cta_pairs(cuda_lib, ashape, bshape, pairs):
    """The fp16-split GEMM on clusters of two CTAs (tcgen05 .cta_group::2; each CTA stages its
    rows of A and half of the weight tile) computes the same products as the one-CTA kernel;
    only the K-slicing of tail tiles (and with it the order of a few additions) can differ.
    pairs 1: each CTA splits its rows of A in registers; pairs 2: A arrives as fp16 hi / lo
    halves written by a kernel in front, and every tile of a stage comes by TMA."""
    a = RNG.standard_normal(ashape).astype(np.float32)
    w = RNG.standard_normal(bshape).astype(np.float32)
    m = single_op_model("MatMul", [a], [w])
    want = run_oracle(m, [a])[0]
    got = run_cuda(m, [a], pairs=pairs)[0]
    bound = 1e-5 * np.abs(want) + 5e-6 * (np.abs(a).reshape(-1, ashape[-1]) @ np.abs(w)).reshape(want.shape)
    assert (np.abs(got - want) <= bound).all()
    single = run_cuda(m, [a], pairs=3)[0]
    assert (np.abs(got - single) <= 2e-6 * (np.abs(a).reshape(-1, ashape[-1]) @ np.abs(w)).reshape(want.shape)).all()


@pytest.mark.parametrize("pairs", [1, 2])
def test_cta_pairs_in_a_model_with_epilogues_and_range_fallback(cuda_lib, pairs):
    from altius_b200 import configs
    from altius_b200.session import CudaSessionBuilder
    model, feeds = configs.vit_base_16(batch=2, depth=2)
    x = next(iter(feeds.values()))
    want = run_cuda(model, [x], pairs=3)[0]
    sess = CudaSessionBuilder(model).with_gemm_pairs(pairs).build()
    try:
        got = sess.run([x])[0]
        assert np.abs(got - want).max() <= 1e-4 and (got.argmax(-1) == want.argmax(-1)).all()
        big = x.copy()
        big[0, 0, 0, 0] = 1e9            # beyond fp16 after the patch embedding: detected, 3xTF32 plan takes over
        out = sess.run([big])[0]
        assert np.isfinite(out).all()
        assert any(e["kind"] == "gemm_tf32x3_tcgen05" for e in sess.schedule())
    finally:
        sess.close()


def test_matmul_tf32x1_is_looser_but_close(cuda_lib):
    a = RNG.standard_normal((512, 768)).astype(np.float32)
    w = RNG.standard_normal((768, 512)).astype(np.float32)
    m = single_op_model("MatMul", [a], [w])
    got, want = both(m, [a], gemm_mode=2)
    err = np.abs(got[0] - want[0]).max()
    assert 1e-4 < err < 0.2          # one TF32 product per term: ~1e-3 relative


def _chain_model(build):
    from altius_b200 import ir
    g = ir.Graph()
    outs = build(g)
    for i, o in enumerate(outs):
        g.values[o].name = f"out{i}"
        g.outputs.append(o)
    return ir.Model(g, 13)


def test_qk_transpose_matmul_scale_softmax(cuda_lib):
    q = RNG.standard_normal((24, 197, 64)).astype(np.float32)
    k = RNG.standard_normal((24, 197, 64)).astype(np.float32)

    def build(g):
        qi, ki = g.add_input("q", q.shape), g.add_input("k", k.shape)
        kt = g.op("Transpose", ki, perm=[0, 2, 1])
        s = g.op("MatMul", qi, kt)
        s = g.op("Mul", s, g.new_init(np.array([0.125], np.float32)))
        return [g.op("Softmax", s, axis=-1)]
    m = _chain_model(build)
    for mode in (0, 1):
        got, want = both(m, [q, k], gemm_mode=mode)
        np.testing.assert_allclose(got[0], want[0], rtol=2e-5, atol=1e-7)


def test_linear_gelu_residual_epilogue(cuda_lib):
    x = RNG.standard_normal((4, 197, 768)).astype(np.float32)
    r = RNG.standard_normal((4, 197, 384)).astype(np.float32)
    w = (0.05 * RNG.standard_normal((768, 384))).astype(np.float32)
    b = RNG.standard_normal(384).astype(np.float32)

    def build(g):
        xi, ri = g.add_input("x", x.shape), g.add_input("r", r.shape)
        h = g.op("MatMul", xi, g.new_init(w))
        h = g.op("Add", h, g.new_init(b))
        h = g.op("Gelu", h)
        return [g.op("Add", ri, h)]
    m = _chain_model(build)
    bound = 5e-6 * (np.abs(x).reshape(-1, 768) @ np.abs(w) + np.abs(b)).reshape(4, 197, 384)
    for opts in (dict(gemm_mode=0), dict(gemm_mode=1), dict(gemm_mode=3), dict(gemm_mode=0, fuse=False)):
        got, want = both(m, [x, r], **opts)
        assert (np.abs(got[0] - want[0]) <= 1e-5 * np.abs(want[0]) + bound).all()


def test_gelu_in_the_gemm_epilogue_equals_the_gelu_kernel_bit_for_bit(cuda_lib):
    # The epilogue evaluates Gelu on pairs with packed fp32 instructions and its own
    # division sequence; the stand-alone kernel uses the scalar formulas. Same MatMul
    # kernel in both sessions, so any difference comes from the activation.
    rng = np.random.default_rng(7)
    x = rng.standard_normal((1024, 64)).astype(np.float32)
    x *= np.exp2(np.arange(1024) % 34 - 30).astype(np.float32)[:, None]   # pre-activations from 1e-9 to 100
    w = (0.3 * rng.standard_normal((64, 512))).astype(np.float32)
    b = np.zeros(512, np.float32)

    def build(g):
        h = g.op("MatMul", g.add_input("x", x.shape), g.new_init(w))
        return [g.op("Gelu", g.op("Add", h, g.new_init(b)))]
    m = _chain_model(build)
    fused = run_cuda(m, [x], gemm_mode=0)[0]
    plain = run_cuda(m, [x], gemm_mode=0, fuse=False)[0]
    assert np.abs(plain).max() > 50 and (np.abs(plain) < 1e-6).any()
    assert_bit_exact(fused, plain)


def test_gemm_transb_constant_weight(cuda_lib):
    a = RNG.standard_normal((300, 1280)).astype(np.float32)
    w = (0.02 * RNG.standard_normal((1000, 1280))).astype(np.float32)
    c = RNG.standard_normal(1000).astype(np.float32)
    m = single_op_model("Gemm", [a], [w, c], alpha=1.0, beta=1.0, trans_a=False, trans_b=True)
    for mode in (0, 1, 3):
        got, want = both(m, [a], gemm_mode=mode)
        bound = 1e-5 * np.abs(want[0]) + 5e-6 * (np.abs(a) @ np.abs(w.T) + np.abs(c))
        assert (np.abs(got[0] - want[0]) <= bound).all()


@pytest.mark.parametrize("scale_op", ["Mul", "Div"])
@pytest.mark.parametrize("B,T,H", [(2, 197, 12), (3, 198, 6), (1, 33, 2), (2, 256, 1), (1, 7, 3), (2, 100, 2), (1, 65, 1),
                                   (1, 208, 2), (1, 209, 1), (1, 129, 2), (2, 128, 1)])
def test_fused_attention_core(cuda_lib, B, T, H, scale_op):
    """Split -> head reshapes/transposes -> Q K^T -> scale -> Softmax -> P V -> merge heads,
    lowered to one kernel when fusion is on; compared with the oracle running the chain."""
    hd, D = 64, 64 * H
    qkv = RNG.standard_normal((B, T, 3 * D)).astype(np.float32)

    def build(g):
        x = g.add_input("qkv", qkv.shape)
        q, k, v = g.add_node("Split", [x, g.new_init(np.array([D, D, D], np.int64))], 3, axis=2)

        def heads(t):
            t = g.op("Reshape", t, g.new_init(np.array([B, T, H, hd], np.int64)))
            t = g.op("Transpose", t, perm=[0, 2, 1, 3])
            return g.op("Reshape", t, g.new_init(np.array([B * H, T, hd], np.int64)))
        q, k, v = heads(q), heads(k), heads(v)
        s = g.op("MatMul", q, g.op("Transpose", k, perm=[0, 2, 1]))
        s = g.op(scale_op, s, g.new_init(np.array([0.125 if scale_op == "Mul" else 8.0], np.float32)))
        p = g.op("Softmax", s, axis=-1)
        o = g.op("MatMul", p, v)
        o = g.op("Reshape", o, g.new_init(np.array([B, H, T, hd], np.int64)))
        o = g.op("Transpose", o, perm=[0, 2, 1, 3])
        return [g.op("Reshape", o, g.new_init(np.array([B, T, D], np.int64)))]
    m = _chain_model(build)
    from altius_b200.session import CudaSessionBuilder
    sess = CudaSessionBuilder(m).build()
    tc = T > 64   # the tcgen05 kernel takes 64 < T <= 256; shorter sequences stay on the CUDA cores
    assert [e["kind"] for e in sess.schedule()] == ["attention_tcgen05" if tc else "attention_fused"]
    sess.close()
    want = run_oracle(m, [qkv])[0]
    got = run_cuda(m, [qkv])[0]
    if tc:
        # 3xTF32 products with the tensor memory accumulator: a score is off by at most
        # 5e-6 * sum|q||k| * scale, which moves every softmax weight by that relative amount
        # (numerator and denominator), and the second product adds 5e-6 * sum p|v|.
        x = qkv.astype(np.float64).reshape(B, T, 3, H, hd).transpose(2, 0, 3, 1, 4)
        q64, k64, v64 = x[0], x[1], x[2]
        s64 = np.einsum("bhid,bhjd->bhij", q64, k64) * 0.125
        err_s = 5e-6 * 0.125 * np.einsum("bhid,bhjd->bhij", np.abs(q64), np.abs(k64)).max(axis=-1, keepdims=True)
        p64 = np.exp(s64 - s64.max(axis=-1, keepdims=True))
        p64 /= p64.sum(axis=-1, keepdims=True)
        pv = np.einsum("bhij,bhjd->bhid", p64, np.abs(v64))
        bound = ((2 * err_s + 5e-6) * pv).transpose(0, 2, 1, 3).reshape(B, T, D) + 1e-5 * np.abs(want) + 1e-6
        assert (np.abs(got.astype(np.float64) - want) <= bound).all(), float(np.abs(got - want).max())
        got = run_cuda(m, [qkv], gemm_mode=1)[0]   # exact fp32 chains: the CUDA-core fused kernel
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-6)
    unfused = run_cuda(m, [qkv], fuse=False, gemm_mode=1)[0]
    np.testing.assert_allclose(unfused, want, rtol=1e-5, atol=1e-6)


def _projection_attention_model(B, T, H, scale_op="Mul", w_scale=0.05, with_out_proj=True):
    """x [B, T, D] -> MatMul + bias to [B, T, 3D] -> the attention core -> (MatMul): the shape
    of a transformer layer between its LayerNormalization and its residual Add."""
    hd, D = 64, 64 * H
    rng = np.random.default_rng(1234 + T + H)
    w_qkv = (w_scale * rng.standard_normal((D, 3 * D))).astype(np.float32)
    b_qkv = (0.1 * rng.standard_normal(3 * D)).astype(np.float32)
    w_o = (0.05 * rng.standard_normal((D, D))).astype(np.float32)

    def build(g):
        x = g.add_input("x", (B, T, D))
        i64 = lambda v: g.new_init(np.asarray(v, np.int64))
        qkv = g.op("Add", g.op("MatMul", x, g.new_init(w_qkv)), g.new_init(b_qkv))
        q, k, v = g.add_node("Split", [qkv, i64([D, D, D])], 3, axis=2)

        def heads(t):
            t = g.op("Reshape", t, i64([B, T, H, hd]))
            t = g.op("Transpose", t, perm=[0, 2, 1, 3])
            return g.op("Reshape", t, i64([B * H, T, hd]))
        q, k, v = heads(q), heads(k), heads(v)
        s_ = g.op("MatMul", q, g.op("Transpose", k, perm=[0, 2, 1]))
        s_ = g.op(scale_op, s_, g.new_init(np.array([hd ** -0.5 if scale_op == "Mul" else hd ** 0.5], np.float32)))
        o = g.op("MatMul", g.op("Softmax", s_, axis=-1), v)
        o = g.op("Reshape", o, i64([B, H, T, hd]))
        o = g.op("Transpose", o, perm=[0, 2, 1, 3])
        o = g.op("Reshape", o, i64([B, T, D]))
        return [g.op("MatMul", o, g.new_init(w_o)) if with_out_proj else o]
    return _chain_model(build)


@pytest.mark.parametrize("B,T,H,scale_op,out_proj", [(32, 197, 12, "Mul", True), (32, 197, 12, "Div", False),
                                                      (64, 198, 6, "Mul", True), (48, 100, 4, "Mul", False),
                                                      (40, 128, 4, "Div", True), (33, 208, 4, "Mul", False),
                                                      (37, 65, 4, "Mul", True), (44, 129, 4, "Mul", False),
                                                      # seven and eight units per CTA: every barrier wraps its parity
                                                      (128, 100, 8, "Mul", False), (96, 197, 12, "Mul", False)])
def test_attention_fed_by_tma_from_the_projection_gemm(cuda_lib, B, T, H, scale_op, out_proj):
    """The projection GEMM writes [B, T, 3D] as fp16 halves on the fixed scale and the attention
    kernel takes Q, K and V from there by TMA (no fp32 copy of the projection exists): checked
    against the oracle, and against the same session with that path switched off."""
    from altius_b200.session import CudaSessionBuilder
    D = 64 * H
    m = _projection_attention_model(B, T, H, scale_op, with_out_proj=out_proj)
    x = np.random.default_rng(T).standard_normal((B, T, D)).astype(np.float32)
    sess = CudaSessionBuilder(m).build()
    try:
        kinds = [e["kind"] for e in sess.schedule() if e["kind"] != "act_f16_split"]
        assert kinds[:2] == ["gemm_f16x3_pair_tcgen05", "attention_tma_tcgen05"], kinds
        got = sess.run([x])[0]
    finally:
        sess.close()
    want = run_oracle(m, [x], sgemm="openblas")[0]
    assert np.isfinite(got).all()
    assert (np.abs(got - want) <= _split_chain_bound(want, 0.3)).all(), float(np.abs(got - want).max())
    os.environ["ALTIUS_CUDA_NO_ATTENTION_TMA"] = "1"
    try:
        sess = CudaSessionBuilder(m).build()
        try:
            assert "attention_tcgen05" in [e["kind"] for e in sess.schedule()]
            other = sess.run([x])[0]
        finally:
            sess.close()
    finally:
        del os.environ["ALTIUS_CUDA_NO_ATTENTION_TMA"]
    assert (np.abs(got - other) <= _split_chain_bound(want, 0.3)).all()


@pytest.mark.parametrize("case", ["beyond_the_fixed_scale", "all_tiny"])
def test_attention_fed_by_tma_falls_back_when_the_projection_leaves_its_range(cuda_lib, case):
    """The fixed scale holds |x| <= 255 with full precision down to 2^-11: a projection beyond
    that (or one whose elements are all tiny) is reported by the GEMM that writes it, and the run
    is repeated on the 3xTF32 plan."""
    B, T, H = 32, 197, 4
    m = _projection_attention_model(B, T, H, w_scale=40.0 if case == "beyond_the_fixed_scale" else 1e-7,
                                    with_out_proj=False)
    rng = np.random.default_rng(5)
    x = rng.standard_normal((B, T, 64 * H)).astype(np.float32)
    if case == "all_tiny":
        for i in list(m.graph.inits):
            if m.graph.inits[i].shape == (3 * 64 * H,):
                m.graph.inits[i] = (1e-6 * m.graph.inits[i]).astype(np.float32)     # the bias too
    got = run_cuda(m, [x])[0]
    want = run_oracle(m, [x], sgemm="openblas")[0]
    assert np.isfinite(got).all()
    np.testing.assert_allclose(got, want, rtol=2e-4, atol=2e-4 * np.abs(want).max())


# ---- Resize / Expand (the interpreter's restricted patterns, session.rs:299-323, 1057-1132) ----
@pytest.mark.parametrize("mode", ["nearest", "linear"])
@pytest.mark.parametrize("ishape,oshape", [((2, 3, 7, 7), (2, 3, 14, 14)), ((1, 5, 16, 16), (1, 5, 8, 8)),
                                            ((2, 2, 9, 9), (2, 2, 21, 21)), ((1, 1, 4, 6), (1, 1, 8, 12))])
def test_resize_with_sizes(cuda_lib, mode, ishape, oshape):
    x = RNG.standard_normal(ishape).astype(np.float32)
    roi = np.zeros(0, np.float32)
    scales = np.zeros(0, np.float32)
    m = single_op_model("Resize", [x], [roi, scales, np.array(oshape, np.int64)], mode=mode,
                        coordinate_transformation_mode="half_pixel", nearest_mode="round_prefer_floor")
    got, want = both(m, [x])
    assert want[0].shape == oshape
    assert_bit_exact(got[0], want[0])


def test_resize_with_scales_nearest_floor(cuda_lib):
    x = RNG.standard_normal((2, 4, 10, 10)).astype(np.float32)
    m = single_op_model("Resize", [x], [np.zeros(0, np.float32), np.array([1, 1, 2, 2], np.float32)], mode="nearest",
                        coordinate_transformation_mode="asymmetric", nearest_mode="floor")
    got, want = both(m, [x])
    assert want[0].shape == (2, 4, 20, 20)
    assert_bit_exact(got[0], want[0])
    assert_bit_exact(got[0], x.repeat(2, axis=2).repeat(2, axis=3))


@pytest.mark.parametrize("ishape,oshape,dtype", [((1, 1, 1, 9), (1, 1, 5, 9), np.int64), ((1, 1, 1, 4), (2, 3, 5, 4), np.int64),
                                                  ((3, 1, 8), (2, 3, 6, 8), np.float32), ((1,), (4, 7), np.float32)])
def test_expand(cuda_lib, ishape, oshape, dtype):
    x = (RNG.standard_normal(ishape) * 100).astype(dtype)
    m = single_op_model("Expand", [x], [np.array(oshape, np.int64)])
    got, want = both(m, [x])
    assert want[0].shape == oshape and want[0].dtype == dtype
    assert_bit_exact(got[0], want[0])
    assert_bit_exact(got[0], np.broadcast_to(x, oshape))


# ---- results written split by their producers for the CTA-pair GEMM that consumes them ------
def _split_chain_bound(want, scale=1.0):
    return 2e-5 * np.abs(want) + 2e-4 * scale


def test_layer_norm_writes_the_split_operand_of_the_next_gemm(cuda_lib):
    """LayerNormalization -> MatMul at the benchmark's row count: the GEMM runs on CTA pairs and
    takes its A operand as fp16 hi / lo halves that the LayerNormalization kernel writes itself
    (no fp32 copy of the normalised rows exists)."""
    from altius_b200.session import CudaSessionBuilder
    x = RNG.standard_normal((32, 197, 768)).astype(np.float32)
    gam = (1 + 0.02 * RNG.standard_normal(768)).astype(np.float32)
    bet = (0.02 * RNG.standard_normal(768)).astype(np.float32)
    w = (0.02 * RNG.standard_normal((768, 2304))).astype(np.float32)

    def build(g):
        xi = g.add_input("x", x.shape)
        h = g.op("LayerNormalization", xi, g.new_init(gam), g.new_init(bet), axis=-1, epsilon=1e-6, stash_type=1)
        return [g.op("MatMul", h, g.new_init(w))]
    m = _chain_model(build)
    sess = CudaSessionBuilder(m).build()
    try:
        assert [e["kind"] for e in sess.schedule()] == ["layer_norm", "gemm_f16x3_pair_tcgen05"]
        got = sess.run([x])[0]
    finally:
        sess.close()
    want = run_oracle(m, [x], sgemm="openblas")[0]
    assert (np.abs(got - want) <= _split_chain_bound(want)).all()


def test_gemm_epilogue_writes_the_split_operand_of_the_next_gemm(cuda_lib):
    """MatMul -> Add -> Gelu -> MatMul -> Add at the benchmark's row count: the first GEMM's
    epilogue (and the fix-up kernel of its K-sliced tail tiles) writes the Gelu result only as
    fp16 hi / lo halves, which the second GEMM takes by TMA."""
    from altius_b200.session import CudaSessionBuilder
    x = RNG.standard_normal((6304, 768)).astype(np.float32)
    w1 = (0.02 * RNG.standard_normal((768, 3072))).astype(np.float32)
    b1 = (0.02 * RNG.standard_normal(3072)).astype(np.float32)
    w2 = (0.02 * RNG.standard_normal((3072, 768))).astype(np.float32)
    b2 = (0.02 * RNG.standard_normal(768)).astype(np.float32)

    def build(g):
        xi = g.add_input("x", x.shape)
        h = g.op("Gelu", g.op("Add", g.op("MatMul", xi, g.new_init(w1)), g.new_init(b1)))
        return [g.op("Add", g.op("MatMul", h, g.new_init(w2)), g.new_init(b2))]
    m = _chain_model(build)
    sess = CudaSessionBuilder(m).build()
    try:
        assert [e["kind"] for e in sess.schedule()] == ["act_f16_split", "gemm_f16x3_pair_tcgen05", "gemm_f16x3_pair_tcgen05"]
        got = sess.run([x])[0]
    finally:
        sess.close()
    want = run_oracle(m, [x], sgemm="openblas")[0]
    assert (np.abs(got - want) <= _split_chain_bound(want)).all()


def test_attention_writes_the_split_operand_of_the_projection(cuda_lib):
    from altius_b200.session import CudaSessionBuilder
    B, T, H, hd = 32, 197, 12, 64
    D = H * hd
    qkv = RNG.standard_normal((B, T, 3 * D)).astype(np.float32)
    w = (0.02 * RNG.standard_normal((D, D))).astype(np.float32)

    def build(g):
        x = g.add_input("qkv", qkv.shape)
        i64 = lambda v: g.new_init(np.asarray(v, np.int64))
        q, k, v = g.add_node("Split", [x, i64([D, D, D])], 3, axis=2)

        def heads(t):
            t = g.op("Reshape", t, i64([B, T, H, hd]))
            t = g.op("Transpose", t, perm=[0, 2, 1, 3])
            return g.op("Reshape", t, i64([B * H, T, hd]))
        q, k, v = heads(q), heads(k), heads(v)
        s_ = g.op("MatMul", q, g.op("Transpose", k, perm=[0, 2, 1]))
        s_ = g.op("Mul", s_, g.new_init(np.array([hd ** -0.5], np.float32)))
        o = g.op("MatMul", g.op("Softmax", s_, axis=-1), v)
        o = g.op("Reshape", o, i64([B, H, T, hd]))
        o = g.op("Transpose", o, perm=[0, 2, 1, 3])
        o = g.op("Reshape", o, i64([B, T, D]))
        return [g.op("MatMul", o, g.new_init(w))]
    m = _chain_model(build)
    sess = CudaSessionBuilder(m).build()
    try:
        assert [e["kind"] for e in sess.schedule()] == ["attention_tcgen05", "gemm_f16x3_pair_tcgen05"]
        got = sess.run([qkv])[0]
    finally:
        sess.close()
    want = run_oracle(m, [qkv], sgemm="openblas")[0]
    assert (np.abs(got - want) <= _split_chain_bound(want, 0.3)).all()


# ---- aliases and host-folded nodes (Squeeze / Unsqueeze / Identity / Shape) --------------------
@pytest.mark.parametrize("opset", [11, 13])
def test_squeeze_unsqueeze_identity_shape_nodes(cuda_lib, opset):
    """Unsqueeze -> ReLU -> Squeeze -> Identity -> Flatten -> Reshape(shape = Shape(x)) -> Add:
    the four alias operators and a Shape node evaluated on the host, with the axes as
    attributes (opset 11) and as inputs (opset 13)."""
    from altius_b200 import ir
    x = RNG.standard_normal((2, 3, 4)).astype(np.float32)
    g = ir.Graph()
    xi = g.add_input("x", x.shape)
    if opset >= 13:
        ax = lambda v: [g.new_init(np.asarray(v, np.int64))]
        u = g.op("Unsqueeze", xi, *ax([1]))
        r = g.op("ReLU", u)
        sq = g.op("Squeeze", r, *ax([1]))
    else:
        u = g.op("Unsqueeze", xi, axes=[1])
        r = g.op("ReLU", u)
        sq = g.op("Squeeze", r, axes=[1])
    idn = g.op("Identity", sq)
    flat = g.op("Flatten", idn, axis=1)
    back = g.op("Reshape", flat, g.op("Shape", xi))
    out = g.op("Add", back, xi)
    g.outputs += [out, u]
    m = ir.Model(g, opset)
    got, want = both(m, [x])
    assert got[0].shape == (2, 3, 4) and got[1].shape == (2, 1, 3, 4)
    assert_bit_exact(got[0], want[0])
    assert_bit_exact(got[1], want[1])
    assert_bit_exact(got[0], np.maximum(x, 0) + x)


def test_shape_node_as_a_graph_output_is_refused_or_right(cuda_lib):
    """Shape with start / end attributes is what the reference's shape inference asserts against."""
    from altius_b200 import ir
    from altius_b200.session import CudaSessionBuilder, SessionError
    g = ir.Graph()
    xi = g.add_input("x", (2, 3))
    g.outputs.append(g.op("Reshape", xi, g.op("Shape", xi, start=1)))
    with pytest.raises(SessionError, match="Shape: start / end"):
        CudaSessionBuilder(ir.Model(g, 15)).with_plan_only(True).build()


# ---- general broadcasting of Where / Greater, every Cast pair (beyond the interpreter's patterns) ----
@pytest.mark.parametrize("cshape,xshape,yshape", [((4, 1, 5), (1, 3, 5), (4, 3, 1)), ((3, 5), (2, 3, 5), (1,)),
                                                   ((2, 1, 1, 7), (2, 3, 4, 7), (3, 1, 7)), ((6,), (6,), (6,))])
def test_where_general_broadcast_bit_exact(cuda_lib, cshape, xshape, yshape):
    cond = RNG.random(cshape) > 0.5
    x = RNG.standard_normal(xshape).astype(np.float32)
    y = RNG.standard_normal(yshape).astype(np.float32)
    m = single_op_model("Where", [cond, x, y])
    got, want = both(m, [cond, x, y])
    assert_bit_exact(got[0], want[0])
    assert_bit_exact(got[0], np.where(cond, x, y))


@pytest.mark.parametrize("xshape,yshape", [((4, 3, 5), (3, 1)), ((2, 7), (2, 7)), ((5,), (3, 1, 5))])
def test_greater_general_broadcast(cuda_lib, xshape, yshape):
    x = RNG.integers(-2, 3, xshape).astype(np.float32)
    y = RNG.integers(-2, 3, yshape).astype(np.float32)
    m = single_op_model("Greater", [x, y])
    got, want = both(m, [x, y])
    assert got[0].dtype == np.bool_ and np.array_equal(got[0], want[0]) and np.array_equal(got[0], x > y)


def test_cast_every_pair(cuda_lib):
    from altius_b200 import ir
    src = {ir.BOOL: np.array([True, False, True, True]), ir.F32: np.array([-2.7, 0.0, 3.9, 1e9], np.float32),
           ir.I32: np.array([-3, 0, 7, 2 ** 30], np.int32), ir.I64: np.array([-3, 0, 7, 2 ** 40], np.int64)}
    for frm, x in src.items():
        for to in (ir.BOOL, ir.F32, ir.I32, ir.I64):
            if frm == to or (frm == ir.I64 and to == ir.I32) or (frm == ir.F32 and to in (ir.I32,) ):
                # out-of-range conversions are undefined in C; keep the values representable
                x2 = np.clip(x, -1000, 1000).astype(x.dtype) if frm != ir.BOOL else x
            else:
                x2 = x
            m = single_op_model("Cast", [x2], to=to)
            got, want = both(m, [x2])
            assert got[0].dtype == want[0].dtype and np.array_equal(got[0], want[0]), (frm, to)


# ---- the two fusions of the metric's list that were still open ----------------------------------
def test_scale_mask_softmax_is_one_kernel(cuda_lib):
    """S * 0.125 -> Where(causal mask [1,1,T,T], ., -1e9) -> Softmax: one kernel; the same
    bits as the three kernels (a selection is exact), within 1e-5 of the oracle."""
    from altius_b200.session import CudaSessionBuilder
    B, H, T = 3, 4, 197
    sc = RNG.standard_normal((B, H, T, T)).astype(np.float32)
    mask = np.tril(np.ones((T, T), bool))[None, None]

    def build(g):
        x = g.add_input("s", sc.shape)
        m = g.op("Mul", x, g.new_init(np.array([0.125], np.float32)))
        w = g.op("Where", g.new_init(mask), m, g.new_init(np.array(-1e9, np.float32)))
        return [g.op("Softmax", w, axis=-1)]
    m = _chain_model(build)
    sess = CudaSessionBuilder(m).build()
    try:
        assert [e["kind"] for e in sess.schedule()] == ["softmax_scaled_masked"]
        got = sess.run([sc])[0]
    finally:
        sess.close()
    unfused = run_cuda(m, [sc], fuse=False)[0]
    assert_bit_exact(got, unfused)
    want = run_oracle(m, [sc])[0]
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-9)
    assert (got[..., 0, 1:] == 0).all() and np.allclose(got.sum(-1), 1, atol=1e-5)


@pytest.mark.parametrize("c,hw,oc", [(72, 28, 40), (120, 28, 40), (480, 14, 112)])
def test_squeeze_excite_gate_folds_into_the_pointwise_convolution(cuda_lib, c, hw, oc):
    """x * gate[n, c, 1, 1] -> 1 x 1 Conv: the multiply happens inside the GEMM's operand split
    (the gated map is never written); bit-identical to the unfused pair on the same kernel."""
    from altius_b200.session import CudaSessionBuilder
    n = 32
    x = RNG.standard_normal((n, c, hw, hw)).astype(np.float32)
    gate = RNG.random((n, c, 1, 1)).astype(np.float32)
    w = (RNG.standard_normal((oc, c, 1, 1)) / np.sqrt(c)).astype(np.float32)
    b = RNG.standard_normal(oc).astype(np.float32)

    def build(g):
        xi, gi = g.add_input("x", x.shape), g.add_input("g", gate.shape)
        y = g.op("Conv2d", g.op("Mul", xi, gi), g.new_init(w), g.new_init(b), kernel_shape=[1, 1], strides=[1, 1],
                 padding=[0, 0, 0, 0], dilations=[1, 1], group=1, auto_pad="")
        return [y]
    m = _chain_model(build)
    sess = CudaSessionBuilder(m).build()
    try:
        assert [e["kind"] for e in sess.schedule()] == ["gemm_tf32x3_tcgen05"]
        got = sess.run([x, gate])[0]
    finally:
        sess.close()
    unfused = run_cuda(m, [x, gate], fuse=False)[0]
    assert_bit_exact(got, unfused)
    want = run_oracle(m, [x, gate], sgemm="openblas")[0]
    kk = np.abs(x * gate).reshape(n, c, -1)
    bound = 1e-5 * np.abs(want) + 5e-6 * np.einsum("oc,nch->noh", np.abs(w[:, :, 0, 0]), kk).reshape(want.shape) + 1e-6
    assert (np.abs(got - want) <= bound).all()


# ---- measured error of the tensor-core GEMM on the models' shapes -------------------------------
GEMM_MODEL_SHAPES = [  # (M, K, N): ViT-B/16 at 32 images, DeiT-S at 64
    (6304, 768, 2304), (6304, 768, 768), (6304, 768, 3072), (6304, 3072, 768),
    (12672, 384, 1152), (12672, 1536, 384)]


@pytest.mark.parametrize("m,k,n", GEMM_MODEL_SHAPES)
def test_gemm_error_on_the_models_shapes_is_measured(cuda_lib, m, k, n, record_property):
    """Activations ~N(0,1), weights ~N(0,0.02) as in the configurations. The error of the
    default tensor-core path and of the oracle's fp32 sgemm are both measured against a float64
    product: relative to sum|a||b| (the scale a dot product's rounding lives on) and relative to
    the result's rms. The fp32 accumulator in tensor memory truncates after every MMA step, so
    the tensor-core error is a few times the sgemm's; an all-positive dot product of K = 3072
    shows the bias directly (3.2e-5 relative, above the 1e-5 a rounding accumulator would
    keep): asserted here so that the figure in the documentation stays a measured one."""
    a = RNG.standard_normal((m, k)).astype(np.float32)
    w = (0.02 * RNG.standard_normal((k, n))).astype(np.float32)
    model = single_op_model("MatMul", [a], [w])
    got = run_cuda(model, [a])[0]
    sg = run_oracle(model, [a], threads=0, sgemm="openblas")[0]
    rows = slice(0, 512)                                   # float64 truth on a slab of rows
    truth = a[rows].astype(np.float64) @ w.astype(np.float64)
    scale = np.abs(a[rows]).astype(np.float64) @ np.abs(w).astype(np.float64)
    rms = np.sqrt((truth ** 2).mean())
    e_tc, e_sg = np.abs(got[rows] - truth), np.abs(sg[rows] - truth)
    figures = dict(tc_over_sum=float((e_tc / scale).max()), sgemm_over_sum=float((e_sg / scale).max()),
                   tc_over_rms=float(e_tc.max() / rms), sgemm_over_rms=float(e_sg.max() / rms))
    for key, val in figures.items():
        record_property(key, val)
    print("gemm error", (m, k, n), figures)
    assert figures["tc_over_sum"] <= 3e-6 and figures["tc_over_rms"] <= 1e-4
    assert (np.abs(got - sg) <= 1e-5 * np.abs(sg) + 5e-6 * (np.abs(a) @ np.abs(w))).all()


@pytest.mark.parametrize("gemm_mode", [0, 3])
def test_tensor_memory_accumulation_bias_is_what_the_documentation_says(cuda_lib, gemm_mode):
    """All-positive operands, K = 3072, the MLP-2 shape: every partial sum in tensor memory is
    rounded the same way, so the result is biased. The measured figure is printed and bounded."""
    a = RNG.random((6304, 3072)).astype(np.float32) + 0.5
    w = (RNG.random((3072, 768)).astype(np.float32) + 0.5) * 0.02
    model = single_op_model("MatMul", [a], [w])
    got = run_cuda(model, [a], gemm_mode=gemm_mode)[0][:256].astype(np.float64)
    truth = a[:256].astype(np.float64) @ w.astype(np.float64)
    rel = (got - truth) / truth
    print("all-positive K=3072, gemm_mode", gemm_mode, ": mean relative error", rel.mean(), "max |.|", np.abs(rel).max())
    assert np.abs(rel).max() < 6e-5
