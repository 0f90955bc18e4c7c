"""CPU-only tests of the session library's host side: the C ABI surface, shape
inference, lowering / fusion and the arena plan (sessions built with
`plan_only`, which touches no GPU), and error reporting at create time."""
import collections
import os
import re

import numpy as np
import pytest

from altius_b200 import configs, ir, session
from altius_b200.session import CudaSessionBuilder, SessionError
from helpers import run_oracle, single_op_model

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def plan(model, fuse=True):
    return CudaSessionBuilder(model).with_plan_only(True).with_fusion(fuse).build()


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "altius_session_cuda.h")).read()
    declared = set(re.findall(r"\b(altius_(?:cuda|model)_\w+)\s*\(", header))
    assert declared == set(session.ABI_SYMBOLS)
    lib = session.load_library()
    for name in declared:
        assert hasattr(lib, name), name


def test_plan_only_session_refuses_to_run():
    model, feeds = configs.mnist_cnn()
    s = plan(model)
    with pytest.raises(SessionError) as e:
        s.run(list(feeds.values()))
    assert e.value.status == 5


@pytest.mark.parametrize("fn,kw", [(configs.mnist_cnn, {}), (configs.micrograph, dict(batch=2)),
                                   (configs.vit_base_16, dict(batch=2, depth=1)),
                                   (configs.deit_small_distilled_16, dict(batch=2, depth=1)),
                                   (configs.mobilenet_v3_large, dict(batch=1))])
def test_inferred_output_shapes_match_the_oracle(fn, kw):
    model, feeds = fn(**kw)
    s = plan(model)
    want = run_oracle(model, feeds.values(), threads=8, sgemm="openblas")
    assert [tuple(shape) for shape, _ in s.output_info] == [w.shape for w in want]
    assert [np.dtype(dt) for _, dt in s.output_info] == [w.dtype for w in want]


def test_fusion_folds_the_expected_chains():
    model, _ = configs.micrograph(batch=2)
    kinds = collections.Counter(e["kind"] for e in plan(model).schedule())
    assert kinds == {"layer_norm_bias_gelu_residual": 1, "softmax_scaled": 1, "reduce_mean_max": 1}
    assert plan(model, fuse=False).launches_per_run == 8
    # algorithmic bytes of the fused kernels at the benchmark's size
    model, _ = configs.micrograph(batch=64)
    by_kind = {e["kind"]: e for e in plan(model).schedule()}
    x_bytes = 64 * 197 * 768 * 4
    assert abs(by_kind["layer_norm_bias_gelu_residual"]["bytes"] - 2 * x_bytes) < 1e5
    assert by_kind["softmax_scaled"]["bytes"] == 2 * 64 * 12 * 197 * 197 * 4
    assert by_kind["reduce_mean_max"]["bytes"] == x_bytes + 2 * 64 * 197 * 4   # one pass over X for both

    model, _ = configs.vit_base_16(batch=2, depth=2)
    kinds = collections.Counter(e["kind"] for e in plan(model).schedule())
    gemms = sum(v for k, v in kinds.items() if k.startswith("gemm"))
    assert gemms == 2 * 4 + 2          # per layer: qkv, proj, mlp1, mlp2; patch embed; head
    # Split/Reshape/Transpose/QK^T/scale/Softmax/PV/merge in one kernel; at this batch the projection
    # GEMM is too small for the CTA-pair kernel that would write its operands as fp16 halves
    assert kinds["attention_tcgen05"] + kinds["attention_tma_tcgen05"] == 2
    big = collections.Counter(e["kind"] for e in plan(configs.vit_base_16(batch=32, depth=2)[0]).schedule())
    assert big["attention_tma_tcgen05"] == 2 and big["attention_tcgen05"] == 0
    assert not any(k in kinds for k in ("split_copy", "transpose_copy", "softmax", "softmax_scaled"))
    unfused = collections.Counter(e["kind"] for e in plan(model, fuse=False).schedule())
    assert unfused["split_copy"] == 6 and unfused["softmax"] == 2
    assert kinds["layer_norm"] == 2 * 2 + 1
    assert kinds.get("binary_Add", 0) == 1        # only the position embedding stays a kernel
    assert "unary_gelu" not in kinds

    model, _ = configs.mobilenet_v3_large(batch=1)
    kinds = collections.Counter(e["kind"] for e in plan(model).schedule())
    assert "unary_hard_sigmoid" not in kinds and "unary_relu" not in kinds and "binary_Add" not in kinds
    # Squeeze-excite gates: folded into the pointwise convolution that follows where that one
    # runs on the tensor cores with the planes as its [K, N] operand (large enough, plane size a
    # multiple of four floats); the rest stay broadcast Mul kernels.
    assert kinds["binary_Mul"] == 6
    assert kinds["conv_depthwise"] == 15

    # At the benchmark's batch the convolution GEMMs are large enough for the tensor cores:
    # pointwise layers read the planes as a [K, N] rhs, the 7 x 7 layers through transposed planes,
    # the first layer (3 x 3 x 3 = 27 taps) with zero-padded filter rows, the squeeze-excite
    # layers (1 x 1 planes) as one product over the batch.
    model, _ = configs.mobilenet_v3_large(batch=32)
    steps = plan(model).schedule()
    kinds = collections.Counter(e["kind"] for e in steps)
    assert kinds["im2col"] == 1 and kinds["transpose_copy"] == 6
    assert kinds["binary_Mul"] == 3                    # gates of the three 7 x 7 blocks (transposed planes)
    assert plan(model, fuse=False).schedule().count is not None
    assert collections.Counter(e["kind"] for e in plan(model, fuse=False).schedule())["binary_Mul"] >= 8
    assert kinds["gemm_tf32x3_tcgen05"] == 31          # the first layer and the 30 pointwise layers on planes
    assert kinds["gemm_f16x3_tcgen05"] == 12           # squeeze-excite, the 1 x 1 head convolution, the classifier
    assert kinds["gemm_fp32_simt"] == 6                # the smallest squeeze-excite products
    assert "weight_pad" not in kinds                   # prepared once at create, not per run
    cuda_cores = CudaSessionBuilder(model).with_plan_only(True).with_gemm_mode(1).build().schedule()
    assert sum(e["kind"] == "gemm_fp32_simt" for e in cuda_cores) == 49
    assert not any(e["kind"].endswith("tcgen05") for e in cuda_cores)


def test_flops_of_vit_match_the_published_count():
    model, _ = configs.vit_base_16(batch=1, depth=12)
    flops = sum(e["flops"] for e in plan(model).schedule())
    assert abs(flops / 1e9 - 35.13) < 0.05


def test_arena_reuses_memory():
    model, _ = configs.vit_base_16(batch=4, depth=12)
    # gemm_mode 1: no transposed / split weight copies live in the arena
    s = CudaSessionBuilder(model).with_plan_only(True).with_gemm_mode(1).build()
    total = 0
    for v in range(len(model.graph.values)):
        if v in model.graph.inits:
            continue
        shape, dt = s.value_info(v)
        total += int(np.prod(shape)) * np.dtype(dt).itemsize
    assert s.arena_bytes < total / 8


def test_constant_only_nodes_are_not_in_the_per_run_schedule():
    model, _ = configs.mnist_cnn()
    kinds = [e["kind"] for e in plan(model).schedule()]
    assert len(kinds) == 7     # 2x (im2col + conv gemm + maxpool) + the final matmul


def test_errors_are_reported_at_create():
    a = np.zeros((1, 3, 28, 28), np.float32)
    b = np.zeros((3, 1, 2), np.float32)
    with pytest.raises(SessionError) as e:
        plan(single_op_model("Add", [a, b]))
    assert e.value.status == 2 and "broadcast" in str(e.value)
    with pytest.raises(SessionError) as e:
        plan(single_op_model("Clip", [a]))
    assert e.value.status == 3 and "Kernel not implemented" in str(e.value)
    x = np.zeros((2, 3, 4), np.float32)
    with pytest.raises(SessionError) as e:
        plan(single_op_model("Softmax", [x], axis=1))
    assert e.value.status == 3
    with pytest.raises(SessionError) as e:                 # dangling value id
        g = ir.Graph()
        i = g.add_input("x", (2, 2))
        g.nodes.append(ir.Node("ReLU", [i], [99]))
        g.outputs.append(99)
        plan(ir.Model(g))
    assert e.value.status == 1
    with pytest.raises(RuntimeError):
        session.InferenceSession(configs.mnist_cnn()[0], backend="interpreter")


def test_resize_and_expand_shapes():
    """shape.rs:148-160 (Expand) and :209-254 (Resize: sizes, or floor(dims * scales) for the
    asymmetric / nearest / floor pattern only)."""
    x = np.zeros((2, 3, 10, 10), np.float32)
    none = np.zeros(0, np.float32)
    s = plan(single_op_model("Resize", [x], [none, none, np.array([2, 3, 25, 15], np.int64)], mode="linear"))
    assert s.output_info[0][0] == (2, 3, 25, 15)
    assert [e["kind"] for e in s.schedule()] == ["resize_bilinear"]
    s = plan(single_op_model("Resize", [x], [none, np.array([1, 1, 2.5, 2.5], np.float32)], mode="nearest",
                             coordinate_transformation_mode="asymmetric", nearest_mode="floor"))
    assert s.output_info[0][0] == (2, 3, 25, 25)
    with pytest.raises(SessionError) as e:               # 3-input form outside the one supported pattern
        plan(single_op_model("Resize", [x], [none, np.array([1, 1, 2, 2], np.float32)], mode="linear",
                             coordinate_transformation_mode="asymmetric", nearest_mode="floor"))
    assert e.value.status == 3 and "Unsupported pattern" in str(e.value)
    i = np.zeros((1, 1, 1, 7), np.int64)
    s = plan(single_op_model("Expand", [i], [np.array([1, 1, 4, 7], np.int64)]))
    assert s.output_info[0][0] == (1, 1, 4, 7) and [e["kind"] for e in s.schedule()] == ["expand_copy"]
    with pytest.raises(SessionError) as e:
        plan(single_op_model("Expand", [np.zeros((3,), np.float32)], [np.array([2, 4], np.int64)]))
    assert e.value.status == 2


def test_create_without_a_gpu_fails_loudly():
    lib = session.load_library()
    if lib.altius_cuda_device_count() > 0:
        pytest.skip("a GPU is visible")
    model, _ = configs.mnist_cnn()
    with pytest.raises(SessionError) as e:
        CudaSessionBuilder(model).build()
    assert e.value.status == 5 and "no CPU fallback" in str(e.value)
