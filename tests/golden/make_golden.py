"""Generates the fixtures in this folder: seeded inputs and the CPU oracle's
outputs for a few small cases of the hot path.

    python tests/golden/make_golden.py

The reference repository holds no golden output files for these kernels and
cannot be run offline (Rust + BLIS), so these are NOT reference outputs: they
freeze the oracle's results so that a later change to either the oracle or the
CUDA kernels shows up as a diff. Contraction cases use the oracle's own sgemm
(documented summation order), so they are reproducible bit for bit on any x86-64
host with FMA.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
sys.path.insert(0, os.path.join(HERE, ".."))

from altius_b200 import configs  # noqa: E402
from helpers import run_oracle, single_op_model  # noqa: E402


def cases():
    rng = np.random.default_rng(20240229)
    x = (rng.standard_normal((3, 7, 50)) * 3).astype(np.float32)
    g = (1 + 0.02 * rng.standard_normal(50)).astype(np.float32)
    b = (0.02 * rng.standard_normal(50)).astype(np.float32)
    yield "gelu", single_op_model("Gelu", [x]), [x]
    yield "sigmoid", single_op_model("Sigmoid", [x]), [x]
    yield "tanh", single_op_model("Tanh", [x]), [x]
    yield "softmax", single_op_model("Softmax", [x], axis=-1), [x]
    yield "layer_norm", single_op_model("LayerNormalization", [x], [g, b], axis=-1, epsilon=1e-6,
                                        stash_type=1), [x]
    yield "hard_sigmoid", single_op_model("HardSigmoid", [x], alpha=1.0 / 6.0, beta=0.5), [x]
    yield "reduce_mean", single_op_model("ReduceMean", [x], axes=[-1], keep_dims=True), [x]
    a = rng.standard_normal((5, 33)).astype(np.float32)
    w = rng.standard_normal((33, 9)).astype(np.float32)
    yield "matmul", single_op_model("MatMul", [a, w]), [a, w]
    img = rng.standard_normal((2, 3, 9, 9)).astype(np.float32)
    k = rng.standard_normal((4, 3, 3, 3)).astype(np.float32)
    cb = rng.standard_normal(4).astype(np.float32)
    yield "conv3x3", single_op_model("Conv2d", [img], [k, cb], kernel_shape=[3, 3], strides=[2, 2],
                                     padding=[1, 1, 1, 1], dilations=[1, 1], group=1, auto_pad=""), [img]
    yield "max_pool", single_op_model("MaxPool", [img], kernel_shape=[3, 3], strides=[2, 2],
                                      padding=[1, 1, 1, 1]), [img]
    model, feeds = configs.mnist_cnn()
    yield "mnist_cnn", model, list(feeds.values())


def main():
    out = {}
    for name, model, inputs in cases():
        res = run_oracle(model, inputs, threads=1, sgemm="own")
        for i, t in enumerate(inputs):
            out[f"{name}/in{i}"] = t
        for i, t in enumerate(res):
            out[f"{name}/out{i}"] = t
    np.savez_compressed(os.path.join(HERE, "oracle_cases.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
