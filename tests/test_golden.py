"""Frozen oracle outputs (tests/golden/oracle_cases.npz, made by
tests/golden/make_golden.py): the oracle must still reproduce them bit for bit
(CPU), and the CUDA session must match them to the per-class bars (GPU)."""
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
from helpers import assert_bit_exact, run_cuda, run_oracle  # noqa: E402
import make_golden  # noqa: E402

GOLD = np.load(os.path.join(HERE, "golden", "oracle_cases.npz"))
CASES = {name: (model, inputs) for name, model, inputs in make_golden.cases()}
EXACT = {"gelu", "sigmoid", "tanh", "hard_sigmoid", "max_pool"}


@pytest.mark.parametrize("name", sorted(CASES))
def test_oracle_reproduces_fixture(name):
    model, inputs = CASES[name]
    for i, t in enumerate(inputs):
        assert_bit_exact(t, GOLD[f"{name}/in{i}"])
    out = run_oracle(model, inputs, threads=1, sgemm="own")
    for i, t in enumerate(out):
        assert_bit_exact(t, GOLD[f"{name}/out{i}"])


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(CASES))
def test_cuda_matches_fixture(cuda_lib, name):
    model, inputs = CASES[name]
    out = run_cuda(model, inputs)
    for i, t in enumerate(out):
        want = GOLD[f"{name}/out{i}"]
        if name in EXACT:
            assert_bit_exact(t, want)
        else:
            np.testing.assert_allclose(t, want, rtol=1e-5, atol=2e-5 if name in ("matmul", "conv3x3", "mnist_cnn") else 1e-6)
