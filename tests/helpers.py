"""Shared helpers for the parity tests: one-node graphs in the style of the
reference's Python op tests (crates/altius_py/tests/test_ops_*.py), run through
the CPU oracle and through the CUDA session's C ABI."""
import numpy as np

from altius_b200 import ir
from altius_b200.session import CudaSessionBuilder
from oracle import InterpreterSessionBuilder


def single_op_model(op, input_arrays, const_arrays=(), n_outputs=1, opset=13, const_first=False,
                    **attrs):
    """Graph with one node. `input_arrays` become run-time inputs, `const_arrays`
    initializers appended after (or before, const_first) them."""
    g = ir.Graph()
    ins = [g.add_input(f"in{i}", a.shape, ir.elem_type_of(a.dtype)) for i, a in enumerate(input_arrays)]
    consts = [g.new_init(np.asarray(c)) if c is not None else -1 for c in const_arrays]
    order = consts + ins if const_first else ins + consts
    outs = g.add_node(op, order, n_outputs, **attrs)
    for i, o in enumerate(outs):
        g.values[o].name = f"out{i}"
        g.outputs.append(o)
    return ir.Model(g, opset)


def run_oracle(model, inputs, threads=4, sgemm="own"):
    return (InterpreterSessionBuilder(model).with_intra_op_num_threads(threads).with_sgemm(sgemm)
            .build().run(list(inputs)))


def run_cuda(model, inputs, **opts):
    b = CudaSessionBuilder(model)
    if "fuse" in opts:
        b = b.with_fusion(opts["fuse"])
    if "graph" in opts:
        b = b.with_cuda_graph(opts["graph"])
    if "gemm_mode" in opts:
        b = b.with_gemm_mode(opts["gemm_mode"])
    if "pairs" in opts:
        b = b.with_gemm_pairs(opts["pairs"])
    sess = b.build()
    try:
        return sess.run(list(inputs))
    finally:
        sess.close()


def assert_bit_exact(got, want):
    got, want = np.ascontiguousarray(got), np.ascontiguousarray(want)
    assert got.shape == want.shape and got.dtype == want.dtype
    if got.dtype == np.float32:
        g, w = got.view(np.uint32), want.view(np.uint32)
        both_nan = np.isnan(got) & np.isnan(want)
        bad = (g != w) & ~both_nan
        assert not bad.any(), f"{bad.sum()} of {bad.size} elements differ bitwise; first at " \
                              f"{np.argwhere(bad)[0]}: {got[bad][0]!r} vs {want[bad][0]!r}"
    else:
        assert np.array_equal(got, want)


def max_rel_err(got, want, floor=1e-30):
    got, want = got.astype(np.float64), want.astype(np.float64)
    return float(np.max(np.abs(got - want) / np.maximum(np.abs(want), floor)))
