"""Whole-graph parity of the CUDA session with the CPU oracle on the benchmark
configurations (synthetic weights and inputs of the configurations' shapes and
distributions). Bars: max absolute logit error 1e-3 with identical top-1 for
the models; the per-op bars for the tensor-op micrograph; fused and unfused
schedules and graph / no-graph replay must agree."""
import numpy as np
import pytest

from altius_b200 import configs
from altius_b200.session import CudaSessionBuilder, InferenceSession
from helpers import assert_bit_exact, max_rel_err, run_cuda, run_oracle

pytestmark = pytest.mark.gpu


def check_logits(got, want):
    assert got.shape == want.shape
    assert np.abs(got - want).max() <= 1e-3
    assert (got.argmax(-1) == want.argmax(-1)).all()


def test_mnist_cnn(cuda_lib):
    model, feeds = configs.mnist_cnn()
    want = run_oracle(model, feeds.values())[0]
    for opts in (dict(), dict(fuse=False), dict(graph=False), dict(gemm_mode=1)):
        check_logits(run_cuda(model, feeds.values(), **opts)[0], want)


def test_inference_session_by_name(cuda_lib):
    model, feeds = configs.mnist_cnn()
    want = run_oracle(model, feeds.values())[0]
    sess = InferenceSession(model, backend="cuda")
    check_logits(sess.run(None, feeds)[0], want)
    with pytest.raises(RuntimeError):
        sess.run(None, {"wrong": feeds["Input3"]})


@pytest.mark.parametrize("batch", [3, 64])
def test_micrograph(cuda_lib, batch):
    model, feeds = configs.micrograph(batch=batch)
    want = run_oracle(model, feeds.values(), threads=0)
    for opts in (dict(), dict(fuse=False)):
        got = run_cuda(model, feeds.values(), **opts)
        np.testing.assert_allclose(got[0], want[0], rtol=1e-5, atol=1e-6)   # fused LN chain
        assert max_rel_err(got[1], want[1]) < 1e-5                          # scale + softmax
        np.testing.assert_allclose(got[2], want[2], rtol=1e-5, atol=1e-7)   # ReduceMean
        assert_bit_exact(got[3], want[3])                                   # ReduceMax
    # size-independent properties at the full size
    assert np.abs(got[1].sum(-1) - 1).max() < 1e-5
    assert np.abs(got[0].mean(-1)).max() < 0.1


def test_repeated_runs_are_identical(cuda_lib):
    model, feeds = configs.vit_base_16(batch=2, depth=2)
    sess = CudaSessionBuilder(model).build()
    a = sess.run(list(feeds.values()))[0].copy()
    b = sess.run(list(feeds.values()))[0].copy()
    assert_bit_exact(a, b)
    sess.close()


@pytest.mark.parametrize("name,fn,kw", [
    ("vit_b16", configs.vit_base_16, dict(batch=2)),
    ("deit_s16", configs.deit_small_distilled_16, dict(batch=3)),
    ("mobilenet_v3", configs.mobilenet_v3_large, dict(batch=2)),
])
def test_models(cuda_lib, name, fn, kw):
    model, feeds = fn(**kw)
    want = run_oracle(model, feeds.values(), threads=0)[0]
    for opts in (dict(), dict(fuse=False), dict(gemm_mode=1)):
        check_logits(run_cuda(model, feeds.values(), **opts)[0], want)


def test_profile_reports_every_kernel_kind(cuda_lib):
    model, feeds = configs.vit_base_16(batch=2, depth=1)
    sess = CudaSessionBuilder(model).with_profiling_enabled(True).build()
    sess.run(list(feeds.values()))
    prof = sess.profile()
    kinds = {e["kind"] for e in sess.schedule()}
    assert set(prof) == kinds
    assert sum(p["launches"] for p in prof.values()) == sess.launches_per_run
    assert all(p["total_ms"] > 0 for p in prof.values())
    sess.close()


def test_run_batches_equals_run_per_batch(cuda_lib):
    """The pipelined queue call returns, batch by batch, exactly what `run` returns; with
    pageable and with page-locked buffers, and for a single batch."""
    from altius_b200.session import alloc_pinned
    model, feeds = configs.vit_base_16(batch=2, depth=2)
    x0 = next(iter(feeds.values()))
    rng = np.random.default_rng(5)
    xs = [x0] + [rng.standard_normal(x0.shape).astype(np.float32) for _ in range(4)]
    sess = CudaSessionBuilder(model).build()
    try:
        want = [sess.run([x])[0].copy() for x in xs]
        got = sess.run_batches([[x] for x in xs])
        for g, w in zip(got, want):
            assert_bit_exact(g[0], w)
        pinned_in = []
        for x in xs:
            p = alloc_pinned(x.shape)
            p[...] = x
            pinned_in.append([p])
        pinned_out = [[alloc_pinned(want[0].shape)] for _ in xs]
        sess.run_batches(pinned_in, outputs=pinned_out)
        for g, w in zip(pinned_out, want):
            assert_bit_exact(np.array(g[0]), w)
        assert_bit_exact(sess.run_batches([[xs[3]]])[0][0], want[3])
        assert sess.run_batches([]) == []
    finally:
        sess.close()


def test_sessions_on_two_devices_in_one_process(cuda_lib):
    """Kernel attributes (dynamic shared memory limits) belong to a device: a second session
    on another GPU of the same process must set them again."""
    from altius_b200 import session
    if session.load_library().altius_cuda_device_count() < 2:
        pytest.skip("needs two GPUs")
    model, feeds = configs.vit_base_16(batch=2, depth=2)
    x = next(iter(feeds.values()))
    outs = []
    for dev in (0, 1):
        sess = CudaSessionBuilder(model).with_device(dev).build()
        try:
            outs.append(sess.run([x])[0].copy())
        finally:
            sess.close()
    assert_bit_exact(outs[0], outs[1])


@pytest.mark.parametrize("name,fn,kw", [
    ("vit_b16_b32", configs.vit_base_16, dict(batch=32)),
    ("deit_s16_b64", configs.deit_small_distilled_16, dict(batch=64)),
    ("mobilenet_v3_b32", configs.mobilenet_v3_large, dict(batch=32)),
])
def test_models_at_the_benchmarked_batch(cuda_lib, name, fn, kw):
    """The configurations at the batch the benchmark runs them at, through the default plan
    (CTA-pair GEMMs with operands split by their producers, K-sliced tail tiles, the tcgen05
    attention kernel, tensor-core convolutions), against the oracle with OpenBLAS sgemm on all
    host threads: max absolute logit error 1e-3, identical top-1."""
    model, feeds = fn(**kw)
    x = list(feeds.values())
    got = run_cuda(model, x)[0]
    want = run_oracle(model, x, threads=0, sgemm="openblas")[0]
    check_logits(got, want)
