"""The allocation-free whole-tensor maximum (`altius_cuda_reduce_max_noalloc`).

Some callers cannot allocate device memory at the point where they need a value
(latency-critical loops and callbacks that cannot absorb cudaMalloc's implicit
synchronisation, plug-ins that own no memory pool). For them the library has one
entry point whose scratch is a fixed array inside the library itself. This file
checks, through the C ABI, that it returns exactly what the regular session
path (a one-node ReduceMax graph, scratch in the session arena) returns -- on
two calls in a row, the second on a smaller tensor with a smaller maximum, so a
stale partial left in the shared scratch by the first call would show -- and that
sizes beyond the fixed scratch are refused with a message.

It is collected last on purpose: a run that stops at the first failure has then
already run every other test.
"""
import numpy as np
import pytest

from altius_b200.session import SessionError, load_library, reduce_max_noalloc
from helpers import run_cuda, single_op_model

MAX_ELEMS = 16384 * 4096


def test_oversized_and_empty_inputs_are_refused():
    # The size checks come before any CUDA call: this runs without a GPU too.
    load_library()
    with pytest.raises(SessionError) as e:
        reduce_max_noalloc(0x1000, MAX_ELEMS + 1, 0x2000)
    assert e.value.status == 1 and "exceed the fixed scratch" in str(e.value)
    with pytest.raises(SessionError) as e:
        reduce_max_noalloc(0x1000, 0, 0x2000)
    assert e.value.status == 1
    with pytest.raises(SessionError):
        reduce_max_noalloc(0, 16, 0x2000)


@pytest.mark.gpu
def test_matches_the_session_path_on_two_calls_in_a_row(cuda_lib):
    import torch
    rng = np.random.default_rng(7)
    first = (rng.standard_normal((5, 1000, 1003)) * 3 + 10).astype(np.float32)   # 5,015,000 elements, max ~ 25
    second = (rng.standard_normal((3, 331)) - 40).astype(np.float32)             # 993 elements, max ~ -37
    out = torch.empty(1, dtype=torch.float32, device="cuda")
    for host in (first, second):
        dev = torch.from_numpy(host).cuda()
        torch.cuda.synchronize()
        reduce_max_noalloc(dev.data_ptr(), host.size, out.data_ptr())     # default stream
        torch.cuda.synchronize()
        got = out.cpu().numpy()
        want = run_cuda(single_op_model("ReduceMax", [host], axes=[], keep_dims=False), [host])[0]
        assert want.shape == (1,) and want[0] == host.max()
        assert got.view(np.uint32)[0] == want.view(np.uint32)[0]          # bit-exact, as the other ReduceMax tests


@pytest.mark.gpu
def test_largest_accepted_size_and_a_side_stream(cuda_lib):
    import torch
    x = torch.full((MAX_ELEMS,), -1.0, dtype=torch.float32, device="cuda")
    x[MAX_ELEMS - 1] = 3.5
    out = torch.empty(1, dtype=torch.float32, device="cuda")
    stream = torch.cuda.Stream()
    torch.cuda.synchronize()
    reduce_max_noalloc(x.data_ptr(), MAX_ELEMS, out.data_ptr(), stream.cuda_stream)
    stream.synchronize()
    assert float(out.cpu()[0]) == 3.5
