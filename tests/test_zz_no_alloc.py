"""GPU: the allocation-free 3xTF32 entry point against the ordinary one.

gt_gemm_3xtf32_noalloc exists for callers that cannot let a library allocate device memory
(their own pool owns the GPU, or an allocation's synchronisation would land inside a timed
step).  It must give what gt_gemm gives in 3xTF32 mode, call after call, although every call
reuses the same built-in scratch array, and it must refuse problems that do not fit.
This file is collected last on purpose: a run that stops at the first failure has then
already run every other test.
"""
import numpy as np
import pytest

from oracle import gemm_oracle as O
from tests import _util as U

pytestmark = pytest.mark.gpu


def _both(layout, a, b, *, bias=None, c0=None, epilogue="none", alpha=1.0):
    from gradtuity_b200 import _lib, gemm as G

    M = a.shape[1] if layout == "TN" else a.shape[0]
    K = a.shape[0] if layout == "TN" else a.shape[1]
    N = b.shape[0] if layout == "NT" else b.shape[1]
    da, db = U.DeviceBuffer(a), U.DeviceBuffer(b)
    dbias = U.DeviceBuffer(bias) if bias is not None else None
    init = c0 if c0 is not None else np.full((M, N), np.nan, np.float32)
    d_ref, d_new = U.DeviceBuffer(init), U.DeviceBuffer(init)
    kw = dict(bias_ptr=dbias.ptr if dbias else 0, alpha=alpha, accumulate=c0 is not None, epilogue=U.EPILOGUES[epilogue])
    G.gemm(U.LAYOUTS[layout], M, N, K, da.ptr, a.shape[1], db.ptr, b.shape[1], d_ref.ptr, N,
           precision=U.PRECISIONS["3xtf32"], **kw)
    G.gemm_3xtf32_noalloc(U.LAYOUTS[layout], M, N, K, da.ptr, a.shape[1], db.ptr, b.shape[1], d_new.ptr, N, **kw)
    _lib.device_status()
    return d_ref.read((M, N)), d_new.read((M, N))


def test_two_calls_in_a_row_match_the_allocating_entry_point(gt):
    # second call: other layout, other shape, smaller operands, so stale scratch contents from
    # the first call would show up if anything depended on them
    calls = [("NN", 384, 640, 520, "bias_gelu", False), ("TN", 200, 136, 96, "none", True)]
    for layout, M, N, K, epilogue, acc in calls:
        a, b, rng = U.make_operands(layout, M, N, K, seed=M + N + K)
        bias = rng.standard_normal(N).astype(np.float32) if epilogue != "none" else None
        c0 = rng.standard_normal((M, N)).astype(np.float32) if acc else None
        ref, new = _both(layout, a, b, bias=bias, c0=c0, epilogue=epilogue, alpha=0.5)
        assert not np.isnan(new).any()
        # same kernels, same inputs: the tolerance is the 3xTF32 bar, the expectation is equality
        assert O.rel_frobenius(new, ref) <= U.TOL["3xtf32"]
        assert np.array_equal(new, ref)
        want = O.gemm(a, b, layout, bias=bias, epilogue=epilogue, c0=c0, alpha=0.5)
        base = c0 if c0 is not None else 0.0
        assert O.rel_frobenius(new - base, want - base) <= U.TOL["3xtf32"]


def _free_device_bytes():
    """Free bytes on the current device as the CUDA runtime reports them."""
    import ctypes

    rt = ctypes.CDLL("libcudart.so.12")
    free, total = ctypes.c_size_t(0), ctypes.c_size_t(0)
    assert rt.cudaMemGetInfo(ctypes.byref(free), ctypes.byref(total)) == 0
    return free.value


def test_a_call_after_the_first_leaves_free_device_memory_unchanged(gt):
    """The property the entry point exists for: once its one-time set-up has run, a call reserves no
    device memory, even for the largest problem it accepts (which in gt_gemm's 3xTF32 mode would
    grow the library's workspace in a fresh process)."""
    from gradtuity_b200 import gemm as G

    small = [U.DeviceBuffer(np.ones((64, 64), np.float32)) for _ in range(3)]
    G.gemm_3xtf32_noalloc(0, 64, 64, 64, small[0].ptr, 64, small[1].ptr, 64, small[2].ptr, 64)     # set-up call
    gt.device_status()
    M = N = K = 1024                                   # 2 * (1 Mi + 1 Mi) * 2 = exactly the 8 Mi floats the array holds
    a, b, _ = U.make_operands("NN", M, N, K, seed=9)
    da, db, dc = U.DeviceBuffer(a), U.DeviceBuffer(b), U.DeviceBuffer(nbytes=M * N * 4)
    gt.device_status()
    for attempt in range(2):                           # a second try in case something else on the box moved memory
        before = _free_device_bytes()
        G.gemm_3xtf32_noalloc(0, M, N, K, da.ptr, K, db.ptr, N, dc.ptr, N)
        gt.device_status()
        after = _free_device_bytes()
        if after == before:
            break
    assert after == before, f"free device memory changed by {before - after} bytes across the call"
    assert O.rel_frobenius(dc.read((M, N)), O.gemm(a, b, "NN")) <= U.TOL["3xtf32"]


def test_oversize_problem_is_refused_and_nothing_is_written(gt):
    from gradtuity_b200 import gemm as G

    M = N = K = 2048              # 2 * (4 Mi + 4 Mi) floats of split scratch: twice the built-in array
    da = U.DeviceBuffer(nbytes=M * K * 4)
    db = U.DeviceBuffer(nbytes=K * N * 4)
    sentinel = np.full((4, 4), 7.0, np.float32)
    dc = U.DeviceBuffer(np.tile(sentinel, (M // 4, N // 4)))
    with pytest.raises(RuntimeError, match="fixed maximum"):
        G.gemm_3xtf32_noalloc(0, M, N, K, da.ptr, K, db.ptr, N, dc.ptr, N)
    gt.device_status()
    assert np.all(dc.read((M, N)) == 7.0)


def test_unaligned_operands_are_served_from_the_same_scratch(gt):
    # the split kernels pack both operands into aligned hi/lo copies, so odd leading dimensions work too
    a, b, _ = U.make_operands("NN", 70, 50, 45, seed=4)
    ref, new = _both("NN", a, b)
    assert np.array_equal(new, ref)
    assert O.rel_frobenius(new, O.gemm(a, b, "NN")) <= U.TOL["3xtf32"]
