"""GPU: the fused causal-attention kernels (head dimension 64) against the float64 oracle, called
through the C ABI on (B, T, H * 64) buffers."""
from ctypes import c_float, c_void_p

import numpy as np
import pytest

from oracle import gemm_oracle as O
from tests import _util as U

pytestmark = pytest.mark.gpu

D = 64


def heads(a, B, S, H):
    return a.reshape(B, S, H, D).transpose(0, 2, 1, 3)


def merge(a, B, S, H):
    return a.transpose(0, 2, 1, 3).reshape(B, S, H * D)


def run_forward(q, k, v, B, S, H, want_p=True, scale=None):
    from gradtuity_b200 import _lib

    lib, ctx = _lib.load_library(), _lib.context()
    scale = 1.0 / np.sqrt(D) if scale is None else scale
    dq, dk, dv = U.DeviceBuffer(q), U.DeviceBuffer(k), U.DeviceBuffer(v)
    do = U.DeviceBuffer(np.full((B, S, H * D), np.nan, np.float32))
    dl = U.DeviceBuffer(np.full((B, H, S), np.nan, np.float32))
    dp = U.DeviceBuffer(np.zeros((B, H, S, S), np.float32)) if want_p else None
    _lib.check(lib.gt_attention_forward(ctx, c_void_p(do.ptr), c_void_p(dp.ptr) if dp else None, c_void_p(dl.ptr),
                                        c_void_p(dq.ptr), c_void_p(dk.ptr), c_void_p(dv.ptr), B, S, H, D,
                                        c_float(scale), None), "gt_attention_forward")
    _lib.device_status()
    return do.read((B, S, H * D)), dl.read((B, H, S)), (dp.read((B, H, S, S)) if dp else None)


@pytest.mark.parametrize("B,H,S", [(1, 1, 128), (2, 3, 256), (1, 2, 512), (2, 12, 1024)])
def test_forward_matches_oracle(gt, B, H, S):
    rng = np.random.default_rng(S + H)
    q, k, v = (rng.standard_normal((B, S, H * D)).astype(np.float32) for _ in range(3))
    o, lse, p = run_forward(q, k, v, B, S, H)
    ref = O.attention_forward_backward(heads(q, B, S, H), heads(k, B, S, H), heads(v, B, S, H), heads(v, B, S, H))
    assert O.rel_frobenius(o, merge(ref["o"], B, S, H)) <= 1e-3
    # P: exact zeros right of the diagonal inside each row's diagonal block, rows sum to one
    iu = np.triu_indices(128, 1)
    for blk in range(S // 128):
        sl = slice(blk * 128, (blk + 1) * 128)
        assert np.all(p[:, :, sl, sl][..., iu[0], iu[1]] == 0.0)
    low = np.tril(np.ones((S, S), bool))
    assert O.rel_frobenius(np.where(low, p, 0.0), ref["p"]) <= 1e-3
    assert np.allclose(np.where(low, p, 0.0).sum(-1), 1.0, atol=2e-3)
    s = ref["s"]
    s = np.where(low, s, -np.inf)
    smax = s.max(-1)
    ref_lse = smax + np.log(np.exp(s - smax[..., None]).sum(-1))
    assert np.allclose(lse, ref_lse, rtol=0, atol=2e-3)


def test_forward_without_p_output_and_large_scores(gt):
    """No P buffer (the form the training step uses), and scores large enough that an unshifted exp
    would overflow: the row maximum found in the first pass keeps the result finite and exact."""
    rng = np.random.default_rng(11)
    B, H, S = 1, 2, 384
    q, k, v = (rng.standard_normal((B, S, H * D)).astype(np.float32) for _ in range(3))
    q *= 12.0
    o, lse, p = run_forward(q, k, v, B, S, H, want_p=False, scale=1.0)
    assert p is None and np.all(np.isfinite(o)) and np.all(np.isfinite(lse))
    qh, kh, vh = heads(q, B, S, H), heads(k, B, S, H), heads(v, B, S, H)
    sc = np.matmul(qh.astype(np.float64), np.swapaxes(kh.astype(np.float64), -1, -2))
    ref_o = np.matmul(O.causal_softmax(sc), vh.astype(np.float64))
    # peaked rows amplify the tf32 rounding of the scores (|s| up to a few hundred): looser bar
    assert O.rel_frobenius(o, merge(ref_o, B, S, H)) <= 2e-2


def test_unsupported_shapes_are_refused(gt):
    from gradtuity_b200 import _lib

    lib, ctx = _lib.load_library(), _lib.context()
    buf = U.DeviceBuffer(np.zeros((1, 100, 64), np.float32))
    rc = lib.gt_attention_forward(ctx, c_void_p(buf.ptr), None, None, c_void_p(buf.ptr), c_void_p(buf.ptr),
                                  c_void_p(buf.ptr), 1, 100, 1, 64, c_float(0.125), None)
    assert rc == _lib.GT_ERR_UNSUPPORTED
    rc = lib.gt_attention_forward(ctx, c_void_p(buf.ptr), None, None, c_void_p(buf.ptr), c_void_p(buf.ptr),
                                  c_void_p(buf.ptr), 1, 128, 2, 32, c_float(0.125), None)
    assert rc == _lib.GT_ERR_UNSUPPORTED


def run_backward(q, k, v, do, B, S, H, accumulate=False):
    from gradtuity_b200 import _lib

    lib, ctx = _lib.load_library(), _lib.context()
    scale = 1.0 / np.sqrt(D)
    bq, bk, bv, bdo = (U.DeviceBuffer(a) for a in (q, k, v, do))
    bo = U.DeviceBuffer(np.zeros((B, S, H * D), np.float32))
    bl = U.DeviceBuffer(np.zeros((B, H, S), np.float32))
    bd = U.DeviceBuffer(np.full((B, H, S), np.nan, np.float32))
    _lib.check(lib.gt_attention_forward(ctx, c_void_p(bo.ptr), None, c_void_p(bl.ptr), c_void_p(bq.ptr), c_void_p(bk.ptr),
                                        c_void_p(bv.ptr), B, S, H, D, c_float(scale), None), "gt_attention_forward")
    init = np.ones((B, S, H * D), np.float32) if accumulate else np.full((B, S, H * D), np.nan, np.float32)
    gq, gk, gv = (U.DeviceBuffer(init) for _ in range(3))
    acc = 1 if accumulate else 0
    _lib.check(lib.gt_attention_backward(ctx, c_void_p(gq.ptr), c_void_p(gk.ptr), c_void_p(gv.ptr), c_void_p(bdo.ptr),
                                         c_void_p(bq.ptr), c_void_p(bk.ptr), c_void_p(bv.ptr), c_void_p(bo.ptr),
                                         c_void_p(bl.ptr), c_void_p(bd.ptr), B, S, H, D, c_float(scale), acc, acc, acc, None),
               "gt_attention_backward")
    _lib.device_status()
    shape = (B, S, H * D)
    return gq.read(shape), gk.read(shape), gv.read(shape), bd.read((B, H, S)), bo.read(shape)


@pytest.mark.parametrize("B,H,S", [(1, 1, 128), (2, 3, 256), (1, 2, 512), (2, 12, 1024), (1, 3, 2048), (40, 4, 128)])
def test_backward_matches_oracle(gt, B, H, S):
    rng = np.random.default_rng(7 * S + H)
    q, k, v, do = (rng.standard_normal((B, S, H * D)).astype(np.float32) for _ in range(4))
    dq, dk, dv, delta, o = run_backward(q, k, v, do, B, S, H)
    ref = O.attention_forward_backward(*(heads(a, B, S, H) for a in (q, k, v, do)))
    ref_delta = (heads(do, B, S, H).astype(np.float64) * ref["o"]).sum(-1)
    assert np.allclose(delta, ref_delta, rtol=0, atol=5e-3 * np.abs(ref_delta).max())
    assert O.rel_frobenius(dv, merge(ref["dv"], B, S, H)) <= 1e-3
    assert O.rel_frobenius(dq, merge(ref["dq"], B, S, H)) <= 2e-3
    assert O.rel_frobenius(dk, merge(ref["dk"], B, S, H)) <= 2e-3


def test_backward_accumulates_into_existing_gradients(gt):
    rng = np.random.default_rng(3)
    B, H, S = 1, 2, 256
    q, k, v, do = (rng.standard_normal((B, S, H * D)).astype(np.float32) for _ in range(4))
    dq0, dk0, dv0, _, _ = run_backward(q, k, v, do, B, S, H)
    dq1, dk1, dv1, _, _ = run_backward(q, k, v, do, B, S, H, accumulate=True)
    for a0, a1 in ((dq0, dq1), (dk0, dk1), (dv0, dv1)):
        assert np.allclose(a1 - 1.0, a0, rtol=0, atol=1e-5 * max(1.0, np.abs(a0).max()))


@pytest.mark.parametrize("B,H,S", [(1, 1, 128), (2, 3, 256), (1, 2, 640), (2, 12, 1024), (1, 3, 2048), (40, 4, 128)])
def test_single_pass_forward_matches_oracle(gt, B, H, S):
    """Without a P output the forward is a single pass with a running reference maximum (O rescaled in tensor
    memory when a tile's maximum jumps): O and the log-sum-exp against float64, with row scales that differ by
    orders of magnitude so that rescaling happens."""
    rng = np.random.default_rng(5 * S + H)
    q, k, v = (rng.standard_normal((B, S, H * D)).astype(np.float32) for _ in range(3))
    q *= np.exp(rng.uniform(-2.0, 2.5, (B, S, 1))).astype(np.float32)          # some rows have scores in the hundreds
    o, lse, _ = run_forward(q, k, v, B, S, H, want_p=False)
    qh, kh, vh = (heads(a, B, S, H).astype(np.float64) for a in (q, k, v))
    sc = np.matmul(qh, np.swapaxes(kh, -1, -2)) / np.sqrt(D)
    p = O.causal_softmax(sc)
    ref_o = np.matmul(p, vh)
    low = np.tril(np.ones((S, S), bool))
    s = np.where(low, sc, -np.inf)
    smax = s.max(-1)
    ref_lse = smax + np.log(np.exp(s - smax[..., None]).sum(-1))
    assert np.all(np.isfinite(o)) and np.all(np.isfinite(lse))
    assert O.rel_frobenius(o, merge(ref_o, B, S, H)) <= 3e-3      # peaked rows amplify the tf32 rounding of the scores
    assert np.allclose(lse, ref_lse, rtol=1e-3, atol=5e-3)      # a score of 40 carries a tf32 rounding error of 0.02


@pytest.mark.parametrize("B,H,S", [(1, 1, 128), (2, 3, 384), (2, 12, 1024)])
def test_backward_adds_the_projection_bias_gradients(gt, B, H, S):
    """gt_attention_backward_bias: dbq / dbk / dbv receive, added to their contents, the column sums over all tokens of the
    dQ / dK / dV the call wrote; a null pointer leaves that one out; dQ, dK, dV themselves are those of the plain call."""
    from gradtuity_b200 import _lib

    lib, ctx = _lib.load_library(), _lib.context()
    rng = np.random.default_rng(S + 5 * H)
    q, k, v, do = (rng.standard_normal((B, S, H * D)).astype(np.float32) for _ in range(4))
    want_dq, want_dk, want_dv, _, _ = run_backward(q, k, v, do, B, S, H)
    scale = 1.0 / np.sqrt(D)
    bq, bk, bv, bdo = (U.DeviceBuffer(a) for a in (q, k, v, do))
    bo, bl = U.DeviceBuffer(np.zeros((B, S, H * D), np.float32)), U.DeviceBuffer(np.zeros((B, H, S), np.float32))
    bd = U.DeviceBuffer(np.zeros((B, H, S), np.float32))
    _lib.check(lib.gt_attention_forward(ctx, c_void_p(bo.ptr), None, c_void_p(bl.ptr), c_void_p(bq.ptr), c_void_p(bk.ptr),
                                        c_void_p(bv.ptr), B, S, H, D, c_float(scale), None), "gt_attention_forward")
    start = rng.standard_normal((3, H * D)).astype(np.float32)
    for present in ((True, True, True), (False, True, False)):
        gq, gk, gv = (U.DeviceBuffer(np.full((B, S, H * D), np.nan, np.float32)) for _ in range(3))
        db = [U.DeviceBuffer(start[i]) for i in range(3)]
        ptrs = [c_void_p(db[i].ptr) if present[i] else None for i in range(3)]
        _lib.check(lib.gt_attention_backward_bias(ctx, c_void_p(gq.ptr), c_void_p(gk.ptr), c_void_p(gv.ptr), ptrs[0], ptrs[1], ptrs[2],
                                                  c_void_p(bdo.ptr), c_void_p(bq.ptr), c_void_p(bk.ptr), c_void_p(bv.ptr), c_void_p(bo.ptr),
                                                  c_void_p(bl.ptr), c_void_p(bd.ptr), B, S, H, D, c_float(scale), 0, 0, 0, None),
                   "gt_attention_backward_bias")
        assert _lib.device_status() == 0
        shape = (B, S, H * D)
        for got, want in ((gq.read(shape), want_dq), (gk.read(shape), want_dk), (gv.read(shape), want_dv)):
            assert np.array_equal(got, want)
        for i, grad in enumerate((want_dq, want_dk, want_dv)):
            have = db[i].read((H * D,))
            if present[i]:
                # the sums nearly cancel (rows of dS sum to about zero): the bar is relative to the magnitudes that were added
                tol = 1e-5 * np.abs(grad).sum((0, 1)).max() + 2e-6 * np.abs(start[i]).max()
                assert np.abs(have - (start[i] + grad.astype(np.float64).sum((0, 1)))).max() <= tol
            else:
                assert np.array_equal(have, start[i])
