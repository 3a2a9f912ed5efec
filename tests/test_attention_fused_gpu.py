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
