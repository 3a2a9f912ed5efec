"""GPU parity: gt_gemm / gt_gemm_batched through the C ABI against the float64 oracle."""
import numpy as np
import pytest

from oracle import gemm_oracle as O
from tests import _util as U

pytestmark = pytest.mark.gpu


# ---- the reference's cross-backend kernel cases, now against absolute goldens ---------------

@pytest.mark.parametrize("precision", ["tf32", "3xtf32", "fp32"])
@pytest.mark.parametrize("kind,M,N,K", U.PHASE4_CASES)
def test_phase4_cases(gt, kind, M, N, K, precision):
    layout, a, b, bias, c0 = U.phase4_inputs(kind, M, N, K)
    epi = {"matmul": "none", "matmul_bias": "bias", "matmul_bias_relu": "bias_relu"}.get(kind, "none")
    out = U.run_gemm(layout, a, b, bias=bias, c0=c0, epilogue=epi, precision=precision)
    gold = U.phase4_vectors()[U.phase4_key(kind, M, N, K)]
    if precision == "tf32":
        # the tolerance the reference itself uses between its TF32 and fp32 backends
        # (gradtuity/tests/test_kernels_cuda_phase4.py:48-52)
        np.testing.assert_allclose(out, gold, rtol=1e-2, atol=1e-3)
    else:
        np.testing.assert_allclose(out, gold, rtol=2e-5, atol=2e-6)


# ---- shape / layout / epilogue sweep ----------------------------------------------------------

SHAPES = [
    (128, 128, 32), (128, 64, 64), (256, 256, 256), (128, 256, 96),
    (1, 1, 1), (1, 64, 8), (3, 5, 7), (17, 33, 19), (40, 24, 36), (63, 65, 127), (129, 257, 255),
    (300, 500, 200), (64, 1000, 72), (520, 136, 1028), (1024, 768, 64), (1024, 64, 1024),
]


@pytest.mark.parametrize("precision", ["tf32", "3xtf32"])
@pytest.mark.parametrize("layout", ["NN", "NT", "TN"])
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_sweep_plain(gt, M, N, K, layout, precision):
    a, b, _ = U.make_operands(layout, M, N, K, seed=M * 7 + N * 3 + K)
    out = U.run_gemm(layout, a, b, precision=precision)
    assert not np.isnan(out).any()
    assert O.rel_frobenius(out, O.gemm(a, b, layout)) <= U.TOL[precision]


@pytest.mark.parametrize("epilogue", ["bias", "bias_relu", "bias_gelu", "causal"])
@pytest.mark.parametrize("layout", ["NN", "NT", "TN"])
@pytest.mark.parametrize("M,N,K", [(256, 512, 128), (200, 328, 72), (17, 33, 19), (512, 512, 64)])
def test_sweep_epilogues(gt, M, N, K, layout, epilogue):
    a, b, rng = U.make_operands(layout, M, N, K, seed=11, scale=1.0 / np.sqrt(K))
    bias = rng.standard_normal(N).astype(np.float32) if epilogue != "causal" else None
    out = U.run_gemm(layout, a, b, bias=bias, epilogue=epilogue)
    ref = O.gemm(a, b, layout, bias=bias, epilogue=epilogue)
    if epilogue == "causal":
        iu = np.triu_indices(M, 1, N)
        assert np.all(out[iu] == np.float32(O.CAUSAL_MASK_VALUE))
        keep = np.tril(np.ones((M, N), bool))
        assert O.rel_frobenius(out[keep], ref[keep]) <= U.TOL["tf32"]
    else:
        assert O.rel_frobenius(out, ref) <= U.TOL["tf32"]
        if epilogue == "bias_relu":
            assert (out >= 0).all()


@pytest.mark.parametrize("layout", ["NN", "NT", "TN"])
def test_gelu_epilogue_stores_preactivation(gt, layout):
    M, N, K = 256, 384, 160
    a, b, rng = U.make_operands(layout, M, N, K, seed=5)
    bias = rng.standard_normal(N).astype(np.float32)
    out, aux = U.run_gemm(layout, a, b, bias=bias, epilogue="bias_gelu", want_aux=True)
    y, pre = O.gemm(a, b, layout, bias=bias, epilogue="bias_gelu", return_pre=True)
    assert O.rel_frobenius(aux, pre) <= U.TOL["tf32"]
    assert O.rel_frobenius(out, y) <= U.TOL["tf32"]
    # the stored activation is the GELU of the stored pre-activation (fast-math exp tolerance)
    np.testing.assert_allclose(out, O.gelu_tanh(aux), rtol=2e-5, atol=2e-6)


@pytest.mark.parametrize("precision", ["tf32", "3xtf32", "fp32"])
@pytest.mark.parametrize("layout", ["NN", "NT", "TN"])
def test_accumulate_and_alpha(gt, layout, precision):
    M, N, K = 192, 320, 256
    a, b, rng = U.make_operands(layout, M, N, K, seed=9)
    c0 = rng.standard_normal((M, N)).astype(np.float32)
    out = U.run_gemm(layout, a, b, c0=c0, alpha=0.125, precision=precision)
    ref = O.gemm(a, b, layout, c0=c0, alpha=0.125)
    # error is measured on the product part, the c0 part is exact
    assert O.rel_frobenius(out - c0, ref - c0) <= U.TOL[precision]


# ---- which kernel runs, alignment, padding ----------------------------------------------------

def test_aligned_operands_take_the_tensor_core_kernel(gt):
    a, b, _ = U.make_operands("NN", 128, 128, 64)
    _, path = U.run_gemm("NN", a, b, return_path=True)
    assert path == 0


@pytest.mark.parametrize("layout", ["NN", "NT", "TN"])
def test_unaligned_operands_take_the_fma_kernel_and_match(gt, layout):
    M, N, K = 70, 50, 45          # leading dimensions 45/50/70: not multiples of 4
    a, b, _ = U.make_operands(layout, M, N, K)
    out, path = U.run_gemm(layout, a, b, return_path=True)
    assert path == 1
    assert O.rel_frobenius(out, O.gemm(a, b, layout)) <= 1e-5   # this kernel is true fp32
    out2, path2 = U.run_gemm(layout, *U.make_operands(layout, 64, 64, 64)[:2], misalign=1, return_path=True)
    assert path2 == 1


@pytest.mark.parametrize("precision", ["tf32", "3xtf32", "fp32"])
@pytest.mark.parametrize("layout", ["NN", "NT", "TN"])
def test_padded_leading_dimensions(gt, layout, precision):
    M, N, K = 150, 200, 100
    a, b, _ = U.make_operands(layout, M, N, K, seed=21)
    out = U.run_gemm(layout, a, b, pad=8, precision=precision)     # NaN padding must never be read
    assert O.rel_frobenius(out, O.gemm(a, b, layout)) <= U.TOL[precision]


@pytest.mark.parametrize("precision", ["tf32", "3xtf32"])
def test_odd_pitch_lm_head_shapes(gt, precision):
    """The tied LM head with an odd vocabulary: logits / dlogits rows are not 16-byte aligned.
    Forward (NT) stores C through the coalesced epilogue; the backward GEMMs read dlogits as an
    unaligned K-major A (NN) and an unaligned MN-major A (TN), copied by the cp.async warps."""
    rng = np.random.default_rng(12)
    M, V, E = 300, 1001, 96
    x = (rng.standard_normal((M, E)) / np.sqrt(E)).astype(np.float32)
    w = (rng.standard_normal((V, E)) / np.sqrt(E)).astype(np.float32)
    dl = (rng.standard_normal((M, V)) / np.sqrt(V)).astype(np.float32)
    logits, path = U.run_gemm("NT", x, w, precision=precision, return_path=True)
    assert path == 0 and O.rel_frobenius(logits, O.gemm(x, w, "NT")) <= U.TOL[precision]
    dx0 = rng.standard_normal((M, E)).astype(np.float32)
    dx, path = U.run_gemm("NN", dl, w, c0=dx0, precision=precision, return_path=True)          # dX += dL W
    assert path == 0 and O.rel_frobenius(dx - dx0, O.gemm(dl, w, "NN")) <= U.TOL[precision]
    dw, path = U.run_gemm("TN", dl, x, precision=precision, return_path=True)                   # dW = dL^T X
    assert path == 0 and O.rel_frobenius(dw, O.gemm(dl, x, "TN")) <= U.TOL[precision]
    # odd pitch plus epilogues on the coalesced path
    bias = rng.standard_normal(V).astype(np.float32)
    for epi in ("bias_gelu", "causal"):
        out = U.run_gemm("NT", x, w, bias=bias if epi != "causal" else None, epilogue=epi, precision=precision)
        ref = O.gemm(x, w, "NT", bias=bias, epilogue=epi)
        keep = np.ones_like(ref, bool) if epi != "causal" else np.tril(np.ones(ref.shape, bool))
        assert O.rel_frobenius(out[keep], ref[keep]) <= U.TOL[precision]
        if epi == "causal":
            assert np.all(out[~keep] == np.float32(O.CAUSAL_MASK_VALUE))


def test_unaligned_a_with_misaligned_base(gt):
    a, b, _ = U.make_operands("NN", 200, 128, 77, seed=6)          # lda = 77
    from gradtuity_b200 import _lib, gemm as G
    da = U.DeviceBuffer(a, offset_elems=3)                          # base 12 bytes off alignment
    db = U.DeviceBuffer(b)
    dc = U.DeviceBuffer(nbytes=200 * 128 * 4)
    G.gemm(0, 200, 128, 77, da.ptr, 77, db.ptr, 128, dc.ptr, 128)
    _lib.device_status()
    assert O.rel_frobenius(dc.read((200, 128)), O.gemm(a, b, "NN")) <= U.TOL["tf32"]


@pytest.mark.parametrize("layout,M,N,K,epilogue,acc", [
    ("TN", 768, 768, 8192, "none", True),        # the dW GEMM of a 768-wide Linear at 8192 tokens
    ("TN", 768, 3072, 4096, "none", True),
    ("TN", 768, 768, 8192, "none", False),       # direct mode without C +=: C is zeroed, then every share adds
    ("NT", 200, 260, 4100, "none", False),       # direct mode with M, N and K tails
    ("NN", 256, 264, 4100, "bias_relu", False),  # K tail, N tail
    ("NT", 130, 500, 2048, "bias_gelu", False),
])
def test_split_k_shapes(gt, layout, M, N, K, epilogue, acc):
    """Few output tiles and a long K: the K range is shared between CTAs.  Without an epilogue every
    CTA adds its partial sum into C (order of the fp32 additions not fixed); with a bias / activation
    the partial sums are added by a second kernel in a fixed order and the epilogue is applied once,
    which is bitwise repeatable."""
    a, b, rng = U.make_operands(layout, M, N, K, seed=K + N)
    bias = rng.standard_normal(N).astype(np.float32) if epilogue != "none" else None
    c0 = rng.standard_normal((M, N)).astype(np.float32) if acc else None
    out = U.run_gemm(layout, a, b, bias=bias, c0=c0, epilogue=epilogue)
    ref = O.gemm(a, b, layout, bias=bias, epilogue=epilogue, c0=c0)
    base = c0 if acc else 0.0
    assert O.rel_frobenius(out - base, ref - base) <= U.TOL["tf32"]
    again = U.run_gemm(layout, a, b, bias=bias, c0=c0, epilogue=epilogue)
    if epilogue != "none":
        assert np.array_equal(out, again)
    else:
        assert O.rel_frobenius(again - base, out - base) <= 1e-5


@pytest.mark.parametrize("layout,M,N,K,epilogue,acc", [
    ("NN", 8192, 768, 768, "bias", False),      # q/k/v/o projection of GPT-2: 192 tiles on 148 SMs, last wave cut in 3
    ("NT", 8200, 768, 768, "none", True),       # dX with C +=, ragged last row tile
    ("NT", 8192, 3072, 800, "none", False),     # 768 tiles: 28 in the last wave, K tail
    ("TN", 8192, 776, 1024, "bias", False),     # N tail inside the last column tile
    ("NN", 8192, 768, 4096, "bias", False),     # 96 tiles of 256 x 256: the big-tile kernel with its tiles cut along K
    ("NT", 8192, 768, 2048, "none", True),      # the same with C += ...
])
def test_last_wave_split_shapes(gt, layout, M, N, K, epilogue, acc):
    """More tiles than SMs with a last wave at most half full: the tiles of that wave are cut along K
    between CTAs that add their partial sums into C (zeroed under those tiles first unless C += ...)."""
    a, b, rng = U.make_operands(layout, M, N, K, seed=M + K)
    bias = rng.standard_normal(N).astype(np.float32) if epilogue != "none" else None
    c0 = rng.standard_normal((M, N)).astype(np.float32) if acc else None
    out = U.run_gemm(layout, a, b, bias=bias, c0=c0, epilogue=epilogue)
    ref = O.gemm(a, b, layout, bias=bias, epilogue=epilogue, c0=c0)
    base = c0 if acc else 0.0
    assert O.rel_frobenius(out - base, ref - base) <= U.TOL["tf32"]
    # every row block on its own, so that an error confined to the last wave's tiles cannot hide in the norm
    for r0 in range(0, M, 1024):
        sl = slice(r0, min(M, r0 + 1024))
        assert O.rel_frobenius((out - base)[sl], (ref - base)[sl]) <= U.TOL["tf32"]


@pytest.mark.parametrize("layout,M,N,K", [("NN", 300, 200, 96), ("NT", 8192, 3072, 768), ("NN", 8192, 768, 3072), ("TN", 260, 132, 64),
                                          ("NT", 2560, 2048, 4128), ("NN", 8192, 768, 768)])
@pytest.mark.parametrize("kind", ["bias_add", "gelu_grad"])
def test_aux_reading_epilogues(gt, layout, M, N, K, kind):
    """BIAS_ADD: C = A B + bias + aux (Linear + residual add); GELU_GRAD: C = (A B) * gelu'(aux) (dX of the second
    MLP layer with the GELU backward).  Shapes with partial chunks (general form), the two GPT-2 MLP shapes and
    the 768-wide projection (CTA pairs with their last wave cut along K: the residual goes in with share 0, the
    gelu' factor with every share), and a long-K shape that takes the same split in the one-CTA kernel."""
    from gradtuity_b200 import _lib, gemm as G

    a, b, rng = U.make_operands(layout, M, N, K, seed=M + N)
    aux = rng.standard_normal((M, N)).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32) if kind == "bias_add" else None
    da, db, dx = U.DeviceBuffer(a), U.DeviceBuffer(b), U.DeviceBuffer(aux)
    dc = U.DeviceBuffer(np.full((M, N), np.nan, np.float32))
    dbias = U.DeviceBuffer(bias) if bias is not None else None
    epi = _lib.EPI_BIAS_ADD if kind == "bias_add" else _lib.EPI_GELU_GRAD
    G.gemm(U.LAYOUTS[layout], M, N, K, da.ptr, a.shape[1], db.ptr, b.shape[1], dc.ptr, N,
           bias_ptr=dbias.ptr if dbias else 0, aux_ptr=dx.ptr, epilogue=epi)
    _lib.device_status()
    out = dc.read((M, N))
    prod = O.gemm(a, b, layout)
    ref = prod + bias + aux if kind == "bias_add" else prod * O.gelu_tanh_grad(aux.astype(np.float64))
    assert O.rel_frobenius(out, ref) <= U.TOL["tf32"]
    assert np.array_equal(dx.read((M, N)), aux)                     # aux is read, never written


@pytest.mark.parametrize("layout,M,N,K", [("NN", 300, 200, 96), ("NT", 8192, 3072, 768), ("TN", 260, 132, 64), ("NT", 2560, 2048, 4128),
                                          ("NN", 8192, 768, 768), ("NT", 1000, 3072, 768)])
def test_gelu_grad_product_with_column_sums(gt, layout, M, N, K):
    """gt_gemm_gelu_grad_colsum: the same C as the GELU_GRAD epilogue, bit for bit where no K share is involved,
    and colsum += the column sums of C (the first layer's bias gradient), taken from the staged output tiles.
    Shapes with partial chunks and row blocks, the GPT-2 MLP shape, and shapes whose last wave is cut along K
    (every share's partial sum passes through a tile: the sums must still add up)."""
    from gradtuity_b200 import _lib, gemm as G

    a, b, rng = U.make_operands(layout, M, N, K, seed=M + N + 1)
    pre = rng.standard_normal((M, N)).astype(np.float32)
    start = rng.standard_normal(N).astype(np.float32)
    da, db, dp = U.DeviceBuffer(a), U.DeviceBuffer(b), U.DeviceBuffer(pre)
    dc = U.DeviceBuffer(np.full((M, N), np.nan, np.float32))
    guard = np.concatenate([start, np.full(40, 7.0, np.float32)])           # nothing may land beyond column N
    ds = U.DeviceBuffer(guard)
    G.gemm_gelu_grad_colsum(U.LAYOUTS[layout], M, N, K, da.ptr, a.shape[1], db.ptr, b.shape[1], dc.ptr, N, dp.ptr, ds.ptr)
    _lib.device_status()
    out = dc.read((M, N))
    ref = O.gemm(a, b, layout) * O.gelu_tanh_grad(pre.astype(np.float64))
    assert O.rel_frobenius(out, ref) <= U.TOL["tf32"]
    sums = ds.read((N + 40,))
    assert np.array_equal(sums[N:], guard[N:])
    want = start.astype(np.float64) + out.astype(np.float64).sum(axis=0)   # sums of what the kernel itself wrote
    scale = np.abs(out.astype(np.float64)).sum(axis=0) + np.abs(start)
    assert np.all(np.abs(sums[:N] - want) <= 2e-5 * scale + 1e-6)
    assert np.array_equal(dp.read((M, N)), pre)


def test_aux_reading_epilogue_needs_aux_and_tensor_core_path(gt):
    from gradtuity_b200 import _lib, gemm as G

    a, b, _ = U.make_operands("NN", 64, 64, 64, seed=1)
    da, db = U.DeviceBuffer(a), U.DeviceBuffer(b)
    dc = U.DeviceBuffer(np.zeros((64, 64), np.float32))
    with pytest.raises(RuntimeError, match="reads aux"):
        G.gemm(0, 64, 64, 64, da.ptr, 64, db.ptr, 64, dc.ptr, 64, epilogue=_lib.EPI_GELU_GRAD)
    with pytest.raises(RuntimeError, match="tensor-core path"):
        G.gemm(0, 64, 64, 64, da.ptr, 64, db.ptr, 64, dc.ptr, 64, aux_ptr=dc.ptr, epilogue=_lib.EPI_GELU_GRAD,
               precision=U.PRECISIONS["fp32"])


@pytest.mark.parametrize("layout,M,N,K,chunks,epilogue", [
    ("NN", 1000, 260, 200, 3, "none"), ("NT", 512, 128, 96, 1, "bias_relu"), ("TN", 900, 300, 130, 4, "bias"), ("NN", 4096, 512, 256, 8, "bias_gelu")])
def test_gemm_on_host_buffers(gt, layout, M, N, K, chunks, epilogue):
    """gt_gemm_host: operands and result in host memory, uploads / products / downloads of row blocks overlapped."""
    from gradtuity_b200 import gemm as G

    a, b, rng = U.make_operands(layout, M, N, K, seed=M + K + chunks)
    bias = rng.standard_normal(N).astype(np.float32) if epilogue != "none" else None
    out = np.full((M, N + 5), np.nan, np.float32)[:, :N]                 # a row pitch larger than N
    G.matmul_host(a, b, out=out, layout=U.LAYOUTS[layout], bias=bias, epilogue=U.EPILOGUES[epilogue], chunks=chunks)
    ref = O.gemm(a, b, layout, bias=bias, epilogue=epilogue)
    assert O.rel_frobenius(out, ref) <= U.TOL["tf32"]
    out2 = G.matmul_host(a, b, layout=U.LAYOUTS[layout], bias=bias, epilogue=U.EPILOGUES[epilogue], chunks=chunks, precision=U.PRECISIONS["3xtf32"])
    assert O.rel_frobenius(out2, ref) <= (2e-5 if epilogue == "bias_gelu" else U.TOL["3xtf32"])


def test_bitwise_deterministic(gt):
    # one CTA per output tile (no shared K range): the summation order is fixed
    a, b, _ = U.make_operands("TN", 1536, 2048, 512, seed=3)
    assert np.array_equal(U.run_gemm("TN", a, b), U.run_gemm("TN", a, b))


def test_tf32_rounding_beats_truncation_margin(gt):
    # operands are rounded to tf32 (nearest) on the way into shared memory, so the error sits
    # near 3e-4, a factor three inside the 1e-3 bar, independent of K
    for K in (256, 4096):
        a, b, _ = U.make_operands("NT", 256, 256, K, seed=K)
        assert O.rel_frobenius(U.run_gemm("NT", a, b), O.gemm(a, b, "NT")) <= 4.5e-4


# ---- batched ----------------------------------------------------------------------------------

def _run_batched(layout, a, b, *, c0=None, epilogue="none", alpha=1.0, precision="tf32"):
    """a, b: (B0, rows, cols) stored per slice contiguously."""
    from gradtuity_b200 import _lib, gemm as G

    Bn = a.shape[0]
    M = a.shape[2] if layout == "TN" else a.shape[1]
    K = a.shape[1] if layout == "TN" else a.shape[2]
    N = b.shape[1] if layout == "NT" else b.shape[2]
    da, db = U.DeviceBuffer(a), U.DeviceBuffer(b)
    dc = U.DeviceBuffer(c0 if c0 is not None else np.full((Bn, M, N), np.nan, np.float32))
    G.gemm_batched(U.LAYOUTS[layout], M, N, K, da.ptr, a.shape[2], a.shape[1] * a.shape[2], 0,
                   db.ptr, b.shape[2], b.shape[1] * b.shape[2], 0, dc.ptr, N, M * N, 0, Bn, 1,
                   alpha=alpha, accumulate=c0 is not None, epilogue=U.EPILOGUES[epilogue],
                   precision=U.PRECISIONS[precision])
    _lib.device_status()
    return dc.read((Bn, M, N))


@pytest.mark.parametrize("precision", ["tf32", "3xtf32"])
@pytest.mark.parametrize("layout", ["NN", "NT", "TN"])
def test_batched_matches_per_slice_oracle(gt, layout, precision):
    rng = np.random.default_rng(42)
    Bn, M, N, K = 6, 96, 80, 64
    ashape = (Bn, K, M) if layout == "TN" else (Bn, M, K)
    bshape = (Bn, N, K) if layout == "NT" else (Bn, K, N)
    a = rng.standard_normal(ashape).astype(np.float32) / 8
    b = rng.standard_normal(bshape).astype(np.float32) / 8
    out = _run_batched(layout, a, b, precision=precision)
    assert O.rel_frobenius(out, O.gemm(a, b, layout)) <= U.TOL[precision]


def test_batched_causal_scores_in_place_heads(gt):
    """S = Q K^T / sqrt(d) with the causal mask, Q and K read in place from a (B, T, H, d)
    projection output through two batch strides (no (B, H, T, d) copy)."""
    from gradtuity_b200 import _lib, gemm as G

    rng = np.random.default_rng(2)
    B, T, H, d = 2, 256, 3, 64
    q = rng.standard_normal((B, T, H, d)).astype(np.float32)
    k = rng.standard_normal((B, T, H, d)).astype(np.float32)
    dq, dk = U.DeviceBuffer(q), U.DeviceBuffer(k)
    ds = U.DeviceBuffer(np.full((B, H, T, T), np.nan, np.float32))
    G.gemm_batched(U.LAYOUTS["NT"], T, T, d, dq.ptr, H * d, d, T * H * d, dk.ptr, H * d, d, T * H * d,
                   ds.ptr, T, T * T, H * T * T, H, B, alpha=1.0 / 8.0, epilogue=U.EPILOGUES["causal"])
    _lib.device_status()
    s = ds.read((B, H, T, T))
    ref = O.gemm(q.transpose(0, 2, 1, 3), k.transpose(0, 2, 1, 3), "NT", alpha=1.0 / 8.0, epilogue="causal")
    keep = np.tril(np.ones((T, T), bool))
    assert np.all(s[..., ~keep] == np.float32(O.CAUSAL_MASK_VALUE))
    assert O.rel_frobenius(s[..., keep], ref[..., keep]) <= U.TOL["tf32"]


def test_triangular_hints_trim_work_not_results(gt):
    """gt_gemm_batched_ex flags: with A declared lower-triangular the k-blocks beyond a row tile's
    diagonal block are never read (NaN there must not show), and causal score tiles wholly above the
    diagonal are left unwritten."""
    from gradtuity_b200 import _lib, gemm as G
    from gradtuity_b200._lib import GEMM_A_LOWER, GEMM_AT_LOWER, GEMM_CAUSAL_SKIP_MASKED

    rng = np.random.default_rng(17)
    Bn, S, D = 3, 384, 64
    tri = np.tril(rng.standard_normal((Bn, S, S))).astype(np.float32)
    poisoned = tri.copy()
    for i in range(S):                                   # beyond the end of row i's 128-wide diagonal block
        poisoned[:, i, (i // 128 + 1) * 128:] = np.nan
    v = rng.standard_normal((Bn, S, D)).astype(np.float32)
    dA, dV, dC = U.DeviceBuffer(poisoned), U.DeviceBuffer(v), U.DeviceBuffer(nbytes=Bn * S * D * 4)
    G.gemm_batched(0, S, D, S, dA.ptr, S, S * S, 0, dV.ptr, D, S * D, 0, dC.ptr, D, S * D, 0, Bn, flags=GEMM_A_LOWER)
    _lib.device_status()
    assert O.rel_frobenius(dC.read((Bn, S, D)), O.gemm(tri, v, "NN")) <= U.TOL["tf32"]
    # transposed use: A stored (K, M) with A[k, m] = 0 for k < m  ->  C = A^T V
    G.gemm_batched(2, S, D, S, dA.ptr, S, S * S, 0, dV.ptr, D, S * D, 0, dC.ptr, D, S * D, 0, Bn, flags=GEMM_AT_LOWER)
    _lib.device_status()
    assert O.rel_frobenius(dC.read((Bn, S, D)), O.gemm(tri, v, "TN")) <= U.TOL["tf32"]
    # causal scores with masked tiles skipped
    q = rng.standard_normal((Bn, S, D)).astype(np.float32); k = rng.standard_normal((Bn, S, D)).astype(np.float32)
    dQ, dK = U.DeviceBuffer(q), U.DeviceBuffer(k)
    dS = U.DeviceBuffer(np.full((Bn, S, S), 7.0, np.float32))
    G.gemm_batched(1, S, S, D, dQ.ptr, D, S * D, 0, dK.ptr, D, S * D, 0, dS.ptr, S, S * S, 0, Bn,
                   epilogue=U.EPILOGUES["causal"], flags=GEMM_CAUSAL_SKIP_MASKED)
    _lib.device_status()
    sc = dS.read((Bn, S, S))
    keep = np.tril(np.ones((S, S), bool))
    assert O.rel_frobenius(sc[:, keep], O.gemm(q, k, "NT")[:, keep]) <= U.TOL["tf32"]
    assert np.all(sc[:, 0:128, 256:384] == 7.0)          # a tile wholly above the diagonal: untouched
    with pytest.raises(RuntimeError, match="square"):
        G.gemm_batched(0, S, D, 128, dA.ptr, S, S * S, 0, dV.ptr, D, S * D, 0, dC.ptr, D, S * D, 0, Bn, flags=GEMM_A_LOWER)


# ---- error behaviour --------------------------------------------------------------------------

def test_bounded_wait_gives_up_and_the_context_survives(gt):
    """A wait that can never be satisfied (a barrier nothing arrives on) runs into its limit, the
    kernel returns, the status word reports the timeout once, and the next GEMM is correct."""
    lib = gt.load_library()
    gt.check(lib.gt_selftest_bounded_wait(gt.context(), 2_000_000), "gt_selftest_bounded_wait")      # about 1 ms
    with pytest.raises(RuntimeError, match="bounded device-side wait"):
        gt.device_status()
    assert gt.device_status() == 0                                  # the word was cleared by the read
    a, b, _ = U.make_operands("NN", 256, 256, 256, seed=2)
    assert O.rel_frobenius(U.run_gemm("NN", a, b), O.gemm(a, b, "NN")) <= U.TOL["tf32"]


def test_invalid_arguments_return_status_not_crash(gt):
    from gradtuity_b200 import gemm as G

    buf = U.DeviceBuffer(np.zeros((64, 64), np.float32))
    with pytest.raises(RuntimeError, match="invalid argument"):
        G.gemm(0, 64, 64, 64, 0, 64, buf.ptr, 64, buf.ptr, 64)            # null A
    with pytest.raises(RuntimeError, match="invalid argument"):
        G.gemm(7, 64, 64, 64, buf.ptr, 64, buf.ptr, 64, buf.ptr, 64)      # bad layout
    with pytest.raises(RuntimeError, match="invalid argument"):
        G.gemm(0, 64, 64, 64, buf.ptr, 32, buf.ptr, 64, buf.ptr, 64)      # lda < K
    with pytest.raises(RuntimeError, match="bias"):
        G.gemm(0, 64, 64, 64, buf.ptr, 64, buf.ptr, 64, buf.ptr, 64, epilogue=1)   # bias epilogue, no bias
    with pytest.raises(RuntimeError, match="invalid argument"):
        G.gemm(0, 0, 64, 64, buf.ptr, 64, buf.ptr, 64, buf.ptr, 64)       # M = 0
    gt.device_status()


# ---- full-size cases: size-independent properties and sampled rows ------------------------------

@pytest.mark.parametrize("precision,M,N,K", [("tf32", 8192, 8192, 8192), ("tf32", 8192, 768, 3072),
                                            ("tf32", 8192, 3072, 768), ("3xtf32", 2048, 2048, 8192)])
def test_full_size_sampled_rows_and_linearity(gt, precision, M, N, K):
    """At the benchmark sizes the float64 oracle is run on 16 sampled rows of C, and the whole
    result is checked through linearity: gemm(A, B1 + B2) == gemm(A, B1) + gemm(A, B2)."""
    from gradtuity_b200 import _lib, gemm as G

    rng = np.random.default_rng(1)
    a = rng.standard_normal((M, K), dtype=np.float32) / np.float32(np.sqrt(K))
    b1 = rng.standard_normal((K, N), dtype=np.float32) / np.float32(np.sqrt(K))
    b2 = rng.standard_normal((K, N), dtype=np.float32) / np.float32(np.sqrt(K))
    da, db1, db2, db12 = U.DeviceBuffer(a), U.DeviceBuffer(b1), U.DeviceBuffer(b2), U.DeviceBuffer(b1 + b2)
    dc1, dc12 = U.DeviceBuffer(nbytes=M * N * 4), U.DeviceBuffer(nbytes=M * N * 4)
    prec = U.PRECISIONS[precision]
    G.gemm(0, M, N, K, da.ptr, K, db1.ptr, N, dc1.ptr, N, precision=prec)
    c1 = dc1.read((M, N))
    G.gemm(0, M, N, K, da.ptr, K, db2.ptr, N, dc1.ptr, N, accumulate=True, precision=prec)   # C1 += A B2
    G.gemm(0, M, N, K, da.ptr, K, db12.ptr, N, dc12.ptr, N, precision=prec)
    _lib.device_status()
    c_sum, c12 = dc1.read((M, N)), dc12.read((M, N))
    rows = np.arange(0, M, M // 16)
    ref = a[rows].astype(np.float64) @ b1.astype(np.float64)
    assert O.rel_frobenius(c1[rows], ref) <= U.TOL[precision]
    # two roundings of B versus one: the bound is twice the single-GEMM bar
    assert O.rel_frobenius(c_sum, c12) <= 2 * U.TOL[precision]


@pytest.mark.parametrize("layout", ["NN", "NT", "TN"])
@pytest.mark.parametrize("M,N,K,epilogue,acc", [(4096, 4096, 2056, "none", False), (4000, 4104, 2048, "bias_gelu", False),
                                                (3968, 4360, 2304, "none", True)])
def test_big_tile_kernel(gt, layout, M, N, K, epilogue, acc):
    """Problems with at least one wave of 256 x 256 tiles and K >= 2048 run on the big-tile kernel:
    ragged M / N / K, every layout, fused epilogue with stored pre-activation, accumulate."""
    from gradtuity_b200 import _lib, gemm as G

    a, b, rng = U.make_operands(layout, M, N, K, seed=M + K)
    bias = rng.standard_normal(N).astype(np.float32) if epilogue != "none" else None
    c0 = rng.standard_normal((M, N)).astype(np.float32) if acc else None
    da, db = U.DeviceBuffer(a), U.DeviceBuffer(b)
    dc = U.DeviceBuffer(c0 if acc else np.full((M, N), np.nan, np.float32))
    dbias = U.DeviceBuffer(bias) if bias is not None else None
    daux = U.DeviceBuffer(np.full((M, N), np.nan, np.float32)) if epilogue == "bias_gelu" else None
    G.gemm(U.LAYOUTS[layout], M, N, K, da.ptr, a.shape[1], db.ptr, b.shape[1], dc.ptr, N,
           bias_ptr=dbias.ptr if dbias else 0, aux_ptr=daux.ptr if daux else 0, accumulate=acc,
           epilogue=U.EPILOGUES[epilogue])
    _lib.device_status()
    out = dc.read((M, N))
    assert not np.isnan(out).any()
    rows = np.unique(np.concatenate([np.arange(0, M, 97), [M - 1, 127, 128, 255, 256]]))
    a_rows = a[:, rows].T if layout == "TN" else a[rows]
    ref, pre = O.gemm(a_rows, b, "NT" if layout == "NT" else "NN", bias=bias, epilogue=epilogue,
                      c0=c0[rows] if acc else None, return_pre=True)
    base = c0[rows] if acc else 0.0
    assert O.rel_frobenius(out[rows] - base, ref - base) <= U.TOL["tf32"]
    if daux is not None:
        assert O.rel_frobenius(daux.read((M, N))[rows], pre) <= U.TOL["tf32"]


def test_3xtf32_error_does_not_grow_with_k(gt):
    """The tensor core truncates on every accumulate; 3xTF32 mode therefore sums K-chunks in
    fp32 registers.  Without that the error at K = 8192 is about 6e-5."""
    for K in (1024, 8192):
        a, b, _ = U.make_operands("NT", 256, 256, K, seed=K)
        assert O.rel_frobenius(U.run_gemm("NT", a, b, precision="3xtf32"), O.gemm(a, b, "NT")) <= 5e-6


def test_two_streams_share_one_context(gt):
    """GEMMs of ONE context enqueued alternately on two streams: the scratch they share (the 3xTF32 operand copies,
    the last-wave flags) is handed from stream to stream in order, so every result is right although nothing on the
    host waits between the calls."""
    import ctypes
    from ctypes import byref, c_void_p

    from gradtuity_b200 import _lib

    rt = ctypes.CDLL("libcudart.so.12")
    rt.cudaStreamCreateWithFlags.argtypes = [ctypes.POINTER(c_void_p), ctypes.c_uint]
    rt.cudaStreamSynchronize.argtypes = [c_void_p]
    rt.cudaStreamDestroy.argtypes = [c_void_p]
    side = c_void_p()
    assert rt.cudaStreamCreateWithFlags(byref(side), 1) == 0             # non-blocking
    lib, ctx = _lib.load_library(), _lib.context()
    cases = []
    for i, (layout, M, N, K, prec) in enumerate([("NN", 384, 640, 520, "3xtf32"), ("NT", 8192, 768, 768, "tf32"),
                                                 ("TN", 200, 136, 96, "3xtf32"), ("NN", 8192, 768, 768, "tf32"),
                                                 ("NT", 640, 384, 1032, "3xtf32"), ("TN", 768, 768, 4096, "tf32")]):
        a, b, _ = U.make_operands(layout, M, N, K, seed=70 + i)
        da, db = U.DeviceBuffer(a), U.DeviceBuffer(b)
        dc = U.DeviceBuffer(np.full((M, N), np.nan, np.float32))
        cases.append((layout, M, N, K, prec, a, b, da, db, dc))
    gt.device_status()
    for rep in range(2):
        for i, (layout, M, N, K, prec, a, b, da, db, dc) in enumerate(cases):
            stream = side if (i + rep) % 2 else None                       # None: the context's own stream
            _lib.check(lib.gt_gemm(ctx, U.LAYOUTS[layout], M, N, K, c_void_p(da.ptr), a.shape[1], c_void_p(db.ptr), b.shape[1],
                                   c_void_p(dc.ptr), N, None, None, 1.0, 0, 0, U.PRECISIONS[prec], stream), "gt_gemm")
    assert rt.cudaStreamSynchronize(side) == 0
    gt.device_status()
    for layout, M, N, K, prec, a, b, da, db, dc in cases:
        assert O.rel_frobenius(dc.read((M, N)), O.gemm(a, b, layout)) <= U.TOL[prec], (layout, M, N, K, prec)
    rt.cudaStreamDestroy(side)
