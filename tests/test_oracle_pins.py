"""CPU: the float64 oracle against the reference's own known answers and the pinned vectors."""
import numpy as np
import pytest

from oracle import gemm_oracle as O
from tests import _util as U


@pytest.mark.parametrize("case", U.known_answers(), ids=lambda c: c["name"])
def test_oracle_matches_reference_known_answers(case):
    op = case["op"]
    if op == "matmul":
        y = O.gemm(np.array(case["a"], float), np.array(case["b"], float), "NN")
        np.testing.assert_allclose(y, np.array(case["y"], float), rtol=1e-6)
    elif op == "matmul_sum_backward":
        a, b = np.array(case["a"], float), np.array(case["b"], float)
        dc = np.ones((a.shape[0], b.shape[1]))
        if case["a_grad"]:
            np.testing.assert_allclose(O.gemm(dc, b, "NT"), np.array(case["da"], float), rtol=1e-6)
        if case["b_grad"]:
            np.testing.assert_allclose(O.gemm(a, dc, "TN"), np.array(case["db"], float), rtol=1e-6)
    elif op in ("linear", "linear_relu"):
        r = O.linear_forward_backward(case["x"], case["w"], case["bias"], np.ones((len(case["x"]), len(case["bias"]))),
                                      activation="relu" if op == "linear_relu" else "none")
        np.testing.assert_allclose(r["y"], np.array(case["y"], float), rtol=1e-6, atol=1e-12)
    elif op in ("linear_sum_backward", "linear_relu_sum_backward"):
        r = O.linear_forward_backward(case["x"], case["w"], case["bias"], np.ones((len(case["x"]), len(case["bias"]))),
                                      activation="relu" if "relu" in op else "none")
        for key, name in (("dx", "dx"), ("dw", "dw"), ("dbias", "db")):
            if key in case:
                np.testing.assert_allclose(r[name], np.array(case[key], float), rtol=1e-6, atol=1e-12)
    else:
        raise AssertionError(op)


@pytest.mark.parametrize("kind,M,N,K", U.PHASE4_CASES)
def test_oracle_matches_phase4_vectors(kind, M, N, K):
    layout, a, b, bias, c0 = U.phase4_inputs(kind, M, N, K)
    epi = {"matmul": "none", "matmul_bias": "bias", "matmul_bias_relu": "bias_relu"}.get(kind, "none")
    y = O.gemm(a, b, layout, bias=bias, epilogue=epi, c0=c0)
    gold = U.phase4_vectors()[U.phase4_key(kind, M, N, K)]
    # fp32 scalar accumulation against float64: a few ulp of the largest partial sum
    np.testing.assert_allclose(y, gold, rtol=2e-5, atol=2e-6)


def test_gelu_matches_reference_formula_points():
    # 0.5 x (1 + tanh(0.79788456 (x + 0.044715 x^3))): gradtuity/kernels_cuda/elemwise_kernels.py:118-124
    x = np.array([-3.0, -1.0, 0.0, 0.5, 2.0])
    want = 0.5 * x * (1 + np.tanh(0.7978845608028654 * (x + 0.044715 * x ** 3)))
    np.testing.assert_allclose(O.gelu_tanh(x), want, rtol=1e-15)
    h = 1e-6
    np.testing.assert_allclose(O.gelu_tanh_grad(x), (O.gelu_tanh(x + h) - O.gelu_tanh(x - h)) / (2 * h), rtol=1e-6, atol=1e-8)


def test_causal_softmax_masks_to_exact_zero():
    # masked probabilities are exactly 0.0: gradtuity/tests/test_fused_softmax.py:70-79
    rng = np.random.default_rng(0)
    s = rng.standard_normal((2, 3, 8, 8))
    p = O.causal_softmax(s)
    iu = np.triu_indices(8, 1)
    assert np.all(p[..., iu[0], iu[1]] == 0.0)
    np.testing.assert_allclose(p.sum(-1), 1.0, rtol=1e-12)


def test_causal_epilogue_and_accumulate():
    rng = np.random.default_rng(1)
    a, b = rng.standard_normal((5, 4)), rng.standard_normal((6, 4))
    y = O.gemm(a, b, "NT", epilogue="causal", alpha=0.5)
    full = 0.5 * a @ b.T
    for i in range(5):
        for j in range(6):
            assert y[i, j] == (O.CAUSAL_MASK_VALUE if j > i else full[i, j])
    c0 = rng.standard_normal((5, 6))
    np.testing.assert_allclose(O.gemm(a, b, "NT", c0=c0), c0 + a @ b.T)


def test_attention_oracle_consistency():
    # backward of the oracle agrees with finite differences of its own forward
    rng = np.random.default_rng(2)
    q, k, v, do = (rng.standard_normal((1, 2, 6, 4)) for _ in range(4))
    r = O.attention_forward_backward(q, k, v, do)
    def loss(qq):
        return (O.attention_forward_backward(qq, k, v, do)["o"] * do).sum()
    h = 1e-6
    e = np.zeros_like(q); e[0, 1, 3, 2] = h
    fd = (loss(q + e) - loss(q - e)) / (2 * h)
    assert abs(fd - r["dq"][0, 1, 3, 2]) < 1e-6


def test_gpt2_oracle_backward_matches_finite_differences():
    from oracle.gpt2_oracle import GPT2Oracle

    rng = np.random.default_rng(3)
    V, S, E, H, L, B = 11, 5, 8, 2, 2, 2
    p = {"wte.weight": rng.standard_normal((V, E)) * 0.3, "wpe.embed.weight": rng.standard_normal((S, E)) * 0.3,
         "ln_f.gamma": 1 + 0.1 * rng.standard_normal(E), "ln_f.beta": 0.1 * rng.standard_normal(E)}
    for l in range(L):
        pre = f"blocks.{l}."
        for ln in ("ln1", "ln2"):
            p[pre + ln + ".gamma"] = 1 + 0.1 * rng.standard_normal(E)
            p[pre + ln + ".beta"] = 0.1 * rng.standard_normal(E)
        for w in ("Wq", "Wk", "Wv", "Wo"):
            p[pre + "attn." + w] = rng.standard_normal((E, E)) * 0.3
            p[pre + "attn.b" + w[1]] = rng.standard_normal(E) * 0.1
        p[pre + "mlp_fc1.weight"] = rng.standard_normal((E, 4 * E)) * 0.3
        p[pre + "mlp_fc1.bias"] = rng.standard_normal(4 * E) * 0.1
        p[pre + "mlp_fc2.weight"] = rng.standard_normal((4 * E, E)) * 0.3
        p[pre + "mlp_fc2.bias"] = rng.standard_normal(E) * 0.1
    ids = rng.integers(0, V, (B, S))
    labels = rng.integers(0, V, B * S)
    orc = GPT2Oracle(L, H)
    loss, g = orc.loss_and_grads(p, ids, labels)
    assert set(g) == set(p)
    h = 1e-6
    for key in ["wte.weight", "wpe.embed.weight", "blocks.0.attn.Wk", "blocks.1.attn.bq", "blocks.0.ln1.gamma",
                "blocks.1.mlp_fc1.weight", "blocks.0.mlp_fc2.bias", "ln_f.beta", "blocks.1.attn.Wo"]:
        idx = tuple(rng.integers(0, s) for s in p[key].shape)
        q = {k: v.copy() for k, v in p.items()}
        q[key][idx] += h
        lp = orc.loss_and_grads(q, ids, labels)[0]
        q[key][idx] -= 2 * h
        lm = orc.loss_and_grads(q, ids, labels)[0]
        assert abs((lp - lm) / (2 * h) - g[key][idx]) < 1e-6, key


def test_conv2d_oracle_against_the_defining_sum_and_finite_differences():
    """The vectorised float64 convolution oracle equals the seven-loop definition, and its gradients
    equal finite differences (no reference test holds conv2d values: gradtuity/tests/test_nn.py:325-380
    checks shapes only)."""
    rng = np.random.default_rng(0)
    N, C, H, W, Co, kH, kW, s, p = 2, 3, 6, 7, 4, 3, 2, 2, 1
    x = rng.standard_normal((N, C, H, W)); w = rng.standard_normal((Co, C, kH, kW)); b = rng.standard_normal(Co)
    Ho, Wo = (H + 2 * p - kH) // s + 1, (W + 2 * p - kW) // s + 1
    dy = rng.standard_normal((N, Co, Ho, Wo))
    r = O.conv2d_forward_backward(x, w, b, dy, s, p)
    y = np.zeros((N, Co, Ho, Wo))
    for n in range(N):
        for co in range(Co):
            for ho in range(Ho):
                for wo in range(Wo):
                    acc = b[co]
                    for c in range(C):
                        for kh in range(kH):
                            for kw in range(kW):
                                h, ww = ho * s - p + kh, wo * s - p + kw
                                if 0 <= h < H and 0 <= ww < W:
                                    acc += x[n, c, h, ww] * w[co, c, kh, kw]
                    y[n, co, ho, wo] = acc
    assert np.abs(y - r["y"]).max() < 1e-12
    eps = 1e-6
    loss = lambda xx, ww_, bb: (O.conv2d_forward_backward(xx, ww_, bb, dy, s, p)["y"] * dy).sum()
    base = loss(x, w, b)
    for idx in [(1, 2, 3, 4), (0, 0, 0, 0)]:
        xp = x.copy(); xp[idx] += eps
        assert abs((loss(xp, w, b) - base) / eps - r["dx"][idx]) < 1e-4
    wp = w.copy(); wp[2, 1, 1, 1] += eps
    assert abs((loss(x, wp, b) - base) / eps - r["dw"][2, 1, 1, 1]) < 1e-4
    bp = b.copy(); bp[3] += eps
    assert abs((loss(x, w, bp) - base) / eps - r["db"][3]) < 1e-4
