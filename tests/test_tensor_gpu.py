"""GPU: the Tensor API on the reference's own known answers and numpy comparisons
(gradtuity/tests/test_tensor.py:1276-1375, 1729-1875; gradtuity/tests/test_nn.py:1165-1450)."""
import numpy as np
import pytest

from oracle import gemm_oracle as O
from tests import _util as U

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def T(gt):
    from gradtuity_b200.tensor import Tensor
    return Tensor


def _f(x):
    return [[float(v) for v in row] for row in x] if isinstance(x[0], list) else [float(v) for v in x]


@pytest.mark.parametrize("case", U.known_answers(), ids=lambda c: c["name"])
def test_reference_known_answers(T, case):
    op = case["op"]
    if op == "matmul":
        y = T(_f(case["a"])).matmul(T(_f(case["b"])))
        assert y.shape == (len(case["a"]), len(case["b"][0]))
        np.testing.assert_allclose(np.array(y.to_list()), np.array(case["y"], float), rtol=1e-6)
    elif op == "matmul_sum_backward":
        a = T(_f(case["a"]), requires_grad=case["a_grad"])
        b = T(_f(case["b"]), requires_grad=case["b_grad"])
        a.matmul(b).sum().backward()
        for t, key in ((a, "da"), (b, "db")):
            if case[key] is None:
                assert t.grad is None
            else:
                np.testing.assert_allclose(np.array(t.grad.to_list()), np.array(case[key], float), rtol=1e-6)
    elif op in ("linear", "linear_relu"):
        x, w, b = T(_f(case["x"])), T(_f(case["w"])), T(_f(case["bias"]))
        y = getattr(x, op)(w, b)
        np.testing.assert_allclose(np.array(y.to_list()), np.array(case["y"], float), rtol=1e-6, atol=1e-7)
    else:
        full = "dw" in case or "dbias" in case
        x = T(_f(case["x"]), requires_grad=True)
        w = T(_f(case["w"]), requires_grad=full)
        b = T(_f(case["bias"]), requires_grad=full)
        y = x.linear_relu(w, b) if "relu" in op else x.linear(w, b)
        y.sum().backward()
        if "dx" in case:
            np.testing.assert_allclose(np.array(x.grad.to_list()), np.array(case["dx"], float), rtol=1e-6, atol=1e-7)
        if "dw" in case:
            np.testing.assert_allclose(np.array(w.grad.to_list()), np.array(case["dw"], float), rtol=1e-6, atol=1e-7)
        if "dbias" in case:
            np.testing.assert_allclose(np.array(b.grad.to_list()), np.array(case["dbias"], float), rtol=1e-6, atol=1e-7)
        if not full:
            assert w.grad is None and b.grad is None


def test_matmul_error_messages(T):
    with pytest.raises(ValueError, match="2D"):
        T([1.0, 2.0, 3.0]).matmul(T([[1.0], [2.0], [3.0]]))
    with pytest.raises(ValueError, match="mismatch"):
        T([[1.0, 2.0]]).matmul(T([[1.0, 2.0, 3.0]]))
    c = T([[1.0, 2.0], [3.0, 4.0]]).matmul(T([[1.0, 0.0], [0.0, 1.0]]))
    assert c.requires_grad is False and c._backward is None


def test_linear_error_messages(T):
    with pytest.raises(ValueError, match="shape mismatch"):
        T([[1.0, 2.0]]).linear(T([[1.0], [2.0], [3.0]]), T([1.0]))
    with pytest.raises(ValueError, match="bias size"):
        T([[1.0, 2.0]]).linear(T([[1.0, 2.0], [3.0, 4.0]]), T([1.0, 2.0, 3.0]))
    with pytest.raises(ValueError, match="shape mismatch"):
        T([[1.0, 2.0]]).linear_relu(T([[1.0], [2.0], [3.0]]), T([1.0]))


def test_linear_matches_matmul_plus_bias(T):
    x = T([[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]])
    w = T([[0.1, 0.2, 0.3], [0.4, 0.5, 0.6]])
    b = T([1.0, 2.0, 3.0])
    np.testing.assert_allclose(np.array(x.linear(w, b).to_list()), np.array(x.matmul(w).add_bias(b).to_list()), rtol=1e-5)


def test_linear_backward_accumulates_into_preset_grads(T):
    x = T([[1.0, 1.0]], requires_grad=True)
    w = T([[1.0, 1.0], [1.0, 1.0]], requires_grad=True)
    b = T([0.0, 0.0], requires_grad=True)
    x.grad, w.grad, b.grad = T._ones((1, 2)), T._ones((2, 2)), T._ones((2,))
    x.linear(w, b).sum().backward()
    np.testing.assert_allclose(np.array(x.grad.to_list()), [[3.0, 3.0]])
    np.testing.assert_allclose(np.array(w.grad.to_list()), [[2.0, 2.0], [2.0, 2.0]])
    np.testing.assert_allclose(np.array(b.grad.to_list()), [2.0, 2.0])


def test_linear_relu_backward_matches_separate_ops(T):
    def build():
        return (T([[1.0, 2.0], [3.0, 4.0]], requires_grad=True), T([[0.5, 0.2], [0.3, 0.4]], requires_grad=True),
                T([0.1, -0.1], requires_grad=True))
    x1, w1, b1 = build()
    x2, w2, b2 = build()
    x1.linear_relu(w1, b1).sum().backward()
    x2.linear(w2, b2).relu().sum().backward()
    for p, q in ((x1, x2), (w1, w2), (b1, b2)):
        np.testing.assert_allclose(np.array(p.grad.to_list()), np.array(q.grad.to_list()), rtol=1e-5)


@pytest.mark.parametrize("shape_a,shape_b", [((3, 5, 7), (3, 7, 4)), ((2, 3, 6, 8), (2, 3, 8, 5))])
def test_bmm_matches_numpy(T, shape_a, shape_b):
    rng = np.random.default_rng(42)
    a = rng.standard_normal(shape_a).astype(np.float32)
    b = rng.standard_normal(shape_b).astype(np.float32)
    out = T.from_numpy(a).bmm(T.from_numpy(b))
    assert out.shape == shape_a[:-1] + (shape_b[-1],)
    np.testing.assert_allclose(out.numpy(), np.matmul(a, b), rtol=0.01, atol=0.01)


def test_bmm_backward_and_double_use(T):
    rng = np.random.default_rng(7)
    a = rng.standard_normal((4, 16, 24)).astype(np.float32)
    b = rng.standard_normal((4, 24, 8)).astype(np.float32)
    ta, tb = T.from_numpy(a, requires_grad=True), T.from_numpy(b, requires_grad=True)
    ta.bmm(tb).sum().backward()
    ones = np.ones((4, 16, 8))
    assert O.rel_frobenius(ta.grad.numpy(), O.gemm(ones, b, "NT")) <= 1e-3
    assert O.rel_frobenius(tb.grad.numpy(), O.gemm(a, ones, "TN")) <= 1e-3
    # the same tensor used twice accumulates twice the gradient (gradtuity/tests/test_tensor.py:1354-1375)
    ta2, tb2 = T.from_numpy(a, requires_grad=True), T.from_numpy(b, requires_grad=True)
    (ta2.bmm(tb2).sum() + ta2.bmm(tb2).sum()).backward()
    np.testing.assert_allclose(ta2.grad.numpy(), 2 * ta.grad.numpy(), rtol=1e-5)


def test_bmm_error_messages(T):
    t3 = T.from_numpy(np.zeros((2, 3, 4), np.float32))
    with pytest.raises(ValueError, match="ndim 3 or 4"):
        T([[1.0]]).bmm(T([[1.0]]))
    with pytest.raises(ValueError, match="same ndim"):
        t3.bmm(T.from_numpy(np.zeros((1, 2, 4, 4), np.float32)))
    with pytest.raises(ValueError, match="batch"):
        t3.bmm(T.from_numpy(np.zeros((3, 4, 4), np.float32)))
    with pytest.raises(ValueError, match="inner"):
        t3.bmm(T.from_numpy(np.zeros((2, 5, 4), np.float32)))


def test_linear_tied_values_and_grads(T):
    rng = np.random.default_rng(0)
    x = rng.standard_normal((48, 32)).astype(np.float32)
    w = rng.standard_normal((100, 32)).astype(np.float32)     # (V, E); V = 100: dL has pitch 100
    dy = rng.standard_normal((48, 100)).astype(np.float32)
    tx, tw = T.from_numpy(x, requires_grad=True), T.from_numpy(w, requires_grad=True)
    y = tx.linear_tied(tw)
    ref = O.linear_tied_forward_backward(x, w, dy)
    assert O.rel_frobenius(y.numpy(), ref["y"]) <= 1e-3
    y.mul(T.from_numpy(dy)).sum().backward()
    assert O.rel_frobenius(tx.grad.numpy(), ref["dx"]) <= 1e-3
    assert O.rel_frobenius(tw.grad.numpy(), ref["dw"]) <= 1e-3


def test_linear_tied_large_odd_vocabulary_repack_path(T):
    """M * V large enough and V odd: the backward copies dL once to a padded pitch so that both of
    its GEMMs read it through TMA."""
    rng = np.random.default_rng(1)
    M, V, E = 2048, 2051, 64
    x = (rng.standard_normal((M, E)) / 8).astype(np.float32)
    w = (rng.standard_normal((V, E)) / 8).astype(np.float32)
    dy = (rng.standard_normal((M, V)) / 45).astype(np.float32)
    tx, tw = T.from_numpy(x, requires_grad=True), T.from_numpy(w, requires_grad=True)
    y = tx.linear_tied(tw)
    y.mul(T.from_numpy(dy)).sum().backward()
    ref = O.linear_tied_forward_backward(x, w, dy)
    assert O.rel_frobenius(y.numpy(), ref["y"]) <= 1e-3
    assert O.rel_frobenius(tx.grad.numpy(), ref["dx"]) <= 1e-3
    assert O.rel_frobenius(tw.grad.numpy(), ref["dw"]) <= 1e-3


def test_linear_tied_padded_logits_through_view_and_cross_entropy(T):
    """Large logits with an odd vocabulary are stored with padded rows; view() and cross_entropy read
    and write them in place (no packed copy), numpy() packs.  Loss, dX and dW against float64."""
    rng = np.random.default_rng(5)
    Bn, S, V, E = 2, 1024, 2051, 64
    M = Bn * S
    x = (rng.standard_normal((M, E)) / 4).astype(np.float32)
    w = (rng.standard_normal((V, E)) / 4).astype(np.float32)
    tgt = rng.integers(0, V, M)
    tx, tw = T.from_numpy(x, requires_grad=True), T.from_numpy(w, requires_grad=True)
    logits = tx.linear_tied(tw).view((Bn, S, V))
    assert logits._pitch == 2080 and logits.shape == (Bn, S, V)
    flat = logits.view((M, V))
    assert flat._pitch == 2080
    loss = flat.cross_entropy(T.from_numpy(tgt.astype(np.float32)), reduction="mean")
    loss.backward()
    z = x.astype(np.float64) @ w.astype(np.float64).T
    zmax = z.max(axis=1, keepdims=True)
    lse = zmax[:, 0] + np.log(np.exp(z - zmax).sum(axis=1))
    ref_loss = float(np.mean(lse - z[np.arange(M), tgt]))
    dz = np.exp(z - lse[:, None])
    dz[np.arange(M), tgt] -= 1.0
    dz /= M
    assert abs(loss.item() - ref_loss) <= 1e-4 * abs(ref_loss)
    assert O.rel_frobenius(tx.grad.numpy(), dz @ w.astype(np.float64)) <= 1e-3
    assert O.rel_frobenius(tw.grad.numpy(), dz.T @ x.astype(np.float64)) <= 1e-3
    # reading the logits packs the rows; the values are the GEMM's
    out = logits.numpy()
    assert out.shape == (Bn, S, V) and logits._pitch is None
    assert O.rel_frobenius(out.reshape(M, V), z) <= 1e-3


@pytest.mark.parametrize("N,C,H,W,Co,k,stride,pad", [
    (2, 1, 28, 28, 8, 3, 1, 1),        # first layer of the MNIST CNN: K = 9, the weight rows are not 16-byte aligned
    (3, 32, 14, 14, 64, 3, 1, 1),      # K = 288: tensor-core path
    (2, 4, 9, 11, 6, (3, 2), 2, 0),    # ragged: rectangular kernel, stride 2, no padding
])
def test_conv2d_forward_and_backward(T, N, C, H, W, Co, k, stride, pad):
    """conv2d through im2col and the GEMM kernels (NT forward with bias, TN for dW, NN for dcol) against a
    float64 NCHW convolution."""
    kH, kW = (k, k) if isinstance(k, int) else k
    rng = np.random.default_rng(N * 100 + C)
    x = rng.standard_normal((N, C, H, W)).astype(np.float32)
    w = (rng.standard_normal((Co, C, kH, kW)) / np.sqrt(C * kH * kW)).astype(np.float32)
    b = rng.standard_normal(Co).astype(np.float32)
    Ho, Wo = (H + 2 * pad - kH) // stride + 1, (W + 2 * pad - kW) // stride + 1
    dy = rng.standard_normal((N, Co, Ho, Wo)).astype(np.float32)
    tx, tw, tb = (T.from_numpy(a, requires_grad=True) for a in (x, w, b))
    y = tx.conv2d(tw, tb, stride=stride, padding=pad)
    assert y.shape == (N, Co, Ho, Wo)
    ref = O.conv2d_forward_backward(x, w, b, dy, stride, pad)
    assert O.rel_frobenius(y.numpy(), ref["y"]) <= 1e-3
    y.mul(T.from_numpy(dy)).sum().backward()
    assert O.rel_frobenius(tx.grad.numpy(), ref["dx"]) <= 1e-3
    assert O.rel_frobenius(tw.grad.numpy(), ref["dw"]) <= 1e-3
    assert O.rel_frobenius(tb.grad.numpy(), ref["db"]) <= 1e-3


def test_conv2d_argument_errors_and_module(T):
    from gradtuity_b200.nn import Conv2d

    x = T.from_numpy(np.zeros((1, 2, 5, 5), np.float32))
    with pytest.raises(ValueError, match="4D input"):
        T.from_numpy(np.zeros((2, 5, 5), np.float32)).conv2d(x, x)
    with pytest.raises(ValueError, match="input channels"):
        x.conv2d(T.from_numpy(np.zeros((3, 1, 3, 3), np.float32)), T.from_numpy(np.zeros(3, np.float32)))
    with pytest.raises(ValueError, match="bias size"):
        x.conv2d(T.from_numpy(np.zeros((3, 2, 3, 3), np.float32)), T.from_numpy(np.zeros(4, np.float32)))
    with pytest.raises(ValueError, match="spatial size invalid"):
        x.conv2d(T.from_numpy(np.zeros((3, 2, 7, 7), np.float32)), T.from_numpy(np.zeros(3, np.float32)))
    conv = Conv2d(1, 4, kernel_size=3, stride=1, padding=1)             # gradtuity/tests/test_nn.py:328-341
    y = conv(T.from_numpy(np.ones((2, 1, 8, 8), np.float32)))
    assert y.shape == (2, 4, 8, 8)
    assert conv.weight.shape == (4, 1, 3, 3) and conv.bias.shape == (4,) and len(conv.parameters()) == 2


def test_maxpool2d_forward_and_backward(T):
    rng = np.random.default_rng(9)
    for shape, k, s in (((2, 3, 8, 10), 2, None), ((1, 2, 9, 9), 3, 2), ((2, 1, 7, 8), (2, 3), (1, 2))):
        x = rng.standard_normal(shape).astype(np.float32)
        tx = T.from_numpy(x, requires_grad=True)
        y = tx.maxpool2d(kernel_size=k, stride=s)
        ref, arg = O.maxpool2d_forward(x, k, s)
        assert np.array_equal(y.numpy(), ref.astype(np.float32))
        dy = rng.standard_normal(ref.shape).astype(np.float32)
        y.mul(T.from_numpy(dy)).sum().backward()
        assert np.allclose(tx.grad.numpy(), O.maxpool2d_backward(dy, arg, shape[2], shape[3]), rtol=0, atol=1e-6)
    with pytest.raises(ValueError, match="4D input"):
        T.from_numpy(np.zeros((3, 4, 4), np.float32)).maxpool2d()
    with pytest.raises(ValueError, match="output size invalid"):
        T.from_numpy(np.zeros((1, 1, 2, 2), np.float32)).maxpool2d(kernel_size=3)


@pytest.mark.parametrize("precision,tol", [("3xtf32", 2e-4), ("tf32", 1e-3)])
def test_mnist_cnn_loss_and_gradients_against_the_oracle(T, precision, tol, monkeypatch):
    """The reference's CNN (two conv + pool stages, two Linear layers) on MNIST-shaped synthetic input: loss and
    the gradient of every parameter against float64; then a few SGD steps lower the loss.  In tf32 mode a
    rounding difference can flip a ReLU mask or the winner of a pooling window for the few elements that sit on a
    boundary, which moves the early layers' gradients by percents although every product is within 1e-3; so the
    tf32 run hands the oracle the masks and winners the GPU run actually took and holds the arithmetic along
    those pieces to 1e-3, while the 3xTF32 run is compared with the oracle's own decisions.  All parameter
    values come from the test's seeded generator."""
    monkeypatch.setenv("GRADTUITY_GEMM_PRECISION", precision)
    from gradtuity_b200.nn import CNN, Flatten
    from gradtuity_b200.optim import SGD

    rng = np.random.default_rng(21)
    model = CNN()
    params = {f"{m}.{a}": getattr(getattr(model, m), a) for m in ("conv1", "conv2", "fc1", "fc2") for a in ("weight", "bias")}
    assert len(model.parameters()) == 8
    host = {}
    for k, p in params.items():
        fan_in = int(np.prod(p.shape[1:])) if p.ndim == 4 else p.shape[0]
        a = (rng.standard_normal(p.shape) * (np.sqrt(2.0 / fan_in) if p.ndim > 1 else 0.05)).astype(np.float32)
        host[k] = a
        from gradtuity_b200.cuda_mem import cuda_memcpy_htod
        cuda_memcpy_htod(p.ptr, np.ascontiguousarray(a))
    N = 8
    x = rng.random((N, 1, 28, 28), dtype=np.float32)
    t = rng.integers(0, 10, N)
    tt = T.from_numpy(t.astype(np.float32))
    # the model's own forward (CNN.__call__), layer by layer so that the pre-activations can be read back
    z1 = model.conv1(T.from_numpy(x)); a1 = z1.relu(); p1 = model.pool1(a1)
    z2 = model.conv2(p1); a2 = z2.relu(); p2 = model.pool2(a2)
    h = model.flatten(p2).linear_relu(model.fc1.weight, model.fc1.bias)
    logits = h.linear(model.fc2.weight, model.fc2.bias)
    assert logits.shape == (N, 10)
    assert np.array_equal(logits.numpy(), model(T.from_numpy(x)).numpy())          # same kernels, same order
    loss = logits.cross_entropy(tt, reduction="mean")
    loss.backward()
    decisions = None
    if precision == "tf32":
        decisions = {"relu1": z1.numpy() > 0, "arg1": O.maxpool2d_forward(a1.numpy(), 2, 2)[1],
                     "relu2": z2.numpy() > 0, "arg2": O.maxpool2d_forward(a2.numpy(), 2, 2)[1], "relu3": h.numpy() > 0}
    ref_loss, ref_g = O.cnn_loss_and_grads(host, x, t, decisions=decisions)
    assert abs(loss.item() - ref_loss) <= 1e-3 * abs(ref_loss)
    for k, p in params.items():
        assert O.rel_frobenius(p.grad.numpy(), ref_g[k]) <= tol, k
    opt = SGD(model.parameters(), lr=0.05)
    first = loss.item()
    for _ in range(15):
        model.zero_grad()
        l2 = model(T.from_numpy(x)).cross_entropy(tt, reduction="mean")
        l2.backward()
        opt.step()
    assert l2.item() < 0.7 * first
    assert Flatten(1)(T.from_numpy(np.zeros((2, 3, 4, 5), np.float32))).shape == (2, 60)


@pytest.mark.parametrize("packed", [True, False])
def test_linear_qkv_matches_three_linears(T, packed):
    """The batched q / k / v projection (shared A, a bias row per batch entry; backward with three batch entries
    adding into one dX and a shared-A dW launch) against the float64 oracle, for parameters that sit side by side
    in memory and for parameters that do not (three `linear` calls)."""
    from gradtuity_b200.nn import CausalSelfAttention

    rng = np.random.default_rng(31)
    Bn, S, E = 2, 192, 128
    attn = CausalSelfAttention(E, 4)
    ws = [(rng.standard_normal((E, E)) / np.sqrt(E)).astype(np.float32) for _ in range(3)]
    bs = [rng.standard_normal(E).astype(np.float32) for _ in range(3)]
    if packed:
        from gradtuity_b200.cuda_mem import cuda_memcpy_htod
        tws, tbs = [attn.Wq, attn.Wk, attn.Wv], [attn.bq, attn.bk, attn.bv]
        assert tws[1].ptr - tws[0].ptr == E * E * 4 and tbs[2].ptr - tbs[1].ptr == E * 4      # the module packs them
        for t, a in zip(tws + tbs, ws + bs):
            cuda_memcpy_htod(t.ptr, a)
    else:
        pad = T.from_numpy(np.zeros(7, np.float32))                                     # breaks the adjacency on purpose
        tws = [T.from_numpy(w, requires_grad=True) for w in ws]
        tbs = [T.from_numpy(b, requires_grad=True) for b in (bs[0], bs[2], bs[1])]
        tbs = [tbs[0], tbs[2], tbs[1]]
        del pad
    x = rng.standard_normal((Bn, S, E)).astype(np.float32)
    dys = [rng.standard_normal((Bn, S, E)).astype(np.float32) for _ in range(3)]
    tx = T.from_numpy(x, requires_grad=True)
    for rep in range(2):                                                                   # second pass accumulates
        outs = tx.linear_qkv(tws[0], tws[1], tws[2], tbs[0], tbs[1], tbs[2])
        loss = None
        for o, dy in zip(outs, dys):
            assert o.shape == (Bn, S, E)
            term = o.mul(T.from_numpy(dy)).sum()
            loss = term if loss is None else loss.add(term)
        loss.backward()
    x2 = x.reshape(-1, E)
    refs = [O.linear_forward_backward(x2, w, b, dy.reshape(-1, E)) for w, b, dy in zip(ws, bs, dys)]
    for o, r in zip(outs, refs):
        assert O.rel_frobenius(o.numpy().reshape(-1, E), r["y"]) <= 1e-3
    assert O.rel_frobenius(tx.grad.numpy().reshape(-1, E), 2 * sum(r["dx"] for r in refs)) <= 1e-3
    for tw, tb, r in zip(tws, tbs, refs):
        assert O.rel_frobenius(tw.grad.numpy(), 2 * r["dw"]) <= 1e-3
        assert O.rel_frobenius(tb.grad.numpy(), 2 * r["db"]) <= 1e-3


def test_linear_qkv_with_one_unused_output(T):
    """Only q feeds the loss: the slices of k and v in the shared gradient buffer are zeroed before the batched
    backward reads them."""
    from gradtuity_b200.nn import CausalSelfAttention

    rng = np.random.default_rng(32)
    E = 64
    attn = CausalSelfAttention(E, 1)
    x = rng.standard_normal((3, 40, E)).astype(np.float32)
    dy = rng.standard_normal((3, 40, E)).astype(np.float32)
    tx = T.from_numpy(x, requires_grad=True)
    q, k, v = tx.linear_qkv(attn.Wq, attn.Wk, attn.Wv, attn.bq, attn.bk, attn.bv)
    q.mul(T.from_numpy(dy)).sum().backward()
    r = O.linear_forward_backward(x.reshape(-1, E), attn.Wq.numpy(), attn.bq.numpy(), dy.reshape(-1, E))
    assert O.rel_frobenius(tx.grad.numpy().reshape(-1, E), r["dx"]) <= 1e-3
    assert O.rel_frobenius(attn.Wq.grad.numpy(), r["dw"]) <= 1e-3
    assert np.all(attn.Wk.grad.numpy() == 0.0) and np.all(attn.bv.grad.numpy() == 0.0)


def test_load_state_dict_keeps_qkv_packed(T):
    from gradtuity_b200.nn import CausalSelfAttention

    rng = np.random.default_rng(33)
    E = 32
    attn = CausalSelfAttention(E, 2)
    state = {k: T.from_numpy(rng.standard_normal(v.shape).astype(np.float32), requires_grad=True) for k, v in attn.state_dict().items()}
    host = {k: v.numpy() for k, v in state.items()}
    attn.load_state_dict(state)
    assert attn.Wk.ptr - attn.Wq.ptr == E * E * 4 and attn.Wv.ptr - attn.Wk.ptr == E * E * 4
    assert attn.bk.ptr - attn.bq.ptr == E * 4
    for k, v in attn.state_dict().items():
        assert np.array_equal(v.numpy(), host[k]) and v.requires_grad


@pytest.mark.parametrize("M,K,I,N", [(256, 64, 192, 64), (100, 20, 36, 12)])
def test_mlp_gelu_and_linear_add_against_the_oracle(T, M, K, I, N):
    """x + fc2(gelu(fc1(h))) with the residual add and the GELU backward inside GEMM epilogues, and
    residual + linear(x), against float64 (second shape: 3xTF32-free general form with partial chunks)."""
    rng = np.random.default_rng(M + I)
    x = rng.standard_normal((M, K)).astype(np.float32)
    w1 = (rng.standard_normal((K, I)) / np.sqrt(K)).astype(np.float32); b1 = rng.standard_normal(I).astype(np.float32)
    w2 = (rng.standard_normal((I, N)) / np.sqrt(I)).astype(np.float32); b2 = rng.standard_normal(N).astype(np.float32)
    res = rng.standard_normal((2, M // 2, N)).astype(np.float32)
    dy = rng.standard_normal((2, M // 2, N)).astype(np.float32)
    tx, tw1, tb1, tw2, tb2, tr = (T.from_numpy(a, requires_grad=True) for a in (x, w1, b1, w2, b2, res))
    y = tx.mlp_gelu(tw1, tb1, tw2, tb2, residual=tr)
    assert y.shape == res.shape
    y.mul(T.from_numpy(dy)).sum().backward()
    x64, dy64 = x.astype(np.float64), dy.reshape(M, N).astype(np.float64)
    pre = x64 @ w1 + b1
    h = O.gelu_tanh(pre)
    ref_y = h @ w2 + b2 + res.reshape(M, N)
    dh = dy64 @ w2.T.astype(np.float64)
    dpre = dh * O.gelu_tanh_grad(pre)
    assert O.rel_frobenius(y.numpy().reshape(M, N), ref_y) <= 1e-3
    assert O.rel_frobenius(tw2.grad.numpy(), h.T @ dy64) <= 1e-3
    assert O.rel_frobenius(tb2.grad.numpy(), dy64.sum(0)) <= 1e-3
    assert O.rel_frobenius(tw1.grad.numpy(), x64.T @ dpre) <= 2e-3
    assert O.rel_frobenius(tb1.grad.numpy(), dpre.sum(0)) <= 2e-3
    assert O.rel_frobenius(tx.grad.numpy(), dpre @ w1.T.astype(np.float64)) <= 2e-3
    assert O.rel_frobenius(tr.grad.numpy().reshape(M, N), dy64) <= 1e-6
    # linear_add
    tx2, tw, tb, tr2 = (T.from_numpy(a, requires_grad=True) for a in (x, w1, b1, rng.standard_normal((M, I)).astype(np.float32)))
    r_host = tr2.numpy()
    z = tx2.linear_add(tw, tb, tr2)
    dz = rng.standard_normal((M, I)).astype(np.float32)
    z.mul(T.from_numpy(dz)).sum().backward()
    ref = O.linear_forward_backward(x, w1, b1, dz)
    assert O.rel_frobenius(z.numpy(), ref["y"] + r_host) <= 1e-3
    assert O.rel_frobenius(tx2.grad.numpy(), ref["dx"]) <= 1e-3
    assert O.rel_frobenius(tw.grad.numpy(), ref["dw"]) <= 1e-3
    assert O.rel_frobenius(tr2.grad.numpy(), dz) <= 1e-6


def test_config0_linear_784_128(T):
    """Config 0: Linear(784 -> 128), batch 128, X ~ U[0,1), W and b ~ U(-1/28, 1/28), dY ~ N(0,1),
    seed 0; y, dX, dW, db against the float64 oracle."""
    rng = np.random.default_rng(0)
    x = rng.random((128, 784), dtype=np.float32)
    w = rng.uniform(-1 / 28, 1 / 28, (784, 128)).astype(np.float32)
    b = rng.uniform(-1 / 28, 1 / 28, (128,)).astype(np.float32)
    dy = rng.standard_normal((128, 128)).astype(np.float32)
    for act, method in (("none", "linear"), ("relu", "linear_relu"), ("gelu", "linear_gelu")):
        tx, tw, tb = (T.from_numpy(v, requires_grad=True) for v in (x, w, b))
        y = getattr(tx, method)(tw, tb)
        y.mul(T.from_numpy(dy)).sum().backward()
        y_gpu = y.numpy()
        ref = O.linear_forward_backward(x, w, b, dy, activation=act, relu_mask=(y_gpu > 0) if act == "relu" else None)
        assert O.rel_frobenius(y_gpu, ref["y"]) <= 1e-3, (act, "y")
        if act == "relu":   # the few outputs within rounding error of zero may differ in sign
            assert np.mean((y_gpu > 0) != (ref["y"] > 0)) < 2e-3
        assert O.rel_frobenius(tx.grad.numpy(), ref["dx"]) <= 1e-3, (act, "dx")
        assert O.rel_frobenius(tw.grad.numpy(), ref["dw"]) <= 1e-3, (act, "dw")
        assert O.rel_frobenius(tb.grad.numpy(), ref["db"]) <= 1e-3, (act, "db")


def test_view_detach_item_roundtrip(T):
    t = T([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]], requires_grad=True)
    v = t.view((3, -1))
    assert v.shape == (3, 2) and v.ptr == t.ptr and not v.owns_memory
    d = t.detach()
    assert d.requires_grad is False and d.ptr == t.ptr
    s = v.sum()
    assert s.item() == pytest.approx(21.0)
    s.backward()
    np.testing.assert_allclose(np.array(t.grad.to_list()), np.ones((2, 3)))
    with pytest.raises(ValueError, match="scalar"):
        t.backward()
    with pytest.raises(ValueError):
        t.view((4, -1))
