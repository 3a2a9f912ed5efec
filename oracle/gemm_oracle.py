"""float64 numpy oracle for the Gradtuity GEMM path. TEST INFRASTRUCTURE, not product code.

Parity status: PINNED for the kernel-level contracts by the reference's own known answers
(tests/test_oracle_pins.py re-states, as data, the expectations of
gradtuity/tests/test_tensor.py:1729-1875 (TestMatmul), gradtuity/tests/test_nn.py:1165-1450
(TestFusedLinear, TestLinearRelu) and the hashed inputs of
gradtuity/tests/test_kernels_cuda_phase4.py:27-167).  UNPINNED for anything larger than those
(GPT-2 activations, loss curves): the reference has no CPU path and no GPU exists in the build
container, so no reference output could be generated for them.

Each function states which reference code it follows.  All arithmetic is float64 unless a
function says otherwise; inputs are whatever numpy arrays the caller holds (usually float32).
"""

from __future__ import annotations

import numpy as np

CAUSAL_MASK_VALUE = -1.0e9  # NEG_INF of causal_mask_inplace, gradtuity/tensor.py:1316


def gelu_tanh(x):
    """GELU, tanh form: gradtuity/kernels_cuda/elemwise_kernels.py:104-125."""
    x = np.asarray(x, dtype=np.float64)
    u = 0.7978845608028654 * (x + 0.044715 * x * x * x)
    return 0.5 * x * (1.0 + np.tanh(u))


def gelu_tanh_grad(x):
    """d gelu / dx: gradtuity/kernels_cuda/elemwise_kernels.py:127-141."""
    x = np.asarray(x, dtype=np.float64)
    u = 0.7978845608028654 * (x + 0.044715 * x * x * x)
    t = np.tanh(u)
    du = 0.7978845608028654 * (1.0 + 3.0 * 0.044715 * x * x)
    return 0.5 * (1.0 + t) + 0.5 * x * (1.0 - t * t) * du


def op_a(a, layout):
    """A as the logical (…, M, K) operand: TN stores it (K, M)."""
    a = np.asarray(a, dtype=np.float64)
    return np.swapaxes(a, -1, -2) if layout == "TN" else a


def op_b(b, layout):
    """B as the logical (…, K, N) operand: NT stores it (N, K)."""
    b = np.asarray(b, dtype=np.float64)
    return np.swapaxes(b, -1, -2) if layout == "NT" else b


def gemm(a, b, layout="NN", *, bias=None, alpha=1.0, epilogue="none", c0=None, return_pre=False):
    """C (+)= epilogue(alpha * op(A) op(B) (+ bias)).

    layout / kernel it restates:
      NN  matmul_kernel               gradtuity/kernels_cuda/matmul_kernels.py:21-63
      NT  matmul_nt_acc_kernel        gradtuity/kernels_cuda/matmul_kernels.py:151-191
      TN  matmul_tn_acc_kernel        gradtuity/kernels_cuda/matmul_kernels.py:195-236
    epilogue:
      "bias"       matmul_bias_kernel       :65-103
      "bias_relu"  matmul_bias_relu_kernel  :105-146
      "bias_gelu"  matmul_bias then gelu_kernel (gpt2/model.py:70)
      "causal"     entries with column > row become CAUSAL_MASK_VALUE (per batch slice)
    c0: previous contents of C for the accumulate kernels (C += …).
    Leading axes of a / b are batch axes (Tensor.bmm, gradtuity/tensor.py:760-896).
    """
    pre = float(alpha) * np.matmul(op_a(a, layout), op_b(b, layout))
    if epilogue in ("bias", "bias_relu", "bias_gelu"):
        pre = pre + np.asarray(bias, dtype=np.float64)
    out = pre
    if epilogue == "bias_relu":
        out = np.maximum(pre, 0.0)
    elif epilogue == "bias_gelu":
        out = gelu_tanh(pre)
    elif epilogue == "causal":
        m, n = pre.shape[-2], pre.shape[-1]
        mask = np.arange(n)[None, :] > np.arange(m)[:, None]
        out = np.where(mask, CAUSAL_MASK_VALUE, pre)
    elif epilogue not in ("none", "bias"):
        raise ValueError(epilogue)
    if c0 is not None:
        out = np.asarray(c0, dtype=np.float64) + out
    return (out, pre) if return_pre else out


def linear_forward_backward(x, w, b, dy, activation="none", relu_mask=None):
    """Tensor.linear / linear_relu and their backward closures.

    Y = act(X W + b) with W stored (in, out)      gradtuity/tensor.py:1604-1621, :1827-1844
    dZ = dY (* [Y>0] for relu)                     gradtuity/tensor.py:1851-1866
    dX = dZ W^T, dW = X^T dZ, db = sum_rows dZ     gradtuity/tensor.py:1632-1679

    relu_mask: optional boolean (M, N) array to use as [Y > 0] instead of the oracle's own.  ReLU
    is discontinuous: an output within rounding error of zero may have either sign, and the
    backward of the implementation under test follows ITS forward (as the reference's does,
    gradtuity/tensor.py:1853-1860), so a backward comparison has to use the same mask.
    """
    x = np.asarray(x, np.float64); w = np.asarray(w, np.float64)
    b = np.asarray(b, np.float64); dy = np.asarray(dy, np.float64)
    z = x @ w + b
    if activation == "relu":
        y = np.maximum(z, 0.0)
        dz = dy * ((y > 0) if relu_mask is None else np.asarray(relu_mask, bool))
    elif activation == "gelu":
        y = gelu_tanh(z)
        dz = dy * gelu_tanh_grad(z)
    else:
        y, dz = z, dy
    return {"y": y, "dx": dz @ w.T, "dw": x.T @ dz, "db": dz.sum(axis=0)}


def linear_tied_forward_backward(x, w, dy):
    """Tensor.linear_tied: logits = X W^T with W stored (V, E); dX = dL W; dW = dL^T X.
    gradtuity/tensor.py:1716-1776."""
    x = np.asarray(x, np.float64); w = np.asarray(w, np.float64); dy = np.asarray(dy, np.float64)
    return {"y": x @ w.T, "dx": dy @ w, "dw": dy.T @ x}


def causal_softmax(s):
    """softmax_with_causal_mask: row i of each (S, S) block attends j <= i, masked outputs are
    exactly 0.  gradtuity/kernels_cuda/softmax_kernels.py:94-129."""
    s = np.asarray(s, np.float64)
    n = s.shape[-1]
    keep = np.arange(n)[None, :] <= np.arange(s.shape[-2])[:, None]
    z = np.where(keep, s, -np.inf)
    z = z - z.max(axis=-1, keepdims=True)
    e = np.where(keep, np.exp(z), 0.0)
    return e / e.sum(axis=-1, keepdims=True)


def softmax_backward(p, dp):
    """dS = P * (dP - sum_j P dP): gradtuity/kernels_cuda/softmax_kernels.py:60-92."""
    p = np.asarray(p, np.float64); dp = np.asarray(dp, np.float64)
    return p * (dp - (p * dp).sum(axis=-1, keepdims=True))


def attention_forward_backward(q, k, v, do):
    """The batched products of CausalSelfAttention (gradtuity/nn.py:539-547) and their
    backward (Tensor.bmm backward, gradtuity/tensor.py:848-893): q, k, v, do are (B, H, T, d)."""
    q = np.asarray(q, np.float64); k = np.asarray(k, np.float64)
    v = np.asarray(v, np.float64); do = np.asarray(do, np.float64)
    scale = 1.0 / np.sqrt(q.shape[-1])
    s = scale * np.matmul(q, np.swapaxes(k, -1, -2))
    p = causal_softmax(s)
    o = np.matmul(p, v)
    dp = np.matmul(do, np.swapaxes(v, -1, -2))
    dv = np.matmul(np.swapaxes(p, -1, -2), do)
    ds = softmax_backward(p, dp) * scale
    dq = np.matmul(ds, k)
    dk = np.matmul(np.swapaxes(ds, -1, -2), q)
    return {"s": s, "p": p, "o": o, "dp": dp, "dv": dv, "ds": ds, "dq": dq, "dk": dk}


def conv2d_forward_backward(x, w, b, dy, stride=1, padding=0):
    """NCHW convolution and its gradients in float64: x (N, C, H, W), w (Co, C, kH, kW), b (Co,), dy
    (N, Co, Ho, Wo).  The arithmetic of gradtuity/tensor.py:1906-2167 (im2col, col @ W_flat^T + b, dW =
    dY^T col, dcol = dY W_flat, col2im) with the output laid out as a true (N, Co, Ho, Wo) tensor."""
    x = np.asarray(x, np.float64); w = np.asarray(w, np.float64); b = np.asarray(b, np.float64); dy = np.asarray(dy, np.float64)
    N, C, H, W = x.shape
    Co, _, kH, kW = w.shape
    Ho = (H + 2 * padding - kH) // stride + 1
    Wo = (W + 2 * padding - kW) // stride + 1
    xp = np.zeros((N, C, H + 2 * padding, W + 2 * padding))
    xp[:, :, padding:padding + H, padding:padding + W] = x
    col = np.empty((N, Ho, Wo, C, kH, kW))
    for kh in range(kH):
        for kw in range(kW):
            col[:, :, :, :, kh, kw] = xp[:, :, kh:kh + stride * Ho:stride, kw:kw + stride * Wo:stride].transpose(0, 2, 3, 1)
    colf = col.reshape(N * Ho * Wo, C * kH * kW)
    wf = w.reshape(Co, -1)
    y = (colf @ wf.T + b).reshape(N, Ho, Wo, Co).transpose(0, 3, 1, 2)
    dyf = dy.transpose(0, 2, 3, 1).reshape(N * Ho * Wo, Co)
    db = dyf.sum(0)
    dw = (dyf.T @ colf).reshape(w.shape)
    dcol = (dyf @ wf).reshape(N, Ho, Wo, C, kH, kW)
    dxp = np.zeros_like(xp)
    for kh in range(kH):
        for kw in range(kW):
            dxp[:, :, kh:kh + stride * Ho:stride, kw:kw + stride * Wo:stride] += dcol[:, :, :, :, kh, kw].transpose(0, 3, 1, 2)
    dx = dxp[:, :, padding:padding + H, padding:padding + W]
    return {"y": y, "dx": dx, "dw": dw, "db": db}


def maxpool2d_forward(x, k=2, stride=None):
    """(N, C, H, W) -> pooled values and, per output, the flat (h * W + w) position of the first maximum of its
    window (gradtuity/tensor.py:2169-2260)."""
    x = np.asarray(x, np.float64)
    kH, kW = (k, k) if isinstance(k, int) else k
    sh, sw = (kH, kW) if stride is None else ((stride, stride) if isinstance(stride, int) else stride)
    N, C, H, W = x.shape
    Ho, Wo = (H - kH) // sh + 1, (W - kW) // sw + 1
    out = np.full((N, C, Ho, Wo), -np.inf)
    arg = np.zeros((N, C, Ho, Wo), np.int64)
    for kh in range(kH):
        for kw in range(kW):
            win = x[:, :, kh:kh + sh * Ho:sh, kw:kw + sw * Wo:sw]
            pos = (np.arange(Ho)[:, None] * sh + kh) * W + (np.arange(Wo)[None, :] * sw + kw)
            better = win > out
            out = np.where(better, win, out)
            arg = np.where(better, pos[None, None], arg)
    return out, arg


def maxpool2d_backward(dy, arg, H, W):
    dy = np.asarray(dy, np.float64)
    N, C, Ho, Wo = dy.shape
    dx = np.zeros((N, C, H * W))
    n, c = np.meshgrid(np.arange(N), np.arange(C), indexing="ij")
    np.add.at(dx, (n[:, :, None, None], c[:, :, None, None], arg), dy)
    return dx.reshape(N, C, H, W)


def _pool_take(a, arg):
    """Values of a (N, C, H, W) at the flat window positions `arg` (N, C, Ho, Wo): pooling with given winners."""
    N, C, H, W = a.shape
    return np.take_along_axis(a.reshape(N, C, H * W), arg.reshape(N, C, -1), axis=2).reshape(arg.shape)


def cnn_loss_and_grads(params, x, targets, decisions=None):
    """The reference's MNIST CNN (gradtuity/nn.py:713-750) with a mean cross-entropy loss, in float64:
    params = dict(conv1.weight, conv1.bias, conv2.weight, conv2.bias, fc1.weight (in, out), fc1.bias, fc2.weight,
    fc2.bias).  Returns the loss and the gradient of every parameter.

    ReLU and max-pooling are piecewise linear: which piece an element is on (sign of the pre-activation, winner of
    a pooling window) is a DISCRETE decision, and an implementation whose products carry tf32 rounding can take a
    different piece for the few elements that lie within rounding error of a boundary, which moves gradients by
    far more than the rounding error itself.  `decisions` = dict(relu1, arg1, relu2, arg2, relu3) fixes those
    choices (boolean masks and window positions, e.g. taken from the implementation under test), so that what is
    compared is the arithmetic along the same piece."""
    P = {k: np.asarray(v, np.float64) for k, v in params.items()}
    x = np.asarray(x, np.float64)
    N = x.shape[0]
    D = decisions
    z1 = conv2d_forward_backward(x, P["conv1.weight"], P["conv1.bias"], np.zeros((N, 32, 28, 28)), 1, 1)["y"]
    relu1 = (z1 > 0) if D is None else np.asarray(D["relu1"], bool)
    a1 = z1 * relu1
    if D is None:
        p1, arg1 = maxpool2d_forward(a1, 2, 2)
    else:
        arg1 = np.asarray(D["arg1"], np.int64); p1 = _pool_take(a1, arg1)
    z2 = conv2d_forward_backward(p1, P["conv2.weight"], P["conv2.bias"], np.zeros((N, 64, 14, 14)), 1, 1)["y"]
    relu2 = (z2 > 0) if D is None else np.asarray(D["relu2"], bool)
    a2 = z2 * relu2
    if D is None:
        p2, arg2 = maxpool2d_forward(a2, 2, 2)
    else:
        arg2 = np.asarray(D["arg2"], np.int64); p2 = _pool_take(a2, arg2)
    f = p2.reshape(N, -1)
    h_pre = f @ P["fc1.weight"] + P["fc1.bias"]
    relu3 = (h_pre > 0) if D is None else np.asarray(D["relu3"], bool)
    h = h_pre * relu3
    logits = h @ P["fc2.weight"] + P["fc2.bias"]
    zmax = logits.max(1, keepdims=True)
    lse = zmax[:, 0] + np.log(np.exp(logits - zmax).sum(1))
    t = np.asarray(targets, np.int64)
    loss = float(np.mean(lse - logits[np.arange(N), t]))
    dlogits = np.exp(logits - lse[:, None])
    dlogits[np.arange(N), t] -= 1
    dlogits /= N
    g = {"fc2.weight": h.T @ dlogits, "fc2.bias": dlogits.sum(0)}
    dh = (dlogits @ P["fc2.weight"].T) * relu3
    g["fc1.weight"] = f.T @ dh
    g["fc1.bias"] = dh.sum(0)
    dp2 = (dh @ P["fc1.weight"].T).reshape(p2.shape)
    dz2 = maxpool2d_backward(dp2, arg2, 14, 14) * relu2
    r2 = conv2d_forward_backward(p1, P["conv2.weight"], P["conv2.bias"], dz2, 1, 1)
    g["conv2.weight"], g["conv2.bias"] = r2["dw"], r2["db"]
    dz1 = maxpool2d_backward(r2["dx"], arg1, 28, 28) * relu1
    r1 = conv2d_forward_backward(x, P["conv1.weight"], P["conv1.bias"], dz1, 1, 1)
    g["conv1.weight"], g["conv1.bias"] = r1["dw"], r1["db"]
    return loss, g


def rel_frobenius(x, ref):
    """||x - ref||_F / ||ref||_F, the parity metric (<= 1e-3 tf32, <= 1e-5 3xTF32)."""
    x = np.asarray(x, np.float64); ref = np.asarray(ref, np.float64)
    den = np.linalg.norm(ref.ravel())
    return float(np.linalg.norm((x - ref).ravel()) / (den if den > 0 else 1.0))


def matmul_f32(a, b):
    """numpy float32 matmul (OpenBLAS): the CPU path the reference's tests compare against
    (np.matmul, gradtuity/tests/test_tensor.py:1284,1301). Timed as the CPU baseline."""
    return np.matmul(np.asarray(a, np.float32), np.asarray(b, np.float32))
