"""float64 numpy oracle for the GPT-2 training step. TEST INFRASTRUCTURE, not product code.

Restates, with hand-written backward passes, the computation of the reference's GPT2Small
(gpt2/model.py:38-149) and train step (gpt2/train.py:111-131): embedding + positional embedding,
pre-LN blocks (LayerNorm -> causal self-attention -> residual; LayerNorm -> Linear -> GELU(tanh)
-> Linear -> residual), final LayerNorm, tied LM head, mean cross-entropy, global-norm gradient
clipping and AdamW.  Parameters are a dict keyed like the reference's `state_dict()`.

Parity status: UNPINNED against the reference (it has no CPU path and its tests hold no values
for the gpt2 package); each building block is checked against finite differences in
tests/test_oracle_pins.py, and the kernels it is built from are pinned in gemm_oracle.py.
"""
from __future__ import annotations

import numpy as np

from .gemm_oracle import causal_softmax, gelu_tanh, gelu_tanh_grad, softmax_backward


def layernorm_forward(x, gamma, beta, eps=1e-5):
    """gradtuity/kernels_cuda/layernorm_kernels.py:21-55 (biased variance over the last axis)."""
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    rstd = 1.0 / np.sqrt(var + eps)
    xhat = (x - mu) * rstd
    return xhat * gamma + beta, (xhat, rstd)


def layernorm_backward(dy, cache, gamma):
    """gradtuity/kernels_cuda/layernorm_kernels.py:57-82."""
    xhat, rstd = cache
    H = dy.shape[-1]
    dxhat = dy * gamma
    s1 = dxhat.sum(-1, keepdims=True)
    s2 = (dxhat * xhat).sum(-1, keepdims=True)
    dx = rstd / H * (H * dxhat - s1 - xhat * s2)
    red = tuple(range(dy.ndim - 1))
    return dx, (dy * xhat).sum(red), dy.sum(red)


def cross_entropy_forward(logits, targets):
    """Mean softmax cross-entropy: gradtuity/kernels_cuda/loss_kernels.py (forward) and the
    1/B scaling of gradtuity/tensor.py:1498-1500."""
    z = logits - logits.max(-1, keepdims=True)
    lse = np.log(np.exp(z).sum(-1, keepdims=True))
    logp = z - lse
    n = logits.shape[0]
    return -logp[np.arange(n), targets].mean(), np.exp(logp)


def cross_entropy_backward(probs, targets):
    """dlogits = (softmax - onehot) / B: gradtuity/tensor.py:1507-1523."""
    n = probs.shape[0]
    d = probs.copy()
    d[np.arange(n), targets] -= 1.0
    return d / n


def adamw_step(p, g, m, v, t, lr, beta1=0.9, beta2=0.999, eps=1e-8, wd=0.01):
    """gradtuity/kernels_cuda/optim_kernels.py:23-46 with bc = 1/(1-beta^t) (gradtuity/optim/__init__.py:131-133)."""
    m = beta1 * m + (1 - beta1) * g
    v = beta2 * v + (1 - beta2) * g * g
    upd = (m / (1 - beta1 ** t)) / (np.sqrt(v / (1 - beta2 ** t)) + eps)
    return p - lr * upd - lr * wd * p, m, v


def clip_grad_norm(grads: dict, max_norm: float, eps: float = 1e-6):
    """gradtuity/optim/utils.py:38-51."""
    total = float(np.sqrt(sum(float((g * g).sum()) for g in grads.values())))
    if total > max_norm:
        s = max_norm / (total + eps)
        grads = {k: g * s for k, g in grads.items()}
    return grads, total


class GPT2Oracle:
    """Forward + backward of GPT2Small for parameters `p` (dict of float64 arrays)."""

    def __init__(self, n_layer: int, n_head: int):
        self.n_layer, self.n_head = n_layer, n_head

    def _attention(self, x, p, pre):
        B, S, E = x.shape
        H = self.n_head
        D = E // H
        xf = x.reshape(B * S, E)
        q = (xf @ p[pre + "Wq"] + p[pre + "bq"]).reshape(B, S, H, D).transpose(0, 2, 1, 3)
        k = (xf @ p[pre + "Wk"] + p[pre + "bk"]).reshape(B, S, H, D).transpose(0, 2, 1, 3)
        v = (xf @ p[pre + "Wv"] + p[pre + "bv"]).reshape(B, S, H, D).transpose(0, 2, 1, 3)
        scale = 1.0 / np.sqrt(D)
        s = scale * (q @ k.transpose(0, 1, 3, 2))
        pr = causal_softmax(s)
        ctx = (pr @ v).transpose(0, 2, 1, 3).reshape(B * S, E)
        out = ctx @ p[pre + "Wo"] + p[pre + "bo"]
        return out.reshape(B, S, E), (xf, q, k, v, pr, ctx, scale)

    def _attention_backward(self, dout, cache, p, pre, g):
        xf, q, k, v, pr, ctx, scale = cache
        B, H, S, D = q.shape
        E = H * D
        do = dout.reshape(B * S, E)
        g[pre + "Wo"] = ctx.T @ do
        g[pre + "bo"] = do.sum(0)
        dctx = (do @ p[pre + "Wo"].T).reshape(B, S, H, D).transpose(0, 2, 1, 3)
        dpr = dctx @ v.transpose(0, 1, 3, 2)
        dv = pr.transpose(0, 1, 3, 2) @ dctx
        ds = softmax_backward(pr, dpr) * scale
        dq = ds @ k
        dk = ds.transpose(0, 1, 3, 2) @ q
        dxf = np.zeros_like(xf)
        for name, d in (("q", dq), ("k", dk), ("v", dv)):
            df = d.transpose(0, 2, 1, 3).reshape(B * S, E)
            g[pre + "W" + name] = xf.T @ df
            g[pre + "b" + name] = df.sum(0)
            dxf += df @ p[pre + "W" + name].T
        return dxf.reshape(B, S, E)

    def loss_and_grads(self, p: dict, input_ids: np.ndarray, labels: np.ndarray):
        """input_ids (B, S) ints, labels (B*S,) ints -> (loss, grads dict keyed like p)."""
        B, S = input_ids.shape
        wte, wpe = p["wte.weight"], p["wpe.embed.weight"]
        E = wte.shape[1]
        x = wte[input_ids] + wpe[np.arange(S)][None, :, :]
        caches = []
        for l in range(self.n_layer):
            pre = f"blocks.{l}."
            h1, c1 = layernorm_forward(x, p[pre + "ln1.gamma"], p[pre + "ln1.beta"])
            a, ca = self._attention(h1, p, pre + "attn.")
            x1 = x + a
            h2, c2 = layernorm_forward(x1, p[pre + "ln2.gamma"], p[pre + "ln2.beta"])
            h2f = h2.reshape(B * S, E)
            z = h2f @ p[pre + "mlp_fc1.weight"] + p[pre + "mlp_fc1.bias"]
            act = gelu_tanh(z)
            m = act @ p[pre + "mlp_fc2.weight"] + p[pre + "mlp_fc2.bias"]
            x2 = x1 + m.reshape(B, S, E)
            caches.append((c1, ca, c2, h2f, z, act))
            x = x2
        hf, cf = layernorm_forward(x, p["ln_f.gamma"], p["ln_f.beta"])
        hff = hf.reshape(B * S, E)
        logits = hff @ wte.T
        loss, probs = cross_entropy_forward(logits, labels)

        g: dict = {}
        dlogits = cross_entropy_backward(probs, labels)
        g["wte.weight"] = dlogits.T @ hff
        dh = (dlogits @ wte).reshape(B, S, E)
        dx, g["ln_f.gamma"], g["ln_f.beta"] = layernorm_backward(dh, cf, p["ln_f.gamma"])
        for l in reversed(range(self.n_layer)):
            pre = f"blocks.{l}."
            c1, ca, c2, h2f, z, act = caches[l]
            dm = dx.reshape(B * S, E)
            g[pre + "mlp_fc2.weight"] = act.T @ dm
            g[pre + "mlp_fc2.bias"] = dm.sum(0)
            dz = (dm @ p[pre + "mlp_fc2.weight"].T) * gelu_tanh_grad(z)
            g[pre + "mlp_fc1.weight"] = h2f.T @ dz
            g[pre + "mlp_fc1.bias"] = dz.sum(0)
            dh2 = (dz @ p[pre + "mlp_fc1.weight"].T).reshape(B, S, E)
            dx1, g[pre + "ln2.gamma"], g[pre + "ln2.beta"] = layernorm_backward(dh2, c2, p[pre + "ln2.gamma"])
            dx1 = dx1 + dx
            dh1 = self._attention_backward(dx1, ca, p, pre + "attn.", g)
            dx0, g[pre + "ln1.gamma"], g[pre + "ln1.beta"] = layernorm_backward(dh1, c1, p[pre + "ln1.gamma"])
            dx = dx0 + dx1
        np.add.at(g["wte.weight"], input_ids.reshape(-1), dx.reshape(B * S, E))
        gw = np.zeros_like(wpe)
        np.add.at(gw, np.tile(np.arange(S), B), dx.reshape(B * S, E))
        g["wpe.embed.weight"] = gw
        return loss, g
