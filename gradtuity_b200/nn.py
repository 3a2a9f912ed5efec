"""Neural-network modules on the GEMM path, with the reference's classes, constructor arguments,
parameter names and storage layouts (gradtuity/nn.py:24-816): `Module`, `Linear` (weight stored
`(in_features, out_features)`), `Embedding`, `PositionalEmbedding`, `TiedLMHead`,
`CausalSelfAttention` (`Wq..Wo`, `bq..bo`), `LayerNorm` (`gamma`, `beta`), `MLP`, `Dropout`.

`state_dict()` keys and `parameters()` order are the reference's, so checkpoints and the
data-parallel gradient exchange see the same lists.  What changes is inside `__call__`: the
attention core is one fused op over in-place head slices, and hidden MLP layers use the fused
bias+ReLU GEMM.  Dropout is the identity at p = 0 (as in the reference, gradtuity/tensor.py:2449-2450);
p > 0 is not on this path and raises.
"""
from __future__ import annotations

from .functional import ones, randn, zero_grad, zeros
from .tensor import Tensor


class Module:
    """Base class: reflection-based parameter discovery (gradtuity/nn.py:24-170)."""

    def __init__(self) -> None:
        self.training = True

    # One walker serves every tree operation below.  The order is the contract: public attributes in dir() order
    # (alphabetical), sub-modules entered depth-first, lists of modules indexed by position, so that paths such
    # as "blocks.3.attn.Wq" and the order of parameters() agree with gradtuity/nn.py:87-114 on every rank.
    def _walk(self, prefix: str = ""):
        """Yields (path, owner, attribute_name, value) for every public attribute of this module and, recursively,
        of its sub-modules; list entries that are modules are walked under "<name>.<index>."."""
        for name in dir(self):
            if name.startswith("_"):
                continue
            try:
                value = getattr(self, name)
            except AttributeError:
                continue
            yield prefix + name, self, name, value
            if isinstance(value, Module):
                yield from value._walk(prefix + name + ".")
            elif isinstance(value, list):
                for i, item in enumerate(value):
                    if isinstance(item, Module):
                        yield from item._walk(f"{prefix}{name}.{i}.")

    def _submodules(self):
        """This module and every module below it, each once."""
        seen = {id(self)}
        yield self
        for _, _, _, value in self._walk():
            for m in (value if isinstance(value, list) else [value]):
                if isinstance(m, Module) and id(m) not in seen:
                    seen.add(id(m))
                    yield m

    def train(self, mode: bool = True) -> "Module":
        for m in self._submodules():
            m.training = mode
        return self

    def eval(self) -> "Module":
        return self.train(False)

    def state_dict(self) -> dict[str, Tensor]:
        """Trainable tensors by dot-separated path, list indices as numeric segments."""
        return {path: value for path, _, _, value in self._walk() if isinstance(value, Tensor) and value.requires_grad}

    def parameters(self) -> list[Tensor]:
        """All trainable tensors in sorted state_dict key order (identical on every rank)."""
        state = self.state_dict()
        return [state[k] for k in sorted(state)]

    def zero_grad(self) -> None:
        zero_grad(self.parameters())

    def load_state_dict(self, state: dict[str, Tensor], strict: bool = True) -> None:
        """Replace parameters by the tensors of `state` (keys as in state_dict()).  strict: the key sets must agree;
        otherwise keys this module does not have are ignored.  Error texts follow gradtuity/nn.py:116-158."""
        slots = {path: (owner, name) for path, owner, name, value in self._walk()
                 if isinstance(value, Tensor) and value.requires_grad}
        if strict:
            extra, lacking = set(state) - set(slots), set(slots) - set(state)
            if extra:
                raise ValueError(f"load_state_dict: unexpected key(s) in state: {extra}")
            if lacking:
                raise ValueError(f"load_state_dict: missing key(s) in state: {lacking}")
        for key, tensor in state.items():
            if key not in slots:
                continue
            owner, name = slots[key]
            try:
                setattr(owner, name, tensor)
            except AttributeError as e:
                raise ValueError(f"load_state_dict: cannot set key {key!r}") from e
        # modules that keep several parameters in one buffer (CausalSelfAttention) restore that layout
        for m in self._submodules():
            hook = getattr(m, "_after_load", None)
            if hook is not None:
                hook()

    def __call__(self, x: Tensor) -> Tensor:
        raise NotImplementedError("Subclasses must implement __call__")


class Linear(Module):
    """Y = X @ W + b; weight (in_features, out_features), Xavier-normal init, zero bias
    (gradtuity/nn.py:173-226)."""

    def __init__(self, in_features: int, out_features: int) -> None:
        self.in_features = in_features
        self.out_features = out_features
        std = (2.0 / (in_features + out_features)) ** 0.5
        self.weight = randn((in_features, out_features), requires_grad=True, std=std)
        self.bias = zeros((out_features,), requires_grad=True)

    def __call__(self, x: Tensor) -> Tensor:
        return x.linear(self.weight, self.bias)

    def parameters(self) -> list[Tensor]:
        return [self.weight, self.bias]

    def __repr__(self) -> str:
        return f"Linear(in_features={self.in_features}, out_features={self.out_features})"


class Dropout(Module):
    """Identity at p = 0 or in eval mode; p > 0 in training is outside this build's path."""

    def __init__(self, p: float = 0.1, rng=None) -> None:
        self.p = p
        self.training = True

    def __call__(self, x: Tensor) -> Tensor:
        if self.p == 0.0 or not self.training:
            return x
        raise NotImplementedError("dropout with p > 0 is not part of the GEMM path; construct models with p = 0")

    def parameters(self) -> list[Tensor]:
        return []

    def __repr__(self) -> str:
        return f"Dropout(p={self.p})"


class Embedding(Module):
    """out = weight[indices]; weight (num_embeddings, embedding_dim), std 1/sqrt(dim)
    (gradtuity/nn.py:305-354)."""

    def __init__(self, num_embeddings: int, embedding_dim: int) -> None:
        self.num_embeddings = num_embeddings
        self.embedding_dim = embedding_dim
        self.weight = randn((num_embeddings, embedding_dim), requires_grad=True, std=1.0 / (embedding_dim ** 0.5))

    def __call__(self, indices) -> Tensor:
        return self.weight.embedding(indices)

    def parameters(self) -> list[Tensor]:
        return [self.weight]

    def __repr__(self) -> str:
        return f"Embedding(num_embeddings={self.num_embeddings}, embedding_dim={self.embedding_dim})"


class PositionalEmbedding(Module):
    """Learned position vectors, repeated across the batch (gradtuity/nn.py:357-412).  The index
    tensor for a given (seq_len, batch, start) is built once and kept on the device."""

    def __init__(self, max_positions: int, embed_dim: int) -> None:
        self.max_positions = max_positions
        self.embed_dim = embed_dim
        self.embed = Embedding(max_positions, embed_dim)
        self._index_cache: dict[tuple[int, int, int], Tensor] = {}

    def __call__(self, seq_len: int, batch_size: int, start_pos: int = 0) -> Tensor:
        if start_pos + seq_len > self.max_positions:
            raise ValueError(f"start_pos ({start_pos}) + seq_len ({seq_len}) > max_positions ({self.max_positions})")
        key = (seq_len, batch_size, start_pos)
        idx = self._index_cache.get(key)
        if idx is None:
            import numpy as np

            pos = np.arange(start_pos, start_pos + seq_len, dtype=np.float32)
            idx = Tensor.from_numpy(np.tile(pos, batch_size))
            self._index_cache[key] = idx
        return self.embed(idx).view((batch_size, seq_len, self.embed_dim))

    def parameters(self) -> list[Tensor]:
        return self.embed.parameters()

    def __repr__(self) -> str:
        return f"PositionalEmbedding(max_positions={self.max_positions}, embed_dim={self.embed_dim})"


class TiedLMHead(Module):
    """logits = h @ wte.weight.T, no weight of its own (gradtuity/nn.py:415-459)."""

    def __init__(self, embedding_module: Embedding) -> None:
        self.embedding_module = embedding_module

    def __call__(self, h: Tensor) -> Tensor:
        B, S, E = h.shape
        wte = self.embedding_module
        if E != wte.embedding_dim:
            raise ValueError(f"input last dim {E} must equal embedding_dim {wte.embedding_dim}")
        logits = h.view((B * S, E)).linear_tied(wte.weight)
        return logits.view((B, S, wte.num_embeddings))

    def parameters(self) -> list[Tensor]:
        return []

    @property
    def weight_ref(self) -> Tensor:
        return self.embedding_module.weight

    def __repr__(self) -> str:
        return "TiedLMHead(tied to Embedding)"


class CausalSelfAttention(Module):
    """Multi-head causal self-attention, (B, S, E) -> (B, S, E) (gradtuity/nn.py:462-569).

    Same parameters (Wq, Wk, Wv, Wo as (E, E); bq, bk, bv, bo) and the same mathematics.  The three
    input projections are one batched launch (`Tensor.linear_qkv`; the three weights, and the three
    biases, live side by side in memory).  The part between the projections runs as
    `Tensor.causal_attention`: fused forward and backward kernels for head dimension 64, else three
    strided-batched GEMM launches and one softmax launch, instead of the reference's three materialised
    transposes, 96 per-slice transposes, two Python loops of 96 GEMM launches, a scale kernel and a
    softmax."""

    def __init__(self, embed_dim: int, num_heads: int, attn_pdrop: float = 0.0, resid_pdrop: float = 0.0) -> None:
        if embed_dim <= 0 or num_heads <= 0:
            raise ValueError("embed_dim and num_heads must be positive")
        if embed_dim % num_heads != 0:
            raise ValueError(f"embed_dim ({embed_dim}) must be divisible by num_heads ({num_heads})")
        self.embed_dim = embed_dim
        self.num_heads = num_heads
        self.head_dim = embed_dim // num_heads
        self.scale = 1.0 / (self.head_dim ** 0.5)
        self.attn_pdrop = attn_pdrop
        self.resid_pdrop = resid_pdrop
        std = (2.0 / (embed_dim + embed_dim)) ** 0.5
        self.Wq = randn((embed_dim, embed_dim), requires_grad=True, std=std)
        self.Wk = randn((embed_dim, embed_dim), requires_grad=True, std=std)
        self.Wv = randn((embed_dim, embed_dim), requires_grad=True, std=std)
        self.Wo = randn((embed_dim, embed_dim), requires_grad=True, std=std)
        self.bq = zeros((embed_dim,), requires_grad=True)
        self.bk = zeros((embed_dim,), requires_grad=True)
        self.bv = zeros((embed_dim,), requires_grad=True)
        self.bo = zeros((embed_dim,), requires_grad=True)
        self.attn_dropout = Dropout(p=attn_pdrop) if attn_pdrop > 0 else None
        self.resid_dropout = Dropout(p=resid_pdrop) if resid_pdrop > 0 else None
        self._pack_qkv()

    def __call__(self, x: Tensor, residual: Tensor | None = None) -> Tensor:
        """attention(x); with `residual` (same shape as x) the result is residual + attention(x), the add done in
        the output projection's epilogue (the reference's block adds afterwards, gpt2/model.py:64-66)."""
        B, S, E = x.shape
        if E != self.embed_dim:
            raise ValueError(f"input last dim {E} must equal embed_dim {self.embed_dim}")
        if self.attn_dropout is not None and self.attn_dropout.p > 0 and self.training:
            raise NotImplementedError("attention dropout with p > 0 is not part of the GEMM path")
        q, k, v = x.linear_qkv(self.Wq, self.Wk, self.Wv, self.bq, self.bk, self.bv)     # one batched launch when packed
        ctx = q.causal_attention(k, v, self.num_heads)
        if residual is not None and self.resid_dropout is None:
            return ctx.view((B * S, E)).linear_add(self.Wo, self.bo, residual)
        out = ctx.view((B * S, E)).linear(self.Wo, self.bo)
        if self.resid_dropout is not None:
            out = self.resid_dropout(out)
        out = out.view((B, S, E))
        return out if residual is None else residual.add(out)

    def parameters(self) -> list[Tensor]:
        return [self.Wq, self.Wk, self.Wv, self.Wo, self.bq, self.bk, self.bv, self.bo]

    def _pack_qkv(self) -> None:
        """Put Wq, Wk, Wv side by side in one buffer, and bq, bk, bv in another, so that `Tensor.linear_qkv`
        can address them as a batch.  The parameters stay three tensors each (same names, shapes, values);
        only where they live changes.  Called at construction and after `load_state_dict`, never later: an
        optimizer holds on to the tensors it was given."""
        from .cuda_mem import cuda_memcpy_dtod
        from .tensor import F32, alloc_storage
        for names in (("Wq", "Wk", "Wv"), ("bq", "bk", "bv")):
            ts = [getattr(self, n) for n in names]
            nbytes = ts[0].numel * F32
            if any(t.shape != ts[0].shape for t in ts):
                continue
            if ts[1].ptr - ts[0].ptr == nbytes and ts[2].ptr - ts[1].ptr == nbytes:
                continue
            block = alloc_storage(3 * nbytes)
            for i, (n, t) in enumerate(zip(names, ts)):
                cuda_memcpy_dtod(block.ptr + i * nbytes, t.ptr, nbytes)
                new = Tensor._from_ptr(block.ptr + i * nbytes, t.shape, owns_memory=False, requires_grad=t.requires_grad,
                                       name=t.name, base=block)
                setattr(self, n, new)

    def _after_load(self) -> None:
        self._pack_qkv()

    def __repr__(self) -> str:
        return f"CausalSelfAttention(embed_dim={self.embed_dim}, num_heads={self.num_heads})"


class Conv2d(Module):
    """2D convolution layer: weight (out_channels, in_channels, kH, kW) ~ N(0, 2 / (in_channels kH kW)), bias
    zeros; forward is `Tensor.conv2d` (gradtuity/nn.py:572-629)."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size, stride: int = 1, padding: int = 0) -> None:
        super().__init__()
        kH, kW = (kernel_size, kernel_size) if isinstance(kernel_size, int) else kernel_size
        self.in_channels = in_channels
        self.out_channels = out_channels
        self.kernel_size = (kH, kW)
        self.stride = stride
        self.padding = padding
        std = (2.0 / (in_channels * kH * kW)) ** 0.5
        self.weight = randn((out_channels, in_channels, kH, kW), requires_grad=True, std=std)
        self.bias = zeros((out_channels,), requires_grad=True)

    def __call__(self, x: Tensor) -> Tensor:
        return x.conv2d(self.weight, self.bias, stride=self.stride, padding=self.padding)

    def __repr__(self) -> str:
        return (f"Conv2d({self.in_channels}, {self.out_channels}, kernel_size={self.kernel_size}, "
                f"stride={self.stride}, padding={self.padding})")


class Flatten(Module):
    """Flatten the dimensions from start_dim on into one: (N, C, H, W) -> (N, C*H*W) (gradtuity/nn.py:229-275)."""

    def __init__(self, start_dim: int = 1) -> None:
        super().__init__()
        self.start_dim = start_dim

    def __call__(self, x: Tensor) -> Tensor:
        s = x.shape
        if len(s) < 2:
            raise ValueError(f"Flatten requires at least 2D input, got shape {s}")
        start_dim = len(s) + self.start_dim if self.start_dim < 0 else self.start_dim
        if start_dim <= 0 or start_dim >= len(s):
            raise ValueError(f"Flatten start_dim must be in [1, {len(s) - 1}], got {self.start_dim}")
        flat = 1
        for d in s[start_dim:]:
            flat *= d
        return x.view(s[:start_dim] + (flat,))

    def parameters(self) -> list[Tensor]:
        return []

    def __repr__(self) -> str:
        return f"Flatten(start_dim={self.start_dim})"


class MaxPool2d(Module):
    """2D max pooling (gradtuity/nn.py:632-659)."""

    def __init__(self, kernel_size=2, stride=None) -> None:
        super().__init__()
        self.kernel_size = kernel_size
        self.stride = stride

    def __call__(self, x: Tensor) -> Tensor:
        return x.maxpool2d(kernel_size=self.kernel_size, stride=self.stride)

    def parameters(self) -> list[Tensor]:
        return []

    def __repr__(self) -> str:
        return f"MaxPool2d(kernel_size={self.kernel_size}, stride={self.stride})"


class CNN(Module):
    """The reference's MNIST model: Conv -> ReLU -> Pool -> Conv -> ReLU -> Pool -> Flatten -> Linear -> ReLU ->
    Linear; input (N, 1, 28, 28), output (N, 10) (gradtuity/nn.py:713-750)."""

    def __init__(self) -> None:
        super().__init__()
        self.conv1 = Conv2d(1, 32, kernel_size=3, stride=1, padding=1)
        self.pool1 = MaxPool2d(kernel_size=2, stride=2)
        self.conv2 = Conv2d(32, 64, kernel_size=3, stride=1, padding=1)
        self.pool2 = MaxPool2d(kernel_size=2, stride=2)
        self.flatten = Flatten(start_dim=1)
        self.fc1 = Linear(64 * 7 * 7, 128)
        self.fc2 = Linear(128, 10)

    def __call__(self, x: Tensor) -> Tensor:
        x = self.pool1(self.conv1(x).relu())
        x = self.pool2(self.conv2(x).relu())
        x = self.flatten(x)
        x = x.linear_relu(self.fc1.weight, self.fc1.bias)
        return x.linear(self.fc2.weight, self.fc2.bias)

    def parameters(self) -> list[Tensor]:
        return self.conv1.parameters() + self.conv2.parameters() + self.fc1.parameters() + self.fc2.parameters()

    def __repr__(self) -> str:
        return "CNN(conv1->relu->pool1->conv2->relu->pool2->flatten->fc1->relu->fc2)"


class LayerNorm(Module):
    """LayerNorm over the last dimension; gamma ones, beta zeros (gradtuity/nn.py:662-710)."""

    def __init__(self, normalized_shape: int, eps: float = 1e-5) -> None:
        self.normalized_shape = normalized_shape
        self.eps = eps
        self.gamma = ones((normalized_shape,), requires_grad=True)
        self.beta = zeros((normalized_shape,), requires_grad=True)

    def __call__(self, x: Tensor) -> Tensor:
        return x.layer_norm(self.gamma, self.beta, eps=self.eps)

    def parameters(self) -> list[Tensor]:
        return [self.gamma, self.beta]

    def __repr__(self) -> str:
        return f"LayerNorm(normalized_shape={self.normalized_shape}, eps={self.eps})"


class MLP(Module):
    """Linear layers with ReLU between them; hidden layers use the fused bias+ReLU GEMM
    (gradtuity/nn.py:753-816)."""

    def __init__(self, nin: int, nouts: list[int]) -> None:
        self.nin = nin
        self.nouts = nouts
        sizes = [nin] + nouts
        self.layers = [Linear(sizes[i], sizes[i + 1]) for i in range(len(nouts))]

    def __call__(self, x: Tensor) -> Tensor:
        for i, layer in enumerate(self.layers):
            if i < len(self.layers) - 1:
                x = x.linear_relu(layer.weight, layer.bias)
            else:
                x = x.linear(layer.weight, layer.bias)
        return x

    def parameters(self) -> list[Tensor]:
        params = []
        for layer in self.layers:
            params.extend(layer.parameters())
        return params

    def __repr__(self) -> str:
        inner = ", ".join(f"Linear({l.in_features}, {l.out_features})" for l in self.layers)
        return f"MLP of [{inner}]"
