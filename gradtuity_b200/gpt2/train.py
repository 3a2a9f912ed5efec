"""GPT-2-small training on synthetic tokens: the train step of gpt2/train.py:111-131
(forward, mean cross-entropy, zero_grad, backward, sync_grads, clip_grad_norm_, AdamW step) on the
gradtuity_b200 modules.

    python -m gradtuity_b200.gpt2.train --steps 20 [--batch_size 8 --seq_len 1024]          (one GPU)
    python -m gradtuity_b200.launch --nproc N gradtuity_b200/gpt2/train.py --steps 20       (N GPUs)

Tokens are uniform random ids (what gpt2/make_test_data.py:37-40 generates), weights are
N(0, 0.02) from a seeded numpy generator, LayerNorm gains 1, biases 0, dropout 0.  Rank r of a
data-parallel job draws its batch for step s from seed (3, s, r).
"""
from __future__ import annotations

import argparse
import math
import time

import os
import sys

import numpy as np

if __package__ in (None, ""):          # run as a script (e.g. by the launcher): make the package importable
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from gradtuity_b200 import _lib
from gradtuity_b200.gpt2.model import GPT2Small
from gradtuity_b200.optim import AdamW, clip_grad_norm_
from gradtuity_b200.tensor import Tensor


def seeded_state(model: GPT2Small, seed: int = 3, std: float = 0.02) -> dict:
    """Parameters as numpy arrays: every matrix ~ N(0, std), LayerNorm gamma 1, vectors 0."""
    rng = np.random.default_rng(seed)
    out = {}
    for key, t in sorted(model.state_dict().items()):
        if key.startswith("lm_head."):
            continue
        if len(t.shape) >= 2:
            out[key] = rng.standard_normal(t.shape, dtype=np.float32) * np.float32(std)
        elif key.endswith("gamma"):
            out[key] = np.ones(t.shape, np.float32)
        else:
            out[key] = np.zeros(t.shape, np.float32)
    return out


def build_model(vocab_size=50257, seq_len=1024, n_embd=768, n_layer=12, n_head=12, seed=3) -> GPT2Small:
    model = GPT2Small(vocab_size=vocab_size, n_positions=seq_len, n_embd=n_embd, n_layer=n_layer, n_head=n_head,
                      embd_pdrop=0.0, attn_pdrop=0.0, resid_pdrop=0.0)
    state = seeded_state(model, seed)
    model.load_state_dict({k: Tensor.from_numpy(v, requires_grad=True) for k, v in state.items()}, strict=False)
    return model


def synthetic_batch(step: int, rank: int, batch_size: int, seq_len: int, vocab_size: int):
    """(input_ids (B, S), labels (B*S,)) as float32 arrays; labels are the next token."""
    rng = np.random.default_rng((3, step, rank))
    tok = rng.integers(0, vocab_size, (batch_size, seq_len + 1))
    return tok[:, :-1].astype(np.float32), tok[:, 1:].reshape(-1).astype(np.float32)


def get_lr(step: int, warmup_steps: int, total_steps: int, base_lr: float) -> float:
    """Linear warm-up then cosine decay (gpt2/train.py get_lr)."""
    if warmup_steps > 0 and step < warmup_steps:
        return base_lr * (step + 1) / warmup_steps
    if total_steps <= warmup_steps:
        return base_lr
    progress = (step - warmup_steps) / max(1, total_steps - warmup_steps)
    return base_lr * 0.5 * (1.0 + math.cos(math.pi * min(1.0, progress)))


def train_step(model: GPT2Small, optimizer: AdamW, params: list, ids_t: Tensor, labels_t: Tensor, max_norm: float = 1.0,
               world_size: int = 1) -> Tensor:
    """One step in the reference's order; returns the loss tensor (still on the device)."""
    logits = model(ids_t)
    B, S, V = logits.shape
    loss = logits.view((B * S, V)).cross_entropy(labels_t, reduction="mean")
    optimizer.zero_grad()
    loss.backward()
    if world_size > 1:
        from gradtuity_b200.dist import sync_grads

        sync_grads(params)
    _, scale = clip_grad_norm_(params, max_norm, eps=1e-6, defer=True)
    optimizer.step(grad_scale=scale)
    return loss


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--batch_size", type=int, default=8)
    ap.add_argument("--seq_len", type=int, default=1024)
    ap.add_argument("--lr", type=float, default=3e-4)
    ap.add_argument("--weight_decay", type=float, default=0.01)
    ap.add_argument("--max_norm", type=float, default=1.0)
    ap.add_argument("--log_every", type=int, default=5)
    ap.add_argument("--n_layer", type=int, default=12)
    ap.add_argument("--vocab_size", type=int, default=50257)
    args = ap.parse_args()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if world > 1:
        from gradtuity_b200 import dist

        dist.init()
    model = build_model(vocab_size=args.vocab_size, seq_len=args.seq_len, n_layer=args.n_layer)
    params = model.parameters()
    if world > 1:
        dist.init_sync(model)
    opt = AdamW(params, lr=args.lr, weight_decay=args.weight_decay)
    t0 = None
    for step in range(args.steps):
        ids, labels = synthetic_batch(step, rank, args.batch_size, args.seq_len, args.vocab_size)
        loss = train_step(model, opt, params, Tensor.from_numpy(ids), Tensor.from_numpy(labels), args.max_norm, world)
        if step == 2:
            _lib.device_status()
            t0 = time.perf_counter()
            s0 = step
        if args.log_every and (step + 1) % args.log_every == 0 and rank == 0:
            print(f"step {step + 1}/{args.steps} loss={loss.item():.4f}", flush=True)
    _lib.device_status()
    if t0 is not None and args.steps - 1 > s0 and rank == 0:
        dt = time.perf_counter() - t0
        n = args.steps - 1 - s0
        print(f"{n} steps in {dt:.3f} s: {dt / n * 1e3:.1f} ms/step, {world * args.batch_size * args.seq_len * n / dt:.0f} tokens/s on {world} GPU(s)")
    if world > 1 and os.environ.get("GRADTUITY_DIST_TIMELINE") == "1" and rank == 0:
        from gradtuity_b200.dist import comm

        rows = comm.get_backend().timeline()
        print("collectives of the last step (MB, enqueued / started / finished, ms after the first one was enqueued):")
        for n, t_enq, t_start, t_end in rows[:-1]:
            print(f"  {n * 4 / 1e6:8.1f} MB  {t_enq:8.3f} {t_start:8.3f} {t_end:8.3f}   ({t_end - t_start:.3f} ms, {n * 4 / 1e6 / max(t_end - t_start, 1e-6):.0f} GB/s)")
        if rows:
            print(f"  compute stream resumed at {rows[-1][1]:.3f} ms; last collective was enqueued at {rows[-2][1]:.3f} ms")
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
