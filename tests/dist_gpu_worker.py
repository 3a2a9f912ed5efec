"""Worker for the 2-GPU tests (spawned through gradtuity_b200.launch by tests/test_dist_gpu.py).
Modes: allreduce | sync_grads | init_sync | init_sync_strict_fail."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402


def tiny(seed, n_layer=2):
    from gradtuity_b200.gpt2.train import build_model
    return build_model(vocab_size=257, seq_len=32, n_embd=64, n_layer=n_layer, n_head=2, seed=seed)


def grads_of(model, ids, labels):
    from gradtuity_b200.tensor import Tensor
    params = model.parameters()
    for p in params:
        p.grad = None
    logits = model(Tensor.from_numpy(ids))
    B, S, V = logits.shape
    loss = logits.view((B * S, V)).cross_entropy(Tensor.from_numpy(labels))
    model.zero_grad()
    loss.backward()
    return params


def main():
    mode = sys.argv[1]
    # The sync_grads check recomputes each gradient a second time and compares at 1e-5: that needs sums in a
    # fixed order (no reduce-add split-K, no last-wave split, no shared-C batch launch).
    os.environ["GRADTUITY_GEMM_DETERMINISTIC"] = "1"
    from gradtuity_b200 import _lib, dist
    from gradtuity_b200.dist import comm, ddp
    from gradtuity_b200.gpt2.train import seeded_state, synthetic_batch
    from gradtuity_b200.tensor import Tensor

    dist.init()
    rank, world = dist.get_rank(), dist.get_world_size()
    if mode == "allreduce":
        t = Tensor([float(rank + 1)] * 5)
        comm.allreduce_inplace(t.ptr, 5)
        assert t.to_list() == [3.0] * 5, t.to_list()            # 1 + 2, as gradtuity/tests/dist_worker.py checks
        dist.barrier()
    elif mode == "sync_grads":
        os.environ["GRADTUITY_BUCKET_MB"] = "0.05"                 # several buckets even for the tiny model
        ddp.SPARSE_MIN_BYTES = 1024                                 # the tied 257 x 64 table takes the row-exchange path
        os.environ["GRADTUITY_SPARSE_EMBED_SYNC"] = "1"
        model = tiny(seed=3)
        ref = tiny(seed=3)                                          # local copy used to compute the peer's gradient
        params = model.parameters()
        for step in range(3):                                       # step 0 builds the arena; 1 and 2 overlap with backward
            mine = synthetic_batch(step, rank, 4, 32, 257)
            peer = synthetic_batch(step, 1 - rank, 4, 32, 257)
            g_peer = [p.grad.numpy() for p in grads_of(ref, *peer)]
            g_mine = [p.grad.numpy() for p in grads_of(ref, *mine)]
            logits = model(Tensor.from_numpy(mine[0]))
            B, S, V = logits.shape
            loss = logits.view((B * S, V)).cross_entropy(Tensor.from_numpy(mine[1]))
            model.zero_grad()
            loss.backward()
            plan = next(iter(ddp._plans.values())) if ddp._plans else None
            sent_early = len(plan.launch_order) if plan is not None else 0
            kept_aside = len(plan.deferred) if plan is not None else 0
            dist.sync_grads(params)
            _lib.device_status()
            for p, a, b in zip(params, g_mine, g_peer):
                np.testing.assert_allclose(p.grad.numpy(), (a + b) / 2, rtol=1e-5, atol=1e-7)
            if step > 0:
                assert sent_early >= 2, f"step {step}: only {sent_early} buckets went out during backward"
                assert kept_aside == 1, f"step {step}: the embedding rows of the tied table were not kept aside ({kept_aside})"
        dist.barrier()
    elif mode == "init_sync":
        model = tiny(seed=3 + 10 * rank)                           # rank 1 starts from different weights
        dist.init_sync(model)
        want = seeded_state(tiny(seed=3), seed=3)
        for k, t in model.state_dict().items():
            if not k.startswith("lm_head."):
                assert np.array_equal(t.numpy(), want[k]), k
        dist.barrier()
    elif mode == "init_sync_strict_fail":
        model = tiny(seed=3, n_layer=2 if rank == 0 else 1)        # different architecture on rank 1
        try:
            dist.init_sync(model, strict=True)
        except RuntimeError as e:
            assert "strict check failed" in str(e), str(e)
        else:
            raise SystemExit("init_sync accepted mismatched models")
        dist.barrier()
    else:
        raise SystemExit(f"unknown mode {mode}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
