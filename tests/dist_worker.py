"""Worker for the world_size-2 CPU tests (spawned by tests/test_dist.py through
gradtuity_b200.launch).  Modes: allreduce | rendezvous | fail."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402


def main():
    mode = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    if mode == "fail":
        if rank == 1:
            sys.exit(3)
        import time
        time.sleep(30)          # must be terminated by the launcher long before this ends
        sys.exit(0)
    if mode == "rendezvous":
        from gradtuity_b200.dist import comm
        uid = comm.exchange_unique_id(rank, lambda: bytes(range(128)), os.environ["GRADTUITY_NCCL_UID_FILE"], timeout=20)
        assert uid == bytes(range(128))
        return
    if mode == "allreduce":
        import torch.distributed as dist
        from gradtuity_b200.dist import comm, ddp
        from tests._dist_host import FakeTensor, GlooBackend, HostMemoryOps

        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{os.environ['MASTER_PORT']}", rank=rank, world_size=world)
        comm.set_backend(GlooBackend())
        ddp._mem_ops = HostMemoryOps()
        rng = np.random.default_rng(100 + rank)
        shapes = [(5, 3), (70,), (2, 2, 2), (129,)]
        params = [FakeTensor(np.zeros(s), requires_grad=True) for s in shapes]
        mine = [rng.standard_normal(s).astype(np.float32) for s in shapes]
        for p, g in zip(params[:-1], mine[:-1]):      # the last parameter has no grad yet: zeros are created
            p.grad = FakeTensor(g)
        os.environ["GRADTUITY_BUCKET_MB"] = str(300 / (1024 * 1024))      # 300-byte buckets
        ddp.sync_grads(params)
        orng = np.random.default_rng(100 + (1 - rank))
        other = [orng.standard_normal(s).astype(np.float32) for s in shapes]
        for i, p in enumerate(params):
            want = (mine[i] + other[i]) / 2 if i < len(shapes) - 1 else np.zeros(shapes[i], np.float32)
            np.testing.assert_allclose(p.grad.array, want, rtol=1e-6, atol=1e-7)
        # second step: the plan is reused, gradients are views of the same arena
        plan = next(iter(ddp._plans.values()))
        assert plan.intact()
        for p, g in zip(params, mine):
            p.grad.array[...] = g
        ddp.sync_grads(params)
        for i, p in enumerate(params):
            np.testing.assert_allclose(p.grad.array, (mine[i] + other[i]) / 2, rtol=1e-6, atol=1e-7)
        dist.destroy_process_group()
        return
    if mode == "accumulate":
        # backward(); backward(); sync_grads() must give the mean over ranks of the SUMMED gradients,
        # although the first backward already sent (and averaged) its buckets.
        import torch.distributed as dist
        from gradtuity_b200.dist import comm, ddp
        from tests._dist_host import FakeTensor, GlooBackend, HostMemoryOps

        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{os.environ['MASTER_PORT']}", rank=rank, world_size=world)
        comm.set_backend(GlooBackend())
        ddp._mem_ops = HostMemoryOps()
        shapes = [(6,), (3, 5), (40,)]
        params = [FakeTensor(np.zeros(s), requires_grad=True) for s in shapes]
        os.environ["GRADTUITY_BUCKET_MB"] = str(64 / (1024 * 1024))
        ddp.sync_grads(params)                                   # builds the plan (zeros)
        plan = next(iter(ddp._plans.values()))

        def grads(r, k):
            g = np.random.default_rng(1000 * k + r)
            return [g.standard_normal(s).astype(np.float32) for s in shapes]

        def backward(k):
            nodes = []
            for p in params:
                n = FakeTensor(np.zeros(1)); n._parents = (p,); nodes.append(n)
            topo = [x for pair in zip(params, nodes) for x in pair]
            plan.begin(topo)
            for p, n, g in reversed(list(zip(params, nodes, grads(rank, k)))):
                p.grad.array[...] += g                          # the node's grad += kernel
                plan.node_done(n._parents)
            plan.end()

        for p in params:
            p.grad.array[...] = 0
        backward(1)
        assert len(plan.launched) == len(plan.buckets)           # the first backward sent everything early
        backward(2)
        assert not plan.launched
        ddp.sync_grads(params)
        for i, p in enumerate(params):
            want = sum(grads(r, k)[i] for r in range(world) for k in (1, 2)) / world
            np.testing.assert_allclose(p.grad.array, want, rtol=1e-5, atol=1e-6)
        dist.destroy_process_group()
        return
    if mode == "embedding":
        # A tied table: dense gradient reduced early, embedding rows gathered from both ranks at sync time.
        import torch.distributed as dist
        from gradtuity_b200.dist import comm, ddp
        from tests._dist_host import FakeTensor, GlooBackend, HostMemoryOps

        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{os.environ['MASTER_PORT']}", rank=rank, world_size=world)
        comm.set_backend(GlooBackend())
        ddp._mem_ops = HostMemoryOps()
        ddp.SPARSE_MIN_BYTES = 64
        os.environ["GRADTUITY_SPARSE_EMBED_SYNC"] = "1"
        V, D, n = 9, 4, 6
        params = [FakeTensor(np.zeros((V, D)), requires_grad=True), FakeTensor(np.zeros(8), requires_grad=True)]
        os.environ["GRADTUITY_BUCKET_MB"] = str(64 / (1024 * 1024))
        ddp.sync_grads(params)
        plan = next(iter(ddp._plans.values()))
        for p in params:
            p.grad.array[...] = 0

        def data(r):
            g = np.random.default_rng(50 + r)
            return (g.standard_normal((V, D)).astype(np.float32), g.integers(0, V, n).astype(np.float32),
                    g.standard_normal((n, D)).astype(np.float32), g.standard_normal(8).astype(np.float32))

        dense, idx, rows, vec = data(rank)
        table = params[0]
        def node(*parents):
            t = FakeTensor(np.zeros(1)); t._parents = parents; return t
        emb, head, other = node(table), node(table), node(params[1])
        emb._embedding_of = table
        plan.begin([table, emb, params[1], other, head])
        table.grad.array[...] += dense
        plan.node_done(head._parents)
        params[1].grad.array[...] += vec
        plan.node_done(other._parents)
        kept_idx, kept_rows = FakeTensor(idx), FakeTensor(rows)
        assert plan.take_embedding_rows(table, kept_idx, kept_rows, n, D, V)
        plan.node_done(emb._parents)
        plan.end()
        ddp.sync_grads(params)
        want = np.zeros((V, D), np.float64)
        for r in range(world):
            d_r, i_r, r_r, _ = data(r)
            full = d_r.astype(np.float64).copy()
            np.add.at(full, i_r.astype(int), r_r)
            want += full / world
        np.testing.assert_allclose(table.grad.array, want, rtol=1e-5, atol=1e-6)
        np.testing.assert_allclose(params[1].grad.array, sum(data(r)[3] for r in range(world)) / world, rtol=1e-6, atol=1e-7)
        dist.destroy_process_group()
        return
    raise SystemExit(f"unknown mode {mode}")


if __name__ == "__main__":
    main()
