#!/usr/bin/env python
"""Runs the UNMODIFIED reference (CutieillFusion/Gradtuity) on a GPU and records what it computes, so that
the parity tests can be pinned to the reference itself and not only to a float64 restatement.

The reference is pure Python over Triton / NVRTC kernels and has no CPU path, so this script needs a GPU.
It imports the reference from a directory given with --ref (a plain copy of the reference's `gradtuity/`
and `gpt2/` packages; `__graft_entry__.build()` makes one under `baseline/_ref/`, which is not committed)
and never changes a line of it.

    python tests/golden/make_reference_fixtures.py gemm  --out OUTDIR [--ref DIR] [--max_dim 8192]
    python tests/golden/make_reference_fixtures.py train --out OUTDIR [--ref DIR] [--steps 200]

`gemm`:  launches the reference's five Triton GEMM kernels (gradtuity/kernels_triton/matmul_kernels.py:18-400)
by raw pointer, the way gradtuity/tests/test_kernels_cuda_phase4.py:37-52 does, on the SAME device buffers that
libgt_b200.so's gt_gemm then reads.  Records, per case, the relative Frobenius error between the two and of
each against float64, and the reference kernel's median-of-50 device time (the convention of
gradtuity/bench/runner.py:107-115).  The NVRTC fp32 kernels (gradtuity/kernels_cuda/matmul_kernels.py) are run
beside the 3xTF32 mode up to 2048^3.  Small reference outputs are saved whole (`reference_gemm_outputs.npz`):
the phase-4 shapes and config 0's Linear(784->128) forward + backward.

`train`: runs the reference's train step (gpt2/train.py:111-131: forward, mean cross-entropy, zero_grad,
backward, sync_grads, clip_grad_norm_, AdamW step) on GPT-2-small (gpt2/model.py:25-35) with dropout 0, the
seeded weights of gradtuity_b200.gpt2.train.seeded_state copied into the reference's parameters, and the seeded
batches of gradtuity_b200.gpt2.train.synthetic_batch; writes the loss of every step and the time of every step
to `reference_gpt2_loss_curve.json`.

Outputs land in OUTDIR; the files the tests read are then copied into tests/golden/.
"""
from __future__ import annotations

import argparse
import glob
import json
import os
import platform
import statistics
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def _setup_reference(ref_dir: str, backend: str = "triton") -> None:
    """Environment the reference needs (gradtuity/cuda_mem.py:13-22, cuda_driver.py:23-34, dist/nccl.py:27-37)."""
    if not os.path.isdir(os.path.join(ref_dir, "gradtuity")):
        raise SystemExit(f"no reference checkout at {ref_dir!r} (expected {ref_dir}/gradtuity)")
    sys.path.insert(0, ref_dir)
    if ROOT not in sys.path:
        sys.path.insert(1, ROOT)
    import site

    def first(patterns):
        for p in patterns:
            hits = sorted(glob.glob(p))
            if hits:
                return hits[0]
        return None

    sp = site.getsitepackages()
    env = os.environ
    env.setdefault("GRADTUITY_KERNEL_BACKEND", backend)
    env.setdefault("GRADTUITY_LIBCUDART_LIBRARY",
                   first([s + "/nvidia/cuda_runtime/lib/libcudart.so*" for s in sp] + ["/usr/local/cuda/lib64/libcudart.so"]) or "libcudart.so")
    env.setdefault("GRADTUITY_LIBNVRTC_LIBRARY",
                   first(["/usr/local/cuda/lib64/libnvrtc.so"] + [s + "/nvidia/cuda_nvrtc/lib/libnvrtc.so*" for s in sp]) or "libnvrtc.so")
    env.setdefault("GRADTUITY_LIBCUDA_LIBRARY", "libcuda.so.1")
    env.setdefault("GRADTUITY_NCCL_LIBRARY", first([s + "/nvidia/nccl/lib/libnccl.so*" for s in sp]) or "libnccl.so.2")
    env.setdefault("RANK", "0")
    env.setdefault("WORLD_SIZE", "1")
    env.setdefault("LOCAL_RANK", "0")


def _versions() -> dict:
    import torch
    import triton

    return {"python": platform.python_version(), "numpy": np.__version__, "torch": torch.__version__, "triton": triton.__version__,
            "gpu": torch.cuda.get_device_name(0) if torch.cuda.is_available() else None}


def rel_fro(x: np.ndarray, ref: np.ndarray) -> float:
    d = np.linalg.norm(x.astype(np.float64) - ref.astype(np.float64))
    n = np.linalg.norm(ref.astype(np.float64))
    return float(d / n) if n > 0 else float(d)


# --------------------------------------------------------------------------------------------------------------
# gemm
# --------------------------------------------------------------------------------------------------------------
def _sample_rows(M: int, n: int = 48) -> np.ndarray:
    if M <= n:
        return np.arange(M)
    return np.unique(np.concatenate([np.arange(0, 4), np.arange(M - 4, M), np.linspace(0, M - 1, n).astype(np.int64)]))


def _f64_rows(layout: str, a: np.ndarray, b: np.ndarray, rows: np.ndarray) -> np.ndarray:
    """float64 product restricted to some output rows (so that 8192^3 needs no 1 TFLOP on the host)."""
    a64 = (a[:, rows].T if layout == "tn" else a[rows]).astype(np.float64)
    b64 = (b.T if layout == "nt" else b).astype(np.float64)
    return a64 @ b64


def cmd_gemm(args) -> None:
    _setup_reference(args.ref, "triton")
    import torch
    import triton

    from gradtuity.kernels_triton import matmul_kernels as TK   # the reference, unmodified
    from gradtuity_b200 import _lib, gemm
    from gradtuity_b200.tensor import Tensor

    try:
        from gradtuity.kernels_cuda import matmul_kernels as CK   # NVRTC fp32 twins
    except Exception as e:  # noqa: BLE001
        CK = None
        print("reference NVRTC kernels unavailable:", repr(e), flush=True)

    torch.cuda.init()
    torch.zeros(1, device="cuda")
    _lib.context()

    def sync_all():
        torch.cuda.synchronize()
        _lib.device_status()

    BLK = 32

    def ref_launch(kernels, kind, M, N, K, a, b, c, bias=0):
        """One launch of a reference kernel with the arguments its own call sites pass
        (gradtuity/tensor.py:576-593 NN, :1632-1648 nt/tn accumulate, :1599-1621 bias)."""
        grid = (triton.cdiv(M, BLK), triton.cdiv(N, BLK))
        tri = kernels is TK
        if kind == "nn":
            argv = (a, b, c, M, N, K, K, 1, N, 1, N, 1)
            fn = TK.matmul_kernel if tri else CK.matmul_kernel_launch
        elif kind == "bias":
            argv = (a, b, bias, c, M, N, K, K, 1, N, 1, N, 1)
            fn = TK.matmul_bias_kernel if tri else CK.matmul_bias_kernel_launch
        elif kind == "bias_relu":
            argv = (a, b, bias, c, M, N, K, K, 1, N, 1, N, 1)
            fn = TK.matmul_bias_relu_kernel if tri else CK.matmul_bias_relu_kernel_launch
        elif kind == "nt":      # C += A (M,K) @ B(N,K)^T
            argv = (a, b, c, M, N, K, K, 1, K, 1, N, 1)
            fn = TK.matmul_nt_acc_kernel if tri else CK.matmul_nt_acc_kernel_launch
        elif kind == "tn":      # C += A(K,M)^T @ B (K,N)
            argv = (a, b, c, M, N, K, M, 1, N, 1, N, 1)
            fn = TK.matmul_tn_acc_kernel if tri else CK.matmul_tn_acc_kernel_launch
        else:
            raise ValueError(kind)
        if tri:
            fn[grid](*argv, BLOCK_M=BLK, BLOCK_N=BLK, BLOCK_K=BLK)
        else:
            fn(grid, *argv, BLK, BLK, BLK)

    def time_ref(fn, iters):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        samples = []
        for _ in range(iters):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            e1.synchronize()
            samples.append(e0.elapsed_time(e1))
        return statistics.median(samples)

    def time_ours(fn, iters):
        lib = _lib.load_library()
        ctx = _lib.context()
        from ctypes import byref, c_float, c_void_p

        for _ in range(3):
            fn()
        _lib.device_status()
        samples = []
        e0, e1 = c_void_p(), c_void_p()
        _lib.check(lib.gt_event_create(ctx, byref(e0)), "event")
        _lib.check(lib.gt_event_create(ctx, byref(e1)), "event")
        for _ in range(iters):
            lib.gt_event_record(ctx, e0)
            fn()
            lib.gt_event_record(ctx, e1)
            _lib.check(lib.gt_sync(ctx), "sync")
            ms = c_float()
            lib.gt_event_elapsed_ms(ctx, e0, e1, byref(ms))
            samples.append(ms.value)
        lib.gt_event_destroy(ctx, e0)
        lib.gt_event_destroy(ctx, e1)
        return statistics.median(samples)

    results = {"versions": _versions(), "cases": []}
    saved = {}
    layout_id = {"nn": _lib.LAYOUT_NN, "nt": _lib.LAYOUT_NT, "tn": _lib.LAYOUT_TN}

    def stored_shapes(layout, M, N, K):
        return {"nn": ((M, K), (K, N)), "nt": ((M, K), (N, K)), "tn": ((K, M), (K, N))}[layout]

    def one_case(tag, layout, M, N, K, a, b, *, kind=None, bias=None, c0=None, save=False, timing=True, cuda_too=False):
        """ours vs the reference kernel on the same A/B device buffers."""
        kind = kind or layout
        acc = kind in ("nt", "tn")
        ta, tb = Tensor.from_numpy(a), Tensor.from_numpy(b)
        tbias = Tensor.from_numpy(bias) if bias is not None else None
        c_init = c0 if c0 is not None else np.zeros((M, N), np.float32)
        t_ref, t_ours, t_x3 = (Tensor.from_numpy(c_init) for _ in range(3))
        lda, ldb = a.shape[1], b.shape[1]
        epi = {"nn": _lib.EPI_NONE, "nt": _lib.EPI_NONE, "tn": _lib.EPI_NONE, "bias": _lib.EPI_BIAS, "bias_relu": _lib.EPI_BIAS_RELU}[kind]
        sync_all()

        def ours(prec, out):
            gemm.gemm(layout_id[layout], M, N, K, ta.ptr, lda, tb.ptr, ldb, out.ptr, N, bias_ptr=tbias.ptr if tbias is not None else 0,
                      accumulate=acc, epilogue=epi, precision=prec)

        ref_launch(TK, kind, M, N, K, ta.ptr, tb.ptr, t_ref.ptr, tbias.ptr if tbias is not None else 0)
        ours(_lib.PREC_TF32, t_ours)
        ours(_lib.PREC_TF32X3, t_x3)
        sync_all()
        c_ref, c_ours, c_x3 = t_ref.numpy(), t_ours.numpy(), t_x3.numpy()
        rows = _sample_rows(M)
        f64 = _f64_rows(layout, a, b, rows)
        if bias is not None:
            f64 = f64 + bias.astype(np.float64)[None, :]
        if kind == "bias_relu":
            f64 = np.maximum(f64, 0.0)
        f64 = f64 + c_init[rows].astype(np.float64)
        rec = {"tag": tag, "kind": kind, "layout": layout, "M": M, "N": N, "K": K, "rows_checked_f64": int(len(rows)),
               "ours_tf32_vs_reference_triton": rel_fro(c_ours, c_ref),
               "reference_triton_vs_f64": rel_fro(c_ref[rows], f64),
               "ours_tf32_vs_f64": rel_fro(c_ours[rows], f64),
               "ours_3xtf32_vs_f64": rel_fro(c_x3[rows], f64)}
        if cuda_too and CK is not None:
            t_c = Tensor.from_numpy(c_init)
            sync_all()
            ref_launch(CK, kind, M, N, K, ta.ptr, tb.ptr, t_c.ptr, tbias.ptr if tbias is not None else 0)
            sync_all()
            c_cuda = t_c.numpy()
            rec["ours_3xtf32_vs_reference_cuda_fp32"] = rel_fro(c_x3, c_cuda)
            rec["reference_cuda_fp32_vs_f64"] = rel_fro(c_cuda[rows], f64)
            if save:
                saved[tag + "/ref_cuda"] = c_cuda
        if timing:
            flops = 2.0 * M * N * K
            iters = 50 if flops < 3e11 else (10 if flops < 6e11 else 5)
            # accumulate kernels keep adding into C while timed: harmless for a duration
            ms_ref = time_ref(lambda: ref_launch(TK, kind, M, N, K, ta.ptr, tb.ptr, t_ref.ptr, tbias.ptr if tbias is not None else 0), iters)
            ms_ours = time_ours(lambda: ours(_lib.PREC_TF32, t_ours), 50)
            rec.update({"reference_triton_ms": ms_ref, "reference_triton_tflops": flops / ms_ref / 1e9, "reference_iters": iters,
                        "ours_tf32_ms": ms_ours, "ours_tf32_tflops": flops / ms_ours / 1e9, "speedup": ms_ref / ms_ours})
        if save == "outputs":          # inputs come from a seed the test repeats; keep the first rows of wide outputs
            keep = 32 if c_ref.size > 128 * 128 else c_ref.shape[0]
            saved[tag + "/ref_triton"] = c_ref[:keep]
            if tag + "/ref_cuda" in saved:
                saved[tag + "/ref_cuda"] = saved[tag + "/ref_cuda"][:keep]
        elif save:
            saved[tag + "/a"], saved[tag + "/b"], saved[tag + "/ref_triton"] = a, b, c_ref
            if bias is not None:
                saved[tag + "/bias"] = bias
            if c0 is not None:
                saved[tag + "/c0"] = c0
        results["cases"].append(rec)
        print(json.dumps(rec), flush=True)
        with open(os.path.join(args.out, "reference_gemm_parity.json"), "w") as f:
            json.dump(results, f, indent=1)

    os.makedirs(args.out, exist_ok=True)

    # 1. the reference's own cross-backend test inputs (gradtuity/tests/test_kernels_cuda_phase4.py:27-167)
    from tests._util import PHASE4_CASES, phase4_inputs, phase4_key

    for (kind4, M, N, K) in PHASE4_CASES:
        lay, a, b, bias, c0 = phase4_inputs(kind4, M, N, K)
        kind = {"matmul": "nn", "matmul_bias": "bias", "matmul_bias_relu": "bias_relu", "matmul_nt_acc": "nt", "matmul_tn_acc": "tn"}[kind4]
        one_case("phase4_" + phase4_key(kind4, M, N, K), lay.lower(), M, N, K, a, b, kind=kind, bias=bias, c0=c0, save=True, timing=False,
                 cuda_too=True)

    # 2. config 0: Linear(784 -> 128), batch 128, seed 0 (forward with bias, dX = dY W^T, dW = X^T dY)
    rng = np.random.default_rng(0)
    x = rng.random((128, 784), dtype=np.float32)
    w = rng.uniform(-1 / 28, 1 / 28, (784, 128)).astype(np.float32)
    bvec = rng.uniform(-1 / 28, 1 / 28, (128,)).astype(np.float32)
    dy = rng.standard_normal((128, 128)).astype(np.float32)
    one_case("config0_y", "nn", 128, 128, 784, x, w, kind="bias", bias=bvec, save="outputs", cuda_too=True)
    one_case("config0_dx", "nt", 128, 784, 128, dy, w, c0=np.zeros((128, 784), np.float32), save="outputs", cuda_too=True)
    one_case("config0_dw", "tn", 784, 128, 128, x, dy, c0=np.zeros((784, 128), np.float32), save="outputs", cuda_too=True)
    np.savez_compressed(os.path.join(args.out, "reference_gemm_outputs.npz"), **saved)

    # 3. config 1: the sweep shapes, three layouts, operands ~ N(0, 1/sqrt(K)), seed 1
    shapes = [(1024, 1024, 1024), (2048, 2048, 2048), (8192, 768, 3072), (8192, 3072, 768), (4096, 4096, 4096), (8192, 8192, 8192)]
    for (M, N, K) in shapes:
        if max(M, N, K) > args.max_dim:
            continue
        rng = np.random.default_rng(1)
        for lay in ("nn", "nt", "tn"):
            if max(M, N, K) == 8192 and min(M, N, K) == 8192 and lay != "nn":
                continue    # 8192^3 once (the reference kernel takes a large fraction of a second per launch)
            sa, sb = stored_shapes(lay, M, N, K)
            a = rng.standard_normal(sa, dtype=np.float32) * np.float32(1.0 / np.sqrt(K))
            b = rng.standard_normal(sb, dtype=np.float32) * np.float32(1.0 / np.sqrt(K))
            c0 = np.zeros((M, N), np.float32) if lay != "nn" else None
            one_case(f"config1_{lay}_{M}x{N}x{K}", lay, M, N, K, a, b, c0=c0, cuda_too=(max(M, N, K) <= 2048))
    print("gemm: done", flush=True)


# --------------------------------------------------------------------------------------------------------------
# train
# --------------------------------------------------------------------------------------------------------------
def cmd_train(args) -> None:
    _setup_reference(args.ref, "triton")
    t_start = time.perf_counter()
    from gpt2.model import GPT2Small                      # the reference's model, unmodified
    from gradtuity import AdamW, Tensor, clip_grad_norm_
    from gradtuity import cuda_mem
    from gradtuity.dist import sync_grads

    # the seeded weights and batches are defined once, in the product's training script (numpy only)
    sys.path.insert(1, ROOT)
    from gradtuity_b200.gpt2.train import synthetic_batch

    B, S, V = args.batch_size, args.seq_len, args.vocab_size
    print(f"building the reference model (n_layer={args.n_layer}, vocab={V}) ...", flush=True)
    model = GPT2Small(vocab_size=V, n_positions=S, n_embd=args.n_embd, n_layer=args.n_layer, n_head=args.n_head,
                      embd_pdrop=0.0, attn_pdrop=0.0, resid_pdrop=0.0)
    print(f"  built in {time.perf_counter() - t_start:.1f} s", flush=True)

    # seeded_state's rule, applied to the reference's own parameter names and shapes
    rng = np.random.default_rng(3)
    state = model.state_dict()
    n_params = 0
    for key in sorted(state):
        if key.startswith("lm_head."):
            continue
        t = state[key]
        if len(t.shape) >= 2:
            arr = rng.standard_normal(t.shape, dtype=np.float32) * np.float32(0.02)
        elif key.endswith("gamma"):
            arr = np.ones(t.shape, np.float32)
        else:
            arr = np.zeros(t.shape, np.float32)
        cuda_mem.cuda_memcpy_htod(t.ptr, arr.tobytes())
        n_params += arr.size
    params = model.parameters()
    opt = AdamW(params, lr=args.lr, weight_decay=args.weight_decay)
    out = {"versions": _versions(), "config": {"batch_size": B, "seq_len": S, "vocab_size": V, "n_layer": args.n_layer, "n_embd": args.n_embd,
                                                  "n_head": args.n_head, "lr": args.lr, "weight_decay": args.weight_decay, "max_norm": args.max_norm,
                                                  "dropout": 0.0, "weights": "numpy default_rng(3): matrices N(0, 0.02), gamma 1, vectors 0",
                                                  "tokens": "numpy default_rng((3, step, 0)).integers(0, V, (B, S + 1))"},
           "backend": os.environ["GRADTUITY_KERNEL_BACKEND"], "parameters": n_params,
           "param_shapes": {k: list(state[k].shape) for k in sorted(state) if not k.startswith("lm_head.")}, "loss": [], "ms_per_step": []}
    os.makedirs(args.out, exist_ok=True)
    path = os.path.join(args.out, args.name)
    for step in range(args.steps):
        ids, labels = synthetic_batch(step, 0, B, S, V)
        cuda_mem.cuda_device_synchronize()
        t0 = time.perf_counter()
        input_ids_t = Tensor(ids.astype(np.int64).tolist())
        labels_t = Tensor(labels.astype(np.int64).tolist())
        logits = model(input_ids_t)
        Bv, Sv, Vv = logits.shape
        loss = logits.view((Bv * Sv, Vv)).cross_entropy(labels_t, reduction="mean")
        opt.zero_grad()
        loss.backward()
        sync_grads(params)
        clip_grad_norm_(params, args.max_norm, eps=1e-6)
        opt.step()
        val = loss.item()
        cuda_mem.cuda_device_synchronize()
        ms = (time.perf_counter() - t0) * 1e3
        out["loss"].append(float(val))
        out["ms_per_step"].append(ms)
        if step % 10 == 0 or step == args.steps - 1:
            print(f"step {step} loss={val:.6f} {ms:.1f} ms", flush=True)
            steady = out["ms_per_step"][min(20, len(out["ms_per_step"]) - 1):]
            out["ms_per_step_median_after_20"] = statistics.median(steady)
            out["tokens_per_s"] = B * S / (out["ms_per_step_median_after_20"] * 1e-3)
            with open(path, "w") as f:
                json.dump(out, f, indent=1)
        if time.perf_counter() - t_start > args.max_seconds:
            print(f"stopping after step {step}: time limit", flush=True)
            break
    out["steps_run"] = len(out["loss"])
    steady = out["ms_per_step"][min(20, len(out["ms_per_step"]) - 1):]
    out["ms_per_step_median_after_20"] = statistics.median(steady)
    out["tokens_per_s"] = B * S / (out["ms_per_step_median_after_20"] * 1e-3)
    with open(path, "w") as f:
        json.dump(out, f, indent=1)
    print("train: done", json.dumps({k: out[k] for k in ("steps_run", "ms_per_step_median_after_20", "tokens_per_s")}), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--max_dim", type=int, default=8192)
    t = sub.add_parser("train")
    t.add_argument("--steps", type=int, default=200)
    t.add_argument("--batch_size", type=int, default=8)
    t.add_argument("--seq_len", type=int, default=1024)
    t.add_argument("--vocab_size", type=int, default=50257)
    t.add_argument("--n_layer", type=int, default=12)
    t.add_argument("--n_embd", type=int, default=768)
    t.add_argument("--n_head", type=int, default=12)
    t.add_argument("--lr", type=float, default=3e-4)
    t.add_argument("--weight_decay", type=float, default=0.01)
    t.add_argument("--max_norm", type=float, default=1.0)
    t.add_argument("--max_seconds", type=float, default=1500.0)
    t.add_argument("--name", type=str, default="reference_gpt2_loss_curve.json")
    for p in (g, t):
        p.add_argument("--ref", type=str, default=os.path.join(ROOT, "baseline", "_ref"))
        p.add_argument("--out", type=str, required=True)
    args = ap.parse_args()
    {"gemm": cmd_gemm, "train": cmd_train}[args.cmd](args)


if __name__ == "__main__":
    main()
