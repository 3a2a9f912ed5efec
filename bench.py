#!/usr/bin/env python
"""Headline benchmark: fp32 GEMM M = N = K = 8192 in tf32 mode on B200, through libgt_b200.so.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One JSON line on stdout (rank 0).  A "step" is one pass of the hot path over one batch of
synthetic input: C = A @ B with A, B ~ N(0, 1/sqrt(K)) from seed 1 (the 8192^3 case of the GEMM
sweep).  `value` times K steps with the operands resident in HBM (CUDA events on the library's
compute stream, which is where the kernels are launched).  `e2e` times the same GEMM with HOST
operands through `gradtuity_b200.gemm.matmul_host` (the C-ABI call gt_gemm_host): every step copies
A and B from pinned host memory, runs the GEMM and copies C back to pinned host memory, the copies
of 8 row blocks overlapped with the products; `e2e.tensor_api` is the same through
`Tensor.from_numpy(...).matmul(...).numpy(out=...)`, where the two uploads, the product and the
download run one after the other.  The operands (805 MB per step) are larger than the 126 MB L2, so
successive steps cannot be served from cache.

N > 1 (launched under torch.distributed.run) runs N independent replicas, one per GPU, with no
data-path collective ("replicas only": a single GEMM does not shard across data-parallel ranks);
torch.distributed is used only for the barrier and the max-over-ranks of the device time.

`--impl reference` times the CPU path the reference's tests check against (numpy float32
matmul, gradtuity/tests/test_tensor.py:1284,1301) on the host cores, on a bounded sample of the
same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

M = N = K = 8192
FLOPS = 2.0 * M * N * K
ALG_BYTES = 4.0 * (M * K + K * N + M * N)
# Rows of A used by the CPU legs: same K and N, a quarter of M (275 GFLOP per pass).
CPU_SAMPLE_ROWS = 2048
# DRAM bytes (read + write) per launch of the 8192^3 GEMM kernel: an ncu `dram__bytes_read.sum +
# dram__bytes_write.sum` capture at the bench size (1.779 GB read + 0.237 GB written).
NCU_TRAFFIC_BYTES_PER_LAUNCH = 2015737344
SUSTAINED_SECONDS = 4.0


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        # The file holds a measured dense bf16 GEMM rate; kind::tf32 runs at half the bf16 rate.
        return p["bf16_tflops"] / 2.0, "measured: MEASURED_PEAKS.json bf16_tflops (burst) / 2 for tf32"
    return 1590.0 / 2.0, "fallback: 1.59 PFLOP/s bf16 / 2 for tf32"


def _peaks_sustained():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        if "bf16_tflops_sustained" in p:
            return p["bf16_tflops_sustained"] / 2.0, "measured: MEASURED_PEAKS.json bf16_tflops_sustained / 2 for tf32"
    return 1400.0 / 2.0, "fallback: 1.4 PFLOP/s sustained bf16 / 2 for tf32"


def _operands():
    import numpy as np

    rng = np.random.default_rng(1)
    a = (rng.standard_normal((M, K), dtype=np.float32) * np.float32(1.0 / np.sqrt(K)))
    b = (rng.standard_normal((K, N), dtype=np.float32) * np.float32(1.0 / np.sqrt(K)))
    return a, b


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device: int):
        self.device = device
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.device}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def _dist_setup(world: int):
    if world <= 1:
        return None
    import torch
    import torch.distributed as dist

    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group(backend="nccl", device_id=torch.device("cuda", local))
    return dist


def _barrier_max(dist, value_ms: float) -> float:
    if dist is None:
        return value_ms
    import torch

    t = torch.tensor([value_ms], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def run_ours(args) -> dict:
    import numpy as np
    from ctypes import byref, c_float, c_void_p

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("for --gpus N > 1 launch with: python -m torch.distributed.run --nproc-per-node N bench.py --gpus N ...")
    dist = _dist_setup(world)

    from gradtuity_b200 import _lib
    from gradtuity_b200 import gemm as G
    from gradtuity_b200.tensor import Tensor

    lib = _lib.load_library()
    ctx = _lib.context()

    a_host, b_host = _operands()
    ta, tb = Tensor.from_numpy(a_host), Tensor.from_numpy(b_host)
    tc = Tensor._zeros((M, N))

    def ev():
        e = c_void_p()
        _lib.check(lib.gt_event_create(ctx, byref(e)), "gt_event_create")
        return e

    def step():
        G.gemm(G.LAYOUT_NN, M, N, K, ta.ptr, K, tb.ptr, N, tc.ptr, N, precision=G.PREC_TF32)

    # ---- device-resident timing ----
    for _ in range(args.warmup):
        step()
    _lib.check(lib.gt_sync(ctx), "gt_sync")
    if dist is not None:
        dist.barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = _lib.launch_count()
    e0, e1 = ev(), ev()
    lib.gt_event_record(ctx, e0)
    for _ in range(args.steps):
        step()
    lib.gt_event_record(ctx, e1)
    ms = c_float()
    _lib.check(lib.gt_event_elapsed_ms(ctx, e0, e1, byref(ms)), "gt_event_elapsed_ms")
    _lib.check(lib.gt_sync(ctx), "gt_sync")
    launches = _lib.launch_count() - launches0
    total_ms = _barrier_max(dist, ms.value)
    _lib.device_status()
    # parity of the device-resident C that was just timed: sampled rows against float64
    rows_dev = np.unique(np.concatenate([np.arange(0, M, M // 16), [1, 127, 128, M - 129, M - 1]]))
    c_dev = tc.numpy()
    ref_dev = a_host[rows_dev].astype(np.float64) @ b_host.astype(np.float64)
    err_dev = float(np.linalg.norm(c_dev[rows_dev] - ref_dev) / np.linalg.norm(ref_dev))
    del c_dev
    if err_dev > 1e-3:
        raise SystemExit(f"parity failure in bench (device-resident C): relative error {err_dev}")

    # ---- sustained: the same GEMM back to back for >= SUSTAINED_SECONDS, clocks sampled meanwhile ----
    sustained = None
    if not args.no_sustained:
        burst_ms = ms.value / args.steps
        n_sus = int(SUSTAINED_SECONDS * 1.6 / (burst_ms * 1e-3))      # headroom: the clock drops under the power cap
        n_sus = max(8, (n_sus + 7) // 8 * 8)
        marks = [ev() for _ in range(9)]
        sus_sampler = ClockSampler(local)
        sus_sampler.start()
        lib.gt_event_record(ctx, marks[0])
        for part in range(8):
            for _ in range(n_sus // 8):
                step()
            lib.gt_event_record(ctx, marks[part + 1])
        _lib.check(lib.gt_sync(ctx), "gt_sync")
        sus_clocks = sus_sampler.stop()
        part_ms = []
        for part in range(8):
            pm = c_float()
            _lib.check(lib.gt_event_elapsed_ms(ctx, marks[part], marks[part + 1], byref(pm)), "gt_event_elapsed_ms")
            part_ms.append(pm.value)
        sus_total = _barrier_max(dist, sum(part_ms))
        sus_step_ms = sus_total / n_sus
        sus_tflops = FLOPS / (sus_step_ms * 1e-3) / 1e12
        peak_s, peak_s_src = _peaks_sustained()
        mhz = sus_clocks.get("sm_mhz")
        sustained = {"seconds": round(sus_total * 1e-3, 2), "launches": n_sus, "ms_per_step": round(sus_step_ms, 4),
                     "tflops": round(sus_tflops, 2), "tflops_by_eighth": [round(FLOPS * (n_sus // 8) / (x * 1e-3) / 1e12, 1) for x in part_ms],
                     "clocks": sus_clocks, "ms_times_mhz": round(sus_step_ms * mhz, 1) if mhz else None,
                     "burst_ms_times_max_mhz": None,
                     "peak": round(peak_s, 2), "peak_source": peak_s_src, "frac": round(sus_tflops / peak_s, 4),
                     "frac_of_nominal_1125": round(sus_tflops / 1125.0, 4)}
        _lib.device_status()

    # ---- end to end through the Tensor API with host buffers ----
    def pinned(shape):
        p = c_void_p()
        nbytes = int(np.prod(shape)) * 4
        _lib.check(lib.gt_host_alloc(ctx, nbytes, byref(p)), "gt_host_alloc")
        import ctypes
        arr = np.ctypeslib.as_array((ctypes.c_float * (nbytes // 4)).from_address(p.value)).reshape(shape)
        return arr, p

    a_pin, pa = pinned((M, K)); b_pin, pb = pinned((K, N)); c_pin, pc = pinned((M, N))
    a_pin[...] = a_host; b_pin[...] = b_host

    def e2e_step_tensor():          # upload A, upload B, multiply, download C, one after the other
        x = Tensor.from_numpy(a_pin)
        w = Tensor.from_numpy(b_pin)
        x.matmul(w).numpy(out=c_pin)

    def e2e_step():                 # the same result with the copies overlapped block by block (gt_gemm_host)
        G.matmul_host(a_pin, b_pin, out=c_pin, precision=G.PREC_TF32, chunks=8)

    e2e_steps = max(1, min(args.steps, 10))

    def time_e2e(fn):
        for _ in range(2):
            fn()
        _lib.check(lib.gt_sync(ctx), "gt_sync")
        if dist is not None:
            dist.barrier()
        # Both forms return with C complete in host memory (they wait for their last copy), so an event
        # recorded on the compute stream after the last call closes the interval.
        f0, f1 = ev(), ev()
        lib.gt_event_record(ctx, f0)
        for _ in range(e2e_steps):
            fn()
        lib.gt_event_record(ctx, f1)
        ems = c_float()
        _lib.check(lib.gt_event_elapsed_ms(ctx, f0, f1, byref(ems)), "gt_event_elapsed_ms")
        return _barrier_max(dist, ems.value)

    e2e_tensor_ms = time_e2e(e2e_step_tensor)
    e2e_total_ms = time_e2e(e2e_step)
    clocks = sampler.stop() if rank == 0 else None
    # parity spot check of what was just timed: 8 rows against float64
    rows = np.arange(0, M, M // 8)
    ref = a_host[rows].astype(np.float64) @ b_host.astype(np.float64)
    err = float(np.linalg.norm(c_pin[rows] - ref) / np.linalg.norm(ref))
    if err > 1e-3:
        raise SystemExit(f"parity failure in bench: relative error {err}")

    ms_per_step = total_ms / args.steps
    value = world * FLOPS / (ms_per_step * 1e-3) / 1e12
    peak, peak_src = _peaks()
    achieved = FLOPS / (ms.value / args.steps * 1e-3) / 1e12
    out = {
        "metric": "gemm_tf32_tflops", "value": round(value, 2), "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "tf32", "data": "synthetic",
        "config": {"workload": "fp32 GEMM sweep, M=N=K=8192, NN, tf32 multiply / fp32 accumulate, one GEMM per step",
                   "parallelism": "replicas only" if world > 1 else "single GPU",
                   "l2": "operands 805 MB per step > 126 MB L2, no flush needed",
                   "inputs": "A, B ~ N(0, 1/sqrt(K)), numpy default_rng(1)"},
        "clocks": clocks,
        "e2e": {"value": round(world * FLOPS / (e2e_total_ms / e2e_steps * 1e-3) / 1e12, 3), "unit": "TFLOP/s",
                "h2d_bytes_per_step": int(4 * (M * K + K * N)), "d2h_bytes_per_step": int(4 * M * N),
                "steps": e2e_steps, "ms_per_step": round(e2e_total_ms / e2e_steps, 3),
                "api": "gradtuity_b200.gemm.matmul_host(A, B, out=C) = gt_gemm_host: pinned host buffers, uploads / products / "
                       "downloads of 8 row blocks overlapped",
                "tensor_api": {"value": round(world * FLOPS / (e2e_tensor_ms / e2e_steps * 1e-3) / 1e12, 3), "unit": "TFLOP/s",
                               "ms_per_step": round(e2e_tensor_ms / e2e_steps, 3),
                               "api": "Tensor.from_numpy(A).matmul(Tensor.from_numpy(B)).numpy(out=C): copies and product in sequence"}},
        "gpu_launches": int(launches),
        "roofline": {"bound": "tensor", "achieved": round(achieved, 2), "peak": round(peak, 2), "unit": "TFLOP/s",
                     "frac": round(achieved / peak, 4), "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH,
                     "peak_source": peak_src, "algorithmic_flops_per_launch": FLOPS,
                     "algorithmic_bytes_per_launch": ALG_BYTES,
                     "frac_of_nominal_1125": round(achieved / 1125.0, 4)},
        "parity_check": {"rel_frobenius_8_rows_vs_float64": err, "device_resident_rows_vs_float64": err_dev,
                         "device_resident_rows": int(len(rows_dev))},
    }
    if sustained is not None:
        if clocks and clocks.get("sm_max_mhz"):
            sustained["burst_ms_times_max_mhz"] = round(ms.value / args.steps * clocks["sm_max_mhz"], 1)
        out["sustained"] = sustained
    if rank == 0 and world == 1 and not args.no_library_peak:
        ta = tb = tc = None
        lib_peak = library_tf32_peak()
        out["library_tf32"] = lib_peak
        if "burst_tflops" in lib_peak:
            out["roofline"]["frac_of_library_tf32_burst"] = round(achieved / lib_peak["burst_tflops"], 4)
            if sustained is not None and lib_peak.get("sustained_tflops"):
                sustained["frac_of_library_tf32_sustained"] = round(sustained["tflops"] / lib_peak["sustained_tflops"], 4)
    if rank == 0 and world == 1:
        out["cpu_baseline"] = cpu_baseline(a_host, b_host, reps=3)
    if not args.no_train:
        # free the GEMM operands before the model is built
        ta = tb = tc = None
        for ptr_ in (pa, pb, pc):
            lib.gt_host_free(ctx, ptr_)
        train = run_train(args, world, rank, lambda v: _barrier_max(dist, v))
        out["train"] = train
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    return out if rank == 0 else None


def library_tf32_peak() -> dict:
    """The TF32 figure a library GEMM reaches on this GPU, measured the way MEASURED_PEAKS.json measured
    bf16: torch.matmul (cuBLAS, allow_tf32) at 8192^3, best of 10 (burst) and back to back for 4 s
    (sustained).  A yardstick beside the roofline only; torch is never on the product path."""
    try:
        import torch

        torch.backends.cuda.matmul.allow_tf32 = True
        dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
        a = torch.randn(M, K, device=dev) / K ** 0.5
        b = torch.randn(K, N, device=dev) / K ** 0.5
        c = torch.empty(M, N, device=dev)
        for _ in range(3):
            torch.matmul(a, b, out=c)
        torch.cuda.synchronize()
        best = float("inf")
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); torch.matmul(a, b, out=c); e1.record(); e1.synchronize()
            best = min(best, e0.elapsed_time(e1))
        n = max(8, int(SUSTAINED_SECONDS * 1.6 / (best * 1e-3)))
        sampler = ClockSampler(dev.index or 0)
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            torch.matmul(a, b, out=c)
        e1.record(); e1.synchronize()
        clocks = sampler.stop()
        sus_ms = e0.elapsed_time(e1) / n
        del a, b, c
        torch.cuda.empty_cache()
        return {"what": "torch.matmul fp32 with allow_tf32 (cuBLAS), 8192^3", "burst_ms": round(best, 4),
                "burst_tflops": round(FLOPS / (best * 1e-3) / 1e12, 2), "sustained_seconds": round(sus_ms * n * 1e-3, 2),
                "sustained_tflops": round(FLOPS / (sus_ms * 1e-3) / 1e12, 2), "sustained_clocks": clocks, "torch": torch.__version__}
    except Exception as e:  # noqa: BLE001
        return {"unavailable": repr(e)[:200]}


TRAIN_FLOPS_PER_STEP = 6.0 * 123532032 * 8192 + 3 * 12 * 2 * (2.0 * 96 * 1024 * 1024 * 64)   # 7.00 TFLOP per GPU


def run_train(args, world: int, rank: int, barrier_max) -> dict:
    """GPT-2-small data-parallel training (configs 3 and 4): batch 8 x 1024 tokens per GPU, uniform random
    tokens, weights N(0, 0.02), dropout 0, AdamW lr 3e-4, clip 1.0.  Every step uploads its token ids
    and labels from host memory and reads the loss back, so the number is end to end."""
    from ctypes import byref, c_float, c_void_p

    from gradtuity_b200 import _lib
    from gradtuity_b200.gpt2.train import build_model, synthetic_batch, train_step
    from gradtuity_b200.optim import AdamW
    from gradtuity_b200.tensor import Tensor

    lib = _lib.load_library()
    ctx = _lib.context()
    if world > 1:
        from gradtuity_b200 import dist as gdist

        gdist.init()
    model = build_model()
    params = model.parameters()
    if world > 1:
        gdist.init_sync(model)
    opt = AdamW(params, lr=3e-4, weight_decay=0.01)
    steps = max(2, args.steps)
    warm = 3
    batches = [synthetic_batch(i, rank, 8, 1024, 50257) for i in range(warm + steps)]
    losses = []
    for i in range(warm):
        losses.append(train_step(model, opt, params, Tensor.from_numpy(batches[i][0]), Tensor.from_numpy(batches[i][1]), 1.0, world).item())
    _lib.check(lib.gt_sync(ctx), "gt_sync")
    barrier_max(0.0)
    l0 = _lib.launch_count()
    e0, e1 = c_void_p(), c_void_p()
    lib.gt_event_create(ctx, byref(e0)); lib.gt_event_create(ctx, byref(e1))
    lib.gt_event_record(ctx, e0)
    for i in range(warm, warm + steps):
        losses.append(train_step(model, opt, params, Tensor.from_numpy(batches[i][0]), Tensor.from_numpy(batches[i][1]), 1.0, world).item())
    lib.gt_event_record(ctx, e1)
    ms = c_float()
    _lib.check(lib.gt_event_elapsed_ms(ctx, e0, e1, byref(ms)), "gt_event_elapsed_ms")
    _lib.device_status()
    launches = _lib.launch_count() - l0
    total_ms = barrier_max(ms.value)
    if world > 1:
        gdist.destroy_process_group()
    step_ms = total_ms / steps
    tokens = world * 8 * 1024
    ref = reference_train_fixture()
    if ref is not None:
        ref["vs_reference_triton"] = round(tokens / (step_ms * 1e-3) / ref["tokens_per_s"], 2)
        ref["vs_reference_triton_per_gpu"] = round(8 * 1024 / (step_ms * 1e-3) / ref["tokens_per_s"], 2)
    return {"reference_triton": ref, "metric": "gpt2_small_train_tokens_per_s", "value": round(tokens / (step_ms * 1e-3), 1), "unit": "tokens/s",
            "ms_per_step": round(step_ms, 3), "steps": steps, "warmup": warm, "n_gpus": world,
            "tflops_per_gpu": round(TRAIN_FLOPS_PER_STEP / (step_ms * 1e-3) / 1e12, 2),
            "frac_of_tf32_peak_measured": round(TRAIN_FLOPS_PER_STEP / (step_ms * 1e-3) / 1e12 / _peaks()[0], 4),
            "h2d_bytes_per_step": int(batches[0][0].nbytes + batches[0][1].nbytes), "d2h_bytes_per_step": 4,
            "gpu_launches_per_step": int(launches // steps), "loss_first": round(losses[0], 4), "loss_last": round(losses[-1], 4),
            "config": {"workload": "GPT-2-small train step, batch 8x1024 per GPU, fp32 storage, tf32 GEMMs, AdamW, clip 1.0",
                       "parallelism": f"dp{world}" if world > 1 else "single GPU",
                       "sync": (f"sync_grads: NCCL all-reduce (avg) of {os.environ.get('GRADTUITY_BUCKET_MB', gdist.ddp.DEFAULT_BUCKET_MB)} MB "
                                "buckets on a side stream, overlapped with backward") if world > 1 else "none"}}


def reference_train_fixture() -> dict | None:
    """The reference's own GPT-2-small train step (its Triton backend, unmodified, one B200), as recorded by
    tests/golden/make_reference_fixtures.py: the 1-GPU figure the tokens/s target is stated against."""
    path = os.path.join(ROOT, "tests", "golden", "reference_gpt2_loss_curve.json")
    try:
        with open(path) as f:
            fx = json.load(f)
        return {"tokens_per_s": round(fx["tokens_per_s"], 1), "ms_per_step": round(fx["ms_per_step_median_after_20"], 1),
                "steps": fx["steps_run"], "n_gpus": 1, "gpu": fx["versions"].get("gpu"), "triton": fx["versions"].get("triton"),
                "source": "tests/golden/reference_gpt2_loss_curve.json (unmodified reference, GRADTUITY_KERNEL_BACKEND=triton, "
                          "same seeded weights and batches, median of the steps after the 20th)"}
    except (OSError, KeyError, ValueError):
        return None


def run_micro(args) -> dict:
    """Kernel-only timing of one GEMM shape (used for sweeps and as the small case for ncu):
    `--shape M N K [--layout NN|NT|TN] [--precision tf32|3xtf32|fp32] [--epilogue ...]`."""
    import numpy as np
    from ctypes import byref, c_float, c_void_p

    from gradtuity_b200 import _lib
    from gradtuity_b200 import gemm as G
    from gradtuity_b200.tensor import Tensor

    lib = _lib.load_library()
    ctx = _lib.context()
    m, n, k = args.shape
    lay = {"NN": 0, "NT": 1, "TN": 2}[args.layout]
    prec = {"tf32": 0, "3xtf32": 1, "fp32": 2}[args.precision]
    epi = {"none": 0, "bias": 1, "bias_relu": 2, "bias_gelu": 3, "causal": 4, "bias_add": 5, "gelu_grad": 6, "gelu_grad_colsum": 6}[args.epilogue]
    rng = np.random.default_rng(1)
    ashape = (k, m) if lay == 2 else (m, k)
    bshape = (n, k) if lay == 1 else (k, n)
    ta = Tensor.from_numpy(rng.standard_normal(ashape, dtype=np.float32) / np.float32(np.sqrt(k)))
    tb = Tensor.from_numpy(rng.standard_normal(bshape, dtype=np.float32) / np.float32(np.sqrt(k)))
    tbias = Tensor.from_numpy(rng.standard_normal((n,), dtype=np.float32))
    tc = Tensor._zeros((m, n))
    taux = Tensor.from_numpy(rng.standard_normal((m, n), dtype=np.float32)) if epi >= 5 else None    # residual / pre-activation
    tsum = Tensor._zeros((n,))

    def step():
        if args.epilogue == "gelu_grad_colsum":
            G.gemm_gelu_grad_colsum(lay, m, n, k, ta.ptr, ashape[1], tb.ptr, bshape[1], tc.ptr, n, taux.ptr, tsum.ptr, precision=prec)
            return
        G.gemm(lay, m, n, k, ta.ptr, ashape[1], tb.ptr, bshape[1], tc.ptr, n, bias_ptr=tbias.ptr if epi in (1, 2, 3, 5) else 0,
               aux_ptr=taux.ptr if taux is not None else 0, accumulate=args.accumulate, epilogue=epi, precision=prec)

    for _ in range(args.warmup):
        step()
    e0, e1 = c_void_p(), c_void_p()
    lib.gt_event_create(ctx, byref(e0)); lib.gt_event_create(ctx, byref(e1))
    lib.gt_event_record(ctx, e0)
    for _ in range(args.steps):
        step()
    lib.gt_event_record(ctx, e1)
    ms = c_float()
    _lib.check(lib.gt_event_elapsed_ms(ctx, e0, e1, byref(ms)), "gt_event_elapsed_ms")
    _lib.device_status()
    t = ms.value / args.steps
    flops = 2.0 * m * n * k
    nbytes = 4.0 * (m * k + k * n + m * n * ((2 if args.accumulate else 1) + (1 if epi >= 5 else 0)))
    return {"micro": True, "shape": [m, n, k], "layout": args.layout, "precision": args.precision, "epilogue": args.epilogue,
            "accumulate": bool(args.accumulate), "ms": round(t, 5), "tflops": round(flops / t / 1e9, 2),
            "gbs": round(nbytes / t / 1e6, 1), "steps": args.steps, "warmup": args.warmup}


def run_sweep(args) -> dict:
    """Config 1: the square and rectangular GEMM sweep, every layout, plain / bias+ReLU / bias+GELU
    epilogues in tf32 mode and the plain product in 3xTF32 mode; kernel-only TFLOP/s and the fraction
    of the measured tf32 peak."""
    import copy

    peak, _ = _peaks()
    shapes = [(1024, 1024, 1024), (2048, 2048, 2048), (4096, 4096, 4096), (8192, 8192, 8192), (8192, 768, 3072), (8192, 3072, 768)]
    rows = []
    for (m, n, k) in shapes:
        for layout in ("NN", "NT", "TN"):
            for prec, epi in (("tf32", "none"), ("tf32", "bias_relu"), ("tf32", "bias_gelu"), ("3xtf32", "none")):
                a = copy.copy(args)
                a.shape, a.layout, a.precision, a.epilogue, a.accumulate = [m, n, k], layout, prec, epi, False
                a.steps = 5 if m * n * k >= 8192 ** 3 else 20
                a.warmup = 3
                r = run_micro(a)
                rows.append({"M": m, "N": n, "K": k, "layout": layout, "precision": prec, "epilogue": epi, "ms": r["ms"],
                             "tflops": r["tflops"], "frac_of_measured_tf32_peak": round(r["tflops"] / peak, 3)})
    return {"sweep": "config 1", "peak_tflops": peak, "rows": rows}


def run_attn(args) -> dict:
    """Kernel-only timing of the batched attention products of config 2 (B=8, H=12, T=1024, d=64),
    reported as achieved GB/s: these GEMMs are HBM-bound (28 FLOP per byte)."""
    import numpy as np
    from ctypes import byref, c_float, c_void_p

    from gradtuity_b200 import _lib
    from gradtuity_b200 import gemm as G
    from gradtuity_b200.tensor import Tensor

    lib = _lib.load_library()
    ctx = _lib.context()
    B, H, S, D = 8, 12, 1024, 64
    E = H * D
    rng = np.random.default_rng(2)
    q, k, v, do = (Tensor.from_numpy(rng.standard_normal((B, S, E), dtype=np.float32)) for _ in range(4))
    p = Tensor._zeros((B, H, S, S)); dp = Tensor._zeros((B, H, S, S)); o = Tensor._zeros((B, S, E))
    hbm = _hbm_peak()
    cases = {
        "S=QK^T*scale+mask (NT)": (lambda: G.gemm_batched(1, S, S, D, q.ptr, E, D, S * E, k.ptr, E, D, S * E, p.ptr, S, S * S, H * S * S, H, B,
                                                            alpha=0.125, epilogue=4), 4.0 * B * H * (2 * S * D + S * S)),
        "O=PV (NN)": (lambda: G.gemm_batched(0, S, D, S, p.ptr, S, S * S, H * S * S, v.ptr, E, D, S * E, o.ptr, E, D, S * E, H, B),
                      4.0 * B * H * (S * S + 2 * S * D)),
        "dP=dO V^T (NT)": (lambda: G.gemm_batched(1, S, S, D, do.ptr, E, D, S * E, v.ptr, E, D, S * E, dp.ptr, S, S * S, H * S * S, H, B, epilogue=4),
                           4.0 * B * H * (2 * S * D + S * S)),
        "dV+=P^T dO (TN)": (lambda: G.gemm_batched(2, S, D, S, p.ptr, S, S * S, H * S * S, do.ptr, E, D, S * E, o.ptr, E, D, S * E, H, B, accumulate=True),
                            4.0 * B * H * (S * S + 3 * S * D)),
        "dQ+=dS K (NN)": (lambda: G.gemm_batched(0, S, D, S, dp.ptr, S, S * S, H * S * S, k.ptr, E, D, S * E, o.ptr, E, D, S * E, H, B, accumulate=True),
                          4.0 * B * H * (S * S + 3 * S * D)),
    }
    lse = Tensor._zeros((B, H, S))
    def fused(p_out):
        _lib.check(lib.gt_attention_forward(ctx, c_void_p(o.ptr), c_void_p(p_out) if p_out else None, c_void_p(lse.ptr),
                                            c_void_p(q.ptr), c_void_p(k.ptr), c_void_p(v.ptr), B, S, H, D, c_float(0.125), None),
                   "gt_attention_forward")
    # fused forward: Q, K, V read, O written (+ the lower-triangular half of P when it is requested)
    cases["fused forward, P written"] = (lambda: fused(p.ptr), 4.0 * B * H * (4 * S * D + S * (S + 128) // 2))
    cases["fused forward, no P"] = (lambda: fused(0), 4.0 * B * H * 4 * S * D)
    dq_, dk_, dv_ = (Tensor._zeros((B, S, E)) for _ in range(3))
    delta = Tensor._zeros((B, H, S))
    # fused backward (two launches): q, k, v, o, dO read (K, Q, dO a second time in the other layout), dq, dk, dv written
    cases["fused backward (dQ + dK/dV kernels)"] = (
        lambda: _lib.check(lib.gt_attention_backward(ctx, c_void_p(dq_.ptr), c_void_p(dk_.ptr), c_void_p(dv_.ptr), c_void_p(do.ptr),
                                                     c_void_p(q.ptr), c_void_p(k.ptr), c_void_p(v.ptr), c_void_p(o.ptr),
                                                     c_void_p(lse.ptr), c_void_p(delta.ptr), B, S, H, D, c_float(0.125), 0, 0, 0, None),
                           "gt_attention_backward"), 4.0 * B * H * 8 * S * D)
    out = {"attn": True, "config": "B=8 H=12 T=1024 d=64, heads read in place from (B,T,H*d)", "hbm_peak_gbs": hbm, "cases": {}}
    for name, (fn, nbytes) in cases.items():
        for _ in range(args.warmup):
            fn()
        e0, e1 = c_void_p(), c_void_p()
        lib.gt_event_create(ctx, byref(e0)); lib.gt_event_create(ctx, byref(e1))
        lib.gt_event_record(ctx, e0)
        for _ in range(args.steps):
            fn()
        lib.gt_event_record(ctx, e1)
        ms = c_float()
        _lib.check(lib.gt_event_elapsed_ms(ctx, e0, e1, byref(ms)), "gt_event_elapsed_ms")
        t = ms.value / args.steps
        out["cases"][name] = {"ms": round(t, 4), "gbs": round(nbytes / t / 1e6, 1), "frac_hbm": round(nbytes / t / 1e6 / hbm, 3),
                              "tflops_dense_equiv": round(2.0 * B * H * S * S * D / t / 1e9, 1)}
    _lib.device_status()
    return out


def run_nn(args) -> dict:
    """Kernel-only timing of the memory-bound kernels of the GPT-2 step at its sizes (8192 tokens, 768 / 3072 / 50257
    columns, 124 M parameters), reported as algorithmic bytes per launch over time against the measured HBM copy
    bandwidth.  Inputs smaller than L2 are rotated through eight copies so that every launch reads from HBM."""
    import numpy as np
    from ctypes import byref, c_float, c_void_p

    from gradtuity_b200 import _lib
    from gradtuity_b200.optim import AdamW, clip_grad_norm_
    from gradtuity_b200.tensor import Tensor

    lib = _lib.load_library()
    ctx = _lib.context()
    rng = np.random.default_rng(4)
    M, E, I, V, LD = 8192, 768, 3072, 50257, 50272
    hbm = _hbm_peak()
    R = 8                                             # copies of the small operands: 8 x 25 MB > 126 MB of L2
    P = lambda t: c_void_p(t.ptr)
    rnd = lambda *shape: Tensor.from_numpy(rng.standard_normal(shape, dtype=np.float32))
    x = [rnd(M, E) for _ in range(R)]; dy = [rnd(M, E) for _ in range(R)]; y = [Tensor._zeros((M, E)) for _ in range(R)]
    gamma, beta = rnd(E), rnd(E)
    mean, rstd = Tensor._zeros((M,)), Tensor._zeros((M,))
    dg, dbt, cs = Tensor._zeros((E,)), Tensor._zeros((E,)), Tensor._zeros((E,))
    wide = [rnd(M, I) for _ in range(2)]; cs_wide = Tensor._zeros((I,))
    _lib.check(lib.gt_layernorm(ctx, P(y[0]), P(mean), P(rstd), P(x[0]), P(gamma), P(beta), M, E, c_float(1e-5)), "gt_layernorm")
    logits = Tensor._zeros((M, LD)); dlogits = Tensor._zeros((M, LD))
    _lib.check(lib.gt_memcpy_h2d(ctx, P(logits), (rng.standard_normal((M, LD), dtype=np.float32) * 3).ctypes.data_as(c_void_p), M * LD * 4), "h2d")
    tgt = Tensor.from_numpy(rng.integers(0, V, M).astype(np.float32))
    loss, row_loss, row_lse = Tensor._zeros((1,)), Tensor._zeros((M,)), Tensor._zeros((M,))
    n_par = 124_439_808
    params = [Tensor.from_numpy(np.zeros(n_par // 8, np.float32), requires_grad=True) for _ in range(8)]
    for q in params:
        q.grad = Tensor.from_numpy(np.full(q.shape, 1e-3, np.float32))
    opt = AdamW(params, lr=1e-4)
    opt.step()                                        # creates m and v
    it = [0]
    def nxt():
        it[0] += 1
        return it[0] % R
    def ln_fwd():
        i = nxt(); _lib.check(lib.gt_layernorm(ctx, P(y[i]), P(mean), P(rstd), P(x[i]), P(gamma), P(beta), M, E, c_float(1e-5)), "ln")
    def ln_bwd(colsum):
        i = nxt()
        _lib.check(lib.gt_layernorm_backward_colsum(ctx, P(y[i]), P(dg), P(dbt), P(cs) if colsum else None, P(dy[i]), P(x[i]), P(mean), P(rstd),
                                                    P(gamma), M, E, 1), "ln bwd")
    cases = {
        "layernorm forward 8192 x 768": (ln_fwd, 2.0 * M * E * 4),
        "layernorm backward 8192 x 768, dx accumulated": (lambda: ln_bwd(False), 4.0 * M * E * 4),
        "the same with the column sums of dx": (lambda: ln_bwd(True), 4.0 * M * E * 4),
        "column sums 8192 x 768": (lambda: _lib.check(lib.gt_colsum_acc(ctx, P(cs), P(dy[nxt()]), M, E, E), "colsum"), 1.0 * M * E * 4),
        "column sums 8192 x 3072": (lambda: _lib.check(lib.gt_colsum_acc(ctx, P(cs_wide), P(wide[nxt() % 2]), M, I, I), "colsum"), 1.0 * M * I * 4),
        "cross-entropy loss + dlogits, one launch, 8192 x 50257": (
            lambda: _lib.check(lib.gt_cross_entropy_fused(ctx, P(loss), P(row_loss), P(row_lse), P(dlogits), LD, P(logits), LD, P(tgt), M, V, 1,
                                                          c_float(1.0 / M)), "ce fused"), 2.0 * M * V * 4),
        "cross-entropy loss alone": (lambda: _lib.check(lib.gt_cross_entropy(ctx, P(loss), P(row_loss), P(row_lse), P(logits), LD, P(tgt), M, V, 1), "ce"),
                                     1.0 * M * V * 4),
        "cross-entropy backward alone": (lambda: _lib.check(lib.gt_cross_entropy_backward(ctx, P(dlogits), LD, P(logits), LD, P(tgt), P(row_lse), None,
                                                                                            c_float(1.0 / M), M, V, 0), "ce bwd"), 2.0 * M * V * 4),
        "AdamW, 124 M parameters, one launch": (lambda: opt.step(), 7.0 * n_par * 4),
        "gradient norm (sum of squares), 124 M": (lambda: clip_grad_norm_(params, 1.0, defer=True), 1.0 * n_par * 4),
    }
    out = {"nn": True, "config": "GPT-2-small step sizes: 8192 tokens, E = 768, 3072, V = 50257 at a pitch of 50272, 124 M parameters",
           "hbm_peak_gbs": hbm, "cases": {}}
    for name, (fn, nbytes) in cases.items():
        for _ in range(args.warmup):
            fn()
        e0, e1 = c_void_p(), c_void_p()
        lib.gt_event_create(ctx, byref(e0)); lib.gt_event_create(ctx, byref(e1))
        lib.gt_event_record(ctx, e0)
        for _ in range(args.steps):
            fn()
        lib.gt_event_record(ctx, e1)
        ms = c_float()
        _lib.check(lib.gt_event_elapsed_ms(ctx, e0, e1, byref(ms)), "gt_event_elapsed_ms")
        t = ms.value / args.steps
        out["cases"][name] = {"ms": round(t, 4), "algorithmic_mb": round(nbytes / 1e6, 1), "gbs": round(nbytes / t / 1e6, 1),
                              "frac_hbm": round(nbytes / t / 1e6 / hbm, 3)}
    _lib.device_status()
    return out


def _hbm_peak() -> float:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"])
    return 6650.0


def _blas_threads() -> int:
    try:
        from threadpoolctl import threadpool_info

        n = [i.get("num_threads", 0) for i in threadpool_info() if i.get("user_api") == "blas"]
        if n:
            return max(n)
    except Exception:
        pass
    return os.cpu_count() or 1


def cpu_baseline(a, b, reps: int) -> dict:
    """numpy float32 matmul (the oracle's `matmul_f32`) on a row slice of the same operands."""
    from oracle import gemm_oracle as O

    _use_all_host_cores()
    a_s = a[:CPU_SAMPLE_ROWS]
    flops = 2.0 * CPU_SAMPLE_ROWS * N * K
    best = float("inf")
    for _ in range(reps):
        t0 = time.perf_counter()
        O.matmul_f32(a_s, b)
        best = min(best, time.perf_counter() - t0)
    return {"value": round(flops / best / 1e12, 4), "unit": "TFLOP/s", "cores": _blas_threads(), "kind": "port",
            "sample": f"numpy float32 A[:{CPU_SAMPLE_ROWS}] @ B of the same 8192^3 operands ({flops / 1e9:.0f} GFLOP), best of {reps}",
            "seconds_per_pass": round(best, 4)}


def _use_all_host_cores() -> int:
    """Give the BLAS behind numpy every core this process may run on.  Launchers such as
    torch.distributed.run export OMP_NUM_THREADS=1, which would turn the CPU arm into a one-thread run."""
    try:
        cores = len(os.sched_getaffinity(0))
    except AttributeError:
        cores = os.cpu_count() or 1
    try:
        from threadpoolctl import threadpool_limits

        threadpool_limits(limits=cores, user_api="blas")
    except Exception:
        pass
    return _blas_threads()


def reference_triton_gemm(iters: int = 5) -> dict:
    """The reference's own GPU GEMM (its Triton `matmul_kernel`, 32x32x32 tiles: gradtuity/tensor.py:569-593,
    gradtuity/kernels_triton/matmul_kernels.py:18-90) on the bench's 8192^3 operands, launched by raw pointer
    from an unmodified copy of the reference under baseline/_ref when that copy and a GPU are present."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "gradtuity")):
        return {"unavailable": "no copy of the reference under baseline/_ref"}
    try:
        import glob
        import site

        import torch

        if not torch.cuda.is_available():
            return {"unavailable": "no GPU"}
        sp = site.getsitepackages()
        cudart = sorted(sum((glob.glob(x + "/nvidia/cuda_runtime/lib/libcudart.so*") for x in sp), [])) or ["libcudart.so"]
        os.environ.setdefault("GRADTUITY_LIBCUDART_LIBRARY", cudart[0])
        os.environ.setdefault("GRADTUITY_KERNEL_BACKEND", "triton")
        if ref not in sys.path:
            sys.path.insert(0, ref)
        import triton
        from gradtuity.kernels_triton.matmul_kernels import matmul_kernel

        a = torch.randn(M, K, device="cuda") / K ** 0.5
        b = torch.randn(K, N, device="cuda") / K ** 0.5
        c = torch.empty(M, N, device="cuda")
        grid = (triton.cdiv(M, 32), triton.cdiv(N, 32))

        def launch():
            matmul_kernel[grid](a.data_ptr(), b.data_ptr(), c.data_ptr(), M, N, K, K, 1, N, 1, N, 1, BLOCK_M=32, BLOCK_N=32, BLOCK_K=32)

        launch()
        torch.cuda.synchronize()
        times = []
        for _ in range(iters):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); launch(); e1.record(); e1.synchronize()
            times.append(e0.elapsed_time(e1))
        ms = statistics.median(times)
        rows = torch.arange(0, M, M // 8, device="cuda")
        want = a[rows].double() @ b.double()
        err = float(torch.linalg.norm(c[rows].double() - want) / torch.linalg.norm(want))
        return {"what": "reference Triton matmul_kernel[grid], BLOCK 32x32x32, fp32 in / tf32 tl.dot, 8192^3 NN, operands resident",
                "ms": round(ms, 3), "tflops": round(FLOPS / (ms * 1e-3) / 1e12, 2), "iters": iters,
                "rel_frobenius_8_rows_vs_float64": err, "triton": triton.__version__}
    except Exception as e:  # noqa: BLE001
        return {"unavailable": repr(e)[:300]}


def run_reference(args) -> dict | None:
    """The reference arm.  The reference has no CPU implementation of the path (it is Triton / NVRTC only), so the
    CPU figure is the numpy float32 matmul its tests check against; the reference's own GPU kernel, which is the
    speed baseline its README implies, is reported beside it under `reference_triton` when it can run here."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return None
    cores = _use_all_host_cores()
    from oracle import gemm_oracle as O

    a, b = _operands()
    a_s = a[:CPU_SAMPLE_ROWS]
    flops = 2.0 * CPU_SAMPLE_ROWS * N * K
    for _ in range(args.warmup):
        O.matmul_f32(a_s, b)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        O.matmul_f32(a_s, b)
    dt = (time.perf_counter() - t0) / args.steps
    value = round(flops / dt / 1e12, 4)
    sample = f"numpy float32 A[:{CPU_SAMPLE_ROWS}] @ B of the 8192^3 operands per step ({flops / 1e9:.0f} GFLOP), {cores} BLAS threads"
    out = {
        "impl": "reference", "metric": "gemm_tf32_tflops", "value": value, "unit": "TFLOP/s",
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "fp32 GEMM sweep, M=N=K=8192, NN (CPU: bounded row slice of the same operands)"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    if not args.no_reference_gpu:
        out["reference_triton"] = reference_triton_gemm()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--shape", type=int, nargs=3, metavar=("M", "N", "K"), help="kernel-only timing of one GEMM shape")
    ap.add_argument("--layout", default="NN", choices=["NN", "NT", "TN"])
    ap.add_argument("--precision", default="tf32", choices=["tf32", "3xtf32", "fp32"])
    ap.add_argument("--epilogue", default="none", choices=["none", "bias", "bias_relu", "bias_gelu", "causal", "bias_add", "gelu_grad", "gelu_grad_colsum"])
    ap.add_argument("--accumulate", action="store_true")
    ap.add_argument("--sweep", action="store_true", help="kernel-only timing of the whole config-1 GEMM sweep")
    ap.add_argument("--attn", action="store_true", help="kernel-only timing of the batched attention products (GB/s)")
    ap.add_argument("--nn", action="store_true", help="kernel-only timing of the memory-bound kernels of the GPT-2 step (GB/s)")
    ap.add_argument("--no-train", dest="no_train", action="store_true", help="skip the GPT-2 training leg")
    ap.add_argument("--no-reference-gpu", dest="no_reference_gpu", action="store_true",
                    help="--impl reference: skip the reference's own Triton GEMM on the GPU")
    ap.add_argument("--no-sustained", dest="no_sustained", action="store_true", help="skip the 4 s back-to-back leg")
    ap.add_argument("--no-library-peak", dest="no_library_peak", action="store_true", help="skip the cuBLAS TF32 yardstick")
    args = ap.parse_args()
    if args.sweep:
        print(json.dumps(run_sweep(args)), flush=True)
        return
    if args.attn:
        print(json.dumps(run_attn(args)), flush=True)
        return
    if args.nn:
        print(json.dumps(run_nn(args)), flush=True)
        return
    if args.shape:
        print(json.dumps(run_micro(args)), flush=True)
        return
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    out = run_reference(args) if args.impl == "reference" else run_ours(args)
    if out is not None:
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
