"""Parity against the reference ITSELF, run unmodified on a B200 by tests/golden/make_reference_fixtures.py:

* `reference_gemm_outputs.npz`: what the reference's Triton kernels (TF32 `tl.dot`) and its NVRTC fp32 kernels
  wrote for the inputs of its own cross-backend tests (gradtuity/tests/test_kernels_cuda_phase4.py:27-167) and
  for config 0's Linear(784 -> 128) forward and backward;
* `reference_gemm_parity.json`: the record of the same-buffer comparison at config 1's sizes (up to 8192^3);
* `reference_gpt2_loss_curve.json`: the loss of each of 200 steps of the reference's train step
  (gpt2/train.py:111-131) on GPT-2-small with seeded weights and batches;
* `reference_gpt2_tiny_loss_curve.json`: the same for a two-layer model small enough for the float64 oracle.

CPU tests pin the float64 oracle to those outputs; GPU tests compare libgt_b200.so with them.
Bars: relative Frobenius error <= 1e-3 in tf32 mode, <= 1e-5 in 3xTF32 mode; on the phase-4 inputs (a few
distinct values, so rounding errors do not average out) the reference's own cross-backend tolerance
rtol 1e-2 / atol 1e-3; loss curves within 1e-3 relative at every step.
"""
import json
import os

import numpy as np
import pytest

from oracle import gemm_oracle as O
from oracle import gpt2_oracle as GO
from tests import _util as U

KIND_OF = {"matmul": ("NN", "none"), "matmul_bias": ("NN", "bias"), "matmul_bias_relu": ("NN", "bias_relu"),
           "matmul_nt_acc": ("NT", "none"), "matmul_tn_acc": ("TN", "none")}


def _outputs():
    return dict(np.load(os.path.join(U.GOLDEN, "reference_gemm_outputs.npz")))


def _json(name):
    with open(os.path.join(U.GOLDEN, name)) as f:
        return json.load(f)


def _phase4_cases(store):
    for (kind, M, N, K) in U.PHASE4_CASES:
        tag = "phase4_" + U.phase4_key(kind, M, N, K)
        layout, a, b, bias, c0 = U.phase4_inputs(kind, M, N, K)
        # the stored inputs are the ones the reference actually read
        assert np.array_equal(store[tag + "/a"], a) and np.array_equal(store[tag + "/b"], b)
        yield tag, kind, layout, a, b, bias, c0


def _config0():
    rng = np.random.default_rng(0)
    x = rng.random((128, 784), dtype=np.float32)
    w = rng.uniform(-1 / 28, 1 / 28, (784, 128)).astype(np.float32)
    b = rng.uniform(-1 / 28, 1 / 28, (128,)).astype(np.float32)
    dy = rng.standard_normal((128, 128)).astype(np.float32)
    zeros = lambda m, n: np.zeros((m, n), np.float32)
    return [("config0_y", "NN", x, w, b, None, "bias"), ("config0_dx", "NT", dy, w, None, zeros(128, 784), "none"),
            ("config0_dw", "TN", x, dy, None, zeros(784, 128), "none")]


# ---- CPU: the oracle against what the reference computed ----------------------------------------------------

def test_oracle_matches_the_reference_outputs_on_its_own_test_inputs():
    store = _outputs()
    n = 0
    for tag, kind, layout, a, b, bias, c0 in _phase4_cases(store):
        want = O.gemm(a, b, layout, bias=bias, epilogue=KIND_OF[kind][1], c0=c0)
        assert np.allclose(store[tag + "/ref_triton"], want, rtol=1e-2, atol=1e-3), tag      # the reference's own tolerance
        assert O.rel_frobenius(store[tag + "/ref_cuda"], want) <= 1e-5, tag                   # its fp32 kernels
        n += 1
    assert n == len(U.PHASE4_CASES)


def test_oracle_matches_the_reference_outputs_for_config0():
    store = _outputs()
    for tag, layout, a, b, bias, c0, epi in _config0():
        want = O.gemm(a, b, layout, bias=bias, epilogue=epi, c0=c0)
        rows = store[tag + "/ref_triton"].shape[0]
        assert O.rel_frobenius(store[tag + "/ref_triton"], want[:rows]) <= 1e-3, tag
        assert O.rel_frobenius(store[tag + "/ref_cuda"], want[:rows]) <= 1e-5, tag


def test_recorded_same_buffer_comparison_meets_the_bars():
    """The record of the run at config 1's sizes: ours vs the reference kernel on the same device buffers."""
    rec = _json("reference_gemm_parity.json")
    cases = {c["tag"]: c for c in rec["cases"]}
    big = [c for t, c in cases.items() if t.startswith("config1_") or t.startswith("config0_")]
    assert any(c["M"] == 8192 and c["N"] == 8192 and c["K"] == 8192 for c in big)
    assert {c["layout"] for c in big} == {"nn", "nt", "tn"}
    for c in big:
        assert c["ours_tf32_vs_reference_triton"] <= 1e-3, c["tag"]
        assert c["ours_tf32_vs_f64"] <= 1e-3 and c["reference_triton_vs_f64"] <= 1e-3, c["tag"]
        assert c["ours_3xtf32_vs_f64"] <= 1e-5, c["tag"]
        if "ours_3xtf32_vs_reference_cuda_fp32" in c:
            assert c["ours_3xtf32_vs_reference_cuda_fp32"] <= 1e-5, c["tag"]


def _seeded_params(shapes: dict) -> dict:
    """The weight rule of tests/golden/make_reference_fixtures.py (and gradtuity_b200.gpt2.train.seeded_state):
    one numpy generator, seed 3, keys in sorted order; matrices N(0, 0.02), gamma 1, other vectors 0."""
    rng = np.random.default_rng(3)
    out = {}
    for key in sorted(shapes):
        shape = tuple(shapes[key])
        if len(shape) >= 2:
            out[key] = rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02)
        elif key.endswith("gamma"):
            out[key] = np.ones(shape, np.float32)
        else:
            out[key] = np.zeros(shape, np.float32)
    return out


def test_gpt2_oracle_tracks_the_reference_on_a_two_layer_model():
    """oracle/gpt2_oracle.py (float64 forward, backward, clip, AdamW) against the loss the reference printed at each
    of 20 steps of its own train step, same seeded weights and batches."""
    from gradtuity_b200.gpt2.train import synthetic_batch

    fx = _json("reference_gpt2_tiny_loss_curve.json")
    cfg = fx["config"]
    p = {k: v.astype(np.float64) for k, v in _seeded_params(fx["param_shapes"]).items()}
    m = {k: np.zeros_like(v) for k, v in p.items()}
    vv = {k: np.zeros_like(v) for k, v in p.items()}
    orc = GO.GPT2Oracle(cfg["n_layer"], cfg["n_head"])
    assert len(fx["loss"]) >= 20
    for step, want in enumerate(fx["loss"]):
        ids, labels = synthetic_batch(step, 0, cfg["batch_size"], cfg["seq_len"], cfg["vocab_size"])
        loss, g = orc.loss_and_grads(p, ids.astype(np.int64), labels.astype(np.int64))
        assert loss == pytest.approx(want, rel=1e-3), f"step {step}"
        g, _ = GO.clip_grad_norm(g, cfg["max_norm"])
        for k in p:
            p[k], m[k], vv[k] = GO.adamw_step(p[k], g[k], m[k], vv[k], step + 1, cfg["lr"], wd=cfg["weight_decay"])


# ---- GPU: libgt_b200.so against what the reference computed ---------------------------------------------------

@pytest.mark.gpu
def test_gemm_matches_the_stored_reference_outputs(gt):
    store = _outputs()
    for tag, kind, layout, a, b, bias, c0 in _phase4_cases(store):
        epi = KIND_OF[kind][1]
        tf = U.run_gemm(layout, a, b, bias=bias, c0=c0, epilogue=epi, precision="tf32")
        x3 = U.run_gemm(layout, a, b, bias=bias, c0=c0, epilogue=epi, precision="3xtf32")
        assert np.allclose(tf, store[tag + "/ref_triton"], rtol=1e-2, atol=1e-3), tag
        assert O.rel_frobenius(x3, store[tag + "/ref_cuda"]) <= 1e-5, tag
    for tag, layout, a, b, bias, c0, epi in _config0():
        rows = store[tag + "/ref_triton"].shape[0]
        tf = U.run_gemm(layout, a, b, bias=bias, c0=c0, epilogue=epi, precision="tf32")
        x3 = U.run_gemm(layout, a, b, bias=bias, c0=c0, epilogue=epi, precision="3xtf32")
        assert O.rel_frobenius(tf[:rows], store[tag + "/ref_triton"]) <= 1e-3, tag
        assert O.rel_frobenius(x3[:rows], store[tag + "/ref_cuda"]) <= 1e-5, tag


def _replay(cfg, steps):
    from gradtuity_b200 import _lib
    from gradtuity_b200.gpt2.train import build_model, synthetic_batch, train_step
    from gradtuity_b200.optim import AdamW
    from gradtuity_b200.tensor import Tensor

    model = build_model(vocab_size=cfg["vocab_size"], seq_len=cfg["seq_len"], n_embd=cfg["n_embd"], n_layer=cfg["n_layer"],
                        n_head=cfg["n_head"], seed=3)
    params = model.parameters()
    opt = AdamW(params, lr=cfg["lr"], weight_decay=cfg["weight_decay"])
    losses = []
    for step in range(steps):
        ids, labels = synthetic_batch(step, 0, cfg["batch_size"], cfg["seq_len"], cfg["vocab_size"])
        losses.append(train_step(model, opt, params, Tensor.from_numpy(ids), Tensor.from_numpy(labels), cfg["max_norm"]).item())
    _lib.device_status()
    return np.array(losses)


@pytest.mark.gpu
@pytest.mark.parametrize("fixture", ["reference_gpt2_tiny_loss_curve.json", "reference_gpt2_loss_curve.json"])
def test_gpt2_loss_curve_tracks_the_reference(gt, fixture, monkeypatch):
    """The end-to-end criterion: our train step, replayed on the reference's seeded weights and batches, gives the
    reference's loss within 1e-3 relative at every step: 200 steps of GPT-2-small (12 layers, vocabulary 50257,
    batch 8 x 1024), and the two-layer model the float64 oracle is pinned with."""
    monkeypatch.setenv("GRADTUITY_GEMM_PRECISION", "tf32")
    fx = _json(fixture)
    want = np.array(fx["loss"])
    if fixture == "reference_gpt2_loss_curve.json":
        assert len(want) == 200 and fx["config"]["n_layer"] == 12 and fx["config"]["vocab_size"] == 50257
    got = _replay(fx["config"], len(want))
    rel = np.abs(got - want) / np.abs(want)
    assert rel.max() <= 1e-3, (int(rel.argmax()), float(rel.max()))
