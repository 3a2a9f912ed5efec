"""Writes phase4_vectors.npz: outputs for the inputs of the reference's cross-backend kernel
tests (gradtuity/tests/test_kernels_cuda_phase4.py:27-167), computed by a scalar restatement
of what the reference's CUDA-C kernels do (gradtuity/kernels_cuda/matmul_kernels.py:21-236):
one fp32 accumulator per output, k ascending, fused multiply-add replaced by float32 multiply
then add (the difference is below 1e-6 here), bias / ReLU / "C +=" applied as there.

The reference test itself compares its two GPU backends with rtol 1e-2 / atol 1e-3 and holds
no absolute numbers; these vectors pin the same inputs to absolute values.

Run:  python tests/golden/make_phase4_vectors.py      (pure Python loops, a few seconds)
"""
import os

import numpy as np

f32 = np.float32


def a_vals(n):
    return [f32((((i * 13) % 41) - 20) / 100.0) for i in range(n)]


def b_vals(n):
    return [f32((((i * 7) % 37) - 18) / 100.0) for i in range(n)]


def bias_vals(n):
    return [f32(0.05 * (i % 7) - 0.2) for i in range(n)]


def kernel(M, N, K, a, b, sam, sak, sbk, sbn, bias=None, relu=False, c0=None):
    out = np.zeros((M, N), dtype=np.float32)
    for m in range(M):
        for n in range(N):
            acc = f32(0.0)
            for k in range(K):
                acc = f32(acc + f32(a[m * sam + k * sak] * b[k * sbk + n * sbn]))
            if bias is not None:
                acc = f32(acc + bias[n])
            if relu:
                acc = max(acc, f32(0.0))
            if c0 is not None:
                acc = f32(c0[m * N + n] + acc)
            out[m, n] = acc
    return out


def main():
    vec = {}
    for (M, K, N) in [(32, 32, 32), (64, 96, 48), (17, 33, 19)]:
        a, b = a_vals(M * K), b_vals(K * N)
        vec[f"matmul_{M}_{K}_{N}"] = kernel(M, N, K, a, b, K, 1, N, 1)
    for (M, K, N) in [(64, 96, 48), (17, 33, 19)]:
        a, b, bias = a_vals(M * K), b_vals(K * N), bias_vals(N)
        vec[f"matmul_bias_{M}_{K}_{N}"] = kernel(M, N, K, a, b, K, 1, N, 1, bias=bias)
        vec[f"matmul_bias_relu_{M}_{K}_{N}"] = kernel(M, N, K, a, b, K, 1, N, 1, bias=bias, relu=True)
    for (M, N, K) in [(48, 32, 64), (19, 17, 33)]:
        c0 = [f32(0.001 * i) for i in range(M * N)]
        a, b = a_vals(M * K), b_vals(N * K)
        vec[f"matmul_nt_acc_{M}_{N}_{K}"] = kernel(M, N, K, a, b, K, 1, 1, K, c0=c0)      # B stored (N, K)
        a, b = a_vals(K * M), b_vals(K * N)
        vec[f"matmul_tn_acc_{M}_{N}_{K}"] = kernel(M, N, K, a, b, 1, M, N, 1, c0=c0)      # A stored (K, M)
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "phase4_vectors.npz")
    np.savez_compressed(out, **vec)
    print("wrote", out, sorted(vec))


if __name__ == "__main__":
    main()
