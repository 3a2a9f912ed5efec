"""Helpers shared by the tests: reference-test input generators and device buffers."""
import json
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = os.path.join(HERE, "golden")

LAYOUTS = {"NN": 0, "NT": 1, "TN": 2}
EPILOGUES = {"none": 0, "bias": 1, "bias_relu": 2, "bias_gelu": 3, "causal": 4}
PRECISIONS = {"tf32": 0, "3xtf32": 1, "fp32": 2}
# Parity bars: relative Frobenius error against the float64 oracle.
TOL = {"tf32": 1e-3, "3xtf32": 1e-5, "fp32": 1e-5}


def known_answers():
    with open(os.path.join(GOLDEN, "reference_known_answers.json")) as f:
        return json.load(f)


def phase4_vectors():
    return dict(np.load(os.path.join(GOLDEN, "phase4_vectors.npz")))


def phase4_inputs(kind, M, N, K):
    """Inputs of gradtuity/tests/test_kernels_cuda_phase4.py:27-167 for one case.
    Returns (layout, a, b, bias, c0) with a/b shaped as stored."""
    def av(n):
        return np.array([(((i * 13) % 41) - 20) / 100.0 for i in range(n)], dtype=np.float32)

    def bv(n):
        return np.array([(((i * 7) % 37) - 18) / 100.0 for i in range(n)], dtype=np.float32)

    bias = np.array([0.05 * (i % 7) - 0.2 for i in range(N)], dtype=np.float32)
    c0 = np.array([0.001 * i for i in range(M * N)], dtype=np.float32).reshape(M, N)
    if kind in ("matmul", "matmul_bias", "matmul_bias_relu"):
        return "NN", av(M * K).reshape(M, K), bv(K * N).reshape(K, N), (bias if kind != "matmul" else None), None
    if kind == "matmul_nt_acc":
        return "NT", av(M * K).reshape(M, K), bv(N * K).reshape(N, K), None, c0
    if kind == "matmul_tn_acc":
        return "TN", av(K * M).reshape(K, M), bv(K * N).reshape(K, N), None, c0
    raise ValueError(kind)


PHASE4_CASES = (
    [("matmul", M, N, K) for (M, K, N) in [(32, 32, 32), (64, 96, 48), (17, 33, 19)]]
    + [("matmul_bias", M, N, K) for (M, K, N) in [(64, 96, 48), (17, 33, 19)]]
    + [("matmul_bias_relu", M, N, K) for (M, K, N) in [(64, 96, 48), (17, 33, 19)]]
    + [("matmul_nt_acc", M, N, K) for (M, N, K) in [(48, 32, 64), (19, 17, 33)]]
    + [("matmul_tn_acc", M, N, K) for (M, N, K) in [(48, 32, 64), (19, 17, 33)]]
)


def phase4_key(kind, M, N, K):
    if kind in ("matmul", "matmul_bias", "matmul_bias_relu"):
        return f"{kind}_{M}_{K}_{N}"
    return f"{kind}_{M}_{N}_{K}"


class DeviceBuffer:
    """A device allocation holding a numpy array's contents (float32)."""

    def __init__(self, array=None, *, nbytes=None, offset_elems=0):
        from gradtuity_b200 import cuda_mem as cm

        self._cm = cm
        if array is not None:
            array = np.ascontiguousarray(array, dtype=np.float32)
            nbytes = array.nbytes
        self.nbytes = nbytes
        self.base = cm.cuda_malloc(nbytes + 4 * offset_elems + 16)
        self.ptr = self.base + 4 * offset_elems
        if array is not None:
            cm.cuda_memcpy_htod(self.ptr, array)

    def read(self, shape):
        out = np.empty(shape, dtype=np.float32)
        self._cm.cuda_memcpy_dtoh_into(self.ptr, out)
        return out

    def free(self):
        if self.base:
            self._cm.cuda_free(self.base)
            self.base = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def _padded(x, pad, fill=np.nan):
    if pad == 0:
        return np.ascontiguousarray(x, dtype=np.float32)
    out = np.full((x.shape[0], x.shape[1] + pad), fill, dtype=np.float32)
    out[:, :x.shape[1]] = x
    return out


def run_gemm(layout, a, b, *, bias=None, c0=None, epilogue="none", precision="tf32", alpha=1.0,
             want_aux=False, misalign=0, pad=0, return_path=False):
    """Upload, call gt_gemm through the C ABI, download. a, b are stored-layout 2-D arrays.

    pad: extra elements per stored row (leading dimension = row length + pad); the padding is
    filled with NaN on the operands (so reading it shows) and with a sentinel on C (so writing
    it shows).  misalign: element offset of the operand base pointers."""
    from ctypes import byref, c_int, c_void_p

    from gradtuity_b200 import _lib, gemm as G

    M = a.shape[1] if layout == "TN" else a.shape[0]
    K = a.shape[0] if layout == "TN" else a.shape[1]
    N = b.shape[0] if layout == "NT" else b.shape[1]
    da = DeviceBuffer(_padded(a, pad), offset_elems=misalign)
    db = DeviceBuffer(_padded(b, pad), offset_elems=misalign)
    SENT = np.float32(-12345.5)
    chost = np.full((M, N), np.nan, np.float32) if c0 is None else np.asarray(c0, np.float32)
    dc = DeviceBuffer(_padded(chost, pad, SENT))
    dbias = DeviceBuffer(bias) if bias is not None else None
    daux = DeviceBuffer(_padded(np.full((M, N), np.nan, np.float32), pad, SENT)) if want_aux else None
    lda, ldb, ldc = a.shape[1] + pad, b.shape[1] + pad, N + pad
    G.gemm(LAYOUTS[layout], M, N, K, da.ptr, lda, db.ptr, ldb, dc.ptr, ldc,
           bias_ptr=dbias.ptr if dbias else 0, aux_ptr=daux.ptr if daux else 0, alpha=alpha,
           accumulate=c0 is not None, epilogue=EPILOGUES[epilogue], precision=PRECISIONS[precision])
    _lib.device_status()
    full = dc.read((M, ldc))
    if pad:
        assert np.all(full[:, N:] == SENT), "GEMM wrote into the padding of C"
    out = np.ascontiguousarray(full[:, :N])
    res = [out]
    if want_aux:
        fa = daux.read((M, ldc))
        if pad:
            assert np.all(fa[:, N:] == SENT), "GEMM wrote into the padding of aux"
        res.append(np.ascontiguousarray(fa[:, :N]))
    if return_path:
        path = c_int(-1)
        _lib.check(_lib.load_library().gt_gemm_path(_lib.context(), LAYOUTS[layout], M, N, K, c_void_p(da.ptr), lda,
                                                    c_void_p(db.ptr), ldb, c_void_p(dc.ptr), ldc,
                                                    PRECISIONS[precision], byref(path)), "gt_gemm_path")
        res.append(path.value)
    return res[0] if len(res) == 1 else tuple(res)


def make_operands(layout, M, N, K, seed=1, scale=None):
    """Seeded operands ~ N(0, 1/sqrt(K)) stored in the layout's native order."""
    rng = np.random.default_rng(seed)
    s = (1.0 / np.sqrt(K)) if scale is None else scale
    ashape = (K, M) if layout == "TN" else (M, K)
    bshape = (N, K) if layout == "NT" else (K, N)
    a = (rng.standard_normal(ashape) * s).astype(np.float32)
    b = (rng.standard_normal(bshape) * s).astype(np.float32)
    return a, b, rng
