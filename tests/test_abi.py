"""CPU: the C-ABI library loads and exports every symbol include/gt_b200.h declares."""
import ctypes
import os
import re

from gradtuity_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "gt_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(gt_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_entry_points():
    syms = declared_symbols()
    for must in ("gt_init", "gt_gemm", "gt_gemm_batched", "gt_strerror", "gt_device_status"):
        assert must in syms


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(_lib.library_path())
    missing = [s for s in declared_symbols() if not hasattr(lib, s)]
    assert not missing, f"declared in include/gt_b200.h but not exported: {missing}"


def test_ctypes_table_covers_the_header():
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_strerror_needs_no_gpu():
    lib = _lib.load_library()
    assert lib.gt_strerror(0) == b"success"
    assert b"invalid" in lib.gt_strerror(_lib.GT_ERR_INVALID_ARG)
    assert b"bounded" in lib.gt_strerror(_lib.GT_ERR_TIMEOUT)


def test_null_context_is_rejected_without_a_gpu():
    lib = _lib.load_library()
    assert lib.gt_sync(None) == _lib.GT_ERR_INVALID_ARG
    assert lib.gt_gemm(None, 0, 1, 1, 1, None, 1, None, 1, None, 1, None, None, 1.0, 0, 0, 0, None) == _lib.GT_ERR_INVALID_ARG
