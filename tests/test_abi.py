"""The C-ABI library loads without a GPU and exports every symbol include/bfuse_b200.h declares."""
import ctypes
import os
import re

import numpy as np

import bfuse_project_b200 as bf

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "bfuse_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bfuse_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported():
    names = declared_symbols()
    assert len(names) >= 30
    L = ctypes.CDLL(bf.LIB_PATH)
    missing = [n for n in names if not hasattr(L, n)]
    assert not missing, missing


def test_check_matrix_follows_the_reference_rule():
    ans = np.array([1.0, 0.0, 100.0, 1e-6], np.float32)
    assert bf.check_matrix(ans, ans) == 0
    # abs error above eps but relative below -> accepted; both above -> counted
    assert bf.check_matrix(np.array([1.0005, 0.0, 100.05, 1e-6], np.float32), ans) == 0
    assert bf.check_matrix(np.array([1.002, 0.0, 100.0, 1e-6], np.float32), ans) == 1
    # answer exactly zero: only the absolute test applies
    assert bf.check_matrix(np.array([1.0, 0.002, 100.0, 1e-6], np.float32), ans) == 1
    assert bf.check_matrix(np.array([np.nan, 0.0, 100.0, 1e-6], np.float32), ans) == 1


def test_context_creation_fails_loudly_without_a_device():
    import torch
    if torch.cuda.is_available():
        return
    try:
        bf.Runtime(0)
    except bf.BfuseError as e:
        assert e.code == 5
    else:
        raise AssertionError("a context must not be created without an sm_100 device")
