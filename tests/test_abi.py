"""CPU-only: the C-ABI library loads and exports every symbol the header declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "jgb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(jg_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_entry_points():
    names = declared_symbols()
    assert "jg_aggregate_f32" in names and "jg_version" in names


def test_library_exports_every_declared_symbol():
    from jittorgeometric_b200 import _build, _lib
    if not os.path.exists(_lib.LIB_PATH):
        _build.build()
    L = ctypes.CDLL(_lib.LIB_PATH)
    missing = [n for n in declared_symbols() if not hasattr(L, n)]
    assert not missing, missing


def test_binding_table_matches_header():
    from jittorgeometric_b200 import _lib
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_host_only_entry_points():
    from jittorgeometric_b200 import _lib
    L = _lib.lib()
    assert L.jg_version() >= 100
    assert L.jg_status_string(0) == b"ok"
    assert L.jg_status_string(-3) == b"workspace missing or too small"
    assert L.jg_spmm_plan_bytes(10, 100, 4) > 0
    assert L.jg_spmm_plan_bytes(10, 100, 0) == 0
    assert L.jg_aggregate_workspace_bytes(10, 100, 8, 0) >= 8


def test_ops_refuse_cpu_tensors():
    import torch
    import jittorgeometric_b200 as jg
    x = torch.zeros((2, 4))
    with pytest.raises(RuntimeError):
        jg.ops.segment_aggregate(x, torch.zeros(1, dtype=torch.int32), torch.tensor([0, 1, 1], dtype=torch.int32),
                                 torch.ones(1))
