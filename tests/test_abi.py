"""The C-ABI library loads and exports every symbol the public header declares (no compute
calls: this runs without a GPU)."""
import importlib
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "xlstm_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(xlstm_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    xl = importlib.import_module("neural-networks_b200")
    names = _declared()
    assert len(names) >= 10
    for n in names:
        assert hasattr(xl._lib.lib, n), "library does not export " + n
        assert n in xl._lib.SIGNATURES, "python binding lacks " + n
    assert sorted(xl._lib.SIGNATURES) == names


def test_version_and_error_text():
    xl = importlib.import_module("neural-networks_b200")
    assert xl._lib.lib.xlstm_version() >= 1
    assert isinstance(xl._lib.lib.xlstm_last_error(), bytes)


def test_argument_errors_are_reported_without_a_device():
    import ctypes
    xl = importlib.import_module("neural-networks_b200")
    lib = xl._lib.lib
    assert lib.xlstm_rmsnorm_fw(None, None, None, None, None, None, 4, 8, 8, 1e-6) == -1
    assert b"null pointer" in lib.xlstm_last_error()
    bad = xl._lib.MlstmShape(0, 1, 1, 1, 1, 1, 0, 0, 0)
    assert lib.xlstm_mlstm_saved_bytes(ctypes.byref(bad)) == 0


def test_ops_refuse_cpu_tensors():
    import pytest
    import torch
    xl = importlib.import_module("neural-networks_b200")
    x = torch.zeros(4, 8)
    with pytest.raises(xl._lib.XlstmError):
        xl.ops.rms_norm_forward_into(x, torch.ones(8), 8, torch.empty(4, 8), torch.empty(4))
