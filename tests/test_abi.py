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
    assert lib.xlstm_rmsnorm_fw(None, None, 0, None, None, 0, None, None, 4, 8, 8, 1e-6) == -1
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


def test_library_exports_nothing_the_header_does_not_declare():
    """Development hooks must not ship: every xlstm_* symbol of the dynamic symbol table is declared."""
    import subprocess
    xl = importlib.import_module("neural-networks_b200")
    out = subprocess.run(["nm", "-D", "--defined-only", xl._lib.LIB_PATH], capture_output=True, text=True, check=True).stdout
    exported = sorted({line.split()[-1] for line in out.splitlines() if line.split() and line.split()[-1].startswith("xlstm_")})
    assert exported == _declared()


def test_no_launch_helper_keeps_a_process_wide_attribute_flag():
    """cudaFuncSetAttribute applies to one device: a launcher that remembers having set it must remember it
    per device, or the second GPU of a process launches without the shared-memory opt-in."""
    csrc = os.path.join(ROOT, "neural-networks_b200", "csrc")
    for f in sorted(os.listdir(csrc)):
        if not f.endswith((".cu", ".cuh")):
            continue
        text = open(os.path.join(csrc, f)).read()
        if "cudaFuncSetAttribute" not in text:
            continue
        assert not re.search(r"static\s+bool\s+\w*attr\w*\s*=", text), f + ": process-wide attribute flag"


def test_dp_entry_points_refuse_use_before_init():
    xl = importlib.import_module("neural-networks_b200")
    lib = xl._lib.lib
    assert lib.xlstm_dp_world() == 0
    assert lib.xlstm_dp_bucket_start(0, None) < 0
    assert lib.xlstm_dp_wait(None) < 0
    assert lib.xlstm_dp_shutdown() == 0
