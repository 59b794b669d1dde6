"""The allocation-free cross-entropy entry point, called through the C ABI.

xlstm_ce_fw_bw_noalloc is for hosts that cannot hand the op a scratch buffer because they cannot
allocate device memory at that point (their pool already owns the device, or the step loop must
not touch the CUDA allocator). Its scratch is a fixed array inside the library, shared by every
call on the device and never cleared, so this test runs it twice in a row on different inputs and
requires both results to equal what the ordinary entry point (caller-owned workspace) produces.
The file name keeps it last in collection order: a run that stops at the first failure has then
already exercised everything else.
"""
import ctypes
import importlib

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _both(lib, rows, C, seed, masked):
    g = torch.Generator(device="cuda").manual_seed(seed)
    logits = torch.randn((rows, C), device="cuda", generator=g) * 3
    targets = torch.randint(0, C, (rows,), device="cuda", generator=g, dtype=torch.int32)
    mask = None
    if masked:
        mask = (torch.rand((rows,), device="cuda", generator=g) > 0.25).to(torch.int32)
    inv = 1.0 / rows
    stream = torch.cuda.current_stream().cuda_stream
    mp = None if mask is None else mask.data_ptr()
    # reference: the existing entry point with a caller-owned workspace
    d_ref = torch.empty_like(logits)
    loss_ref = torch.zeros((1,), device="cuda")
    ws = torch.empty((lib.xlstm_ce_workspace_bytes(rows),), dtype=torch.uint8, device="cuda")
    assert lib.xlstm_ce_fw_bw(stream, logits.data_ptr(), targets.data_ptr(), mp, d_ref.data_ptr(), loss_ref.data_ptr(),
                              rows, C, inv, ws.data_ptr(), ws.numel()) == 0, lib.xlstm_last_error()
    # the allocation-free entry point: inputs and outputs only
    d_new = torch.full_like(logits, float("nan"))
    loss_new = torch.zeros((1,), device="cuda")
    assert lib.xlstm_ce_fw_bw_noalloc(stream, logits.data_ptr(), targets.data_ptr(), mp, d_new.data_ptr(),
                                      loss_new.data_ptr(), rows, C, inv) == 0, lib.xlstm_last_error()
    torch.cuda.synchronize()
    return d_ref, loss_ref, d_new, loss_new


def test_noalloc_matches_workspace_entry_point_on_two_calls_in_a_row():
    xl = importlib.import_module("neural-networks_b200")
    lib = xl._lib.lib
    # second call is smaller and masked: leftovers of the first call sit in the shared scratch
    for rows, C, seed, masked in [(4096, 1000, 1, False), (1500, 50304, 2, True)]:
        d_ref, loss_ref, d_new, loss_new = _both(lib, rows, C, seed, masked)
        # same kernels, same order of operations: 1e-4 is the bar of the other CE tests, equality is expected
        err = (d_new - d_ref).abs().max().item() / max(d_ref.abs().max().item(), 1e-30)
        assert err <= 1e-4, err
        assert abs(loss_new.item() - loss_ref.item()) <= 1e-4 * max(1.0, abs(loss_ref.item()))
        assert torch.isfinite(d_new).all()


def test_noalloc_refuses_more_rows_than_its_scratch_holds():
    xl = importlib.import_module("neural-networks_b200")
    lib = xl._lib.lib
    rows = 65536 + 1
    x = torch.zeros((8,), device="cuda")
    rc = lib.xlstm_ce_fw_bw_noalloc(torch.cuda.current_stream().cuda_stream, x.data_ptr(), x.data_ptr(), None, x.data_ptr(),
                                    x.data_ptr(), rows, 1, 1.0)
    assert rc == -1
    assert b"exceed" in lib.xlstm_last_error()
