"""GPU parity of the chunkwise mLSTM core against the CPU oracle (recurrent form, float64),
through the C ABI. Shapes and invariants follow the reference's own GPU tests:
mlstm_matches_cpu, mlstm_fused_tiled_matches_cpu, mlstm_fused_ragged_chunk_matches_cpu,
mlstm_chunking_matches_single_chunk, mlstm_chunked_carry_matches_whole,
mlstm_chunked_backward_matches_whole (src/gpu/mlstm.rs:1004-1533).

Bars: rel-to-max 1e-4 for fp32 storage, 2e-2 for bf16 storage."""
import numpy as np
import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-4, torch.bfloat16: 2e-2}


def _run(shape, L, dtype, gdtype, seed=0, flags=0, save_states=True, carry=None, dstate=None):
    from gpu_util import ops, dev, host, mlstm_inputs, bf16_round
    B, H, T, dqk, dhv = shape
    bf = dtype == torch.bfloat16
    q, k, v, ig, fg, dy = mlstm_inputs(*shape, seed=seed, bf16=bf)
    if gdtype == torch.bfloat16:
        dy = bf16_round(dy)
    st = ops.MlstmShape(B, H, T, dqk, dhv, L, dtype, gdtype, flags)
    dq_, dk_, dv_ = dev(q, dtype), dev(k, dtype), dev(v, dtype)
    di_, df_ = dev(ig), dev(fg)
    cin = None if carry is None else tuple(dev(a) for a in carry)
    fused = ops.mlstm_fused_fw(dq_, dk_, dv_, di_, df_, st, carry_in=cin, save_states=save_states)
    din = None if dstate is None else tuple(dev(a) for a in dstate)
    grads = ops.mlstm_fused_bw(fused, dq_, dk_, dv_, di_, df_, dev(dy, gdtype), st, carry_in=cin, dstate_in=din)
    torch.cuda.synchronize()
    c0 = dict(C0=None, n0=None, m0=None) if carry is None else dict(C0=carry[0], n0=carry[1], m0=carry[2])
    d0 = dict(dC_in=None, dn_in=None) if dstate is None else dict(dC_in=dstate[0], dn_in=dstate[1])
    ofw = O.mlstm_core_fw(q, k, v, ig, fg, B, H, T, dqk, dhv, **c0)
    obw = O.mlstm_core_bw(q, k, v, ig, fg, dy, B, H, T, dqk, dhv, **c0, **d0)
    got = dict(ytil=host(fused.ytil), m=host(fused.msv), psi=host(fused.psiv), nq=host(fused.qnv),
               C=host(fused.state[0]), n=host(fused.state[1]), mlast=host(fused.state[2]),
               dq=host(grads[0]), dk=host(grads[1]), dv=host(grads[2]), dig=host(grads[3]), dfg=host(grads[4]),
               dC=host(grads[5][0]), dn=host(grads[5][1]))
    ref = dict(ofw)
    ref.update(obw)
    return got, ref


def _assert_close(got, ref, tol, names):
    from gpu_util import rel_to_max
    for n in names:
        e = rel_to_max(got[n], ref[n])
        assert e <= tol, "%s: rel-to-max error %.3e > %.1e" % (n, e, tol)


FW = ("ytil", "m", "psi", "C", "n", "mlast")
BW = ("dq", "dk", "dv", "dig", "dfg", "dC", "dn")


@pytest.mark.parametrize("shape,L", [((2, 2, 6, 4, 4), 64), ((2, 2, 20, 4, 4), 8), ((2, 8, 70, 96, 96), 32),
                                     ((2, 8, 200, 64, 64), 32), ((1, 2, 130, 32, 48), 64)])
def test_fp32_matches_oracle(shape, L):
    got, ref = _run(shape, L, torch.float32, torch.float32)
    _assert_close(got, ref, 1e-4, FW + BW)


@pytest.mark.parametrize("L", [1, 3, 8, 16, 32, 64, 200])
def test_chunk_length_does_not_change_results(L):
    got, ref = _run((2, 2, 70, 8, 12), L, torch.float32, torch.float32, seed=5)
    _assert_close(got, ref, 1e-4, FW + BW)


@pytest.mark.parametrize("shape,L", [((2, 2, 20, 4, 4), 8), ((2, 4, 200, 64, 64), 64), ((1, 2, 256, 128, 128), 64)])
@pytest.mark.parametrize("gdtype", [torch.float32, torch.bfloat16])
def test_bf16_storage_matches_oracle(shape, L, gdtype):
    got, ref = _run(shape, L, torch.bfloat16, gdtype, flags=1)
    _assert_close(got, ref, 2e-2, FW + BW)


def test_carry_in_and_bptt_state_in():
    """A call that continues a recurrence (state in) and receives BPTT state from its right."""
    B, H, T, dqk, dhv = 2, 2, 40, 8, 8
    r = np.random.default_rng(11)
    carry = (r.standard_normal((B * H, dhv, dqk)), r.standard_normal((B * H, dqk)), r.standard_normal((B * H,)))
    dstate = (r.standard_normal((B * H, dhv, dqk)) * 0.1, r.standard_normal((B * H, dqk)) * 0.1)
    carry = tuple(a.astype(np.float32).astype(np.float64) for a in carry)
    dstate = tuple(a.astype(np.float32).astype(np.float64) for a in dstate)
    got, ref = _run((B, H, T, dqk, dhv), 16, torch.float32, torch.float32, carry=carry, dstate=dstate)
    _assert_close(got, ref, 1e-4, FW + BW)


def test_recomputed_states_equal_saved_states():
    a, _ = _run((2, 2, 100, 16, 16), 32, torch.float32, torch.float32, save_states=True)
    b, _ = _run((2, 2, 100, 16, 16), 32, torch.float32, torch.float32, save_states=False)
    for n in BW:
        assert np.array_equal(a[n], b[n]), n


def test_bit_repeatable():
    a, _ = _run((2, 4, 130, 32, 32), 64, torch.bfloat16, torch.float32, flags=1)
    b, _ = _run((2, 4, 130, 32, 32), 64, torch.bfloat16, torch.float32, flags=1)
    for n in FW + BW:
        assert np.array_equal(a[n], b[n]), n


def test_declines_oversized_tile_without_launching():
    from gpu_util import ops, xl
    st = ops.MlstmShape(1, 1, 64, 512, 512, 64, torch.float32, torch.float32, flags=1)
    z = torch.zeros((64, 512), device="cuda")
    g = torch.zeros((64, 1), device="cuda")
    before = xl._lib.lib.xlstm_launch_count()
    with pytest.raises(xl._lib.Declined):
        ops.mlstm_fused_fw(z, z, z, g, g, st)
    assert xl._lib.lib.xlstm_launch_count() == before


# ---- tensor-core path (dqk = dhv = 128, L = 64, bf16 storage; flags = 0 selects it) -----------
@pytest.mark.parametrize("shape", [(1, 2, 64, 128, 128), (1, 2, 256, 128, 128), (2, 3, 200, 128, 128), (2, 2, 40, 128, 128),
                                   (5, 2, 9, 128, 128), (8, 4, 1, 128, 128), (2, 1, 9, 256, 128)])
@pytest.mark.parametrize("gdtype", [torch.float32, torch.bfloat16])
def test_tensor_core_path_matches_oracle(shape, gdtype):
    from gpu_util import xl
    got, ref = _run(shape, 64, torch.bfloat16, gdtype, seed=21)
    assert xl._lib.lib.xlstm_device_status() == 0, xl._lib.lib.xlstm_last_error()
    _assert_close(got, ref, 2e-2, FW + BW)


def test_tensor_core_path_with_carry():
    from gpu_util import xl
    B, H, T, d = 2, 2, 150, 128
    r = np.random.default_rng(12)
    f32 = lambda a: a.astype(np.float32).astype(np.float64)
    carry = (f32(r.standard_normal((B * H, d, d))), f32(r.standard_normal((B * H, d))), f32(r.standard_normal((B * H,))))
    dstate = (f32(r.standard_normal((B * H, d, d)) * 0.1), f32(r.standard_normal((B * H, d)) * 0.1))
    got, ref = _run((B, H, T, d, d), 64, torch.bfloat16, torch.float32, carry=carry, dstate=dstate)
    assert xl._lib.lib.xlstm_device_status() == 0, xl._lib.lib.xlstm_last_error()
    _assert_close(got, ref, 2e-2, FW + BW)


def test_tensor_core_path_agrees_with_cuda_core_path():
    a, _ = _run((2, 4, 256, 128, 128), 64, torch.bfloat16, torch.float32, seed=22, flags=0)
    b, _ = _run((2, 4, 256, 128, 128), 64, torch.bfloat16, torch.float32, seed=22, flags=1)
    _assert_close(a, b, 2e-2, FW + BW)


def test_tensor_core_path_bit_repeatable():
    a, _ = _run((2, 2, 200, 128, 128), 64, torch.bfloat16, torch.float32, seed=23)
    b, _ = _run((2, 2, 200, 128, 128), 64, torch.bfloat16, torch.float32, seed=23)
    for n in FW + BW:
        assert np.array_equal(a[n], b[n]), n


def test_tensor_core_backward_recomputes_chunk_states_when_no_record_is_kept():
    """saved = NULL: the backward rebuilds the chunk-boundary states with the forward's state-only pass;
    the gradients are bit-identical to the saved-record path."""
    a, _ = _run((2, 2, 200, 128, 128), 64, torch.bfloat16, torch.float32, seed=24, save_states=True)
    b, _ = _run((2, 2, 200, 128, 128), 64, torch.bfloat16, torch.float32, seed=24, save_states=False)
    for n in BW:
        assert np.array_equal(a[n], b[n]), n


# ---- heads wider than 128: run as 128 x 128 sub-heads whose partial results are summed ---------
@pytest.mark.parametrize("shape", [(1, 2, 200, 256, 256), (2, 1, 70, 128, 256), (1, 2, 130, 256, 128), (1, 1, 64, 384, 256)])
@pytest.mark.parametrize("gdtype", [torch.float32, torch.bfloat16])
def test_wide_heads_match_oracle(shape, gdtype):
    from gpu_util import xl
    got, ref = _run(shape, 64, torch.bfloat16, gdtype, seed=31)
    assert xl._lib.lib.xlstm_device_status() == 0, xl._lib.lib.xlstm_last_error()
    _assert_close(got, ref, 2e-2, FW + BW)


def test_wide_heads_with_carry_and_recompute():
    from gpu_util import xl
    B, H, T, dqk, dhv = 2, 2, 150, 256, 256
    r = np.random.default_rng(13)
    f32 = lambda a: a.astype(np.float32).astype(np.float64)
    carry = (f32(r.standard_normal((B * H, dhv, dqk))), f32(r.standard_normal((B * H, dqk))), f32(r.standard_normal((B * H,))))
    dstate = (f32(r.standard_normal((B * H, dhv, dqk)) * 0.1), f32(r.standard_normal((B * H, dqk)) * 0.1))
    got, ref = _run((B, H, T, dqk, dhv), 64, torch.bfloat16, torch.float32, carry=carry, dstate=dstate, save_states=False)
    assert xl._lib.lib.xlstm_device_status() == 0, xl._lib.lib.xlstm_last_error()
    _assert_close(got, ref, 2e-2, FW + BW)


@pytest.mark.parametrize("shape,L,dtype", [((2, 2, 70, 8, 12), 16, torch.float32), ((2, 2, 150, 128, 128), 64, torch.bfloat16),
                                           ((1, 2, 130, 256, 128), 64, torch.bfloat16), ((3, 2, 9, 128, 128), 64, torch.bfloat16)])
def test_final_state_alone_equals_the_forwards_final_state(shape, L, dtype):
    """The states-only entry point walks the same recurrence as the forward: bit-identical (C, n, m), with a carry."""
    from gpu_util import ops, dev, mlstm_inputs, xl
    B, H, T, dqk, dhv = shape
    q, k, v, ig, fg, _ = mlstm_inputs(*shape, seed=61, bf16=dtype == torch.bfloat16)
    r = np.random.default_rng(62)
    carry = tuple(dev(a) for a in (r.standard_normal((B * H, dhv, dqk)), r.standard_normal((B * H, dqk)), r.standard_normal((B * H,))))
    st = ops.MlstmShape(B, H, T, dqk, dhv, L, dtype, torch.float32)
    args = (dev(q, dtype), dev(k, dtype), dev(v, dtype), dev(ig), dev(fg), st)
    for cin in (None, carry):
        full = ops.mlstm_fused_fw(*args, carry_in=cin, save_states=False, want_state=True).state
        alone = ops.mlstm_final_state(*args, carry_in=cin)
        torch.cuda.synchronize()
        assert xl._lib.lib.xlstm_device_status() == 0
        for a, b in zip(alone, full):
            assert torch.equal(a, b)


def test_caller_buffers_reused_across_shapes_with_stale_contents():
    """The boundary's ownership rule (caller allocates every buffer, possibly larger than the shape and holding
    stale data; the callee writes every element of its outputs; src/gpu/buf.rs:24-30, and the reference's own
    pooled-buffer test src/gpu/slstm.rs:1615-1647): one set of oversized, NaN-poisoned output, record and
    workspace buffers serves calls of three different shapes in a row, and each call's results are bit-identical
    to the same call on fresh exact-size buffers."""
    import ctypes
    from gpu_util import ops, xl
    lib, L = xl._lib.lib, xl._lib
    shapes = [(2, 2, 200, 128, 128), (1, 4, 64, 128, 128), (2, 1, 130, 256, 256), (2, 2, 200, 128, 128)]
    big = 1 << 26  # bytes per pooled buffer
    pool = {n: torch.empty(big, dtype=torch.uint8, device="cuda") for n in
            ("ytil", "msv", "psiv", "qnv", "saved", "ws", "dq", "dk", "dv", "dig", "dfg", "wsb")}
    gen = torch.Generator(device="cuda").manual_seed(5)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    for (B, H, T, dqk, dhv) in shapes:
        st = ops.MlstmShape(B, H, T, dqk, dhv, 64, torch.bfloat16, torch.float32)
        rnd = lambda *s: torch.randn(s, device="cuda", generator=gen)
        q, v = rnd(B * T, H * dqk).to(torch.bfloat16), rnd(B * T, H * dhv).to(torch.bfloat16)
        k = (rnd(B * T, H * dqk) / dqk ** 0.5).to(torch.bfloat16)
        ig, fg, dy = rnd(B * T, H), rnd(B * T, H) + 3.0, rnd(B * T, H * dhv)
        fused = ops.mlstm_fused_fw(q, k, v, ig, fg, st, want_state=False)
        want = ops.mlstm_fused_bw(fused, q, k, v, ig, fg, dy, st, want_dstate=False)
        for t in pool.values():
            t.view(torch.float32).fill_(float("nan"))
        wsf = lib.xlstm_mlstm_fw_workspace_bytes(ctypes.byref(st.c))
        assert lib.xlstm_mlstm_saved_bytes(ctypes.byref(st.c)) <= big and wsf <= big
        stream = torch.cuda.current_stream().cuda_stream
        L.check(lib.xlstm_mlstm_fw(stream, ctypes.byref(st.c), p(q), p(k), p(v), p(ig), p(fg), None, None, None, p(pool["ytil"]),
                                   p(pool["msv"]), p(pool["psiv"]), p(pool["qnv"]), p(pool["saved"]), None, None, None,
                                   p(pool["ws"]), big), "fw")
        L.check(lib.xlstm_mlstm_bw(stream, ctypes.byref(st.c), p(q), p(k), p(v), p(ig), p(fg), None, None, None, p(pool["ytil"]),
                                   p(pool["msv"]), p(pool["psiv"]), p(pool["qnv"]), p(pool["saved"]), p(dy), None, None,
                                   p(pool["dq"]), p(pool["dk"]), p(pool["dv"]), p(pool["dig"]), p(pool["dfg"]), None, None,
                                   p(pool["wsb"]), big), "bw")
        torch.cuda.synchronize()
        n = B * T
        got_y = pool["ytil"].view(torch.bfloat16)[:n * H * dhv].view(n, H * dhv)
        assert torch.equal(got_y, fused.ytil)
        for name, ref in zip(("dq", "dk", "dv", "dig", "dfg"), want[:5]):
            got = pool[name].view(torch.float32)[:ref.numel()].view(ref.shape)
            assert torch.equal(got, ref), name
        assert xl._lib.lib.xlstm_device_status() == 0


@pytest.mark.parametrize("B,T", [(20, 9), (14, 9), (7, 9), (130, 1), (5, 32), (19, 7), (23, 3), (64, 16), (3, 21)])
@pytest.mark.parametrize("gdtype,save", [(torch.float32, True), (torch.bfloat16, False)])
def test_packed_short_sequences_equal_the_unpacked_call_and_the_oracle(B, T, gdtype, save):
    """XLSTM_PACK_SHORT: 64 // T carry-less sequences share a chunk tile (the hierarchical model's word rectangles).
    Same arithmetic per sequence up to the summation order of the gate scans, so the packed call agrees with the
    unpacked one to fp32 round-off (one bf16 ulp where the result is stored as bf16); both sit inside the bf16 bar of
    the float64 oracle. Covers batch
    sizes below, at and off a multiple of the tile's capacity (the remainder runs unpacked on the tail), T = 1 (64 to
    a tile), T = 32 (two), T = 21 (three, with one idle row), and both ways of getting the chunk states."""
    from gpu_util import ops, dev, host, mlstm_inputs, bf16_round, rel_to_max
    H, d = 2, 128
    q, k, v, ig, fg, dy = mlstm_inputs(B, H, T, d, d, seed=31 + B + T, bf16=True)
    if gdtype == torch.bfloat16:
        dy = bf16_round(dy)
    dt = torch.bfloat16
    args = (dev(q, dt), dev(k, dt), dev(v, dt), dev(ig), dev(fg))
    out = {}
    for name, flags in (("packed", ops.PACK_SHORT), ("plain", 0)):
        st = ops.MlstmShape(B, H, T, d, d, 64, dt, gdtype, flags)
        fused = ops.mlstm_fused_fw(*args, st, save_states=save, want_state=False)
        grads = ops.mlstm_fused_bw(fused, *args, dev(dy, gdtype), st, want_dstate=False)
        torch.cuda.synchronize()
        out[name] = (fused, grads)
    assert ops.lib.xlstm_device_status() == 0
    fp, gp = out["packed"]
    fu, gu = out["plain"]
    # (a position's place in the tile changes the order of the gate scans' additions: last-bit differences in m)
    for a, b, n, bar in ((fp.ytil, fu.ytil, "ytil", 2.0 ** -8), (fp.msv, fu.msv, "m", 1e-6), (fp.psiv, fu.psiv, "psi", 1e-6),
                         (fp.qnv, fu.qnv, "qn", 1e-5)):
        assert rel_to_max(host(a), host(b)) <= bar, n
    for i, n in enumerate(("dq", "dk", "dv", "dig", "dfg")):
        assert rel_to_max(host(gp[i]), host(gu[i])) <= (1e-5 if gdtype == torch.float32 else 2.0 ** -8), n
    ofw = O.mlstm_core_fw(q, k, v, ig, fg, B, H, T, d, d, C0=None, n0=None, m0=None)
    obw = O.mlstm_core_bw(q, k, v, ig, fg, dy, B, H, T, d, d, C0=None, n0=None, m0=None, dC_in=None, dn_in=None)
    got = dict(ytil=host(fp.ytil), m=host(fp.msv), psi=host(fp.psiv), dq=host(gp[0]), dk=host(gp[1]), dv=host(gp[2]),
               dig=host(gp[3]), dfg=host(gp[4]))
    ref = dict(ofw)
    ref.update(obw)
    _assert_close(got, ref, TOL[torch.bfloat16], ("ytil", "m", "psi", "dq", "dk", "dv", "dig", "dfg"))


def test_packed_flag_is_refused_with_a_carry_or_a_state_request_and_ignored_where_it_does_not_apply():
    from gpu_util import ops, dev, mlstm_inputs
    B, H, T, d = 8, 2, 9, 128
    q, k, v, ig, fg, dy = mlstm_inputs(B, H, T, d, d, seed=5, bf16=True)
    dt = torch.bfloat16
    args = (dev(q, dt), dev(k, dt), dev(v, dt), dev(ig), dev(fg))
    st = ops.MlstmShape(B, H, T, d, d, 64, dt, torch.float32, ops.PACK_SHORT)
    with pytest.raises(Exception, match="PACK_SHORT"):
        ops.mlstm_fused_fw(*args, st, want_state=True)
    fused = ops.mlstm_fused_fw(*args, st, want_state=False)
    with pytest.raises(Exception, match="PACK_SHORT"):
        ops.mlstm_fused_bw(fused, *args, dev(dy), st, want_dstate=True)
    # CUDA-core path (fp32 storage, small heads): the flag changes nothing
    q, k, v, ig, fg, dy = mlstm_inputs(4, 2, 6, 8, 8, seed=6)
    a32 = (dev(q), dev(k), dev(v), dev(ig), dev(fg))
    res = []
    for flags in (ops.PACK_SHORT, 0):
        s32 = ops.MlstmShape(4, 2, 6, 8, 8, 64, torch.float32, torch.float32, flags)
        res.append(ops.mlstm_fused_fw(*a32, s32, want_state=True).ytil)
    assert torch.equal(res[0], res[1])
