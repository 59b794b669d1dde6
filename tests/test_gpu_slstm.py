"""GPU parity of the persistent sLSTM loop against the CPU oracle, through the C ABI. Cases
follow the reference's slstm_matches_cpu_layer, slstm_long_t_matches_cpu, the fused == per-step
sweep over B in {1,64,256}, and slstm_chunked_carry (src/gpu/slstm.rs:1508-1938); block-diagonal
heads are checked against both the block oracle and the masked-dense identity. Bar: 1e-4
rel-to-max (all fp32)."""
import numpy as np
import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _case(B, H, NH, T, seed=0, carry=False):
    from gpu_util import ops, dev, host
    r = np.random.default_rng(seed)
    dh = H // NH
    f32 = lambda a: a.astype(np.float32).astype(np.float64)
    wh = f32(r.standard_normal((NH, dh, 4 * dh)) / np.sqrt(dh)) if NH > 1 else f32(r.standard_normal((H, 4 * H)) / np.sqrt(H))
    g = f32(r.standard_normal((B, T, 4 * H)))
    bcat = f32(np.concatenate([np.zeros(2 * H), np.full(H, 4.5), np.zeros(H)]) + 0.1 * r.standard_normal(4 * H))
    dy = f32(r.standard_normal((B, T, H)))
    state = dstate = None
    if carry:
        c = f32(r.standard_normal((B, H))); n = f32(np.abs(r.standard_normal((B, H))) + 0.5)
        m = f32(r.standard_normal((B, H))); h = f32(np.tanh(r.standard_normal((B, H))))
        state = (c, n, m, h)
        dstate = tuple(f32(0.1 * r.standard_normal((B, H))) for _ in range(3))
    fw = O.slstm_fw(wh, g, bcat, B, H, NH, T, state=state)
    bw = O.slstm_bw(wh, dy, fw, B, H, NH, T, dstate=dstate)

    dwh, dg, db = dev(wh), dev(g), dev(bcat)
    if carry:
        dst = tuple(dev(a) for a in state); dds = tuple(dev(a) for a in dstate)
    else:  # poisoned: the kernel must not read them
        dst = tuple(torch.full((B, H), float("nan"), device="cuda") for _ in range(4))
        dds = tuple(torch.full((B, H), float("nan"), device="cuda") for _ in range(3))
    out = torch.full((B, T, H), float("nan"), device="cuda")
    slabs = ops.SlstmSlabs(B, T, H, "cuda")
    ops.slstm_fused_time(dwh, dg, db, dst, out, slabs, nh=NH, carry=carry)
    g_after_fw = host(dg)
    ops.slstm_fused_time_bwd(dwh, dev(dy), dg, dds, slabs, nh=NH, carry=carry)
    torch.cuda.synchronize()
    got = dict(out=host(out), gf=g_after_fw[..., 2 * H:3 * H], dg=host(dg), c=host(dst[0]), n=host(dst[1]), m=host(dst[2]),
               h=host(dst[3]), dh=host(dds[0]), dc=host(dds[1]), dn=host(dds[2]))
    for nme in ("c_prev", "n_prev", "ipr", "fpr", "zt", "ot", "h_prev"):
        got[nme] = host(slabs.t[nme])
    ref = dict(out=fw["out"], gf=fw["g"][..., 2 * H:3 * H], dg=bw["dg"], c=fw["state"][0], n=fw["state"][1], m=fw["state"][2],
               h=fw["state"][3], dh=bw["dstate"][0], dc=bw["dstate"][1], dn=bw["dstate"][2])
    for nme in ("c_prev", "n_prev", "ipr", "fpr", "zt", "ot", "h_prev"):
        ref[nme] = fw[nme]
    return got, ref


def _check(got, ref, tol=1e-4):
    from gpu_util import rel_to_max
    for k in ref:
        e = rel_to_max(got[k], ref[k])
        assert e <= tol, "%s: rel-to-max error %.3e > %.1e" % (k, e, tol)


@pytest.mark.parametrize("B,H,T", [(2, 6, 5), (2, 12, 64), (1, 64, 64), (64, 64, 64), (256, 64, 33), (3, 40, 17)])
def test_dense_matches_oracle(B, H, T):
    _check(*_case(B, H, 1, T))


@pytest.mark.parametrize("B,H,NH,T", [(3, 32, 4, 17), (8, 256, 4, 40), (32, 1024, 4, 24), (5, 512, 2, 12)])
def test_block_diagonal_matches_oracle(B, H, NH, T):
    _check(*_case(B, H, NH, T, seed=1))


def test_carry_state_in_and_out():
    _check(*_case(4, 64, 2, 30, seed=2, carry=True))


# Heads too wide for one cluster's shared memory run on the grid-cooperative kernels, which split a
# head over up to all SMs and exchange through `out` / `g` in global memory.
@pytest.mark.parametrize("B,H,NH,T,carry", [(4, 1024, 1, 9, False), (3, 2048, 4, 7, False), (8, 2048, 4, 5, True),
                                            (11, 1024, 1, 4, True), (2, 1024, 2, 1, True)])
def test_wide_heads_match_oracle(B, H, NH, T, carry):
    _check(*_case(B, H, NH, T, seed=4, carry=carry))


def test_dense_too_wide_is_declined():
    from gpu_util import ops, xl
    B, H, T = 1, 4096, 4  # 256 MB of recurrent weights: more than the GPU's shared memory holds
    z = lambda *s: torch.zeros(s, device="cuda")
    before = xl._lib.lib.xlstm_launch_count()
    with pytest.raises(xl._lib.Declined):
        ops.slstm_fused_time(z(H, 4 * H), z(B, T, 4 * H), z(4 * H), tuple(z(B, H) for _ in range(4)), z(B, T, H),
                             ops.SlstmSlabs(B, T, H, "cuda"), nh=1)
    assert xl._lib.lib.xlstm_launch_count() == before


def test_bit_repeatable():
    a, _ = _case(8, 256, 4, 20, seed=3)
    b, _ = _case(8, 256, 4, 20, seed=3)
    for k in a:
        assert np.array_equal(a[k], b[k]), k


def test_grid_kernels_alternating_batch_sizes_and_very_short_sequences():
    """The grid kernels' flagged exchange tags every word with a launch number and a step. Calls that alternate
    between batch sizes (different kernel instantiations writing the same exchange array) and run for only two or
    three steps must never accept a word an earlier launch left behind: every call equals the oracle."""
    for i, (B, T) in enumerate([(8, 3), (4, 2), (8, 2), (4, 3), (8, 3), (2, 2)]):
        got, ref = _case(B, 1024, 1, T, seed=40 + i)
        _check(got, ref)
