"""A trained model written as an NNM1 container and read back runs to the same bits, and the CPU oracle built
from the same file agrees with the GPU model within the fp32 bar."""
import importlib

import numpy as np
import pytest
import torch

from oracle import model as M

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("nh_s,tied", [(1, True), (2, True), (1, False)])
def test_saved_model_reloads_to_identical_logits(tmp_path, nh_s, tied):
    xl = importlib.import_module("neural-networks_b200")
    layers = importlib.import_module("neural-networks_b200.layers")
    ck = importlib.import_module("neural-networks_b200.checkpoint")
    vocab, d, nb, heads, dqk, dhv, up, B, T = 64, 32, 3, 2, 16, 16, 48, 2, 16
    rng = np.random.default_rng(11)
    p = layers.init_lm_params(rng, vocab, d, nb, heads, dqk, dhv, up, std=0.2, slstm_at=(1,), nh_s=nh_s)
    head = {} if tied else dict(head_w=rng.standard_normal((d, vocab)).astype(np.float32) * 0.2,
                                head_b=rng.standard_normal(vocab).astype(np.float32) * 0.2)
    lm = layers.build_lm(p, heads, dqk, dhv, nh_s=nh_s, cap=12.0, tied=tied, **head)
    ids = torch.from_numpy(rng.integers(0, vocab, B * T)).cuda()
    tg = torch.from_numpy(rng.integers(0, vocab, B * T).astype(np.int32)).cuda()
    lm.train_step(ids, tg, B, T, xl.ops.AdamCfg(1e-2, 0.1, t=1))  # the file must hold the updated weights
    want = lm.forward(ids, B, T).clone()

    path = str(tmp_path / "lm.nnm")
    ck.save_lm(path, lm, heads, dqk)
    again = ck.load_lm(path, nh_s=nh_s)
    assert again.tied == tied and again.cap == 12.0
    got = again.forward(ids, B, T)
    assert torch.equal(got, want)

    q, info = ck.lm_from_container(ck.load(path), nh_s=nh_s)
    ref = M.build_lm(q, info["heads"], info["dqk"], info["dhv"], nh_s=nh_s, cap=info["cap"], tied=info["tied"],
                     head_w=info["head_w"], head_b=info["head_b"])
    cpu = ref.forward(ids.cpu().numpy(), B, T)
    err = np.abs(got.cpu().numpy() - cpu).max() / np.abs(cpu).max()
    assert err < 1e-4, err  # fp32 parity bar
