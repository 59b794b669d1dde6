"""Host-side logic of head-sharded inference (no GPU): the per-rank parameter slices tile the full cell, and
the sum over ranks of (local heads' output) x (local rows of W_out) is the full output projection."""
import importlib.util
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load_shard_fn():
    # infer.py imports the CUDA-backed package; the slicing helper itself is pure numpy indexing, so it is
    # taken from the source file without importing the package (which needs the built library to load).
    src = open(os.path.join(ROOT, "neural-networks_b200", "infer.py")).read()
    start = src.index("def shard_mlstm_params")
    end = src.index("def build_lm_head_sharded")
    ns = {}
    exec(src[start:end], ns)
    return ns["shard_mlstm_params"]


def test_head_shards_tile_the_cell_and_sum_to_the_full_projection():
    shard = _load_shard_fn()
    r = np.random.default_rng(0)
    d, heads, dqk, dhv, world, rows = 24, 4, 3, 5, 2, 7
    cell = dict(kind="mlstm")
    for n, w in (("q", dqk), ("k", dqk), ("v", dhv), ("o", dhv), ("i", 1), ("f", 1)):
        cell["w" + n] = r.standard_normal((d, heads * w))
        cell["b" + n] = r.standard_normal(heads * w)
    cell["gamma"] = r.standard_normal(heads * dhv)
    cell["w_out"] = r.standard_normal((heads * dhv, d))
    cell["b_out"] = r.standard_normal(d)
    parts = [shard(cell, heads, dqk, dhv, k, world) for k in range(world)]
    for n in ("wq", "wk", "wv", "wo", "wi", "wf"):
        assert np.array_equal(np.concatenate([p[n] for p in parts], axis=1), cell[n])
    for n in ("bq", "bk", "bv", "bo", "bi", "bf", "gamma"):
        assert np.array_equal(np.concatenate([p[n] for p in parts]), cell[n])
    assert np.array_equal(np.concatenate([p["w_out"] for p in parts], axis=0), cell["w_out"])
    hc = r.standard_normal((rows, heads * dhv))  # gated head outputs, heads side by side
    hl = heads // world
    partial = sum(hc[:, k * hl * dhv:(k + 1) * hl * dhv] @ parts[k]["w_out"] for k in range(world))
    assert np.allclose(partial + cell["b_out"], hc @ cell["w_out"] + cell["b_out"], rtol=1e-12, atol=1e-12)


def test_package_weight_generator_matches_the_oracles_layout():
    """bench.py draws its LM weights with the package's own generator (the product path may not import the
    oracle); the dictionary it returns must have the oracle generator's keys and shapes, block by block."""
    import importlib
    from oracle import model as M
    layers = importlib.import_module("neural-networks_b200.layers")
    args = (50, 32, 3, 2, 16, 16, 88)
    a = layers.init_lm_params(np.random.default_rng(0), *args, slstm_at=(1,), nh_s=2)
    b = M.init_lm_params(np.random.default_rng(0), *args, slstm_at=(1,), nh_s=2)
    assert a["table"].shape == b["table"].shape and a["gamma"].shape == b["gamma"].shape
    assert len(a["blocks"]) == len(b["blocks"])
    for x, y in zip(a["blocks"], b["blocks"]):
        assert set(x) == set(y)
        assert x["cell"]["kind"] == y["cell"]["kind"] and set(x["cell"]) == set(y["cell"])
        for k in x:
            if k != "cell":
                assert np.shape(x[k]) == np.shape(y[k]), k
        for k in x["cell"]:
            if k != "kind":
                assert np.shape(x["cell"][k]) == np.shape(y["cell"][k]), k
