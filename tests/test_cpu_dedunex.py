"""cpu: the plain restatement of the Dedunex design is consistent with itself (one call, token by token, portions), its
helpers do what their docstrings say, and the registry knows the family."""
import ctypes
import math
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import dedunex_oracle as O  # noqa: E402
import dedunex_util as U  # noqa: E402


def test_oracle_cut_invariance_and_layer_runs():
    layers = [U.gru(mlp=U.dense()), U.attn(mlp=U.dense(ff=5)), U.latent(), U.attn(heads=2, kv_heads=1, window=0, mlp=None)]
    cfg = U.make_config(layers, width=12, vocab=19, groups=3, loop=(1, 3, 2))
    assert O.layer_runs(cfg) == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (3, None)]
    assert O.layer_runs(U.make_config(layers, loop=(2, 2, 5))) == [(0, None), (1, None), (2, None), (3, None)]
    assert O.layer_runs(U.make_config(layers)) == [(i, None) for i in range(4)]
    w = U.values(U.random_weights(cfg, seed=1))
    toks = [int(t) for t in np.random.default_rng(0).integers(0, 19, 21)]
    whole, stream = O.forward(cfg, w, toks)
    assert stream.shape == (6, 21, 12)
    st, rows, lay = O.Stepper(cfg, w), [], []
    for c0, c1 in ((0, 5), (5, 7), (7, 8), (8, 21)):
        lg, af = st.run(toks[c0:c1])
        rows.append(lg)
        lay.append(af)
    assert np.allclose(np.concatenate(rows), whole, rtol=1e-12, atol=1e-12)
    assert np.allclose(np.concatenate(lay, axis=1), stream, rtol=1e-12, atol=1e-12)


def test_norm_helpers():
    x = np.array([3.0, 4.0, 0.0, 2.0, 1.0, 1.0])
    w = np.arange(1.0, 7.0)
    assert np.allclose(O.group_rms_norm(x, w, 1, 0.0), O.rms_norm(x, w, 0.0))
    g = O.group_rms_norm(x, np.ones(6), 3, 0.0)
    assert np.allclose(g, [3 / math.sqrt(12.5), 4 / math.sqrt(12.5), 0, math.sqrt(2.0), 1, 1])
    assert np.allclose(O.group_rms_norm(x, np.ones(6), 6, 1.0), x / np.sqrt(x * x + 1.0))  # eps sits inside the root


def test_rotation_pairs_and_scaling():
    rot = {"base": 100.0, "dims": 4}
    v = np.array([1.0, 2.0, 3.0, 4.0, 5.0])
    assert np.allclose(O.rotate_half(v, 0, rot), v)
    f, mag = O.rotary_frequencies(rot)
    assert np.allclose(f, [1.0, 0.1]) and mag == 1.0
    out = O.rotate_half(v, 3, rot)
    assert np.isclose(out[0], 1.0 * math.cos(3.0) - 3.0 * math.sin(3.0)) and np.isclose(out[2], 3.0 * math.cos(3.0) + 1.0 * math.sin(3.0))
    assert np.isclose(out[1], 2.0 * math.cos(0.3) - 4.0 * math.sin(0.3)) and out[4] == 5.0
    # a score depends on the distance of the two positions only
    q, k = np.arange(1.0, 5.0), np.array([0.5, -1.0, 2.0, 0.25])
    assert np.isclose(O.rotate_half(q, 9, rot) @ O.rotate_half(k, 4, rot), O.rotate_half(q, 25, rot) @ O.rotate_half(k, 20, rot))
    # scaling: factor 1 changes nothing; fast dimensions keep their frequency, slow ones are divided by the factor
    same = dict(rot, scaling={"factor": 1.0, "fast": 16.0, "original": 64, "slow": 2.0})
    f1, m1 = O.rotary_frequencies(same)
    assert np.allclose(f1, f) and m1 == 1.0
    big = {"base": 10000.0, "dims": 16, "scaling": {"factor": 4.0, "fast": 8.0, "original": 256, "slow": 1.0}}
    plain, _ = O.rotary_frequencies({"base": 10000.0, "dims": 16})
    f2, m2 = O.rotary_frequencies(big)
    assert np.isclose(f2[0], plain[0]) and np.isclose(f2[-1], plain[-1] / 4.0) and np.isclose(m2, 0.1 * math.log(4.0) + 1.0)
    assert all(plain[i] / 4.0 - 1e-15 <= f2[i] <= plain[i] + 1e-15 for i in range(8))


def test_window_counts_the_token_itself_and_cap_bounds_scores():
    # one head, keys equal, values one-hot: the output shows which keys took part
    cfg = U.make_config([U.attn(heads=1, kv_heads=1, dim=2, vdim=6, window=3, rot_dims=0, diff=0.0)], width=4, vocab=5)
    w = U.values(U.random_weights(cfg, seed=2))
    p, mx, cache = "l0.mix.", cfg["layers"][0]["mixer"], []
    w[p + "lq1"] = w[p + "lk1"] = w[p + "lq2"] = w[p + "lk2"] = np.zeros(2)  # lambda = diff = 0: the first map alone
    w[p + "v"] = np.zeros((6, 4))
    w[p + "o"] = np.eye(4, 6)
    seen = []
    for t in range(6):
        w[p + "v.b"] = np.eye(6)[t]
        y = O.differential_attention_step(w, p, mx, np.ones(4), t, cache, 1e-5)
        seen.append([j for j in range(4) if abs(y[j]) > 1e-9])
    assert seen[0] == [0] and seen[1] == [0, 1] and seen[3] == [1, 2, 3]
    assert len(cache) == 6
    big = O.softmax_attend(np.array([100.0]), [np.array([1.0]), np.array([-1.0])], [np.array([1.0]), np.array([0.0])], 1.0, cap=2.0)
    assert np.isclose(big[0], 1.0 / (1.0 + math.exp(-4.0)), rtol=1e-6)  # scores 100 and -100 are capped to 2 and -2


def test_mingru_candidate_and_state():
    w = {"m.z": np.zeros((2, 1)), "m.z.b": np.array([0.0, 50.0]), "m.x": np.zeros((2, 1)), "m.x.b": np.array([-1e-9, 2.0]),
         "m.g": np.zeros((2, 1)), "m.o": np.eye(2)}
    st = np.array([4.0, 4.0])
    O.mingru_step(w, "m.", np.ones(1), st)
    assert np.isclose(st[0], 0.5 * 4.0 + 0.5 * 0.5)   # below zero the candidate is sigmoid(u): it meets u + 1/2 at zero
    assert np.isclose(st[1], 2.5)                     # an open gate replaces the state by the candidate u + 1/2


def test_registry_knows_the_family():
    so = os.path.join(ROOT, "qwen_inference_engine_b200", "libqie_b200.so")
    if not os.path.exists(so):
        pytest.skip("library not built")
    lib = ctypes.CDLL(so)
    lib.qie_model_families.restype = ctypes.c_char_p
    assert "Dedunex" in lib.qie_model_families().decode().split(",")
