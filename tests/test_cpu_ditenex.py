"""cpu: the plain restatement of the Ditenex design is consistent with itself (one call, token by token, portions), its
helpers do what their docstrings say, the identity the engine's attention rests on holds, and the registry knows the
family."""
import ctypes
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import ditenex_oracle as O  # noqa: E402
import ditenex_util as U  # noqa: E402


def test_oracle_cut_invariance():
    layers = [U.attn(v_mix=False, mlp=U.dense()), U.attn(mlp=U.moe()), U.attn(heads=2, kv_heads=1, window=0, v_mix=False, mlp=None), U.attn(mlp=U.dense(ff=5))]
    cfg = U.make_config(layers, width=12, vocab=19)
    w = U.values(U.random_weights(cfg, seed=1))
    toks = [int(t) for t in np.random.default_rng(0).integers(0, 19, 21)]
    whole, layers_whole = O.forward(cfg, w, toks)
    st, rows, lay = O.Stepper(cfg, w), [], []
    for c0, c1 in ((0, 5), (5, 7), (7, 8), (8, 21)):
        lg, af = st.run(toks[c0:c1])
        rows.append(lg)
        lay.append(af)
    assert np.allclose(np.concatenate(rows), whole, rtol=1e-9, atol=1e-9)
    assert np.allclose(np.concatenate(lay, axis=1), layers_whole, rtol=1e-9, atol=1e-9)


def test_token_shift_and_activation_helpers():
    h = np.array([[1.0, 10.0], [2.0, 20.0], [4.0, 40.0]])
    out = O.token_shift(h, np.array([0.0, 100.0]), np.array([0.5, 1.0]))
    assert np.allclose(out, [[0.5, 100.0], [1.5, 10.0], [3.0, 20.0]])
    # both branches meet at zero with slope 1/2, the positive one is a parabola, the negative one levels off linearly
    z = np.array([-30.0, -1e-9, 0.0, 1e-9, 2.0])
    y = O.xielu(z, 0.3, -0.2)
    assert abs(y[2]) == 0.0 and np.allclose(y[[1, 3]], [-0.5e-9, 0.5e-9], atol=1e-15)
    assert np.isclose(y[4], O.softplus(0.3) * 4.0 + 1.0)
    assert np.isclose(y[0], (0.5 + O.softplus(-0.2)) * (np.expm1(-30.0) + 30.0) - 15.0)


def test_router_groups_correction_and_negative_scores():
    # 6 experts in 3 groups, 1 group kept: the correction (not the plain score) decides group and expert, the weight
    # is the plain score; with every choice score negative the dropped groups must not win by counting as zero
    h = np.eye(6)[:1]
    router = np.zeros((6, 6))
    router[:, 0] = [2.0, 1.9, 0.0, 0.1, -1.0, -1.1]
    s = O.sigmoid(router[:, 0])
    chosen, wts = O.route(h, router, np.array([0.0, 0.0, 0.1, 0.1, 0.0, 0.0]), 2, 3, 1, 2.0)
    assert chosen[0].tolist() == [0, 1]           # a small correction leaves group 0 ahead
    chosen, wts = O.route(h, router, np.array([0.0, 0.0, 0.9, 0.8, 0.0, 0.0]), 2, 3, 1, 2.0)
    assert chosen[0].tolist() == [2, 3] and np.allclose(wts[0], 2.0 * s[[2, 3]])   # chosen by correction, weighed without it
    chosen, _ = O.route(h, router, np.full(6, -5.0), 2, 3, 1, 1.0)
    assert chosen[0].tolist() == [0, 1]           # all choice scores negative: a dropped group counting as 0 would win
    chosen, _ = O.route(h, router, np.array([0.0, -3.0, 0.0, 0.0, 0.0, 0.0]), 3, 3, 2, 1.0)
    assert chosen[0].tolist() == [3, 2, 4]        # group sums -1.25, 1.02, 0.52: the best single expert (0) falls with its group


def test_mixing_scores_equals_mixing_queries():
    # score'_h = sum_g T[h, g] (q_g . k_c(g) s - m_g dist) is one dot product of a longer query with ALL kv heads' keys,
    # minus a mixed slope times the distance: what the engine's attention computes
    rng = np.random.default_rng(3)
    H, G, d, dv, T = 6, 3, 4, 5, 9
    q, k, v = rng.standard_normal((T, H, d)), rng.standard_normal((T, G, d)), rng.standard_normal((T, G, dv))
    talk = np.eye(H) + 0.5 * rng.standard_normal((H, H))
    pos = np.arange(T)
    want = O.talking_window_attention(q, k, v, pos, pos, 0.7, 4, talk)
    rep = H // G
    qt = np.zeros((T, H, G * d))
    for h in range(H):
        for g in range(H):
            qt[:, h, (g // rep) * d:(g // rep + 1) * d] += talk[h, g] * q[:, g]
    slopes = talk @ O.distance_slopes(H)
    got = np.zeros((T, H, dv))
    for i in range(T):
        for h in range(H):
            js = [j for j in range(T) if 0 <= i - j < 4]
            sc = np.array([qt[i, h] @ k[j].reshape(-1) * 0.7 - slopes[h] * (i - j) for j in js])
            p = np.exp(sc - sc.max())
            p /= p.sum()
            got[i, h] = sum(pj * v[j, h // rep] for pj, j in zip(p, js))
    assert np.allclose(got, want, rtol=1e-10, atol=1e-10)


def test_window_counts_the_token_itself():
    # a window of w keys is the token and the w - 1 before it: with distinct one-hot values the output shows which keys took part
    T, w = 6, 3
    q = np.zeros((T, 1, 2))
    k = np.zeros((T, 1, 2))
    v = np.eye(T)[:, None, :]
    out = O.talking_window_attention(q, k, v, np.arange(T), np.arange(T), 1.0, w, np.ones((1, 1)))
    assert [j for j in range(T) if out[5, 0, j] > 0] == [3, 4, 5]
    assert [j for j in range(T) if out[1, 0, j] > 0] == [0, 1]
    # nearer keys weigh more: the distance penalty of the only head is 2^-8 per position
    assert np.isclose(out[5, 0, 4] / out[5, 0, 5], np.exp(-2.0 ** -8))


def test_registry_knows_the_family():
    so = os.path.join(ROOT, "qwen_inference_engine_b200", "libqie_b200.so")
    if not os.path.exists(so):
        pytest.skip("library not built")
    lib = ctypes.CDLL(so)
    lib.qie_model_families.restype = ctypes.c_char_p
    assert "Ditenex" in lib.qie_model_families().decode().split(",")
