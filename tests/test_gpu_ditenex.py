"""gpu: the Ditenex family against the plain float64 restatement in tests/ditenex_oracle.py.

Every test builds its own small configuration and random bf16-exact weights, writes them as a model folder and loads
that through the model registry.  Most run in float32 so that a wrong key, window edge, carried row or router choice
shows at 1e-4; where random weights would hide a fault the test first proves that the fault WOULD show (the oracle with
the window moved by one differs from the right answer by far more than the tolerance)."""
import copy
import os
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
pytestmark = pytest.mark.gpu

import ditenex_oracle as O  # noqa: E402
import ditenex_util as U  # noqa: E402

TOL32 = 2e-4


def _engine(tmp_path, cfg, weights, dtype="float32", page_size=16, max_pages=32, max_seqs=4, rows=256, name="m", use_graph=False):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import qwen_inference_engine_b200 as q
    folder = U.write_model(str(tmp_path / name), cfg, weights)
    return q.Engine(model_dir=folder, dtype=dtype, page_size=page_size, max_pages=max_pages, max_seqs=max_seqs,
                    max_batch_tokens=rows, context=page_size * max_pages, use_graph=use_graph)


def _tokens(cfg, n, seed):
    return [int(t) for t in np.random.default_rng(seed).integers(0, cfg["vocab"], n)]


def _oracle_logits(cfg, weights, tokens):
    return O.forward(cfg, U.values(weights), tokens)[0]


def _whole(eng, tokens):
    s = eng.new_sequence()
    try:
        return eng.forward_batch([(s, tokens)], range(len(tokens)))
    finally:
        eng.free_sequence(s)


def _cuts(eng, tokens, cuts):
    assert sum(cuts) == len(tokens)
    s, at, rows = eng.new_sequence(), 0, []
    for c in cuts:
        rows.append(eng.forward_batch([(s, tokens[at:at + c])], range(c)))
        at += c
    eng.free_sequence(s)
    return np.concatenate(rows)


MIXED = [U.attn(mlp=U.dense()), U.attn(heads=6, kv_heads=2, dim=4, vdim=5, window=5, mlp=U.moe()), U.attn(v_mix=False, window=0, mlp=None),
         U.attn(heads=2, kv_heads=2, dim=8, vdim=5, window=11, mlp=U.moe(experts=4, top=1, ff=7, groups=0, shared_ff=0)),
         U.attn(heads=4, kv_heads=1, dim=3, vdim=10, window=3, mlp=U.dense(ff=9))]


# ---------------------------------------------------------------------------------------------- each mechanism alone
@pytest.mark.parametrize("layers", [
    [U.attn(v_mix=False)],                                                      # the mixer alone: shift, biases, slopes, head mixing, window, gate
    [U.attn(heads=3, kv_heads=3, dim=5, vdim=3, window=0, v_mix=False)],        # no head sharing, no window
    [U.attn(heads=8, kv_heads=1, dim=4, vdim=40, window=1, v_mix=False)],       # one kv head for all, a window of the token itself
    [U.attn(heads=1, kv_heads=1, dim=7, vdim=2, window=4, v_mix=False)],        # a single head: nothing to mix
    [U.attn(heads=12, kv_heads=4, dim=16, vdim=24, window=9, v_mix=False)],     # larger heads, four kv heads side by side in the key row
    [U.attn(v_mix=False), U.attn(), U.attn(v_mix=False), U.attn()],             # values blended with those of layer 1, not of layer 0
    [U.attn(v_mix=False, mlp=U.dense())],                                       # both branches of the activation
    [U.attn(v_mix=False, mlp=U.moe())],                                         # groups, correction, shared expert
    [U.attn(v_mix=False, mlp=U.moe(experts=8, top=3, ff=5, groups=4, keep=3, scale=0.7, shared_ff=0))],
    [U.attn(v_mix=False, mlp=U.moe(experts=5, top=5, ff=6, groups=1, keep=1, shared_ff=33))],   # every expert chosen, one group
    [U.attn(v_mix=False, mlp=U.moe(experts=40, top=2, ff=3, groups=0, shared_ff=4))],           # more experts than a warp has lanes
], ids=["mixer", "no_groups_no_window", "mqa_window1", "one_head", "wide_heads", "value_blend", "dense", "moe", "moe_keep3", "moe_all", "moe_40"])
def test_single_mechanism_matches_oracle(tmp_path, layers):
    cfg = U.make_config(copy.deepcopy(layers), width=20, vocab=37)
    w = U.random_weights(cfg, seed=3)
    toks = _tokens(cfg, 23, 1)
    eng = _engine(tmp_path, cfg, w)
    eng.set_int("dump_layers", 1)
    got = _whole(eng, toks)
    nl = len(layers)
    stream = eng.read_activation("layers", nl * 256 * cfg["width"], np.float32).reshape(nl, 256, cfg["width"])[:, :len(toks)]
    want, stream_want = O.forward(cfg, U.values(w), toks)
    eng.close()
    for i in range(nl):
        assert U.rel_err(stream[i], stream_want[i]) < TOL32, i
    assert U.rel_err(got, want) < TOL32


def test_router_choice_follows_the_correction_and_the_groups(tmp_path):
    # corrections as large as the scores, some so negative that every choice score of a group is below zero: an expert
    # weighed by its corrected score, groups ranked by one best score, or dropped groups counted as zero would all differ
    mlp = U.moe(experts=12, top=3, ff=6, groups=4, keep=2, scale=2.5, shared_ff=0)
    cfg = U.make_config([U.attn(v_mix=False, mlp=mlp)], width=16, vocab=29)
    w = U.random_weights(cfg, seed=23)
    rng = np.random.default_rng(5)
    U.set_values(w, "l0.mlp.correction", np.concatenate([rng.uniform(-0.5, 0.5, 6), rng.uniform(-3.0, -1.5, 6)]))
    toks = _tokens(cfg, 60, 2)
    right = _oracle_logits(cfg, w, toks)
    vals = U.values(w)
    saved = O.route

    def uncorrected(h, router, correction, top, n_groups, keep, scale):
        return saved(h, router, np.zeros_like(correction), top, n_groups, keep, scale)
    O.route = uncorrected
    try:
        assert U.rel_err(O.forward(cfg, vals, toks)[0], right) > 50 * TOL32
    finally:
        O.route = saved
    eng = _engine(tmp_path, cfg, w)
    got = _whole(eng, toks)
    eng.close()
    assert U.rel_err(got, right) < TOL32


def test_other_sizes_and_constants(tmp_path):
    # odd widths, another eps and residual multiplier (also 1), mixed order ending in a layer without feed-forward
    for width, eps, mult in ((28, 1e-3, 1.0), (36, 1e-6, 0.15)):
        layers = copy.deepcopy(MIXED) + [U.attn(v_mix=False, window=2, mlp=None)]
        cfg = U.make_config(layers, width=width, vocab=41, eps=eps, res_mult=mult)
        w = U.random_weights(cfg, seed=11 + width)
        toks = _tokens(cfg, 30, 2)
        eng = _engine(tmp_path, cfg, w, name=f"m{width}")
        got = _whole(eng, toks)
        eng.close()
        assert U.rel_err(got, _oracle_logits(cfg, w, toks)) < TOL32


# ---------------------------------------------------------------------------------------------- cutting and batching
def test_prefill_decode_portions_and_batches_agree(tmp_path):
    cfg = U.make_config(copy.deepcopy(MIXED), width=24, vocab=53)
    w = U.random_weights(cfg, seed=5)
    reqs = [_tokens(cfg, n, 10 + i) for i, n in enumerate([41, 17, 2, 29])]
    want = [_oracle_logits(cfg, w, t) for t in reqs]
    eng = _engine(tmp_path, cfg, w, page_size=8, max_pages=24, rows=32)  # 41 tokens > 32 rows: the engine cuts, too
    for t, e in zip(reqs, want):
        assert U.rel_err(_whole(eng, t), e) < TOL32
    # token by token
    assert U.rel_err(_cuts(eng, reqs[0], [1] * 41), want[0]) < TOL32
    # portions of several sizes, down to two tokens, then single tokens
    for cuts in ([2, 2, 3, 9, 2, 16, 1, 1, 5], [7, 7, 7, 7, 7, 6], [40, 1], [1, 38, 2]):
        assert U.rel_err(_cuts(eng, reqs[0], cuts), want[0]) < TOL32
    # unequal requests together: portions of some beside single tokens of others
    seqs = [eng.new_sequence() for _ in reqs]
    at = [0] * len(reqs)
    got = [[] for _ in reqs]
    plan = [[5, 17, 1, 3], [1, 0, 1, 9], [20, 0, 0, 1], [1, 0, 0, 16], [14, 0, 0, 0]]
    for step in plan:
        entries, owner = [], []
        for i, c in enumerate(step):
            if c:
                entries.append((seqs[i], reqs[i][at[i]:at[i] + c]))
                owner += [i] * c
                at[i] += c
        lg = eng.forward_batch(entries, range(len(owner)))
        for row, i in zip(lg, owner):
            got[i].append(row)
    assert at == [len(t) for t in reqs]
    eng.close()
    for i in range(len(reqs)):
        assert U.rel_err(np.stack(got[i]), want[i]) < TOL32


def test_pages_and_slots_are_reused(tmp_path):
    # a pool of 8 pages of 8 positions and 2 slots: requests come and go, pages and carried rows get new owners
    cfg = U.make_config(copy.deepcopy(MIXED[:3]), width=20, vocab=31)
    w = U.random_weights(cfg, seed=7)
    eng = _engine(tmp_path, cfg, w, page_size=8, max_pages=8, max_seqs=2, rows=64)
    reqs = [_tokens(cfg, n, 30 + i) for i, n in enumerate([20, 27, 9, 24, 15, 30])]
    want = [_oracle_logits(cfg, w, t) for t in reqs]
    a = eng.new_sequence()
    b = eng.new_sequence()
    ga = [eng.forward_batch([(a, reqs[0][:11])], range(11))]
    gb = [eng.forward_batch([(b, reqs[1])], range(27))]
    ga.append(eng.forward_batch([(a, reqs[0][11:])], range(9)))
    assert U.rel_err(np.concatenate(ga), want[0]) < TOL32 and U.rel_err(gb[0], want[1]) < TOL32
    assert eng.pages_free() == 8 - 3 - 4
    with pytest.raises(Exception):
        eng.new_sequence()  # both slots live
    eng.free_sequence(a)
    for i in (2, 3):  # slot and pages of `a` serve two more requests while b stays: a stale carried row would shift their first token
        s = eng.new_sequence()
        lg = np.concatenate([eng.forward_batch([(s, reqs[i][:4])], range(4)), eng.forward_batch([(s, reqs[i][4:])], range(len(reqs[i]) - 4))])
        assert U.rel_err(lg, want[i]) < TOL32, i
        eng.free_sequence(s)
    eng.free_sequence(b)
    assert eng.pages_free() == 8
    s, t = eng.new_sequence(), eng.new_sequence()
    lg = eng.forward_batch([(s, reqs[4]), (t, reqs[5][:17])], range(15 + 17))
    lg2 = eng.forward_batch([(t, reqs[5][17:])], range(13))
    eng.close()
    assert U.rel_err(lg[:15], want[4]) < TOL32
    assert U.rel_err(np.concatenate([lg[15:], lg2]), want[5]) < TOL32


# ---------------------------------------------------------------------------------------------- edges that random weights hide
def _sharpen(w, layer, factor):
    """scales the query and key projections so that single keys carry the softmax"""
    for name in ("mix.q", "mix.k"):
        U.set_values(w, f"l{layer}.{name}", w[f"l{layer}.{name}"][1] * factor)


def test_window_edges_in_prompts_and_decoding(tmp_path):
    # window 7 over pages of 4: the edge never coincides with a page border for long.  No token shift (mu = 0), so
    # that nothing but the window carries older tokens, and sharp scores
    cfg = U.make_config([U.attn(heads=2, kv_heads=1, dim=8, vdim=6, window=7, scale=1.0, v_mix=False)], width=16, vocab=29)
    w = U.random_weights(cfg, seed=9, gain=2.0)
    U.set_values(w, "l0.shift", np.zeros(16))
    _sharpen(w, 0, 3.0)
    toks = _tokens(cfg, 40, 4)
    right = _oracle_logits(cfg, w, toks)
    for size in (8, 6):  # the fault this test is about WOULD show
        bad = copy.deepcopy(cfg)
        bad["layers"][0]["mixer"]["mask"]["size"] = size
        assert U.rel_err(_oracle_logits(bad, w, toks)[12:], right[12:]) > 50 * TOL32, size
    eng = _engine(tmp_path, cfg, w, page_size=4, max_pages=16, rows=64)
    assert U.rel_err(_whole(eng, toks), right) < TOL32                 # edges inside a prompt
    assert U.rel_err(_cuts(eng, toks, [5] + [1] * 35), right) < TOL32   # the window passes over decoded tokens
    assert U.rel_err(_cuts(eng, toks, [2, 9, 3, 11, 2, 13]), right) < TOL32
    eng.close()


def test_token_shift_carries_across_cuts(tmp_path):
    # mu = 1 in half of the channels: the mixer reads the previous token there and nothing of its own; a lost or stale
    # carried row at a cut, or the shifted row carried instead of the unshifted one, changes every token after a cut
    cfg = U.make_config([U.attn(v_mix=False, mlp=U.dense()), U.attn(v_mix=False, window=0)], width=16, vocab=29)
    w = U.random_weights(cfg, seed=19)
    for i in (0, 1):
        U.set_values(w, f"l{i}.shift", np.where(np.arange(16) % 2 == 0, 1.0, 0.25))
    toks = _tokens(cfg, 33, 5)
    right = _oracle_logits(cfg, w, toks)
    eng = _engine(tmp_path, cfg, w, page_size=8, max_pages=16, rows=64)
    assert U.rel_err(_whole(eng, toks), right) < TOL32
    assert U.rel_err(_cuts(eng, toks, [1] * 33), right) < TOL32
    assert U.rel_err(_cuts(eng, toks, [2, 1, 7, 2, 1, 20]), right) < TOL32
    eng.close()


def test_far_key_among_hundreds(tmp_path):
    # full causal attention over 300 keys (several key tiles and pages, key splits when decoding); the slopes of the
    # distance penalty reach 75 at that distance for the steepest head, the flattest still sees the first key
    cfg = U.make_config([U.attn(heads=2, kv_heads=1, dim=8, vdim=6, window=0, scale=1.0, v_mix=False)], width=16, vocab=23)
    w = U.random_weights(cfg, seed=13)
    _sharpen(w, 0, 2.5)
    toks = _tokens(cfg, 300, 6)
    right = _oracle_logits(cfg, w, toks)
    eng = _engine(tmp_path, cfg, w, page_size=16, max_pages=24, rows=512)
    assert U.rel_err(_whole(eng, toks), right) < TOL32
    assert U.rel_err(_cuts(eng, toks, [255] + [1] * 45), right) < TOL32
    assert U.rel_err(_cuts(eng, toks, [100, 2, 61, 97, 40]), right) < TOL32
    eng.close()


def test_first_tokens_and_long_decoding(tmp_path):
    # the first tokens (zero carried row, a single key) and 200 decoded tokens with windows passing over them
    cfg = U.make_config(copy.deepcopy(MIXED[:4]), width=20, vocab=31)
    w = U.random_weights(cfg, seed=17)
    toks = _tokens(cfg, 203, 8)
    right = _oracle_logits(cfg, w, toks)
    eng = _engine(tmp_path, cfg, w, page_size=16, max_pages=16, rows=64)
    got = _cuts(eng, toks, [1, 1, 1] + [1] * 200)
    eng.close()
    assert U.rel_err(got[:4], right[:4]) < TOL32
    assert U.rel_err(got, right) < TOL32


# ---------------------------------------------------------------------------------------------- generation and serving precision
def test_greedy_generation_through_engine_and_scheduler(tmp_path):
    import qwen_inference_engine_b200 as q
    cfg = U.make_config(copy.deepcopy(MIXED[:4]), width=24, vocab=61)
    w = U.random_weights(cfg, seed=21, gain=1.5)
    vals = U.values(w)
    prompts = [_tokens(cfg, n, 40 + i) for i, n in enumerate([9, 14, 5])]

    def greedy(prompt, n_new):
        st, out = O.Stepper(cfg, vals), []
        z = st.run(prompt)[0][-1]
        for _ in range(n_new):
            srt = np.sort(z)
            if srt[-1] - srt[-2] < 1e-3:  # a close call is not a fault of either side
                break
            out.append(int(np.argmax(z)))
            z = st.run([out[-1]])[0][-1]
        return out

    want = [greedy(p, 12) for p in prompts]
    assert sum(len(e) for e in want) > 20
    for use_graph in (False, True):  # eager launches, then decode steps replayed from CUDA graphs
        eng = _engine(tmp_path, cfg, w, page_size=8, max_pages=12, max_seqs=2, rows=64, name=f"g{int(use_graph)}", use_graph=use_graph)
        assert eng.family == "ditenex"
        for p, e in zip(prompts, want):  # the engine's own entry point: prefill + decode steps
            assert eng.generate(p, 12)[:len(e)] == e
        free0 = eng.pages_free()
        sch = q.Scheduler(eng, max_running=2, eos_token=-1)  # three requests over two slots: the third waits for a slot
        rids = [sch.submit(p, 12) for p in prompts]
        sch.run()
        for rid, e in zip(rids, want):
            toks, fin = sch.result(rid)
            assert fin and toks[:len(e)] == e
        sch.close()
        assert eng.pages_free() == free0
        eng.close()


def test_bf16_prompt_attention_on_tensor_cores_keeps_the_edges(tmp_path):
    # portions of 64 rows and more over the bf16 cache run 64 rows at a time on tensor cores: a window edge that falls
    # inside a 64-key block, two sequences of unequal length in one batch, key rows that are padded (2 x 24 -> 64),
    # projections wide enough for the tcgen05 GEMM and experts that take the grouped tensor-core GEMM (tiles wider than
    # the 32 gated columns and the 64 output columns).  The tolerance is bf16's; the fault it guards against is far larger.
    layers = [U.attn(heads=4, kv_heads=2, dim=24, vdim=20, window=37, scale=0.6, mlp=U.dense(ff=128)),
              U.attn(heads=2, kv_heads=1, dim=32, vdim=16, window=0, scale=0.4, v_mix=False, mlp=None),  # no mask: tiles in pairs
              # last, so that an expert chosen otherwise at bf16 precision (a close call) stays in its own row
              U.attn(heads=4, kv_heads=2, dim=16, vdim=20, window=70, scale=0.5, mlp=U.moe(experts=6, top=2, ff=32, shared_ff=64))]
    cfg = U.make_config(layers, width=64, vocab=29)
    w = U.random_weights(cfg, seed=31, gain=1.5)
    for i in range(3):
        U.set_values(w, f"l{i}.shift", np.zeros(64))
    U.set_values(w, "l2.mlp.router", 4.0 * w["l2.mlp.router"][1])  # a decisive router: few close calls for bf16 to turn
    reqs = [_tokens(cfg, 150, 4), _tokens(cfg, 81, 5)]
    right = [_oracle_logits(cfg, w, t) for t in reqs]
    tol = 4e-2  # nine tenths of the rows; the median row stays under half of it through three bf16 layers

    def rows(got, want):
        return np.sqrt(((got - want) ** 2).mean(-1)) / np.sqrt((want ** 2).mean(-1))
    for size in (38, 36):  # a window one key off moves the MEDIAN row four times further than the median may go
        bad = copy.deepcopy(cfg)
        bad["layers"][0]["mixer"]["mask"]["size"] = size
        assert np.median(rows(_oracle_logits(bad, w, reqs[0]), right[0])[40:]) > 2 * tol, size
    eng = _engine(tmp_path, cfg, w, dtype="bfloat16", page_size=16, max_pages=24, rows=256)
    a, b = eng.new_sequence(), eng.new_sequence()
    lg = eng.forward_batch([(a, reqs[0]), (b, reqs[1][:70])], range(220))
    lg2 = eng.forward_batch([(b, reqs[1][70:])], range(11))  # the per-row kernel over the same bf16 rows
    eng.close()
    ea = rows(lg[:150], right[0])
    eb = rows(np.concatenate([lg[150:], lg2]), right[1])
    assert np.median(ea) < tol / 2 and np.quantile(ea, 0.9) < tol, (np.median(ea), ea.max())
    assert np.median(eb) < tol / 2 and np.quantile(eb, 0.9) < tol, (np.median(eb), eb.max())


def test_bf16_other_sizes_and_wide_key_rows(tmp_path):
    # bf16 serving precision away from the tensor-core shapes: a width that is no multiple of 64 (the tile GEMM instead
    # of tcgen05), key rows of 4 x 40 = 160 elements and values of 136 (beyond the tensor-core attention's tiles: the
    # per-row kernel serves portions of 64 rows and more, too), portions against the whole prompt
    layers = [U.attn(heads=4, kv_heads=4, dim=40, vdim=12, window=50, scale=0.3, mlp=U.dense(ff=30)),
              U.attn(heads=2, kv_heads=1, dim=24, vdim=136, window=0, scale=0.4, v_mix=False, mlp=U.moe(experts=6, top=2, ff=10, shared_ff=20)),
              U.attn(heads=4, kv_heads=4, dim=40, vdim=12, window=70, scale=0.3, mlp=None)]
    cfg = U.make_config(layers, width=36, vocab=41)
    w = U.random_weights(cfg, seed=37)
    toks = _tokens(cfg, 120, 9)
    right = _oracle_logits(cfg, w, toks)
    eng = _engine(tmp_path, cfg, w, dtype="bfloat16", page_size=16, max_pages=24, rows=256)
    whole = _whole(eng, toks)
    cut = _cuts(eng, toks, [70, 3, 1, 46])
    eng.close()
    for got in (whole, cut):
        err = np.sqrt(((got - right) ** 2).mean(-1)) / np.sqrt((right ** 2).mean(-1))
        assert np.median(err) < 1e-2 and np.quantile(err, 0.95) < 3e-2, (np.median(err), err.max())
