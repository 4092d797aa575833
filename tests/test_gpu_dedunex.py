"""gpu: the Dedunex family against the plain float64 restatement in tests/dedunex_oracle.py.

Every test builds its own small configuration and random bf16-exact weights, writes them as a model folder and loads
that through the model registry.  Most run in float32 so that a wrong key, window edge, rotation, lost state or pass of
the loop shows at 1e-4; where random weights would hide a fault the test first proves that the fault WOULD show (the
oracle with the window moved by one, another pairing of the rotated dimensions, no frequency scaling, no soft cap or a
state lost at a cut differs from the right answer by far more than the tolerance)."""
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

import dedunex_oracle as O  # noqa: E402
import dedunex_util as U  # noqa: E402

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


def _oracle_logits(cfg, weights, tokens, **kw):
    return O.forward(cfg, U.values(weights), tokens, **kw)[0]


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


def _mixed_layers():
    return [U.gru(width=14, mlp=U.dense()), U.attn(mlp=U.dense(ff=9)), U.latent(mlp=U.dense(ff=11)),
            U.attn(heads=6, kv_heads=2, dim=4, vdim=5, window=5, rot_dims=2, scaling=U.YARN, mlp=None), U.gru(width=9, mlp=None),
            U.latent(heads=2, dim=8, vdim=3, rot_dim=2, kv_rank=6, q_rank=5, mlp=U.dense(ff=6))]


# ---------------------------------------------------------------------------------------------- each mechanism alone
SINGLE = {
    "attention": ([U.attn()], None, 2),                                        # GQA, partial rotation, window, cap, lambda
    "attention_plain": ([U.attn(heads=3, kv_heads=3, dim=5, vdim=3, window=0, softcap=0.0, diff=0.0, rot_dims=0)], None, 1),
    "attention_mqa_window1": ([U.attn(heads=8, kv_heads=1, dim=4, vdim=40, window=1, rot_dims=4, scaling=U.YARN)], None, 4),
    "attention_one_head": ([U.attn(heads=1, kv_heads=1, dim=7, vdim=2, window=4, rot_dims=6, diff=0.8)], None, 5),
    "attention_wide": ([U.attn(heads=12, kv_heads=4, dim=16, vdim=24, window=9, rot_dims=8, scaling=U.YARN, mlp=U.dense())], None, 2),
    "latent": ([U.latent()], None, 2),
    "latent_one_head_no_rotation": ([U.latent(heads=1, dim=7, vdim=2, rot_dim=0, kv_rank=5, q_rank=3)], None, 10),
    "latent_20_heads": ([U.latent(heads=20, dim=4, vdim=6, rot_dim=8, kv_rank=24, q_rank=40, scaling=U.YARN, mlp=U.dense(ff=5))], None, 20),
    "mingru": ([U.gru()], None, 2),
    "mingru_70_channels": ([U.gru(width=70, mlp=U.dense(ff=3))], None, 1),
    "mingru_one_channel": ([U.gru(width=1)], None, 2),
    "loop_inner": ([U.gru(), U.attn(), U.latent(), U.gru(width=5)], (1, 3, 2), 2),      # two passes, caches and state per pass
    "loop_whole_model": ([U.attn(mlp=U.dense()), U.gru(), U.latent()], (0, 3, 3), 2),
    "loop_once": ([U.gru(), U.attn(), U.latent()], (1, 2, 1), 2),                       # one pass still adds its vector
    "loop_empty": ([U.gru(), U.attn()], (1, 1, 4), 2),                                   # nothing inside: no pass, no vector
    "loop_at_the_end": ([U.latent(), U.gru(mlp=U.dense())], (1, 2, 3), 2),
}


@pytest.mark.parametrize("name", list(SINGLE))
def test_single_mechanism_matches_oracle(tmp_path, name):
    layers, loop, groups = SINGLE[name]
    cfg = U.make_config(copy.deepcopy(layers), width=20, vocab=37, groups=groups, loop=loop)
    w = U.random_weights(cfg, seed=3)
    toks = _tokens(cfg, 23, 1)
    eng = _engine(tmp_path, cfg, w)
    assert eng.family == "dedunex"
    eng.set_int("dump_layers", 1)
    got = _whole(eng, toks)
    want, stream_want = O.forward(cfg, U.values(w), toks)
    nr = stream_want.shape[0]
    assert nr == len(O.layer_runs(cfg))
    stream = eng.read_activation("layers", nr * 256 * cfg["width"], np.float32).reshape(nr, 256, cfg["width"])[:, :len(toks)]
    eng.close()
    for i in range(nr):
        assert U.rel_err(stream[i], stream_want[i]) < TOL32, i
    assert U.rel_err(got, want) < TOL32


def test_other_sizes_and_constants(tmp_path):
    # other widths, eps, norm groups (one group; as many groups as elements), mixed order ending without a feed-forward
    # (widths 30 and 17 are no multiples of 4: the scalar paths of the norm and of the GEMV)
    for width, eps, groups, loop in ((28, 1e-3, 7, (2, 5, 2)), (36, 1e-6, 1, None), (24, 1e-2, 24, (0, 1, 2)), (30, 1e-5, 5, (3, 6, 2)), (17, 1e-5, 1, None)):
        cfg = U.make_config(_mixed_layers(), width=width, vocab=41, eps=eps, groups=groups, loop=loop)
        w = U.random_weights(cfg, seed=11 + width)
        toks = _tokens(cfg, 30, 2)
        eng = _engine(tmp_path, cfg, w, name=f"m{width}")
        got = _whole(eng, toks)
        eng.close()
        assert U.rel_err(got, _oracle_logits(cfg, w, toks)) < TOL32


# ---------------------------------------------------------------------------------------------- cutting and batching
def test_prefill_decode_portions_and_batches_agree(tmp_path):
    cfg = U.make_config(_mixed_layers(), width=24, vocab=53, groups=3, loop=(1, 4, 2))
    w = U.random_weights(cfg, seed=5)
    reqs = [_tokens(cfg, n, 10 + i) for i, n in enumerate([41, 17, 2, 29])]
    want = [_oracle_logits(cfg, w, t) for t in reqs]
    eng = _engine(tmp_path, cfg, w, page_size=8, max_pages=24, rows=32)  # 41 tokens > 32 rows: the engine cuts, too
    for t, e in zip(reqs, want):
        assert U.rel_err(_whole(eng, t), e) < TOL32
    assert U.rel_err(_cuts(eng, reqs[0], [1] * 41), want[0]) < TOL32  # token by token
    for cuts in ([2, 2, 3, 9, 2, 16, 1, 1, 5], [7, 7, 7, 7, 7, 6], [40, 1], [1, 38, 2]):  # portions down to two tokens
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
    # a pool of 8 pages of 8 positions and 2 slots: requests come and go, pages and recurrent states get new owners
    cfg = U.make_config(_mixed_layers()[:3], width=20, vocab=31, loop=(0, 2, 2))
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
    for i in (2, 3):  # slot and pages of `a` serve two more requests while b stays: a stale state would move every token
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
def test_window_edges_in_prompts_and_decoding(tmp_path):
    # window 7 over pages of 4: the edge never coincides with a page border for long.  Queries and keys are normed, so
    # the norm weights and the scale sharpen the scores until single keys carry the softmax
    cfg = U.make_config([U.attn(heads=2, kv_heads=1, dim=8, vdim=6, window=7, scale=1.5, softcap=40.0, rot_dims=4)], width=16, vocab=29)
    w = U.random_weights(cfg, seed=9, gain=2.0)
    for nm in ("l0.mix.q.norm", "l0.mix.k.norm"):
        U.set_values(w, nm, 1.6 * w[nm][1])
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


def test_far_key_among_hundreds(tmp_path):
    # latent attention sees every earlier token, the differential attention here a window longer than the prompt: 300
    # keys are several key tiles and pages, and key splits when decoding; sharp scores make single far keys count
    layers = [U.latent(heads=2, dim=8, vdim=6, rot_dim=4, kv_rank=12, q_rank=10, scale=1.0),
              U.attn(heads=2, kv_heads=1, dim=8, vdim=6, window=1000, scale=1.5, softcap=50.0, rot_dims=8, scaling=U.YARN)]
    cfg = U.make_config(layers, width=16, vocab=23)
    w = U.random_weights(cfg, seed=13)
    for nm in ("l0.mix.uq", "l0.mix.uk"):
        U.set_values(w, nm, 2.5 * w[nm][1])
    for nm in ("l1.mix.q.norm", "l1.mix.k.norm"):
        U.set_values(w, nm, 1.8 * w[nm][1])
    toks = _tokens(cfg, 300, 6)
    right = _oracle_logits(cfg, w, toks)
    eng = _engine(tmp_path, cfg, w, page_size=16, max_pages=24, rows=512)
    assert U.rel_err(_whole(eng, toks), right) < TOL32
    assert U.rel_err(_cuts(eng, toks, [255] + [1] * 45), right) < TOL32
    assert U.rel_err(_cuts(eng, toks, [100, 2, 61, 97, 40]), right) < TOL32
    eng.close()


def test_rotation_scaling_cap_and_lambda_are_what_decides(tmp_path):
    # each of these would go unnoticed with tame weights: the pairing of the rotated dimensions, the blended frequencies
    # and their magnitude, the soft cap (scores well beyond it), the two maps' weights in lambda
    layers = [U.attn(heads=2, kv_heads=2, dim=8, vdim=6, window=0, scale=2.0, softcap=4.0, diff=0.4, rot_dims=8, base=50.0, scaling=U.YARN),
              U.latent(heads=2, dim=4, vdim=6, rot_dim=8, kv_rank=8, q_rank=8, scale=1.0, base=50.0, scaling=U.YARN)]
    cfg = U.make_config(layers, width=16, vocab=23)
    w = U.random_weights(cfg, seed=23)
    for nm in ("l0.mix.q.norm", "l0.mix.k.norm"):
        U.set_values(w, nm, 1.5 * w[nm][1])
    U.set_values(w, "l0.mix.lq1", 0.9 * np.ones(8)), U.set_values(w, "l0.mix.lk1", 0.25 * np.ones(8))  # exp(1.8) - exp(-0.6) + 0.4
    U.set_values(w, "l0.mix.lq2", -0.3 * np.ones(8)), U.set_values(w, "l0.mix.lk2", 0.25 * np.ones(8))
    toks = _tokens(cfg, 90, 3)
    right = _oracle_logits(cfg, w, toks)
    assert U.rel_err(_oracle_logits(cfg, w, toks, pairing="neighbours")[20:], right[20:]) > 50 * TOL32
    for what in ("scaling", "softcap", "lambda"):
        bad, wb = copy.deepcopy(cfg), copy.deepcopy(w)
        if what == "scaling":
            for ly in bad["layers"]:
                del ly["mixer"]["rot"]["scaling"]
        elif what == "softcap":
            del bad["layers"][0]["mixer"]["softcap"]
        else:
            U.set_values(wb, "l0.mix.lq1", np.zeros(8))
        assert U.rel_err(_oracle_logits(bad, wb, toks)[20:], right[20:]) > 50 * TOL32, what
    eng = _engine(tmp_path, cfg, w, page_size=16, max_pages=8, rows=128)
    assert U.rel_err(_whole(eng, toks), right) < TOL32
    assert U.rel_err(_cuts(eng, toks, [70] + [1] * 20), right) < TOL32
    eng.close()


def test_mingru_state_survives_cuts_batches_and_long_portions(tmp_path):
    # half of the channels forget slowly (gate bias -6: a token keeps 99.75% of the state), so a state lost or mixed up at
    # a cut moves everything after it; 300 + 130 rows of two sequences in one batch take the chunk-parallel scan
    cfg = U.make_config([U.gru(width=70, mlp=U.dense(ff=8)), U.gru(width=12)], width=16, vocab=29)
    w = U.random_weights(cfg, seed=29)
    for i, c in ((0, 70), (1, 12)):
        U.set_values(w, f"l{i}.mix.z.b", np.where(np.arange(c) % 2 == 0, -6.0, 0.5))
    a, b = _tokens(cfg, 340, 7), _tokens(cfg, 150, 8)
    ra, rb = _oracle_logits(cfg, w, a), _oracle_logits(cfg, w, b)
    st = O.Stepper(cfg, U.values(w))  # the fault WOULD show: the second portion from a zero state
    assert U.rel_err(st.run(a[300:])[0], ra[300:]) > 50 * TOL32
    eng = _engine(tmp_path, cfg, w, page_size=16, max_pages=40, rows=512)
    sa, sb = eng.new_sequence(), eng.new_sequence()
    lg = eng.forward_batch([(sa, a[:300]), (sb, b[:130])], range(430))
    assert U.rel_err(lg[:300], ra[:300]) < TOL32 and U.rel_err(lg[300:], rb[:130]) < TOL32
    lg = eng.forward_batch([(sb, b[130:]), (sa, a[300:302])], range(22))  # the carried states go on, in another order
    assert U.rel_err(lg[:20], rb[130:]) < TOL32 and U.rel_err(lg[20:], ra[300:302]) < TOL32
    tail = np.concatenate([eng.forward_batch([(sa, [t])], [0]) for t in a[302:]])
    assert U.rel_err(tail, ra[302:]) < TOL32
    eng.close()


def test_first_tokens_and_long_decoding(tmp_path):
    # the first tokens (a single key, a zero state) and 200 decoded tokens with windows passing over them
    cfg = U.make_config(_mixed_layers()[:4], width=20, vocab=31, loop=(1, 4, 2))
    w = U.random_weights(cfg, seed=17)
    toks = _tokens(cfg, 203, 8)
    right = _oracle_logits(cfg, w, toks)
    eng = _engine(tmp_path, cfg, w, page_size=16, max_pages=16, rows=64)
    got = _cuts(eng, toks, [1] * 203)
    eng.close()
    assert U.rel_err(got[:4], right[:4]) < TOL32
    assert U.rel_err(got, right) < TOL32


# ---------------------------------------------------------------------------------------------- generation and serving precision
def test_greedy_generation_through_engine_and_scheduler(tmp_path):
    import qwen_inference_engine_b200 as q
    cfg = U.make_config(_mixed_layers()[:4], width=24, vocab=61, groups=4, loop=(0, 3, 2))
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


def test_top_k_sampling_draws_from_the_best_tokens(tmp_path):
    # the engine's sampler on this family's logits: with top-k 3 every drawn token is among the three largest logits of
    # its position (the oracle's, where the third and fourth are clearly apart), and top-k 1 is the greedy choice
    cfg = U.make_config(_mixed_layers()[:3], width=24, vocab=61, groups=4, loop=(1, 3, 2))
    w = U.random_weights(cfg, seed=41, gain=1.5)
    prompt = _tokens(cfg, 11, 3)
    eng = _engine(tmp_path, cfg, w, page_size=8, max_pages=12, max_seqs=2, rows=64)
    greedy = eng.generate(prompt, 6)
    eng.set_sampling(topk=1)
    assert eng.generate(prompt, 6) == greedy
    eng.set_sampling(topk=3, temperature_prefill=1.0, temperature_decode=1.0, seed=7)
    drawn = eng.generate(prompt, 8)
    eng.close()
    st = O.Stepper(cfg, U.values(w))
    z = st.run(prompt)[0][-1]
    for t in drawn:
        order = np.argsort(z)[::-1]
        if z[order[2]] - z[order[3]] > 1e-3:
            assert t in order[:3]
        z = st.run([t])[0][-1]


def _row_err(got, want):
    return np.sqrt(((got - want) ** 2).mean(-1)) / np.sqrt((want ** 2).mean(-1))


def test_bf16_tensor_core_paths_keep_the_edges(tmp_path):
    # bf16 serving precision with shapes the tensor-core kernels take: width 64 and input projections of 128 columns and
    # more (tcgen05 GEMMs between bf16 rows), portions of 64 rows and more over the bf16 cache (tensor-core attention of both
    # kinds: a window edge inside a 64-key block, two sequences of unequal length, padded head sizes), 300 rows through the
    # chunk-parallel scan reading bf16 rows.  The tolerance is bf16's; the faults it guards against are far larger.
    layers = [U.gru(width=64, mlp=U.dense(ff=64)),
              U.attn(heads=4, kv_heads=2, dim=24, vdim=20, window=37, scale=1.0, softcap=20.0, rot_dims=8, mlp=U.dense(ff=128)),
              U.latent(heads=4, dim=16, vdim=16, rot_dim=8, kv_rank=32, q_rank=64, scale=0.3, mlp=U.dense(ff=64)),
              U.attn(heads=2, kv_heads=1, dim=32, vdim=16, window=0, scale=0.4, rot_dims=16, scaling=U.YARN, mlp=None)]
    cfg = U.make_config(layers, width=64, vocab=29, groups=4, loop=(1, 3, 2))
    w = U.random_weights(cfg, seed=31, gain=1.5)
    for nm in ("l1.mix.q.norm", "l1.mix.k.norm"):  # sharper scores and a louder mixer: the window's edge carries weight
        U.set_values(w, nm, 2.5 * w[nm][1])
    U.set_values(w, "l1.mix.o", 3.0 * w["l1.mix.o"][1])
    reqs = [_tokens(cfg, 300, 4), _tokens(cfg, 81, 5)]
    right = [_oracle_logits(cfg, w, t) for t in reqs]
    tol = 4e-2
    for size in (38, 36):  # a window one key off moves the MEDIAN row further than the median may go
        bad = copy.deepcopy(cfg)
        bad["layers"][1]["mixer"]["mask"]["size"] = size
        assert np.median(_row_err(_oracle_logits(bad, w, reqs[0][:120]), right[0][:120])[40:]) > tol, size
    eng = _engine(tmp_path, cfg, w, dtype="bfloat16", page_size=16, max_pages=40, rows=512)
    a, b = eng.new_sequence(), eng.new_sequence()
    lg = eng.forward_batch([(a, reqs[0]), (b, reqs[1][:70])], range(370))
    lg2 = eng.forward_batch([(b, reqs[1][70:])], range(11))  # the per-row kernels over the same bf16 rows
    eng.close()
    ea = _row_err(lg[:300], right[0])
    eb = _row_err(np.concatenate([lg[300:], lg2]), right[1])
    assert np.median(ea) < tol / 2 and np.quantile(ea, 0.9) < tol, (np.median(ea), ea.max())
    assert np.median(eb) < tol / 2 and np.quantile(eb, 0.9) < tol, (np.median(eb), eb.max())


def test_bf16_other_sizes(tmp_path):
    # bf16 serving precision away from the tensor-core shapes: a width that is no multiple of 64, head sizes beyond the
    # tensor-core attention's tiles (the per-row kernel serves portions of 64 rows and more, too), portions against the whole
    layers = [U.attn(heads=4, kv_heads=4, dim=40, vdim=136, window=50, scale=0.3, rot_dims=10, mlp=U.dense(ff=30)),
              U.gru(width=33, mlp=None),
              U.latent(heads=3, dim=12, vdim=10, rot_dim=6, kv_rank=20, q_rank=18, scale=0.3, mlp=U.dense(ff=10))]
    cfg = U.make_config(layers, width=36, vocab=41, groups=3, loop=(0, 2, 2))
    w = U.random_weights(cfg, seed=37)
    toks = _tokens(cfg, 120, 9)
    right = _oracle_logits(cfg, w, toks)
    eng = _engine(tmp_path, cfg, w, dtype="bfloat16", page_size=16, max_pages=24, rows=256)
    whole = _whole(eng, toks)
    cut = _cuts(eng, toks, [70, 3, 1, 46])
    eng.close()
    for got in (whole, cut):
        err = _row_err(got, right)
        assert np.median(err) < 1e-2 and np.quantile(err, 0.95) < 3e-2, (np.median(err), err.max())


@pytest.mark.parametrize("heads,kv_rank,rot_dim", [(20, 40, 8), (3, 264, 16), (2, 8, 0)], ids=["two_head_groups", "latent_over_two_warps", "tiny_no_rotation"])
def test_bf16_latent_prompt_kernel_shapes(tmp_path, heads, kv_rank, rot_dim):
    # the tensor-core latent attention of prompt portions takes eight rows per CTA: more than 16 heads (two head groups), a latent
    # too wide for one warp's accumulators, rows of three sequences in one batch (a CTA then holds rows of two sequences and
    # serves them in passes), a portion that continues a cached prefix
    cfg = U.make_config([U.latent(heads=heads, dim=8, vdim=8, rot_dim=rot_dim, kv_rank=kv_rank, q_rank=24, scale=0.4)], width=32, vocab=29, groups=2)
    w = U.random_weights(cfg, seed=43, gain=1.5)
    reqs = [_tokens(cfg, n, 50 + i) for i, n in enumerate([83, 5, 97])]
    right = [_oracle_logits(cfg, w, t) for t in reqs]
    eng = _engine(tmp_path, cfg, w, dtype="bfloat16", page_size=16, max_pages=24, rows=256)
    seqs = [eng.new_sequence() for _ in reqs]
    lg = eng.forward_batch([(seqs[0], reqs[0][:70]), (seqs[1], reqs[1]), (seqs[2], reqs[2][:20])], range(95))
    lg2 = eng.forward_batch([(seqs[2], reqs[2][20:]), (seqs[0], reqs[0][70:])], range(90))
    eng.close()
    got = [np.concatenate([lg[:70], lg2[77:]]), lg[70:75], np.concatenate([lg[75:], lg2[:77]])]
    for g, r in zip(got, right):
        err = _row_err(g, r)
        assert np.median(err) < 1e-2 and err.max() < 4e-2, (np.median(err), err.max())
