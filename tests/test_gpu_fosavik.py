"""gpu: the Fosavik family against the plain float64 restatement in tests/fosavik_oracle.py.

Every test builds its own small configuration and random bf16-exact weights, writes them as a model folder and loads
that through the model registry.  Most run in float32 so that a wrong key, window edge, state or sink shows at 1e-4;
where random weights would hide a fault the test first proves that the fault WOULD show (the oracle with the window
moved by one, or without the sink, differs from the right answer by far more than the tolerance)."""
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

import fosavik_oracle as O  # noqa: E402
import fosavik_util as U  # noqa: E402

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
    m = O.Model(cfg, U.values(weights))
    return m.forward(tokens, m.new_state())


def _row_errors(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    return np.sqrt(((got - want) ** 2).mean(-1)) / (np.sqrt((want ** 2).mean(-1)) + 1e-30)


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


MIXED = [U.diff_layer(mlp=U.dense()), U.parallel_layer(mlp=U.dense(ff=9, limit=0.5)), U.mamba_layer(mlp=None),
         U.diff_layer(kv_from=0, mlp=U.dense(ff=11, limit=2.0)), U.parallel_layer(heads=2, kv_heads=2, dim=5, window=4, keep_first=0, width=10,
                                                                                    blocks=1, conv=2, mlp=None),
         U.mamba_layer(heads=3, vdim=4, state=7, groups=1, norm_groups=1, conv=2, mlp=U.dense())]


# ---------------------------------------------------------------------------------------------- each mechanism alone
@pytest.mark.parametrize("layers,streams", [
    ([U.diff_layer()], 1),                                                        # differential attention alone, one stream
    ([U.diff_layer(heads=3, kv_heads=3, dim=5, vdim=3, diff=0.0)], 2),            # no head sharing, diff 0
    ([U.diff_layer(heads=8, kv_heads=1, dim=4, vdim=40, diff=0.8)], 4),           # one kv head for all
    ([U.diff_layer(), U.diff_layer(kv_from=0)], 3),                               # a layer on another layer's keys and values
    ([U.parallel_layer()], 3),                                                    # window + kept tokens + sink + gate | recurrence
    ([U.parallel_layer(heads=1, kv_heads=1, dim=3, window=1, keep_first=0, width=4, blocks=4, conv=1)], 2),  # a window of the token itself, one tap
    ([U.parallel_layer(window=5, keep_first=9, width=130, blocks=2, conv=8)], 4),  # more kept tokens than the window, 8 taps, > 128 channels
    ([U.mamba_layer()], 3),
    ([U.mamba_layer(heads=1, vdim=70, state=40, groups=1, norm_groups=5, conv=1)], 1),  # columns beyond one block, state rows beyond 32
    ([U.mamba_layer(heads=6, vdim=3, state=2, groups=3, norm_groups=1, conv=8)], 8),
    ([U.diff_layer(mlp=U.dense())], 4),                                           # the feed-forward and its clamps
    ([U.mamba_layer(mlp=U.dense(ff=33, limit=0.05))], 2),
], ids=["diff", "diff_nogroup", "diff_mqa", "diff_kv_from", "parallel", "parallel_min", "parallel_keep_gt_window", "mamba", "mamba_wide",
        "mamba_groups", "diff_ff", "mamba_ff_tight"])
def test_single_mechanism_matches_oracle(tmp_path, layers, streams):
    cfg = U.make_config(copy.deepcopy(layers), width=20, vocab=37, streams=streams)
    w = U.random_weights(cfg, seed=3)
    toks = _tokens(cfg, 23, 1)
    eng = _engine(tmp_path, cfg, w)
    eng.set_int("dump_layers", 1)
    got = _whole(eng, toks)
    nl = len(layers)
    stream = eng.read_activation("layers", nl * 256 * cfg["width"], np.float32).reshape(nl, 256, cfg["width"])[:, :len(toks)]
    m = O.Model(cfg, U.values(w))
    want, streams_want = m.forward(toks, m.new_state(), want_layers=True)
    eng.close()
    for i in range(nl):
        assert U.rel_err(stream[i], streams_want[i]) < TOL32, i
    assert U.rel_err(got, want) < TOL32


def test_other_sizes_and_constants(tmp_path):
    # odd width, another eps, one stream vs many, mixed order ending in a feed-forward
    for streams, width in ((1, 28), (5, 36)):
        cfg = U.make_config(copy.deepcopy(MIXED), width=width, vocab=41, streams=streams, eps=1e-3)
        w = U.random_weights(cfg, seed=11 + streams)
        toks = _tokens(cfg, 30, 2)
        eng = _engine(tmp_path, cfg, w, name=f"m{streams}")
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
    # a pool of 8 pages of 8 positions and 2 slots: requests come and go, pages and state slots get new owners
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
    for i in (2, 3):  # slot and pages of `a` serve two more requests while b stays
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
def _spiky(cfg, w, layer, q_name, k_name, rows_q, rows_k, factor=12.0):
    """scales the query and key projections of one head so that its scores stand out"""
    for name, rows in ((q_name, rows_q), (k_name, rows_k)):
        bits, vals = w[f"l{layer}.{name}"]
        v = vals.copy()
        v[rows] *= factor
        w[f"l{layer}.{name}"] = U.bf16_round(v.astype(np.float32))


def test_window_edges_kept_tokens_and_sink(tmp_path):
    # window 7 and 3 kept tokens over pages of 4: the edges never coincide with a page border for long
    layer = U.parallel_layer(heads=2, kv_heads=1, dim=8, window=7, keep_first=3, scale=1.0, width=8, blocks=2, conv=2, left_scale=1.0, right_scale=0.1)
    cfg = U.make_config([layer], width=16, vocab=29, streams=2)
    w = U.random_weights(cfg, seed=9, gain=2.0)
    toks = _tokens(cfg, 40, 4)
    right = _oracle_logits(cfg, w, toks)
    # the faults this test is about WOULD show: a window one key longer or shorter, one kept token more or less, no sink
    for key, val in (("size", 8), ("size", 6), ("keep_first", 4), ("keep_first", 2)):
        bad = copy.deepcopy(cfg)
        bad["layers"][0]["mixer"]["left"]["mask"][key] = val
        assert U.rel_err(_oracle_logits(bad, w, toks)[12:], right[12:]) > 50 * TOL32, (key, val)
    saved = O.attend

    def no_sink(q, K, V, pos, scale, window=0, keep_first=0, unit_sink=False):
        return saved(q, K, V, pos, scale, window, keep_first, False)
    O.attend = no_sink
    try:
        assert U.rel_err(_oracle_logits(cfg, w, toks), right) > 50 * TOL32
    finally:
        O.attend = saved
    eng = _engine(tmp_path, cfg, w, page_size=4, max_pages=16, rows=64)
    assert U.rel_err(_whole(eng, toks), right) < TOL32                 # edges inside a prompt
    assert U.rel_err(_cuts(eng, toks, [5] + [1] * 35), right) < TOL32   # the window passes over decoded tokens
    assert U.rel_err(_cuts(eng, toks, [2, 9, 3, 11, 2, 13]), right) < TOL32
    eng.close()


def test_far_key_among_hundreds(tmp_path):
    # full causal attention over 300 keys (several key tiles and pages, key splits when decoding): head 0's first map
    # is made sharp, so single far keys carry the output
    cfg = U.make_config([U.diff_layer(heads=2, kv_heads=1, dim=8, vdim=6, scale=1.0, diff=0.2)], width=16, vocab=23, streams=2)
    w = U.random_weights(cfg, seed=13)
    _spiky(cfg, w, 0, "mix.q", "mix.k", slice(0, 8), slice(0, 8), 6.0)
    toks = _tokens(cfg, 300, 6)
    right = _oracle_logits(cfg, w, toks)
    eng = _engine(tmp_path, cfg, w, page_size=16, max_pages=24, rows=512)
    assert U.rel_err(_whole(eng, toks), right) < TOL32
    assert U.rel_err(_cuts(eng, toks, [255] + [1] * 45), right) < TOL32
    assert U.rel_err(_cuts(eng, toks, [100, 2, 61, 97, 40]), right) < TOL32
    eng.close()


def test_long_portions_run_the_chunked_recurrence(tmp_path):
    # portions of 256 rows and more take the chunk-parallel form of both recurrences (chunks of 64 rows from the
    # segment's start, a carry pass); two sequences in one batch, a state carried in from an earlier portion and out to
    # decoded tokens, a decay near one (slow channels) beside fast ones
    cfg = U.make_config([U.parallel_layer(heads=2, kv_heads=1, dim=8, window=9, keep_first=0, width=70, blocks=2, conv=3, left_scale=0.2,
                                          right_scale=1.5, mlp=U.dense()),
                         U.mamba_layer(heads=4, vdim=10, state=12, groups=2, norm_groups=1, conv=3),   # state rows divide evenly
                         U.mamba_layer(heads=2, vdim=70, state=7, groups=1, norm_groups=2, conv=2)],   # bound-checked rows, two column blocks
                        width=20, vocab=31, streams=2)
    w = U.random_weights(cfg, seed=41)
    for i in (1, 2):  # slow heads: exp(A) dt small, the state remembers hundreds of tokens
        bits, al = w[f"l{i}.mix.A_log"]
        al = al.copy()
        al[0] = -6.0
        w[f"l{i}.mix.A_log"] = U.bf16_round(al.astype(np.float32))
    bits, lam = w["l0.mix.right.lam"]
    lam = lam.copy()
    lam[:10] = -9.0  # softplus ~ 1e-4: a stays within 1e-3 of one, the state remembers hundreds of tokens
    w["l0.mix.right.lam"] = U.bf16_round(lam.astype(np.float32))
    reqs = [_tokens(cfg, 430, 3), _tokens(cfg, 141, 4)]
    right = [_oracle_logits(cfg, w, t) for t in reqs]
    eng = _engine(tmp_path, cfg, w, page_size=16, max_pages=40, rows=512)
    a, b = eng.new_sequence(), eng.new_sequence()
    g0 = eng.forward_batch([(a, reqs[0][:37])], range(37))                            # row by row kernel
    g1 = eng.forward_batch([(a, reqs[0][37:337]), (b, reqs[1][:130])], range(430))    # 300 + 130 rows: chunked, ragged last chunks
    g2 = eng.forward_batch([(a, reqs[0][337:]), (b, reqs[1][130:])], range(93 + 11))  # below 256 rows again
    eng.close()
    assert U.rel_err(np.concatenate([g0, g1[:300], g2[:93]]), right[0]) < TOL32
    assert U.rel_err(np.concatenate([g1[300:], g2[93:]]), right[1]) < TOL32


def test_first_tokens_and_long_decoding(tmp_path):
    # the first tokens (empty history: zero state, zero convolution tail, a single key) and 200 decoded tokens
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
    m = O.Model(cfg, U.values(w))
    prompts = [_tokens(cfg, n, 40 + i) for i, n in enumerate([9, 14, 5])]

    def greedy(prompt, n_new):
        st, out = m.new_state(), []
        z = m.forward(prompt, st)[-1]
        for _ in range(n_new):
            srt = np.sort(z)
            if srt[-1] - srt[-2] < 1e-3:  # a close call is not a fault of either side
                break
            out.append(int(np.argmax(z)))
            z = m.forward([out[-1]], st)[-1]
        return out

    want = [greedy(p, 12) for p in prompts]
    for use_graph in (False, True):  # eager launches, then decode steps replayed from CUDA graphs
        eng = _engine(tmp_path, cfg, w, page_size=8, max_pages=12, max_seqs=2, rows=64, name=f"g{int(use_graph)}", use_graph=use_graph)
        assert eng.family == "fosavik"
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
    # portions of 64 rows and more over the bf16 cache run 64 rows at a time on tensor cores: window and kept-token
    # edges that fall inside a 64-key block, a sink, two sequences of unequal length in one batch, head sizes that are
    # padded (24 -> 32).  The tolerance is bf16's; the faults it guards against are shown to be far larger.
    layer = U.parallel_layer(heads=4, kv_heads=2, dim=24, window=37, keep_first=5, scale=0.6, width=16, blocks=2, conv=2, left_scale=1.0,
                             right_scale=0.05)
    cfg = U.make_config([layer, U.diff_layer(heads=2, kv_heads=1, dim=24, vdim=40, scale=0.5, diff=0.3)], width=32, vocab=29, streams=2)
    w = U.random_weights(cfg, seed=31, gain=2.0)
    reqs = [_tokens(cfg, 150, 4), _tokens(cfg, 81, 5)]
    right = [_oracle_logits(cfg, w, t) for t in reqs]
    tol = 3e-2
    for key, val in (("size", 38), ("size", 36), ("keep_first", 6), ("keep_first", 4)):
        bad = copy.deepcopy(cfg)
        bad["layers"][0]["mixer"]["left"]["mask"][key] = val
        assert np.quantile(_row_errors(_oracle_logits(bad, w, reqs[0])[60:], right[0][60:]), 0.9) > 8 * tol, (key, val)
    eng = _engine(tmp_path, cfg, w, dtype="bfloat16", page_size=16, max_pages=32, rows=256)
    a, b = eng.new_sequence(), eng.new_sequence()
    lg = eng.forward_batch([(a, reqs[0][:100]), (b, reqs[1])], range(181))  # 100 + 81 rows: four tiles, two of them ragged
    lg2 = eng.forward_batch([(a, reqs[0][100:])], range(50))                 # below 64 rows: the per-row kernel over the same cache
    eng.close()
    got = [np.concatenate([lg[:100], lg2]), lg[100:]]
    for g, r in zip(got, right):
        err = _row_errors(g, r)
        assert np.median(err) < tol and np.quantile(err, 0.9) < 2.5 * tol, (np.median(err), np.quantile(err, 0.9))


@pytest.mark.parametrize("dim,vdim", [(12, 20), (36, 44), (136, 132)], ids=["unaligned_small", "unaligned_padded", "beyond_tensor_core_tiles"])
def test_bf16_prompt_attention_odd_head_sizes(tmp_path, dim, vdim):
    # head sizes that are no multiple of 8 (cache rows without 16-byte pieces: element-wise staging) and head sizes beyond the
    # tensor-core kernel's tiles (the per-row kernel takes the prompt); 70 rows in one portion, then single tokens
    cfg = U.make_config([U.diff_layer(heads=2, kv_heads=1, dim=dim, vdim=vdim, scale=dim ** -0.5, diff=0.4),
                         U.parallel_layer(heads=2, kv_heads=2, dim=dim, window=19, keep_first=2, scale=dim ** -0.5, width=12, blocks=1, conv=2)],
                        width=40, vocab=31, streams=2)
    w = U.random_weights(cfg, seed=37)
    toks = _tokens(cfg, 80, 12)
    right = _oracle_logits(cfg, w, toks)
    eng = _engine(tmp_path, cfg, w, dtype="bfloat16", page_size=16, max_pages=16, rows=128)
    got = _cuts(eng, toks, [70] + [1] * 10)
    eng.close()
    err = _row_errors(got, right)
    assert np.median(err) < 2e-2 and np.quantile(err, 0.9) < 6e-2, (np.median(err), np.quantile(err, 0.9))


def test_bf16_serving_precision(tmp_path):
    # bf16 products (tensor-core projections for portions above 16 rows), bf16 cache rows; the stream, softmax, norms and
    # recurrences stay fp32, so logits stay close to the float64 restatement and cutting changes them by rounding only
    cfg = U.make_config([U.diff_layer(heads=4, kv_heads=2, dim=16, vdim=32, mlp=U.dense(ff=128, limit=1.0)),
                         U.parallel_layer(heads=4, kv_heads=2, dim=16, window=24, keep_first=4, width=64, blocks=2, mlp=U.dense(ff=128, limit=1.0)),
                         U.mamba_layer(heads=4, vdim=16, state=16, groups=1, norm_groups=1, mlp=None)], width=64, vocab=200, streams=2)
    w = U.random_weights(cfg, seed=23)
    toks = _tokens(cfg, 90, 9)
    right = _oracle_logits(cfg, w, toks)
    eng = _engine(tmp_path, cfg, w, dtype="bfloat16", page_size=16, max_pages=16, rows=128)
    a = _whole(eng, toks)
    b = _cuts(eng, toks, [40, 2, 30] + [1] * 18)
    eng.close()
    for got in (a, b):  # judged by the bulk of the rows: random weights amplify single bf16 flips
        err = _row_errors(got, right)
        assert np.median(err) < 2e-2 and np.quantile(err, 0.8) < 6e-2 and err.max() < 0.5
    err = _row_errors(b, a)
    assert np.median(err) < 2e-2 and err.max() < 0.5
