"""Puzonex (sublayers that read the stream itself and are normalised on their way back; capped, distance-penalised sink attention,
Mamba-1, windowed attention beside a matrix memory) against the plain oracle of oracle/puzonex.py.

Small configurations with their own random weights; the oracle runs in float64.  The engine's "f32" precision is held to a tight
bar (a window one token off, a lost sink, a state of the wrong slot, a bias on the wrong row shows), the serving precision to the
bar its operand rounding allows.
"""
import copy
import math

import numpy as np
import pytest
import torch

from oracle import puzonex as P

T64 = torch.float64


# ---------------------------------------------------------------------------------------------------- configurations
def attention(heads=6, kv_heads=2, dim=24, vdim=40, window=37, scale=0.2, softcap=20.0):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if softcap:
        m["softcap"] = softcap
    if window:
        m["mask"] = {"size": window}
    return {"type": "attention", "mixer": m}


def mamba1(inner=88, state=12, dt_rank=6, conv=4):
    return {"type": "mamba1", "mixer": {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}}


def parallel(heads=4, kv_heads=2, dim=20, window=29, scale=0.25, softcap=15.0, bias_max=50, rel_rows=10, rheads=3, rdim=12, rvdim=20, gate_cap=10.0):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale, "bias_max": bias_max, "rel_rows": rel_rows}
    if softcap:
        left["softcap"] = softcap
    if window:
        left["mask"] = {"size": window}
    return {"type": "parallel", "mixer": {"left": left, "right": {"heads": rheads, "dim": rdim, "vdim": rvdim, "gate_cap": gate_cap}}}


def layer(mx, ff=52):
    return dict(copy.deepcopy(mx), mlp={"kind": "dense", "ff": ff} if ff else None)


def config(layers, width=120, vocab=211, eps=1e-5):
    return {"architecture": "Puzonex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": copy.deepcopy(layers)}


# five layers of unequal geometry, every mixer at least once, one layer without a feed-forward
FULL = config([layer(mamba1()),
               layer(parallel()),
               layer(attention()),
               layer(mamba1(inner=60, state=7, dt_rank=3, conv=3), None),
               layer(attention(heads=2, kv_heads=2, dim=16, vdim=8, window=70, scale=0.3, softcap=40.0), 30)])
SINGLE = {
    "attention_only": config([layer(attention(), None)]),
    "attention_every_head_its_own_keys": config([layer(attention(heads=3, kv_heads=3, dim=18, vdim=9, window=5), None)], width=72, vocab=90),
    "attention_one_head_window_one": config([layer(attention(heads=1, kv_heads=1, dim=16, vdim=16, window=1), 24)], width=64, vocab=70),
    "attention_no_window_no_cap": config([layer(attention(heads=4, kv_heads=1, dim=13, vdim=21, window=0, softcap=0.0), None)], width=66, vocab=90),
    "attention_window_longer_than_the_prompt": config([layer(attention(window=500))]),
    "mamba1_only": config([layer(mamba1(), None)]),
    "mamba1_odd_sizes_one_tap": config([layer(mamba1(inner=50, state=5, dt_rank=1, conv=1), None)], width=66, vocab=90),
    "mamba1_wide_state_five_taps": config([layer(mamba1(inner=48, state=40, dt_rank=9, conv=5))], width=64, vocab=128),
    "mamba1_state_one": config([layer(mamba1(inner=32, state=1, dt_rank=2, conv=2), None)], width=32, vocab=50),
    "parallel_only": config([layer(parallel(), None)]),
    "parallel_odd_table_far_bias": config([layer(parallel(heads=3, kv_heads=1, dim=14, window=90, bias_max=33, rel_rows=7, rheads=1, rdim=9, rvdim=7))], width=72, vocab=90),
    "parallel_table_longer_than_the_window": config([layer(parallel(heads=2, kv_heads=2, dim=16, window=6, bias_max=100, rel_rows=32, rheads=2, rdim=16, rvdim=16, gate_cap=2.0), None)], width=64, vocab=70),
    "parallel_no_window_one_row_table": config([layer(parallel(window=0, bias_max=8, rel_rows=1, rheads=2, rdim=40, rvdim=24), None)]),
    "dense_only_after_a_small_mixer": config([layer(mamba1(inner=16, state=2, dt_rank=1, conv=2), 200)], width=96, vocab=100),
}

F32_TOL, SPLIT_TOL = 2e-5, 2e-3


def tokens(n, vocab, seed):
    return np.random.default_rng(seed).integers(0, vocab, n).tolist()


def rel(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


def oracle_logits(cfg, w, ids, state=None):
    return P.forward(cfg, w, ids, state).numpy()


def sharp_model(seed, window=33, far=False):
    """Scores with a spread of several units (a query looks at one or two keys of its window, wherever they are), slow decays and
    forget gates near one (the recurrent states remember hundreds of tokens): a key just inside or just outside a window, a lost
    sink, a state that was not carried moves the logits by O(1).  far: no window and a weak distance penalty -- single keys
    hundreds of tokens back carry the output."""
    cfg = config([layer(attention(heads=4, kv_heads=2, dim=24, vdim=24, window=0 if far else window, scale=1.1, softcap=40.0), None),
                  layer(mamba1(inner=64, state=8, dt_rank=4, conv=4)),
                  layer(parallel(heads=4, kv_heads=2, dim=16, window=0 if far else window + 8, scale=1.3, softcap=40.0, bias_max=60, rel_rows=12), None),
                  layer(attention(heads=2, kv_heads=1, dim=32, vdim=16, window=0 if far else 64, scale=0.9, softcap=25.0))], width=128, vocab=200)
    w = P.random_weights(cfg, seed)
    for k in w:
        if k.endswith("right.f.b"):
            w[k] = w[k] + 3.0
        if far and (k.endswith(".r1") or k.endswith(".rel")):
            w[k] = (w[k] * 0.05).to(torch.bfloat16).to(T64)
    return cfg, w


# ---------------------------------------------------------------------------------------------------- CPU: the oracle itself
def test_oracle_prefill_equals_token_by_token():
    w = P.random_weights(FULL, 1)
    ids = tokens(90, FULL["vocab"], 2)
    whole = oracle_logits(FULL, w, ids)
    s = P.State(FULL)
    step = np.concatenate([oracle_logits(FULL, w, ids[:3], s)] + [oracle_logits(FULL, w, [t], s) for t in ids[3:]])
    assert rel(step, whole) < 1e-9


def test_oracle_mechanisms_on_known_answers():
    # distance table rows: one per distance below half the table, then logarithmic steps up to the last row at `far`
    assert [P.bucket(n, 8, 64) for n in (0, 1, 3, 4, 7, 8, 15, 16, 31, 32, 63, 64, 1000)] == [0, 1, 3, 4, 4, 5, 5, 6, 6, 7, 7, 7, 7]
    assert [P.bucket(n, 7, 30) for n in (0, 2, 3, 29, 30)] == [0, 2, 3, 6, 6]
    # position vector: sine at the even entry, cosine of the same angle at the odd one; the first pair turns once per 2 pi positions
    pv = P.position_vector([0, 1, 5], 6, T64)
    assert torch.allclose(pv[0], torch.tensor([0., 1., 0., 1., 0., 1.], dtype=T64))
    assert abs(pv[2, 0] - math.sin(5.0)) < 1e-12 and abs(pv[2, 1] - math.cos(5.0)) < 1e-12
    assert abs(pv[1, 2] - math.sin(10000.0 ** (-2 / 6))) < 1e-7 and abs(pv[1, 5] - math.cos(10000.0 ** (-4 / 6))) < 1e-7      # (the angle is a float32 number)
    # a softmax with a sink: two keys with equal scores and a sink of the same size leave a third of the weight on each value
    q = torch.ones(1, 1, 2, dtype=T64)
    k = torch.tensor([[[1., 0.]], [[0., 1.]]], dtype=T64)
    v = torch.tensor([[[3., 0.]], [[0., 6.]]], dtype=T64)
    o = P.attend(q, k, v, [1], 0, lambda s: s, lambda h, dist: torch.zeros(len(dist), dtype=T64), sink=torch.tensor([1.0], dtype=T64))
    assert torch.allclose(o[0, 0], torch.tensor([1., 2.], dtype=T64))
    # a window of one sees the row's own key only; the distance term then is that of distance zero
    o = P.attend(q, k, v, [1], 1, lambda s: s, lambda h, dist: -5.0 * dist.to(T64))
    assert torch.allclose(o[0, 0], torch.tensor([0., 6.], dtype=T64))
    # the cap: far below it a score passes, far above it the cap itself comes out
    assert abs(P.cap(torch.tensor(0.01, dtype=T64), 30.0) - 0.01) < 1e-8 and abs(P.cap(torch.tensor(1e4, dtype=T64), 30.0) - 30.0) < 1e-9
    # causal convolution: the last column weighs the current token, the window carries the inputs before the portion
    u = torch.tensor([[1.], [2.], [4.]], dtype=T64)
    cv, win = P.causal_conv(u, torch.tensor([[100., 10., 1.]], dtype=T64), torch.tensor([0.5], dtype=T64), torch.tensor([[7.], [8.]], dtype=T64))
    assert cv[:, 0].tolist() == [781.5, 812.5, 124.5] and win[:, 0].tolist() == [2., 4.]
    # selective scan, one channel, one state entry: S = e^{dt A} S + dt u B by hand
    y, S = P.selective_scan(torch.tensor([[2.], [1.]], dtype=T64), torch.tensor([[0.5], [1.0]], dtype=T64), torch.tensor([[-1.0]], dtype=T64),
                            torch.tensor([[1.], [2.]], dtype=T64), torch.tensor([[3.], [1.]], dtype=T64), torch.tensor([10.], dtype=T64), torch.zeros(1, 1, dtype=T64))
    s1 = 0.5 * 2 * 1
    s2 = math.exp(-1.0) * s1 + 1 * 1 * 2
    assert abs(y[0, 0] - (3 * s1 + 20)) < 1e-12 and abs(y[1, 0] - (s2 + 10)) < 1e-12 and abs(S[0, 0] - s2) < 1e-12
    # matrix memory, first token from an empty memory with m_0 = 0: m_1 = max(f, i); the output's denominator is max(|n . q|, e^{-m})
    ig, fg = torch.tensor([2.0], dtype=T64), torch.tensor([-0.5], dtype=T64)
    o, S, n, m = P.matrix_memory(torch.tensor([[1., 0.]], dtype=T64), torch.tensor([[0.1, 3.]], dtype=T64), torch.tensor([[5.]], dtype=T64), ig, fg,
                                 torch.zeros(2, 1, dtype=T64), torch.zeros(2, dtype=T64), torch.zeros((), dtype=T64))
    assert float(m) == 2.0 and abs(S[0, 0] - 0.5) < 1e-12 and abs(n[1] - 3.0) < 1e-12
    assert abs(o[0, 0] - 0.5 / (max(0.1, math.exp(-2.0)) + 1e-6)) < 1e-12
    ig = torch.tensor([-3.0], dtype=T64)                              # a closed input gate: m_1 = f + m_0 = -0.5, the weight e^{i - m}
    o, S, n, m = P.matrix_memory(torch.tensor([[1., 0.]], dtype=T64), torch.tensor([[0.1, 3.]], dtype=T64), torch.tensor([[5.]], dtype=T64), ig, fg,
                                 torch.zeros(2, 1, dtype=T64), torch.zeros(2, dtype=T64), torch.zeros((), dtype=T64))
    assert float(m) == -0.5 and abs(o[0, 0] - 0.5 * math.exp(-2.5) / (math.exp(0.5) + 1e-6)) < 1e-12
    # the gated unit
    x = torch.tensor([[1.0, -2.0]], dtype=T64)
    eye = torch.eye(2, dtype=T64)
    g = 0.5 * x * (1 + torch.tanh(math.sqrt(2 / math.pi) * (x + 0.044715 * x ** 3)))
    assert torch.allclose(P.feed_forward(x, eye, 3 * eye, eye), g * 3 * x)


def test_oracle_sees_what_the_sharp_tests_are_about(monkeypatch):
    cfg, w = sharp_model(41)
    ids = tokens(200, cfg["vocab"], 42)
    base = oracle_logits(cfg, w, ids)
    wider = copy.deepcopy(cfg)
    wider["layers"][0]["mixer"]["mask"]["size"] += 1                 # a window one key too long
    assert rel(oracle_logits(wider, w, ids)[40:], base[40:]) > 1e-2
    wider = copy.deepcopy(cfg)
    wider["layers"][2]["mixer"]["left"]["mask"]["size"] -= 1         # ... one key too short, in the left mixer
    assert rel(oracle_logits(wider, w, ids)[50:], base[50:]) > 1e-2
    no_sink = dict(w)
    no_sink["l0.mix.sink"] = w["l0.mix.sink"] - 30.0                  # a sink that is left out
    assert rel(oracle_logits(cfg, no_sink, ids), base) > 1e-2
    lost = P.State(cfg)                                              # recurrent states that were not carried over a cut
    a = oracle_logits(cfg, w, ids[:120], lost)
    lost.S[1] = torch.zeros_like(lost.S[1])
    assert rel(oracle_logits(cfg, w, ids[120:], lost), base[120:]) > 1e-2
    lost = P.State(cfg)
    oracle_logits(cfg, w, ids[:120], lost)
    lost.mem[2] = [(torch.zeros_like(S), torch.zeros_like(n), torch.zeros_like(m)) for S, n, m in lost.mem[2]]
    assert rel(oracle_logits(cfg, w, ids[120:], lost), base[120:]) > 1e-2
    monkeypatch.setattr(P, "bucket", lambda n, rows, far: min(n, rows - 1))       # a distance table read without its logarithmic rows
    assert rel(oracle_logits(cfg, w, ids), base) > 1e-2
    monkeypatch.undo()
    cfg, w = sharp_model(43, far=True)                                # no window: single keys hundreds of tokens back carry the output
    ids = tokens(400, cfg["vocab"], 44)
    base = oracle_logits(cfg, w, ids)
    near = copy.deepcopy(cfg)
    for i in (0, 3):
        near["layers"][i]["mixer"]["mask"] = {"size": 200}
    assert rel(oracle_logits(near, w, ids)[300:], base[300:]) > 1e-2


# ---------------------------------------------------------------------------------------------------- GPU
def make(cfg, seed=0, weights=None, **opts):
    import crane_b200
    w = weights or P.random_weights(cfg, seed)
    opts.setdefault("max_tokens", 1024)
    opts.setdefault("max_batch", 4)
    m = crane_b200.PuzonexModel(cfg, device=0, **opts)
    m.load_checkpoint((k, t.to(torch.float32).numpy()) for k, t in w.items())
    return m, w


def all_rows(n):
    return list(range(n))


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(SINGLE))
def test_each_mechanism_alone(name):
    cfg = SINGLE[name]
    m, w = make(cfg, 3, precision="f32")
    ids = tokens(100, cfg["vocab"], 4)
    want = oracle_logits(cfg, w, ids)
    assert rel(m.step_batch([(0, ids, all_rows(100))]), want) < F32_TOL
    m.clear_kv_cache()
    rows = [m.step_batch([(0, ids[:2], [0, 1])])] + [m.step_batch([(0, [t], [0])]) for t in ids[2:50]]
    assert rel(np.concatenate(rows), want[:50]) < F32_TOL
    m.close()


@pytest.mark.gpu
@pytest.mark.parametrize("precision,tol", [("f32", F32_TOL), ("split", SPLIT_TOL)])
def test_whole_model_prefill_and_token_by_token_decoding(precision, tol):
    m, w = make(FULL, 5, precision=precision)
    ids = tokens(170, FULL["vocab"], 6)
    want = oracle_logits(FULL, w, ids)
    got = m.step_batch([(0, ids, all_rows(len(ids)))])
    assert rel(got, want) < tol
    m.clear_kv_cache()
    rows = [m.step_batch([(0, ids[:3], [0, 1, 2])])]
    rows += [m.step_batch([(0, [t], [0])]) for t in ids[3:]]       # long decoding through two page borders, every window passed, every state carried 167 times
    step = np.concatenate(rows)
    assert rel(step, want) < tol
    if precision == "f32":
        assert rel(step, got) < 1e-5
    m.close()


@pytest.mark.gpu
def test_plain_bf16_precision_is_close():
    m, w = make(FULL, 7, precision="bf16")
    ids = tokens(90, FULL["vocab"], 8)
    got, want = m.step_batch([(0, ids, all_rows(90))]), oracle_logits(FULL, w, ids)
    assert rel(got, want) < 6e-2
    m.close()


@pytest.mark.gpu
@pytest.mark.parametrize("cuts", [[2, 2, 2, 61, 3, 64, 1, 1, 30, 2], [63, 1, 1, 63, 2, 36], [1] * 5 + [95, 66], [31, 33, 32, 64, 6], [17, 18, 19, 112]])
def test_portions_of_any_size_match_the_whole_prompt(cuts):
    m, w = make(FULL, 9, precision="f32")
    n = sum(cuts)
    ids = tokens(n, FULL["vocab"], 10)
    want = oracle_logits(FULL, w, ids)
    at, rows = 0, []
    for c in cuts:
        rows.append(m.step_batch([(0, ids[at:at + c], all_rows(c))]))
        at += c
    assert rel(np.concatenate(rows), want) < F32_TOL
    m.close()


@pytest.mark.gpu
@pytest.mark.parametrize("precision,tol", [("f32", F32_TOL), ("split", SPLIT_TOL)])
def test_unequal_requests_in_one_batch_match_each_alone(precision, tol):
    m, w = make(FULL, 11, precision=precision, max_tokens=1024)
    lens = [97, 5, 130, 64]
    prompts = [tokens(n, FULL["vocab"], 20 + i) for i, n in enumerate(lens)]
    want = [oracle_logits(FULL, w, p) for p in prompts]
    seqs = [0] + [m.seq_create() for _ in range(3)]
    got = [[] for _ in lens]
    at = [0] * 4
    # a different mixture every step: portions of some beside single tokens of others, one request sitting a step out
    plan = [[(0, 40), (1, 2), (2, 1)], [(2, 64), (3, 63), (0, 1)], [(1, 1), (3, 1), (0, 56), (2, 2)], [(1, 2), (2, 63)]]
    for stepn in plan:
        entries = [(seqs[i], prompts[i][at[i]:at[i] + c], all_rows(c)) for i, c in stepn]
        lg = m.step_batch(entries)
        r = 0
        for i, c in stepn:
            got[i].append(lg[r:r + c]); r += c; at[i] += c
    for i in range(4):
        g = np.concatenate(got[i])
        assert rel(g, want[i][:len(g)]) < tol, i
    m.close()


@pytest.mark.gpu
def test_pages_and_slots_are_used_again():
    m, w = make(FULL, 13, precision="f32", max_tokens=256, max_batch=2)        # 4 pages, 2 slots
    a, b, c = (tokens(n, FULL["vocab"], 30 + i) for i, n in enumerate((130, 120, 100)))
    s1 = m.seq_create()
    m.step_batch([(0, a, []), (s1, b[:60], [])])                # 3 + 1 pages: the pool is full
    with pytest.raises(Exception):
        m.step_batch([(s1, b[60:], [])])                        # needs a fifth page: refused, nothing changes
    assert m.seq_len(s1) == 60
    m.clear_kv_cache()                                          # sequence 0 gives its three pages back
    got_b = m.step_batch([(s1, b[60:], [len(b) - 61])])
    assert rel(got_b[0], oracle_logits(FULL, w, b)[-1]) < F32_TOL
    m.seq_free(s1)
    s2 = m.seq_create()                                         # same slot: windows, states and running maxima start from zero, pages still hold b's rows
    assert s2 == s1
    got_c = m.step_batch([(s2, c[:50], []), (0, a[:64], [63])])
    got_c2 = m.step_batch([(s2, c[50:], [49])])
    assert rel(got_c2[0], oracle_logits(FULL, w, c)[-1]) < F32_TOL
    assert rel(got_c[0], oracle_logits(FULL, w, a[:64])[-1]) < F32_TOL
    m.close()


@pytest.mark.gpu
def test_window_edges_page_borders_and_carried_states_with_sharp_scores():
    cfg, w = sharp_model(41)                                    # windows of 33, 41 and 64 keys
    m, _ = make(cfg, weights=w, max_tokens=1024, max_batch=2, precision="f32")
    ids = tokens(330, cfg["vocab"], 42)
    want = oracle_logits(cfg, w, ids)
    got = m.step_batch([(0, ids, all_rows(330))])
    assert rel(got, want) < F32_TOL
    # decode over the borders of 32-key tiles and 64-token pages and the places where a window's far edge crosses them, after a
    # prompt that ends just before / on / after them
    for start in (1, 2, 3, 31, 32, 33, 34, 40, 41, 42, 63, 64, 65, 66, 72, 73, 95, 96, 97, 104, 105, 127, 128, 129, 191, 192, 193, 255, 256, 257):
        m.clear_kv_cache()
        m.step_batch([(0, ids[:start], [])])
        rows = np.concatenate([m.step_batch([(0, [t], [0])]) for t in ids[start:start + 4]])
        assert rel(rows, want[start:start + 4]) < F32_TOL, start
    # the same edges inside portions of a prompt, the second portion as short as two tokens
    for cut in (33, 34, 41, 64, 65, 97, 129, 256):
        m.clear_kv_cache()
        a = m.step_batch([(0, ids[:cut - 1], [cut - 2])])
        b = m.step_batch([(0, ids[cut - 1:cut + 1], all_rows(2))])
        c = m.step_batch([(0, ids[cut + 1:cut + 40], all_rows(39))])
        assert rel(np.concatenate([a, b, c]), want[cut - 2:cut + 40]) < F32_TOL, cut
    m.close()


@pytest.mark.gpu
def test_keys_far_away_without_a_window():
    cfg, w = sharp_model(43, far=True)
    m, _ = make(cfg, weights=w, max_tokens=2048, precision="f32")
    ids = tokens(1500, cfg["vocab"], 44)
    want = oracle_logits(cfg, w, ids)
    got = m.step_batch([(0, ids[:1200], [500, 900, 1199])])
    assert rel(got, want[[500, 900, 1199]]) < F32_TOL
    rows = np.concatenate([m.step_batch([(0, [t], [0])]) for t in ids[1200:]])          # 300 decoded tokens, the context split over blocks
    assert rel(rows, want[1200:]) < F32_TOL
    m.close()


@pytest.mark.gpu
@pytest.mark.parametrize("precision,tol", [("f32", F32_TOL), ("split", SPLIT_TOL)])
def test_long_portions_scan_in_segments(precision, tol):
    # from 512 rows on a portion's recurrences run as four segments side by side; here on carried states, beside a short request,
    # with lengths that leave the last segment ragged, a state width that is not a multiple of four and a one-segment entry
    cfg = config([layer(mamba1(inner=72, state=6, dt_rank=5, conv=3), None),
                  layer(parallel(heads=2, kv_heads=1, dim=16, window=50, rheads=2, rdim=18, rvdim=21, gate_cap=6.0), 40),
                  layer(mamba1(inner=64, state=16, dt_rank=8, conv=4), None)], width=96, vocab=150)
    m, w = make(cfg, 27, precision=precision, max_tokens=2048)
    ids, other = tokens(1400, cfg["vocab"], 28), tokens(40, cfg["vocab"], 29)
    want, want2 = oracle_logits(cfg, w, ids), oracle_logits(cfg, w, other)
    s1 = m.seq_create()
    a = m.step_batch([(0, ids[:100], [99])])
    b = m.step_batch([(s1, other[:30], [29]), (0, ids[100:803], [0, 350, 702])])
    c = m.step_batch([(0, ids[803:1399], [0, 595]), (s1, other[30:], [9])])
    d = m.step_batch([(0, ids[1399:], [0])])
    assert rel(np.concatenate([a, b[1:], c[:2], d]), want[[99, 100, 450, 802, 803, 1398, 1399]]) < tol
    assert rel(np.stack([b[0], c[2]]), want2[[29, 39]]) < tol
    m.close()


@pytest.mark.gpu
def test_first_tokens_of_a_sequence():
    m, w = make(FULL, 15, precision="f32")
    ids = tokens(7, FULL["vocab"], 16)
    want = oracle_logits(FULL, w, ids)
    assert rel(m.step_batch([(0, ids[:1], [0])]), want[:1]) < F32_TOL           # a one-token prompt: zeros in every window, an empty memory
    assert rel(m.step_batch([(0, ids[1:2], [0])]), want[1:2]) < F32_TOL
    assert rel(m.step_batch([(0, ids[2:4], [0, 1])]), want[2:4]) < F32_TOL      # a portion shorter than the convolution's window
    assert rel(m.step_batch([(0, ids[4:], [0, 1, 2])]), want[4:]) < F32_TOL
    m.close()


@pytest.mark.gpu
def test_greedy_generation_through_generate_and_the_scheduler():
    from crane_b200.scheduler import BatchScheduler
    m, w = make(FULL, 19, precision="f32", max_tokens=512)

    def oracle_greedy(prompt, n):
        s = P.State(FULL)
        lg = oracle_logits(FULL, w, prompt, s)[-1]
        out, margins = [], []
        for _ in range(n):
            top = np.sort(lg)[-2:]
            margins.append(top[1] - top[0])
            out.append(int(lg.argmax()))
            lg = oracle_logits(FULL, w, [out[-1]], s)[-1]
        return out, min(margins)

    prompts = [tokens(n, FULL["vocab"], 50 + i) for i, n in enumerate((70, 9, 33, 130, 20, 64))]
    want = [oracle_greedy(p, 12) for p in prompts]
    assert min(mg for _, mg in want) > 1e-4                     # no decision of this test is a close call
    assert m.generate(prompts[0], max_new_tokens=12).tolist() == want[0][0]
    m.clear_kv_cache()
    sch = BatchScheduler(m, chunk=48, max_live=3, token_budget=80)
    rids = [sch.add(p, 12) for p in prompts]
    out = sch.run()
    for rid, (toks, _) in zip(rids, want):
        assert out[rid] == toks, rid
    sch = BatchScheduler(m, chunk=32, max_live=2)
    rid = sch.add(prompts[1], 6, temperature=0.8, top_k=1, seed=3)         # top-k 1 is greedy whatever the draw
    assert sch.run()[rid] == want[1][0][:6]
    m.clear_kv_cache()
    s1 = m.seq_create()
    m.step_batch([(0, prompts[2], []), (s1, prompts[4], [])])
    first = [want[2][0][0], want[4][0][0]]
    toks, _ = m.decode_batch([0, s1], first, n_steps=5)                     # the graph-replayed loop, two sequences side by side
    assert toks[0].tolist() == want[2][0][1:6] and toks[1].tolist() == want[4][0][1:6]
    m.close()


@pytest.mark.gpu
def test_wide_layers_take_the_tensor_core_paths():
    # widths the tensor-core kernels take: 64- and 128-wide heads, many rows; a wide scan state and a 128 x 64 matrix memory
    cfg = config([layer(attention(heads=4, kv_heads=2, dim=64, vdim=64, window=100, scale=0.12), 352),
                  layer(mamba1(inner=256, state=16, dt_rank=8, conv=4), 64),
                  layer(parallel(heads=2, kv_heads=1, dim=128, window=150, scale=0.09, rheads=2, rdim=128, rvdim=64), 128),
                  layer(attention(heads=4, kv_heads=4, dim=128, vdim=128, window=0, scale=0.09), None)], width=256, vocab=300)
    m, w = make(cfg, 21, precision="split")
    ids = tokens(400, cfg["vocab"], 22)
    want = oracle_logits(cfg, w, ids)
    assert rel(m.step_batch([(0, ids, all_rows(400))]), want) < SPLIT_TOL
    m.clear_kv_cache()
    a = m.step_batch([(0, ids[:333], all_rows(333))])
    b = m.step_batch([(0, ids[333:], all_rows(67))])
    assert rel(np.concatenate([a, b]), want) < SPLIT_TOL
    m.close()


def random_config(seed):
    """A layer list drawn at random: the three mixers in any order, widths that are and are not multiples of 4 and 8, every grouping
    of query heads, windows around tile and page sizes, with and without a feed-forward."""
    r = np.random.default_rng(seed)
    pick = lambda *xs: xs[int(r.integers(len(xs)))]
    width = pick(72, 96, 120, 160)
    layers = []
    for _ in range(int(r.integers(1, 6))):
        kind = int(r.integers(3))
        if kind == 0:
            G = pick(1, 2, 3)
            mx = attention(heads=G * pick(1, 2, 4), kv_heads=G, dim=pick(8, 18, 32, 40), vdim=pick(8, 20, 24, 64), window=pick(0, 1, 5, 31, 32, 33, 64, 100),
                           scale=float(pick(0.1, 0.3, 0.6)), softcap=float(pick(0.0, 5.0, 30.0)))
        elif kind == 1:
            mx = mamba1(inner=pick(24, 50, 96, 130), state=pick(1, 4, 8, 16, 19), dt_rank=pick(1, 3, 8), conv=pick(1, 2, 3, 4, 6))
        else:
            G = pick(1, 2)
            rows = pick(2, 5, 8, 16)
            mx = parallel(heads=G * pick(1, 3), kv_heads=G, dim=pick(8, 12, 20, 32), window=pick(0, 1, 7, 32, 33, 65), scale=float(pick(0.1, 0.4)),
                          softcap=float(pick(0.0, 8.0, 50.0)), bias_max=rows // 2 + pick(1, 7, 40), rel_rows=rows, rheads=pick(1, 2, 4), rdim=pick(4, 10, 16, 36),
                          rvdim=pick(6, 16, 20, 33), gate_cap=float(pick(1.0, 8.0, 20.0)))
        layers.append(layer(mx, pick(0, 12, 30, 64)))
    return config(layers, width=width, vocab=pick(90, 211, 300), eps=float(pick(1e-6, 1e-5)))


@pytest.mark.gpu
@pytest.mark.parametrize("seed", range(10))
def test_random_layer_lists(seed):
    cfg = random_config(100 + seed)
    r = np.random.default_rng(seed)
    ids, other = tokens(150, cfg["vocab"], 200 + seed), tokens(70, cfg["vocab"], 300 + seed)
    for precision, tol in (("f32", F32_TOL), ("split", SPLIT_TOL)):
        m, w = make(cfg, 400 + seed, precision=precision)
        want, want2 = oracle_logits(cfg, w, ids), oracle_logits(cfg, w, other)
        assert rel(m.step_batch([(0, ids, all_rows(150))]), want) < tol, (precision, "whole")
        m.clear_kv_cache()
        s1 = m.seq_create()
        at, at2, rows, rows2 = 0, 0, [], []
        while at < 150:                                      # random cuts, the second request beside some of them
            c = int(min(150 - at, r.choice([1, 2, 3, 17, 40, 64])))
            entries = [(0, ids[at:at + c], all_rows(c))]
            c2 = int(min(70 - at2, r.choice([0, 1, 2, 30])))
            if c2:
                entries.append((s1, other[at2:at2 + c2], all_rows(c2)))
            lg = m.step_batch(entries)
            rows.append(lg[:c]); rows2.append(lg[c:]); at += c; at2 += c2
        assert rel(np.concatenate(rows), want) < tol, (precision, "cuts")
        got2 = np.concatenate(rows2)
        assert rel(got2, want2[:len(got2)]) < tol, (precision, "beside")
        m.close()


@pytest.mark.gpu
def test_model_folder_loader_and_trace_runner(tmp_path):
    import json, os, subprocess, sys
    cfg = copy.deepcopy(FULL)
    for lc in cfg["layers"]:                                    # the rows of a distance table come with its tensor, not with config.json
        if lc["type"] == "parallel":
            lc["mixer"]["left"].pop("rel_rows")
    w = P.random_weights(FULL, 23)
    hdr, blob = {}, b""
    for k, t in w.items():
        bits = P.to_numpy_bf16_bits(t).tobytes()
        hdr[k] = {"dtype": "BF16", "shape": list(t.shape), "data_offsets": [len(blob), len(blob) + len(bits)]}
        blob += bits
    mdir = tmp_path / "model"; mdir.mkdir()
    (mdir / "config.json").write_text(json.dumps(cfg))
    h = json.dumps(hdr).encode()
    (mdir / "model.safetensors").write_bytes(len(h).to_bytes(8, "little") + h + blob)
    a, b = tokens(80, cfg["vocab"], 24), tokens(70, cfg["vocab"], 25)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:50], "want": [49]}, {"id": "b", "tokens": b[:2], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "b", "tokens": b[2:], "want": [0, 67]}, {"id": "a", "tokens": a[50:51], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[51:], "want": []}], "end": ["a"]},
             {"step": 3, "entries": [{"id": "c", "tokens": b, "want": [69]}], "end": ["c"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(mdir), "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "192"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2", "done 3"]
    wa, wb = oracle_logits(FULL, w, a), oracle_logits(FULL, w, b)
    read = lambda n: np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(-1, cfg["vocab"])
    assert rel(read(0), wa[49:50]) < F32_TOL
    assert rel(read(1), np.stack([wb[2], wb[69], wa[50]])) < F32_TOL
    assert not (out / "2.f32").exists()
    assert rel(read(3), wb[69:70]) < F32_TOL                    # request c runs on the slot and pages b gave back
