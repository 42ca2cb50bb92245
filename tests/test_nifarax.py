"""Nifarax (sequential gated sublayers behind carried convolutions; latent attention and gated linear attention; input-weighted
clamped experts) against the plain oracle of oracle/nifarax.py.

Small configurations with their own random weights; the oracle runs in float64.  The engine's "f32" precision is held to a tight
bar (a lost latent row, a convolution window that was not carried, a state of the wrong layer or slot, a weight on the wrong
side of an expert shows), the serving precision to the bar its operand rounding allows.
"""
import copy
import math

import numpy as np
import pytest
import torch

from oracle import nifarax as N

T64 = torch.float64


# ---------------------------------------------------------------------------------------------------- configurations
def latent(heads=5, dim=24, vdim=40, q_rank=56, kv_rank=72, scale=0.25):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale}}


def gla(heads=3, dim=20, vdim=36, tau=8.0, decay_rank=12):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "decay_rank": decay_rank}}


def moe(ff=44, experts=6, top=2, limit=1.5, shared=52, shared_limit=2.5):
    f = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared:
        f["shared"] = {"ff": shared, "limit": shared_limit}
    return f


def layer(mx, mlp="default", weights_of=None):
    l = dict(copy.deepcopy(mx), mlp=moe() if mlp == "default" else mlp)
    if weights_of is not None:
        l["weights_of"] = weights_of
    return l


def config(layers, width=120, vocab=211, taps=3, groups=3, eps=1e-5, cap=20.0):
    return {"architecture": "Nifarax", "vocab": vocab, "width": width, "norm": {"eps": eps, "groups": groups}, "canon": {"taps": taps},
            "logit_softcap": cap, "layers": copy.deepcopy(layers)}


# six layers of unequal geometry; layer 4 reads layer 1's tensors (a gla with a state of its own), layer 5 reads layer 0's
FULL = config([layer(latent()),
               layer(gla()),
               layer(latent(heads=2, dim=40, vdim=16, q_rank=30, kv_rank=64, scale=0.2), moe(ff=20, experts=8, top=3, shared=0)),
               layer(gla(heads=4, dim=16, vdim=24, tau=3.0, decay_rank=5), None),
               layer(gla(), weights_of=1),
               layer(latent(), weights_of=0)])
SINGLE = {
    "latent_attention_only": config([layer(latent(), None)]),
    "gla_only": config([layer(gla(), None)]),
    "latent_odd_widths_one_group": config([layer(latent(heads=3, dim=18, vdim=9, q_rank=21, kv_rank=35), None)], width=72, vocab=90, groups=1, taps=2),
    "gla_odd_widths_five_taps": config([layer(gla(heads=2, dim=13, vdim=21, tau=1.0, decay_rank=3), None)], width=66, vocab=90, groups=2, taps=5),
    "gla_wide_keys": config([layer(gla(heads=2, dim=72, vdim=40, tau=16.0, decay_rank=16), None)], width=96, vocab=128, groups=4, taps=4),
    "one_tap": config([layer(latent(), None), layer(gla(), None)], taps=1),
    "experts_top1_no_shared": config([layer(latent(), moe(ff=30, experts=5, top=1, shared=0))]),
    "experts_all_chosen": config([layer(gla(), moe(ff=28, experts=4, top=4, shared=16))]),
    "experts_shared": config([layer(latent(), moe())]),
    "one_expert_one_head": config([layer(latent(heads=1, dim=16, vdim=12, q_rank=8, kv_rank=20), moe(ff=16, experts=1, top=1, shared=0)),
                                   layer(gla(heads=1, dim=8, vdim=8, tau=2.0, decay_rank=1), moe(ff=8, experts=1, top=1, shared=8))], width=64, vocab=70, groups=1, taps=2),
    "shared_weights": config([layer(gla()), layer(latent()), layer(gla(), weights_of=0), layer(latent(), weights_of=1)]),
    "shared_weights_from_a_later_layer_and_through_another": config([layer(latent(), weights_of=2), layer(latent(), weights_of=0), layer(latent())]),
    "no_cap_needed": config([layer(latent()), layer(gla())], cap=500.0),
}


def tokens(n, vocab, seed):
    return np.random.default_rng(seed).integers(0, vocab, n).tolist()


def rel(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


F32_TOL, SPLIT_TOL = 2e-5, 2e-3


def oracle_logits(cfg, w, ids, state=None):
    return N.forward(cfg, w, ids, state).numpy()


def sharp_model(seed):
    """Attention scores with a spread of several units (a query looks at one or two latent rows anywhere in its past) and decays
    close to one (the recurrent state remembers hundreds of tokens): a lost row, a row of another page or a state that was not
    carried moves the logits by O(1)."""
    cfg = config([layer(latent(scale=1.6), None),
                  layer(gla(tau=40.0)),
                  layer(latent(heads=4, dim=32, vdim=32, q_rank=48, kv_rank=64, scale=1.2)),
                  layer(gla(tau=40.0), weights_of=1)], width=128, vocab=200, groups=2, taps=4)
    return cfg, N.random_weights(cfg, seed)


# ---------------------------------------------------------------------------------------------------- CPU: the oracle itself
def test_oracle_prefill_equals_token_by_token():
    w = N.random_weights(FULL, 1)
    ids = tokens(90, FULL["vocab"], 2)
    whole = oracle_logits(FULL, w, ids)
    s = N.State(FULL)
    parts = [oracle_logits(FULL, w, ids[a:b], s) for a, b in ((0, 7), (7, 9), (9, 10), (10, 70), (70, 71), (71, 90))]
    assert rel(np.concatenate(parts), whole) < 1e-11


def test_oracle_mechanisms_on_known_answers():
    t = lambda a: torch.tensor(a, dtype=T64)
    # norm in two groups: (3, 4) and (0, 5) each by its own root mean square
    x = t([[3.0, 4.0, 0.0, 5.0]])
    out = N.group_norm(x, t([1.0, 1.0, 2.0, 2.0]), 2, 0.0)[0]
    assert torch.allclose(out, t([3 / math.sqrt(12.5), 4 / math.sqrt(12.5), 0.0, 2 * 5 / math.sqrt(12.5)]))
    assert torch.allclose(N.group_norm(x, torch.ones(4, dtype=T64), 1, 0.0), x / math.sqrt(12.5))
    # convolution with taps (w0, w1, w2): out_t = w0 h_(t-2) + w1 h_(t-1) + w2 h_t, zeros before the start, the window carried
    h = t([[1.0], [2.0], [3.0], [4.0]])
    w = t([[0.5, 10.0, 100.0]])
    full, win = N.causal_conv(h, w, torch.zeros(2, 1, dtype=T64))
    assert full[:, 0].tolist() == [100.0, 210.0, 320.5, 431.0] and win[:, 0].tolist() == [3.0, 4.0]
    a, wa = N.causal_conv(h[:1], w, torch.zeros(2, 1, dtype=T64))
    b, wb = N.causal_conv(h[1:], w, wa)
    assert torch.allclose(torch.cat([a, b]), full) and wb[:, 0].tolist() == [3.0, 4.0]
    # recurrence: one head, one key channel, decay 1/2, k = v = q = 1: o_t = sum_{i<=t} 2^-(t-i)
    one = torch.ones(3, 1, 1, dtype=T64)
    o, S = N.gla_scan(one, one, one, one * 0.5, torch.zeros(1, 1, 1, dtype=T64))
    assert o.flatten().tolist() == [1.0, 1.5, 1.75] and float(S) == 1.75
    # the decay acts on key channels (rows of S): channel 0 forgets, channel 1 keeps
    q = t([[[1.0, 1.0]], [[1.0, 1.0]]]); k = t([[[1.0, 1.0]], [[0.0, 0.0]]]); v = t([[[2.0, 3.0]], [[0.0, 0.0]]]); al = t([[[0.0, 1.0]], [[0.0, 1.0]]])
    o, S = N.gla_scan(q, k, v, al, torch.zeros(1, 2, 2, dtype=T64))
    assert o[1, 0].tolist() == [2.0, 3.0] and S[0].tolist() == [[0.0, 0.0], [2.0, 3.0]]
    # decay = sigmoid(z)^(1/tau), z = a2 (a1 u) + b
    d = N.gla_decay(torch.ones(1, 1, dtype=T64), t([[2.0]]), t([[1.0], [-3.0]]), t([0.5, 0.0]), 4.0)
    sig = lambda z: 1 / (1 + math.exp(-z))
    assert torch.allclose(d, t([[sig(2.5) ** 0.25, sig(-6.0) ** 0.25]]))
    # expert: gate clamped from above only, up on both sides, (up + 1)
    y = N.expert(torch.ones(1, 1, dtype=T64), t([[5.0], [-5.0]]), t([[9.0], [-9.0]]), torch.eye(2, dtype=T64), 2.0)
    g0, g1 = 2.0, -5.0
    assert torch.allclose(y[0], t([g0 * sig(1.702 * g0) * 3.0, g1 * sig(1.702 * g1) * -1.0]))
    # routing: the largest sigmoid scores, kept as they are (no renormalisation)
    idx, wt = N.route(torch.ones(1, 1, dtype=T64), t([[0.0], [2.0], [-1.0], [1.0]]), 2)
    assert idx.tolist() == [[1, 3]] and torch.allclose(wt[0], t([sig(2.0), sig(1.0)]))
    # the weight multiplies the expert's input: with a gate that saturates at the limit this is not weight * expert(h)
    p = {"m.router": t([[3.0], [-30.0]]), "m.e0.gate": t([[8.0]]), "m.e0.up": t([[0.25]]), "m.e0.down": t([[1.0]]),
         "m.e1.gate": t([[1.0]]), "m.e1.up": t([[1.0]]), "m.e1.down": t([[1.0]])}
    cfg = {"expert": {"ff": 1, "limit": 2.0}, "router": {"experts": 2, "top": 1}}
    s = sig(3.0)
    got = float(N.moe(torch.ones(1, 1, dtype=T64), p, "m.", cfg))
    inside = 2.0 * sig(1.702 * 2.0) * (0.25 * s + 1.0)
    outside = s * 2.0 * sig(1.702 * 2.0) * 1.25
    assert abs(got - inside) < 1e-12 and abs(got - outside) > 1e-2
    # soft cap and causal attention
    assert torch.allclose(N.softcap(t([0.0, 1e9, -3.0]), 2.0), t([0.0, 2.0, 2.0 * math.tanh(-1.5)]))
    k = torch.zeros(4, 1, 2, dtype=T64); v = torch.arange(4, dtype=T64).reshape(4, 1, 1)
    out = N.causal_attention(torch.zeros(2, 1, 2, dtype=T64), k, v, torch.tensor([1, 3]), 1.0)
    assert torch.allclose(out.flatten(), t([0.5, 1.5]))
    assert [N.weight_layer(FULL, i) for i in range(6)] == [0, 1, 2, 3, 1, 0]


def test_oracle_sees_what_the_sharp_tests_are_about(monkeypatch):
    cfg, w = sharp_model(3)
    ids = tokens(150, cfg["vocab"], 4)
    want = oracle_logits(cfg, w, ids)
    s = N.State(cfg)
    oracle_logits(cfg, w, ids[:120], s)
    keep = copy.deepcopy(s)
    s.latent[0] = torch.cat([s.latent[0][:7], s.latent[0][8:9], s.latent[0][8:]])        # one far latent row replaced by its neighbour
    assert rel(oracle_logits(cfg, w, ids[120:], s), want[120:]) > 1e-3
    s = copy.deepcopy(keep)
    s.S[1], s.S[3] = s.S[3], s.S[1]                                                       # the two layers that share tensors swap their states
    assert rel(oracle_logits(cfg, w, ids[120:], s), want[120:]) > 1e-3
    s = copy.deepcopy(keep)
    s.win[2][1] = torch.zeros_like(s.win[2][1])                                           # a convolution window that was not carried
    assert rel(oracle_logits(cfg, w, ids[120:121], s), want[120:121]) > 1e-3
    s = copy.deepcopy(keep)
    s.S[1] = s.S[1] * 0.0                                                                 # a recurrent state that was lost
    assert rel(oracle_logits(cfg, w, ids[120:], s), want[120:]) > 1e-2
    orig = N.expert
    monkeypatch.setattr(N, "moe", weight_on_the_output)                                   # the score on the wrong side of the expert
    assert rel(oracle_logits(cfg, w, ids), want) > 1e-3
    monkeypatch.setattr(N, "expert", orig)


def weight_on_the_output(u, p, pre, cfg):
    idx, wts = N.route(u, p[pre + "router"], cfg["router"]["top"])
    out = torch.zeros(u.shape[0], p[pre + "e0.down"].shape[0], dtype=u.dtype)
    for r in range(u.shape[0]):
        for kk in range(idx.shape[1]):
            e = int(idx[r, kk])
            out[r] += wts[r, kk] * N.expert(u[r:r + 1], p[f"{pre}e{e}.gate"], p[f"{pre}e{e}.up"], p[f"{pre}e{e}.down"], cfg["expert"]["limit"])[0]
    sh = cfg.get("shared")
    if sh:
        out = out + torch.sigmoid(u @ p[pre + "shared.sg"].T) * N.expert(u, p[pre + "shared.gate"], p[pre + "shared.up"], p[pre + "shared.down"], sh["limit"])
    return out


# ---------------------------------------------------------------------------------------------------- GPU
def make(cfg, seed=0, weights=None, **opts):
    import crane_b200
    w = weights or N.random_weights(cfg, seed)
    opts.setdefault("max_tokens", 1024)
    opts.setdefault("max_batch", 4)
    m = crane_b200.NifaraxModel(cfg, device=0, **opts)
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
    rows = [m.step_batch([(0, ids[:2], [0, 1])])] + [m.step_batch([(0, [t], [0])]) for t in ids[2:40]]
    assert rel(np.concatenate(rows), want[:40]) < F32_TOL
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
    rows += [m.step_batch([(0, [t], [0])]) for t in ids[3:]]       # long decoding through two page borders, every state carried 167 times
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
    # operands rounded to 8 bits move a router score across its neighbour's here and there, and that row then runs another expert:
    # the bar is on the bulk of the rows, not on the worst one
    err = np.abs(got - want).max(-1) / np.abs(want).max()
    assert np.median(err) < 4e-2 and (err < 8e-2).mean() > 0.8
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
    s2 = m.seq_create()                                         # same slot: windows and states must start from zero, pages still hold b's rows
    assert s2 == s1
    got_c = m.step_batch([(s2, c[:50], []), (0, a[:64], [63])])
    got_c2 = m.step_batch([(s2, c[50:], [49])])
    assert rel(got_c2[0], oracle_logits(FULL, w, c)[-1]) < F32_TOL
    assert rel(got_c[0], oracle_logits(FULL, w, a[:64])[-1]) < F32_TOL
    m.close()


@pytest.mark.gpu
def test_far_rows_page_borders_and_carried_states_with_sharp_scores():
    cfg, w = sharp_model(41)
    m, _ = make(cfg, weights=w, max_tokens=1024, max_batch=2, precision="f32")
    ids = tokens(330, cfg["vocab"], 42)
    want = oracle_logits(cfg, w, ids)
    got = m.step_batch([(0, ids, all_rows(330))])
    assert rel(got, want) < F32_TOL
    # decode over the borders of 32-key tiles and 64-token pages, after a prompt that ends just before / on / after them
    for start in (1, 2, 3, 4, 31, 32, 33, 63, 64, 65, 95, 96, 97, 127, 128, 129, 191, 192, 193, 255, 256, 257):
        m.clear_kv_cache()
        m.step_batch([(0, ids[:start], [])])
        rows = np.concatenate([m.step_batch([(0, [t], [0])]) for t in ids[start:start + 4]])
        assert rel(rows, want[start:start + 4]) < F32_TOL, start
    # the same edges inside portions of a prompt, the second portion as short as two tokens
    for cut in (33, 64, 65, 129, 256):
        m.clear_kv_cache()
        a = m.step_batch([(0, ids[:cut - 1], [cut - 2])])
        b = m.step_batch([(0, ids[cut - 1:cut + 1], all_rows(2))])
        c = m.step_batch([(0, ids[cut + 1:cut + 40], all_rows(39))])
        assert rel(np.concatenate([a, b, c]), want[cut - 2:cut + 40]) < F32_TOL, cut
    m.close()


@pytest.mark.gpu
def test_first_tokens_of_a_sequence():
    m, w = make(FULL, 15, precision="f32")
    ids = tokens(7, FULL["vocab"], 16)
    want = oracle_logits(FULL, w, ids)
    assert rel(m.step_batch([(0, ids[:1], [0])]), want[:1]) < F32_TOL           # a one-token prompt: zeros in every convolution window
    assert rel(m.step_batch([(0, ids[1:2], [0])]), want[1:2]) < F32_TOL
    assert rel(m.step_batch([(0, ids[2:4], [0, 1])]), want[2:4]) < F32_TOL      # a portion shorter than the window
    assert rel(m.step_batch([(0, ids[4:], [0, 1, 2])]), want[4:]) < F32_TOL
    m.close()


@pytest.mark.gpu
def test_long_context_decode():
    cfg = config([layer(latent(scale=0.9), None), layer(gla(tau=30.0)), layer(latent(heads=2, dim=16, vdim=16, q_rank=24, kv_rank=40, scale=0.9), None)],
                 width=128, vocab=150, groups=2, taps=4)
    m, w = make(cfg, 17, precision="f32", max_tokens=2048)
    ids = tokens(1500, cfg["vocab"], 18)
    want = oracle_logits(cfg, w, ids)
    m.step_batch([(0, ids[:1200], [])])
    rows = np.concatenate([m.step_batch([(0, [t], [0])]) for t in ids[1200:]])          # 300 decoded tokens, the context split over blocks
    assert rel(rows, want[1200:]) < F32_TOL
    m.close()


@pytest.mark.gpu
@pytest.mark.parametrize("precision,tol", [("f32", F32_TOL), ("split", SPLIT_TOL)])
def test_long_portions_scan_in_segments(precision, tol):
    # from 512 rows on a portion's recurrence runs as four segments side by side; here on a carried state, beside a short request,
    # with lengths that leave the last segment ragged and one key width that is not a multiple of four
    cfg = config([layer(gla(heads=2, dim=32, vdim=40, tau=50.0, decay_rank=8), None), layer(gla(heads=3, dim=18, vdim=20, tau=20.0, decay_rank=4), moe(ff=24, experts=4, top=1, shared=0))],
                 width=96, vocab=150, groups=2, taps=4)
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
def test_greedy_generation_through_generate_and_the_scheduler():
    from crane_b200.scheduler import BatchScheduler
    m, w = make(FULL, 19, precision="f32", max_tokens=512)

    def oracle_greedy(prompt, n):
        s = N.State(FULL)
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
@pytest.mark.parametrize("att", [latent(heads=4, dim=64, vdim=64, q_rank=96, kv_rank=128, scale=0.12), latent(heads=3, dim=128, vdim=128, q_rank=40, kv_rank=256, scale=0.09),
                                 latent(heads=2, dim=64, vdim=32, q_rank=64, kv_rank=64, scale=0.12)])
def test_wide_latents_and_many_rows_take_the_tensor_core_paths(att):
    # a 64-, 128- or 256-wide latent through the flash kernel (whole prompts with equal key and value widths: keys and values built
    # outright), enough (row, expert) pairs for the per-expert GEMMs
    cfg = config([layer(att, moe(ff=64, experts=4, top=2, shared=96)),
                  layer(gla(heads=2, dim=64, vdim=128, tau=12.0, decay_rank=16), moe(ff=64, experts=4, top=2, shared=0))], width=256, vocab=300, groups=2, taps=4)
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
    """A layer list drawn at random: both mixers in any order, widths that are and are not multiples of 4 and 8, every number of
    taps and norm groups, every shape of expert choice, layers that read another layer's tensors."""
    r = np.random.default_rng(seed)
    pick = lambda *xs: xs[int(r.integers(len(xs)))]
    width = pick(72, 96, 120, 160)
    layers = []
    for i in range(int(r.integers(1, 6))):
        same = [j for j, L in enumerate(layers) if "weights_of" not in L]
        if same and r.random() < 0.25:
            j = pick(*same)
            layers.append(layer({"type": layers[j]["type"], "mixer": layers[j]["mixer"]}, layers[j]["mlp"], weights_of=j))
            continue
        if r.random() < 0.5:
            mx = latent(heads=pick(1, 2, 3, 6), dim=pick(8, 18, 32, 40), vdim=pick(8, 20, 24, 64), q_rank=pick(16, 30, 64), kv_rank=pick(16, 36, 64, 100),
                        scale=float(pick(0.1, 0.3, 0.6)))
        else:
            mx = gla(heads=pick(1, 2, 4), dim=pick(8, 12, 20, 32, 70), vdim=pick(8, 18, 32, 40), tau=float(pick(1.0, 4.0, 16.0, 64.0)), decay_rank=pick(1, 4, 16, 24))
        f = None
        if r.random() < 0.75:
            E = pick(2, 4, 6, 9)
            f = moe(ff=pick(12, 30, 64), experts=E, top=int(r.integers(1, E + 1)), limit=float(pick(0.5, 2.0, 7.0)), shared=pick(0, 20, 64), shared_limit=float(pick(1.0, 3.0)))
        layers.append(layer(mx, f))
    groups = pick(*[g for g in (1, 2, 3, 4, 8) if width % g == 0])
    return config(layers, width=width, vocab=pick(90, 211, 300), taps=pick(1, 2, 3, 4, 6), groups=groups, eps=float(pick(1e-6, 1e-5)), cap=float(pick(5.0, 30.0, 50.0)))


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
    cfg = SINGLE["shared_weights"]
    w = N.random_weights(cfg, 23)
    hdr, blob = {}, b""
    for k, t in w.items():
        bits = N.to_numpy_bf16_bits(t).tobytes()
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
    wa, wb = oracle_logits(cfg, w, a), oracle_logits(cfg, w, b)
    read = lambda n: np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(-1, cfg["vocab"])
    assert rel(read(0), wa[49:50]) < F32_TOL
    assert rel(read(1), np.stack([wb[2], wb[69], wa[50]])) < F32_TOL
    assert not (out / "2.f32").exists()
    assert rel(read(3), wb[69:70]) < F32_TOL                    # request c runs on the slot and pages b gave back
