"""CPU oracle for the Puzonex decoder -- TEST INFRASTRUCTURE ONLY (plain, slow, one function per mechanism).

Puzonex is a decoder-only model whose layer list comes from config.json.  The stream starts as the embedding row plus a
sinusoidal position vector.  A layer runs a mixer and then (optionally) a feed-forward; neither reads a norm of the stream, both
read the stream itself, and the norm sits on the way back:

  x <- x + rms(mixer(x), w_norm1);   x <- x + rms(ff(x), w_norm2)

Notation (weights W are [out, in], applied as W x):
  rms(y, w)     = y / sqrt(mean(y^2) + eps) * w;      unit(y) = y / sqrt(mean(y^2) + eps)
  cap(s, c)     = c tanh(s / c)   (a configuration without "softcap" has no cap, one without "mask" no window)
  position      : entry 2i = sin(p f_i), entry 2i + 1 = cos(p f_i), f_i = 10000^(-2i / width); p, f_i and p f_i are float32 numbers
  attention     : q = W_q x + b_q, k = W_k x + b_k, v = W_v x + b_v;  q, k under rms per head (one weight vector of size dim shared
                  by the heads), v under unit() per head;  s_ij = cap(scale q_i . k_j) - r1_h ln(1 + r2_h (i - j));  keys with
                  0 <= i - j < window;  softmax whose denominator also holds exp(sink_h);  W_o on the heads
  mamba1        : [u | z] = W_in x;  u <- silu(conv(u) + b_conv);  [dt | B | C] = W_x u;  dt <- softplus(W_dt dt + b_dt);
                  S_t[c, n] = exp(dt_c A[c, n]) S_(t-1)[c, n] + dt_c u_c B_n,  A = -exp(A_log);  y_c = S_t[c, :] . C + D_c u_c;
                  W_o (y silu(z))
  parallel      : out = (rms(left(x), w_left) + rms(right(x), w_right)) / 2
    left        : q = W_q x + b_q, k = W_k x + b_k, the values are k as projected;  q and k under ONE rms over all their heads
                  (weights of the whole projection's size);  s_ij = cap(scale temp_h q_i . k_j) + rel[bucket(i - j), h];  window;
                  plain softmax;  (W_o (heads * sigmoid(W_g x))) + b_o
    right       : matrix memory per head.  q = W_q x / sqrt(dim), k = W_k x, v = W_v x;  i_t = cap(w_i . x + b_i, c),
                  f_t = log sigmoid(cap(w_f . x + b_f, c));  m_t = max(f_t + m_(t-1), i_t) with m_0 = 0;
                  S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(i_t - m_t) k_t v_t^T,  n_t likewise from k_t;
                  o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6);  W_o (unit(o) per head * w_norm * sigmoid(W_g x))
  feed-forward  : W_down (gelu_tanh(W_gate x) * (W_up x))
  head          : W_head rms(x, w_final)

Everything runs in the dtype of the weights handed in (float64 in the tests), whole prompts or token by token; `State` makes the
two forms comparable.
"""
from __future__ import annotations

import math

import numpy as np
import torch


# ---------------------------------------------------------------------------------------------- mechanisms
def rms(y, w, eps):
    return y / torch.sqrt(y.pow(2).mean(-1, keepdim=True) + eps) * w


def unit(y, eps):
    return y / torch.sqrt(y.pow(2).mean(-1, keepdim=True) + eps)


def cap(s, c):
    return c * torch.tanh(s / c)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def position_vector(pos, width, dtype):
    """pos [S] -> [S, width]: sines at the even entries, cosines of the same angles at the odd ones.  Positions, frequencies and
    their product (the angle) are float32 numbers, as the design has them; the sine and cosine of that angle are taken in `dtype`."""
    out = torch.zeros(len(pos), width, dtype=dtype)
    p = np.asarray(pos, dtype=np.float32)
    for c in range(width):
        f = np.float32(10000.0 ** (-(2 * (c // 2)) / width))
        ang = torch.from_numpy((p * f).astype(np.float32)).to(dtype)
        out[:, c] = torch.sin(ang) if c % 2 == 0 else torch.cos(ang)
    return out


def bucket(n, rows, far):
    """Row of a learned distance table for the distance n >= 0: one row per distance up to rows / 2, then logarithmic steps that
    reach the last row at the distance `far`."""
    half = rows // 2
    if n < half or half == 0:
        return min(n, rows - 1)
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def windowed_scores(q, k, q_pos, window, capf, biasf):
    """-> list over rows of (first key, scores [H, keys]).  capf caps a vector of raw scores; biasf(h, dist) gives what head h adds
    at the distances `dist` (a vector of i - j)."""
    S, H, d = q.shape
    G = k.shape[1]
    out = []
    for i in range(S):
        p = int(q_pos[i])
        j0 = max(0, p - window + 1) if window > 0 else 0
        sc = torch.zeros(H, p + 1 - j0, dtype=q.dtype)
        for h in range(H):
            g = h // (H // G)
            dist = p - torch.arange(j0, p + 1)
            sc[h] = capf(k[j0:p + 1, g] @ q[i, h]) + biasf(h, dist)
        out.append((j0, sc))
    return out


def attend(q, k, v, q_pos, window, capf, biasf, sink=None):
    """Softmax attention of rows at positions q_pos over the keys 0 .. pos inside the window.  q [S, H, d] carries every factor
    of the score that comes before the cap; sink [H]: one more term exp(sink_h) in the denominator, without a value."""
    S, H, _ = q.shape
    G, dv = v.shape[1], v.shape[2]
    out = torch.zeros(S, H, dv, dtype=q.dtype)
    for i, (j0, sc) in enumerate(windowed_scores(q, k, q_pos, window, capf, biasf)):
        p = int(q_pos[i])
        for h in range(H):
            g = h // (H // G)
            s = sc[h]
            m = s.max() if sink is None else torch.maximum(s.max(), sink[h])
            e = torch.exp(s - m)
            den = e.sum() if sink is None else e.sum() + torch.exp(sink[h] - m)
            out[i, h] = (e / den) @ v[j0:p + 1, g]
    return out


def causal_conv(u, w, b, before):
    """u [S, C] the new inputs, before [taps - 1, C] the inputs ahead of them (zeros at a sequence's start), w [C, taps] with the
    last column on the current token -> (conv [S, C], the last taps - 1 inputs)."""
    taps = w.shape[1]
    full = torch.cat([before, u], 0)
    out = torch.zeros_like(u)
    for t in range(u.shape[0]):
        out[t] = b
        for j in range(taps):
            out[t] = out[t] + w[:, j] * full[t + j]
    return out, full[full.shape[0] - (taps - 1):].clone()


def selective_scan(u, dt, A, B, C, D, S0):
    """u, dt [S, inner]; A [inner, N]; B, C [S, N]; D [inner]; S0 [inner, N] -> (y [S, inner], S_end)."""
    S = S0.clone()
    y = torch.zeros_like(u)
    for t in range(u.shape[0]):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * u[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + D * u[t]
    return y, S


def matrix_memory(q, k, v, ig, fg, S0, n0, m0):
    """One head.  q, k [S, d]; v [S, dv]; ig, fg [S] the log input / log forget gates; S0 [d, dv], n0 [d], m0 scalar
    -> (o [S, dv], S, n, m)."""
    S, n, m = S0.clone(), n0.clone(), m0.clone()
    o = torch.zeros(q.shape[0], v.shape[1], dtype=q.dtype)
    for t in range(q.shape[0]):
        m_new = torch.maximum(fg[t] + m, ig[t])
        a, b = torch.exp(fg[t] + m - m_new), torch.exp(ig[t] - m_new)
        S = a * S + b * torch.outer(k[t], v[t])
        n = a * n + b * k[t]
        m = m_new
        o[t] = (S.T @ q[t]) / (torch.maximum(torch.abs(n @ q[t]), torch.exp(-m)) + 1e-6)
    return o, S, n, m


def feed_forward(x, w_gate, w_up, w_down):
    return (gelu_tanh(x @ w_gate.T) * (x @ w_up.T)) @ w_down.T


# ---------------------------------------------------------------------------------------------- the model
class State:
    """What a sequence carries: per layer the keys and values (attention), the convolution window and the scan's state
    (mamba1), or both mixers' parts (parallel)."""

    def __init__(self, config, dtype=torch.float64):
        n = len(config["layers"])
        self.k = [None] * n
        self.v = [None] * n
        self.win = [None] * n
        self.S = [None] * n
        self.mem = [None] * n
        self.len = 0


def _grow(old, new):
    return new if old is None else torch.cat([old, new], 0)


def attention_mixer(x, pos, p, pre, mc, eps, state, li):
    H, G, d, dv = mc["heads"], mc["kv_heads"], mc["dim"], mc["vdim"]
    S = x.shape[0]
    q = (x @ p[pre + "q"].T + p[pre + "q.b"]).reshape(S, H, d)
    k = (x @ p[pre + "k"].T + p[pre + "k.b"]).reshape(S, G, d)
    v = (x @ p[pre + "v"].T + p[pre + "v.b"]).reshape(S, G, dv)
    q, k, v = rms(q, p[pre + "q.norm"], eps), rms(k, p[pre + "k.norm"], eps), unit(v, eps)
    state.k[li], state.v[li] = _grow(state.k[li], k), _grow(state.v[li], v)
    r1, r2, c = p[pre + "r1"], p[pre + "r2"], mc.get("softcap")
    window = mc["mask"]["size"] if mc.get("mask") else 0
    o = attend(q * mc["scale"], state.k[li], state.v[li], pos, window, (lambda s: cap(s, c)) if c else (lambda s: s),
               lambda h, dist: -r1[h] * torch.log(1.0 + r2[h] * dist), p[pre + "sink"])
    return o.reshape(S, H * dv) @ p[pre + "o"].T


def mamba1_mixer(x, p, pre, mc, state, li):
    inner, N, R = mc["inner"], mc["state"], mc["dt_rank"]
    uz = x @ p[pre + "in"].T
    u, z = uz[:, :inner], uz[:, inner:]
    if state.win[li] is None:
        state.win[li] = torch.zeros(mc["conv"] - 1, inner, dtype=x.dtype)
        state.S[li] = torch.zeros(inner, N, dtype=x.dtype)
    cv, state.win[li] = causal_conv(u, p[pre + "conv"], p[pre + "conv.b"], state.win[li])
    u = silu(cv)
    low = u @ p[pre + "x"].T
    dt = torch.nn.functional.softplus(low[:, :R] @ p[pre + "dt"].T + p[pre + "dt.b"], threshold=1e9)
    y, state.S[li] = selective_scan(u, dt, -torch.exp(p[pre + "A_log"]), low[:, R:R + N], low[:, R + N:R + 2 * N], p[pre + "D"], state.S[li])
    return (y * silu(z)) @ p[pre + "o"].T


def left_mixer(x, pos, p, pre, mc, eps, state, li):
    H, G, d = mc["heads"], mc["kv_heads"], mc["dim"]
    S = x.shape[0]
    q = x @ p[pre + "q"].T + p[pre + "q.b"]
    k = x @ p[pre + "k"].T + p[pre + "k.b"]
    v = k.reshape(S, G, d)
    q, k = rms(q, p[pre + "q.norm"], eps).reshape(S, H, d), rms(k, p[pre + "k.norm"], eps).reshape(S, G, d)
    state.k[li], state.v[li] = _grow(state.k[li], k), _grow(state.v[li], v)
    table, c = p[pre + "rel"], mc.get("softcap")
    window = mc["mask"]["size"] if mc.get("mask") else 0
    rows = torch.tensor([bucket(n, table.shape[0], mc["bias_max"]) for n in range(int(pos[-1]) + 1)])
    o = attend(q * mc["scale"] * p[pre + "temp"][None, :, None], state.k[li], state.v[li], pos, window, (lambda s: cap(s, c)) if c else (lambda s: s),
               lambda h, dist: table[rows[dist], h])
    o = o.reshape(S, H * d) * torch.sigmoid(x @ p[pre + "g"].T)
    return o @ p[pre + "o"].T + p[pre + "o.b"]


def right_mixer(x, p, pre, mc, eps, state, li):
    H, d, dv, c = mc["heads"], mc["dim"], mc["vdim"], mc["gate_cap"]
    S = x.shape[0]
    q = (x @ p[pre + "q"].T).reshape(S, H, d) * d ** -0.5
    k = (x @ p[pre + "k"].T).reshape(S, H, d)
    v = (x @ p[pre + "v"].T).reshape(S, H, dv)
    ig = cap(x @ p[pre + "i"].T + p[pre + "i.b"], c)
    fg = torch.nn.functional.logsigmoid(cap(x @ p[pre + "f"].T + p[pre + "f.b"], c))
    if state.mem[li] is None:
        state.mem[li] = [(torch.zeros(d, dv, dtype=x.dtype), torch.zeros(d, dtype=x.dtype), torch.zeros((), dtype=x.dtype)) for _ in range(H)]
    o = torch.zeros(S, H, dv, dtype=x.dtype)
    for h in range(H):
        o[:, h], Sm, n, m = matrix_memory(q[:, h], k[:, h], v[:, h], ig[:, h], fg[:, h], *state.mem[li][h])
        state.mem[li][h] = (Sm, n, m)
    o = unit(o, eps).reshape(S, H * dv) * p[pre + "norm"] * torch.sigmoid(x @ p[pre + "g"].T)
    return o @ p[pre + "o"].T


def parallel_mixer(x, pos, p, pre, mc, eps, state, li):
    a = left_mixer(x, pos, p, pre + "left.", mc["left"], eps, state, li)
    b = right_mixer(x, p, pre + "right.", mc["right"], eps, state, li)
    return 0.5 * (rms(a, p[pre + "left.out"], eps) + rms(b, p[pre + "right.out"], eps))


def forward(config, p, tokens, state=None, trace=None):
    """tokens: the next tokens of one sequence -> logits [S, vocab].  `p`: name -> tensor.  `trace`, a list, receives the
    stream after every layer."""
    dtype = p["embed"].dtype
    state = state or State(config, dtype)
    eps = config["norm"]["eps"]
    ids = torch.as_tensor(tokens, dtype=torch.long)
    pos = torch.arange(state.len, state.len + ids.numel())
    x = p["embed"][ids] + position_vector(pos, config["width"], dtype)
    for li, lc in enumerate(config["layers"]):
        pre = f"l{li}."
        if lc["type"] == "attention":
            y = attention_mixer(x, pos, p, pre + "mix.", lc["mixer"], eps, state, li)
        elif lc["type"] == "mamba1":
            y = mamba1_mixer(x, p, pre + "mix.", lc["mixer"], state, li)
        elif lc["type"] == "parallel":
            y = parallel_mixer(x, pos, p, pre + "mix.", lc["mixer"], eps, state, li)
        else:
            raise ValueError(lc["type"])
        x = x + rms(y, p[pre + "norm1"], eps)
        if lc.get("mlp"):
            x = x + rms(feed_forward(x, p[pre + "mlp.gate"], p[pre + "mlp.up"], p[pre + "mlp.down"]), p[pre + "norm2"], eps)
        if trace is not None:
            trace.append(x.clone())
    state.len += ids.numel()
    return rms(x, p["final.norm"], eps) @ p["head"].T


# ---------------------------------------------------------------------------------------------- random models for tests
def tensor_shapes(config):
    W, V = config["width"], config["vocab"]
    out = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    for i, lc in enumerate(config["layers"]):
        m, pre = lc["mixer"], f"l{i}."
        out[pre + "norm1"] = (W,)
        if lc["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out.update({pre + "mix.q": (H * d, W), pre + "mix.q.b": (H * d,), pre + "mix.k": (G * d, W), pre + "mix.k.b": (G * d,),
                        pre + "mix.v": (G * dv, W), pre + "mix.v.b": (G * dv,), pre + "mix.q.norm": (d,), pre + "mix.k.norm": (d,),
                        pre + "mix.r1": (H,), pre + "mix.r2": (H,), pre + "mix.sink": (H,), pre + "mix.o": (W, H * dv)})
        elif lc["type"] == "mamba1":
            I, N, R, taps = m["inner"], m["state"], m["dt_rank"], m["conv"]
            out.update({pre + "mix.in": (2 * I, W), pre + "mix.conv": (I, taps), pre + "mix.conv.b": (I,), pre + "mix.x": (R + 2 * N, I),
                        pre + "mix.dt": (I, R), pre + "mix.dt.b": (I,), pre + "mix.A_log": (I, N), pre + "mix.D": (I,), pre + "mix.o": (W, I)})
        else:
            a, b = m["left"], m["right"]
            H, G, d = a["heads"], a["kv_heads"], a["dim"]
            out.update({pre + "mix.left.q": (H * d, W), pre + "mix.left.q.b": (H * d,), pre + "mix.left.k": (G * d, W), pre + "mix.left.k.b": (G * d,),
                        pre + "mix.left.q.norm": (H * d,), pre + "mix.left.k.norm": (G * d,), pre + "mix.left.rel": (a["rel_rows"], H),
                        pre + "mix.left.temp": (H,), pre + "mix.left.g": (H * d, W), pre + "mix.left.o": (W, H * d), pre + "mix.left.o.b": (W,),
                        pre + "mix.left.out": (W,), pre + "mix.right.out": (W,)})
            H, d, dv = b["heads"], b["dim"], b["vdim"]
            out.update({pre + "mix.right.q": (H * d, W), pre + "mix.right.k": (H * d, W), pre + "mix.right.v": (H * dv, W),
                        pre + "mix.right.g": (H * dv, W), pre + "mix.right.o": (W, H * dv), pre + "mix.right.norm": (H * dv,),
                        pre + "mix.right.i": (H, W), pre + "mix.right.i.b": (H,), pre + "mix.right.f": (H, W), pre + "mix.right.f.b": (H,)})
        if lc.get("mlp"):
            F = lc["mlp"]["ff"]
            out.update({pre + "norm2": (W,), pre + "mlp.gate": (F, W), pre + "mlp.up": (F, W), pre + "mlp.down": (W, F)})
    return out


def random_weights(config, seed=0):
    """bf16-representable float64 tensors: norms around one, projections ~ 1/sqrt(in), positive distance-bias numbers, forget
    gates that keep most of the memory, step sizes and decays spread over a few orders."""
    g = torch.Generator().manual_seed(seed)
    p = {}
    for name, shape in tensor_shapes(config).items():
        last = name.rsplit(".", 1)[-1]
        if name == "embed":
            t = torch.randn(shape, generator=g)
        elif last in ("norm1", "norm2", "norm", "out", "temp"):
            t = 1.0 + torch.randn(shape, generator=g) * 0.1
        elif last in ("r1", "r2"):
            t = 0.1 + torch.rand(shape, generator=g)
        elif last in ("sink", "rel"):
            t = torch.randn(shape, generator=g)
        elif last == "conv":
            t = torch.randn(shape, generator=g) * 0.4
        elif last == "A_log":
            t = torch.log(torch.rand(shape, generator=g) * 3.0 + 0.05)
        elif last == "D":
            t = 1.0 + torch.randn(shape, generator=g) * 0.2
        elif name.endswith("dt.b"):
            t = torch.log(torch.expm1(torch.rand(shape, generator=g) * 0.2 + 0.01))
        elif name.endswith("f.b"):
            t = 3.0 + torch.randn(shape, generator=g)
        elif last == "b":
            t = torch.randn(shape, generator=g) * 0.3
        elif last == "dt":
            t = torch.randn(shape, generator=g) * (0.5 / math.sqrt(shape[-1]))
        else:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[-1])
        p[name] = t.to(torch.bfloat16).to(torch.float64)
    return p


def to_numpy_bf16_bits(t):
    return t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
