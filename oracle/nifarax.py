"""CPU oracle for the Nifarax decoder -- TEST INFRASTRUCTURE ONLY (plain, slow, one function per mechanism).

Nifarax is a decoder-only model whose layer list comes from config.json.  The stream starts as the normalised embedding;
every layer runs two sublayers one after the other, `x += gate1 * mixer(in1)` and then `x += gate2 * ff(in2)`, where for
sublayer s with h = norm_s(x):

  in_s   = h + conv_s(h)                    a short causal depthwise convolution over time (taps from the configuration)
  gate_s = sigmoid(R_s h + b_s)             one gate per channel, from the norm's output before the convolution

Notation (weights W are [out, in], applied as W x):
  group_norm(x, w)  : x cut into `groups` equal consecutive parts, each part / sqrt(mean(part^2) + eps), the whole times w
  rms(x, w)         = x / sqrt(mean(x^2) + eps) * w
  conv(h)_t         = sum_j w[:, j] * h_(t - taps + 1 + j),  zeros before the sequence starts
  gla               : q = W_q u / sqrt(dim), k = W_k u, v = W_v u, a = sigmoid(W_a2 W_a1 u + b)^(1/tau)  (per head and key channel)
                      S_t = diag(a_t) S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t;  out = W_o (rms_per_head(o) * silu(W_g u))
  latent attention  : cq = rms(W_dq u), q = W_uq cq;  c = rms(W_dkv u) (the only thing kept per token);
                      k_j = W_uk c_j, v_j = W_uv c_j;  causal softmax of scale * q_i . k_j;  out = W_o [heads]
  expert(u)         : g = min(W_gate u, L), p = clamp(W_up u, -L, L);  W_down (g * sigmoid(1.702 g) * (p + 1))
  moe(u)            : s = sigmoid(W_r u); the `top` largest s choose the experts; sum_e expert_e(s_e * u)
                      + sigmoid(w_sg . u) * shared_expert(u)
  head              : cap * tanh((E group_norm(x, w_final)) / cap) with E the embedding table

A layer entry with "weights_of": j reads layer j's tensors and keeps a state of its own.  Everything runs in the dtype of the
weights handed in (float64 in the tests), whole prompts or token by token; `State` makes the two forms comparable.
"""
from __future__ import annotations

import math

import numpy as np
import torch


# ---------------------------------------------------------------------------------------------- mechanisms
def group_norm(x, w, groups, eps):
    """x [S, W]: every one of `groups` equal consecutive parts is divided by its own root mean square."""
    S, W = x.shape
    parts = x.reshape(S, groups, W // groups)
    parts = parts / torch.sqrt(parts.pow(2).mean(-1, keepdim=True) + eps)
    return parts.reshape(S, W) * w


def rms(x, w, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def causal_conv(h, w, before):
    """h [S, C] the new inputs, before [taps - 1, C] the inputs ahead of them (zeros at a sequence's start), w [C, taps].
    -> (conv(h) [S, C], the last taps - 1 inputs)."""
    taps = w.shape[1]
    full = torch.cat([before, h], 0)                                        # row i of h is row i + taps - 1 of full
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(taps):
            out[t] += w[:, j] * full[t + j]
    return out, full[full.shape[0] - (taps - 1):].clone()


def gla_decay(u, w_a1, w_a2, b, tau):
    """-> a [S, channels] in (0, 1): sigmoid(z)^(1/tau) as exp(log_sigmoid(z) / tau)."""
    z = (u @ w_a1.T) @ w_a2.T + b
    return torch.exp(torch.nn.functional.logsigmoid(z) / tau)


def gla_scan(q, k, v, a, S0):
    """q, k, a [S, H, d], v [S, H, dv], S0 [H, d, dv] -> (o [S, H, dv], the state after the last token)."""
    S = S0.clone()
    o = torch.zeros(q.shape[0], q.shape[1], v.shape[-1], dtype=q.dtype)
    for t in range(q.shape[0]):
        S = a[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return o, S


def silu(z):
    return z * torch.sigmoid(z)


def causal_attention(q, k, v, q_pos, scale):
    """q [S, H, d] at positions q_pos; k [T, H, d], v [T, H, dv] the rows of positions 0 .. T-1; row i sees j <= i."""
    S, H, _ = q.shape
    T = k.shape[0]
    hidden = torch.arange(T)[None, :] > q_pos[:, None]
    out = torch.zeros(S, H, v.shape[-1], dtype=q.dtype)
    for h in range(H):
        s = (q[:, h, :] @ k[:, h, :].T) * scale
        s = s.masked_fill(hidden, float("-inf"))
        out[:, h, :] = torch.softmax(s, -1) @ v[:, h, :]
    return out


def expert(u, w_gate, w_up, w_down, limit):
    g = torch.clamp(u @ w_gate.T, max=limit)
    p = torch.clamp(u @ w_up.T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (p + 1.0)) @ w_down.T


def route(u, w_router, top):
    """-> (indices [S, top], weights [S, top]): the largest sigmoid scores and those scores themselves."""
    s = torch.sigmoid(u @ w_router.T)
    idx = torch.topk(s, top, dim=-1).indices
    return idx, torch.gather(s, 1, idx)


def moe(u, p, pre, cfg):
    """The chosen experts read the input times their score; the shared expert's output is scaled by one sigmoid per token."""
    idx, wts = route(u, p[pre + "router"], cfg["router"]["top"])
    L = cfg["expert"]["limit"]
    out = torch.zeros(u.shape[0], p[pre + "e0.down"].shape[0], dtype=u.dtype)
    for t in range(u.shape[0]):
        for kk in range(idx.shape[1]):
            e = int(idx[t, kk])
            out[t] += expert(wts[t, kk] * u[t:t + 1], p[f"{pre}e{e}.gate"], p[f"{pre}e{e}.up"], p[f"{pre}e{e}.down"], L)[0]
    sh = cfg.get("shared")
    if sh:
        y = expert(u, p[pre + "shared.gate"], p[pre + "shared.up"], p[pre + "shared.down"], sh["limit"])
        out = out + torch.sigmoid(u @ p[pre + "shared.sg"].T) * y
    return out


def softcap(z, cap):
    return cap * torch.tanh(z / cap)


# ---------------------------------------------------------------------------------------------- the model
def weight_layer(config, i):
    """The layer whose tensors layer i reads."""
    while config["layers"][i].get("weights_of") is not None:
        i = int(config["layers"][i]["weights_of"])
    return i


class State:
    """What a sequence carries: per layer the two convolution windows, the latent rows (latent attention) or the
    recurrent matrix (gla)."""

    def __init__(self, config, dtype=torch.float64):
        W, taps = config["width"], config["canon"]["taps"]
        n = len(config["layers"])
        self.win = [[torch.zeros(taps - 1, W, dtype=dtype) for _ in range(2)] for _ in range(n)]
        self.latent = [None] * n
        self.S = [None] * n
        self.len = 0


def gla_mixer(u, p, pre, mc, eps, state, li):
    H, d, dv = mc["heads"], mc["dim"], mc["vdim"]
    S = u.shape[0]
    q = (u @ p[pre + "q"].T).reshape(S, H, d) * d ** -0.5
    k = (u @ p[pre + "k"].T).reshape(S, H, d)
    v = (u @ p[pre + "v"].T).reshape(S, H, dv)
    a = gla_decay(u, p[pre + "a1"], p[pre + "a2"], p[pre + "a2.b"], mc["tau"]).reshape(S, H, d)
    S0 = state.S[li] if state.S[li] is not None else torch.zeros(H, d, dv, dtype=u.dtype)
    o, state.S[li] = gla_scan(q, k, v, a, S0)
    o = rms(o, p[pre + "norm"], eps).reshape(S, H * dv)
    return (o * silu(u @ p[pre + "g"].T)) @ p[pre + "o"].T


def latent_mixer(u, pos, p, pre, mc, eps, state, li):
    H, d, dv = mc["heads"], mc["dim"], mc["vdim"]
    S = u.shape[0]
    cq = rms(u @ p[pre + "dq"].T, p[pre + "dq.norm"], eps)
    q = (cq @ p[pre + "uq"].T).reshape(S, H, d)
    c = rms(u @ p[pre + "dkv"].T, p[pre + "dkv.norm"], eps)
    if state.latent[li] is not None:
        c = torch.cat([state.latent[li], c], 0)
    state.latent[li] = c
    k = (c @ p[pre + "uk"].T).reshape(-1, H, d)
    v = (c @ p[pre + "uv"].T).reshape(-1, H, dv)
    o = causal_attention(q, k, v, pos, mc["scale"]).reshape(S, H * dv)
    return o @ p[pre + "o"].T


def sublayer_input(x, p, pre, which, config, state, li):
    """-> (what the sublayer reads, its output gate)."""
    h = group_norm(x, p[f"{pre}norm{which}"], config["norm"]["groups"], config["norm"]["eps"])
    cv, state.win[li][which - 1] = causal_conv(h, p[f"{pre}canon{which}"], state.win[li][which - 1])
    gate = torch.sigmoid(h @ p[f"{pre}rg{which}"].T + p[f"{pre}rg{which}.b"])
    return h + cv, gate


def forward(config, p, tokens, state=None, trace=None):
    """tokens: the next tokens of one sequence -> logits [S, vocab].  `p`: name -> tensor.  `trace`, a list, receives the
    stream after every layer."""
    state = state or State(config, p["embed"].dtype)
    eps, groups = config["norm"]["eps"], config["norm"]["groups"]
    ids = torch.as_tensor(tokens, dtype=torch.long)
    pos = torch.arange(state.len, state.len + ids.numel())
    x = group_norm(p["embed"][ids], p["embed.norm"], groups, eps)
    for li, lc in enumerate(config["layers"]):
        pre = f"l{weight_layer(config, li)}."
        u, gate = sublayer_input(x, p, pre, 1, config, state, li)
        if lc["type"] == "gla":
            y = gla_mixer(u, p, pre + "mix.", lc["mixer"], eps, state, li)
        elif lc["type"] == "latent_attention":
            y = latent_mixer(u, pos, p, pre + "mix.", lc["mixer"], eps, state, li)
        else:
            raise ValueError(lc["type"])
        x = x + gate * y
        if lc.get("mlp"):
            u, gate = sublayer_input(x, p, pre, 2, config, state, li)
            x = x + gate * moe(u, p, pre + "mlp.", lc["mlp"])
        if trace is not None:
            trace.append(x.clone())
    state.len += ids.numel()
    z = group_norm(x, p["final.norm"], groups, eps) @ p["embed"].T
    return softcap(z, config["logit_softcap"])


# ---------------------------------------------------------------------------------------------- random models for tests
def tensor_shapes(config):
    W, V, taps = config["width"], config["vocab"], config["canon"]["taps"]
    out = {"embed": (V, W), "embed.norm": (W,), "final.norm": (W,)}
    for i, lc in enumerate(config["layers"]):
        if lc.get("weights_of") is not None:
            continue
        m, pre = lc["mixer"], f"l{i}."
        out.update({pre + "norm1": (W,), pre + "canon1": (W, taps), pre + "rg1": (W, W), pre + "rg1.b": (W,)})
        H, d, dv = m["heads"], m["dim"], m["vdim"]
        if lc["type"] == "gla":
            ar = m["decay_rank"]
            out.update({pre + "mix.q": (H * d, W), pre + "mix.k": (H * d, W), pre + "mix.v": (H * dv, W), pre + "mix.g": (H * dv, W),
                        pre + "mix.o": (W, H * dv), pre + "mix.norm": (dv,), pre + "mix.a1": (ar, W), pre + "mix.a2": (H * d, ar),
                        pre + "mix.a2.b": (H * d,)})
        else:
            qr, kr = m["q_rank"], m["kv_rank"]
            out.update({pre + "mix.dq": (qr, W), pre + "mix.dq.norm": (qr,), pre + "mix.uq": (H * d, qr), pre + "mix.dkv": (kr, W),
                        pre + "mix.dkv.norm": (kr,), pre + "mix.uk": (H * d, kr), pre + "mix.uv": (H * dv, kr), pre + "mix.o": (W, H * dv)})
        f = lc.get("mlp")
        if f:
            F, E = f["expert"]["ff"], f["router"]["experts"]
            out.update({pre + "norm2": (W,), pre + "canon2": (W, taps), pre + "rg2": (W, W), pre + "rg2.b": (W,), pre + "mlp.router": (E, W)})
            for e in range(E):
                out.update({f"{pre}mlp.e{e}.gate": (F, W), f"{pre}mlp.e{e}.up": (F, W), f"{pre}mlp.e{e}.down": (W, F)})
            if f.get("shared"):
                Fs = f["shared"]["ff"]
                out.update({pre + "mlp.shared.gate": (Fs, W), pre + "mlp.shared.up": (Fs, W), pre + "mlp.shared.down": (W, Fs),
                            pre + "mlp.shared.sg": (1, W)})
    return out


def random_weights(config, seed=0):
    """bf16-representable float64 tensors; norms around one, projections ~ 1/sqrt(in), decay biases so that the decays spread
    over (0, 1), convolution taps and gate biases of order one."""
    g = torch.Generator().manual_seed(seed)
    p = {}
    for name, shape in tensor_shapes(config).items():
        last = name.rsplit(".", 1)[-1]
        if name == "embed":
            t = torch.randn(shape, generator=g)
        elif last in ("norm1", "norm2", "norm") or name in ("final.norm", "embed.norm"):
            t = 1.0 + torch.randn(shape, generator=g) * 0.1
        elif last in ("canon1", "canon2"):
            t = torch.randn(shape, generator=g) * 0.3
        elif name.endswith("a2.b"):
            t = 2.0 + torch.randn(shape, generator=g) * 2.0
        elif last == "b":
            t = torch.randn(shape, generator=g) * 0.5
        elif last in ("router", "sg"):
            t = torch.randn(shape, generator=g) * (2.0 / math.sqrt(shape[-1]))
        elif last in ("gate", "up"):
            t = torch.randn(shape, generator=g) * (1.5 / math.sqrt(shape[-1]))
        else:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[-1])
        p[name] = t.to(torch.bfloat16).to(torch.float64)
    return p


def to_numpy_bf16_bits(t):
    return t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
