"""A plain, slow statement of the Torirax decoder on the CPU, one function per mechanism, written from the
design's equations and sharing no code with the engine. Everything is float64 torch on whole sequences (or token
by token where a function says so); nothing is paged, batched, cached or fused. The GPU tests compare the engine
with these functions.

Notation: T tokens, W the model's width, H query heads, G key/value heads, D the query/key size of a head,
E the value size of a head, P positions p = 0..T-1 of one sequence.

  embedding        x[p] = s * table[token[p]] + position_table[p]
  layer norm       y = (x - mean(x)) / sqrt(mean((x - mean(x))^2) + eps) * weight          (no bias)
  layer            x += ls1 * mixer(norm1(x));   x += ls2 * ff(norm2(x))   (the second only where there is a ff)
  delta mixer      per head, with state S [D, D] starting at 0:
                     u = k / sqrt(sum(k^2) + 1e-6)
                     S' = diag(w) S - (a * u) (u^T S) + k v^T,   o = S'^T r
                     w = exp(-exp(-1/2) * sigmoid(W2 tanh(W1 h) + w0)),   a = sigmoid(Wa h + ba)
                   o of a head / rms(o) (eps), all heads * weight * sigmoid(Wg h), then Wo
  differential     two softmax maps over the same values: a1 - lambda * a2, lambda = exp(lq1.lk1) - exp(lq2.lk2) + c,
  attention        then / rms over the head's E values (no weight), * (1 - c), * sigmoid(Wg h), then Wo.
                   Key j is visible from position i iff j <= i and (i - j < window or j < keep_first).
  PolyNorm ff      z = Wup h;  act = a N(z) + b N(z^2) + c N(z^3) + e,  N(t) = t / rms(t) over the ff values;  Wdown act
  output           logits = head @ layer_norm(x)
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def rms_div(t, eps):
    """t divided by its root mean square over the last axis, eps inside the root."""
    return t / torch.sqrt((t * t).mean(-1, keepdim=True) + eps)


def layer_norm(x, weight, eps):
    d = x - x.mean(-1, keepdim=True)
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * weight


def embed(tokens, table, position_table, scale, first_position=0):
    p = torch.arange(first_position, first_position + len(tokens))
    return table[torch.as_tensor(tokens, dtype=torch.long)] * scale + position_table[p]


def visible(i, j, window, keep_first):
    """Whether the query at position i sees the key at position j."""
    return j <= i and (window is None or i - j < window or j < keep_first)


def softmax_over_visible(scores, window, keep_first, first_query=0):
    """scores [Tq, Tk] (query rows at positions first_query.., keys at 0..): plain softmax over each row's visible keys."""
    Tq, Tk = scores.shape
    i = torch.arange(first_query, first_query + Tq)[:, None]
    j = torch.arange(Tk)[None, :]
    seen = j <= i
    if window is not None:
        seen = seen & ((i - j < window) | (j < keep_first))
    return torch.softmax(scores.masked_fill(~seen, float("-inf")), -1)


def differential_lambda(lq1, lk1, lq2, lk2, c):
    return math.exp(float((lq1 * lk1).sum())) - math.exp(float((lq2 * lk2).sum())) + c


def differential_attention(q, k, v, H, G, D, E, scale, window, keep_first, lam, c, eps, first_query=0):
    """q [Tq, H*2*D], k [Tk, G*2*D], v [Tk, G*E] (a head's rows are [map 1, map 2]); returns [Tq, H*E] before the gate."""
    Tq, Tk = q.shape[0], k.shape[0]
    q, k, v = q.view(Tq, H, 2, D), k.view(Tk, G, 2, D), v.view(Tk, G, E)
    out = torch.zeros(Tq, H, E, dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        maps = []
        for m in range(2):
            s = (q[:, h, m] @ k[:, g, m].T) * scale
            maps.append(softmax_over_visible(s, window, keep_first, first_query) @ v[:, g])
        o = maps[0] - lam * maps[1]
        out[:, h] = rms_div(o, eps) * (1.0 - c)
    return out.reshape(Tq, H * E)


def attention_mixer(h, p, prefix, m, eps, kv=None, first_query=0):
    """h [T, W] (normed rows at positions first_query..). kv: (k, v) of all positions so far, for a layer that has
    no key/value projections of its own or for rows that continue a sequence. Returns (output [T, W], (k, v))."""
    w = lambda n: p[prefix + "mix." + n].to(F)
    H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = h @ w("q").T + w("q.b")
    if kv is None:
        kv = (h @ w("k").T + w("k.b"), h @ w("v").T + w("v.b"))
    mask = m.get("mask") or {}
    lam = differential_lambda(w("lq1"), w("lk1"), w("lq2"), w("lk2"), m["diff"])
    o = differential_attention(q, kv[0], kv[1], H, G, D, E, m["scale"], mask.get("size"), mask.get("keep_first", 0), lam,
                               m["diff"], eps, first_query)
    o = o * torch.sigmoid(h @ w("g").T)
    return o @ w("o").T, kv


def delta_decay(h, w1, w2, w0):
    return torch.exp(-math.exp(-0.5) * torch.sigmoid(torch.tanh(h @ w1.T) @ w2.T + w0))


def delta_rule_step(S, r, k, v, w, a):
    """One token of one head. S [D, D] (key channel, value channel); r, k, v, w, a [D]. Returns (S', o)."""
    u = k / torch.sqrt((k * k).sum() + 1e-6)
    S = w[:, None] * S - (a * u)[:, None] * (u @ S)[None, :] + k[:, None] * v[None, :]
    return S, S.T @ r


def delta_mixer(h, p, prefix, m, eps, state=None):
    """h [T, W]; state [heads, D, D] or None (zero). Returns (output [T, W], state after the last token)."""
    w = lambda n: p[prefix + "mix." + n].to(F)
    Hh, D = m["heads"], m["dim"]
    T = h.shape[0]
    r, k, v = [(h @ w(n).T).view(T, Hh, D) for n in ("r", "k", "v")]
    dec = delta_decay(h, w("w1"), w("w2"), w("w0")).view(T, Hh, D)
    a = torch.sigmoid(h @ w("a").T + w("a.b")).view(T, Hh, D)
    S = torch.zeros(Hh, D, D, dtype=F) if state is None else state.clone()
    o = torch.zeros(T, Hh, D, dtype=F)
    for t in range(T):
        for hd in range(Hh):
            S[hd], o[t, hd] = delta_rule_step(S[hd], r[t, hd], k[t, hd], v[t, hd], dec[t, hd], a[t, hd])
    o = rms_div(o, eps).reshape(T, Hh * D) * w("norm") * torch.sigmoid(h @ w("g").T)
    return o @ w("o").T, S


def polynorm(z, coef, eps):
    a, b, c, e = (float(t) for t in coef)
    return a * rms_div(z, eps) + b * rms_div(z * z, eps) + c * rms_div(z * z * z, eps) + e


def feed_forward(h, p, prefix, eps):
    return polynorm(h @ p[prefix + "mlp.up"].to(F).T, p[prefix + "mlp.act"].to(F), eps) @ p[prefix + "mlp.down"].to(F).T


class PlainTorirax:
    """The whole model over one sequence, fed in any portions: `forward(tokens)` continues where the last call ended.
    `layers_out` (a list) receives the residual stream after every layer of the call."""

    def __init__(self, config: dict, params: dict):
        self.c, self.p = config, {k: v.to(F) if v.is_floating_point() else v for k, v in params.items()}
        self.eps = config["norm"]["eps"]
        self.reset()

    def reset(self):
        self.n = 0
        self.kv = {}        # layer index -> (k, v) of all positions so far
        self.state = {}     # layer index -> delta state

    def forward(self, tokens, layers_out=None):
        c, p, eps = self.c, self.p, self.eps
        x = embed(tokens, p["embed"], p["pos"], c["embedding"]["scale"], self.n)
        for i, layer in enumerate(c["layers"]):
            pre, m = f"l{i}.", layer["mixer"]
            h = layer_norm(x, p[pre + "norm1"], eps)
            if layer["type"] == "general_delta":
                y, self.state[i] = delta_mixer(h, p, pre, m, eps, self.state.get(i))
            elif layer["type"] == "attention":
                src = m.get("kv_from")
                if src is None:
                    k = h @ p[pre + "mix.k"].T + p[pre + "mix.k.b"]
                    v = h @ p[pre + "mix.v"].T + p[pre + "mix.v.b"]
                    if i in self.kv:
                        k, v = torch.cat([self.kv[i][0], k]), torch.cat([self.kv[i][1], v])
                    self.kv[i] = (k, v)
                    src = i
                y, _ = attention_mixer(h, p, pre, m, eps, self.kv[src], self.n)
            else:
                raise ValueError(f"unknown layer type {layer['type']!r}")
            x = x + p[pre + "ls1"] * y
            if layer.get("mlp") is not None:
                if layer["mlp"]["kind"] != "dense":
                    raise ValueError(f"unknown feed-forward kind {layer['mlp']['kind']!r}")
                x = x + p[pre + "ls2"] * feed_forward(layer_norm(x, p[pre + "norm2"], eps), p, pre, eps)
            if layers_out is not None:
                layers_out.append(x.clone())
        self.n += len(tokens)
        return layer_norm(x, p["final.norm"], eps) @ p["head"].T
