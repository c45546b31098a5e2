"""A plain, slow statement of the Vegodra decoder on the CPU, one function per mechanism, written from the design's
equations and sharing no code with the engine. Everything is float64 torch on whole sequences (the recurrence token by
token); nothing is paged, batched, cached or fused. The GPU tests compare the engine with these functions.

Notation: T tokens at positions p = 0..T-1 of one sequence, W the model's width, H heads, G key/value heads, D the
query/key size of a head, E its value size, R the latent size, Dr the rotated size of latent attention.

  layer norm        y = (x - mean(x)) / sqrt(mean((x - mean(x))^2) + eps) * weight + bias
  rms               y = x / sqrt(mean(x^2) + eps)   (times a weight where one is named)
  embedding         x = layer_norm(table[token])
  layer             h = layer_norm(x);  x <- x + mixer(h) + ff(h)      (one norm, two readers)
  rotation          the pair (u, v) at position p becomes (u cos a - v sin a, v cos a + u sin a), a = p * base^(-2i/dims);
                    pairs are (i, i + dims/2) ("half") or (2i, 2i + 1) ("interleaved"), i < dims/2; the rest passes
  latent attention  cq = rms(Wdq h) * wq;  q = Wuq cq, per head [D plain | Dr rotated (interleaved)]
                    [c_raw | kr_raw] = Wdkv h;  c = rms(c_raw) * wc;  kr = rotated(kr_raw), one for all heads
                    k_h = Wuk_h c, v_h = Wuv_h c;  score = (q_plain . k_h + q_rot . kr) * scale;  causal softmax
                    out = Wo (concat(heads) * sigmoid(Wg h))
  attention         q, k, v = Wq h, Wk h, Wv h;  q, k rotated ("half") on their first dims, then divided by their rms
                    over D;  score = q . k * scale;  key j seen from i iff j <= i and floor(i / C) == floor(j / C);
                    softmax whose denominator also holds exp(sink_h);  head h times sigmoid(Wg h)_h;  Wo.
                    A layer may take keys and values from an earlier layer instead of projecting its own.
  gated linear      q = Wq h / sqrt(D), k = Wk h, v = Wv h;  alpha = sigmoid(Wa2 (Wa1 h) + b)^(1 / tau)  per key channel
  attention         S <- diag(alpha) S + k v^T;  o = S^T q;  o <- rms(o) * w over E;  out = Wo (concat(o) * silu(Wg h))
  feed-forward      Wdown (gelu_tanh(Wgate h) * (Wup h))
  output            logits = head @ layer_norm(x)
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def layer_norm(x, weight, bias, eps):
    d = x - x.mean(-1, keepdim=True)
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * weight + bias


def rms_div(t, eps):
    return t / torch.sqrt((t * t).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate(t, positions, dims, base, pairing):
    """t [T, ..., D]: the first `dims` of the last axis rotated by each row's position; the rest passes unchanged."""
    out = t.clone()
    half = dims // 2
    for i in range(half):
        a, b = (i, i + half) if pairing == "half" else (2 * i, 2 * i + 1)
        ang = positions.to(F) * (float(base) ** (-2.0 * i / dims))
        shape = (-1,) + (1,) * (t.dim() - 2)
        c, s = torch.cos(ang).view(shape), torch.sin(ang).view(shape)
        u, v = t[..., a], t[..., b]
        out[..., a] = u * c - v * s
        out[..., b] = v * c + u * s
    return out


def softmax_with_sink(scores, seen, sink=None):
    """scores [Tq, Tk], seen a boolean mask of the same shape: each row's softmax over its seen keys; with a sink the
    denominator also holds exp(sink), which has no key and no value."""
    s = scores.masked_fill(~seen, float("-inf"))
    m = s.max(-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, torch.full_like(m, float(sink)))
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + math.exp(float(sink)) * torch.exp(-m)
    return e / den


def causal_mask(Tq, Tk, first_query=0, chunk=None):
    i = torch.arange(first_query, first_query + Tq)[:, None]
    j = torch.arange(Tk)[None, :]
    seen = j <= i
    if chunk:
        seen = seen & (i // chunk == j // chunk)
    return seen


def dense_ff(h, w, pre):
    return (gelu_tanh(h @ w[pre + "gate"].T) * (h @ w[pre + "up"].T)) @ w[pre + "down"].T


def latent_attention(h, w, pre, m, eps, positions=None):
    T = h.shape[0]
    pos = torch.arange(T) if positions is None else positions
    H, D, Dr, E, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = rms_div(h @ w[pre + "dq"].T, eps) * w[pre + "dq.norm"]
    q = (cq @ w[pre + "uq"].T).view(T, H, D + Dr)
    q_plain = q[..., :D]
    q_rot = rotate(q[..., D:], pos, m["rot"]["dims"], m["rot"]["base"], "interleaved")
    ckr = h @ w[pre + "dkv"].T
    c = rms_div(ckr[:, :R], eps) * w[pre + "dkv.norm"]
    kr = rotate(ckr[:, R:], pos, m["rot"]["dims"], m["rot"]["base"], "interleaved")
    k = (c @ w[pre + "uk"].T).view(T, H, D)
    v = (c @ w[pre + "uv"].T).view(T, H, E)
    seen = causal_mask(T, T)
    out = torch.zeros(T, H, E, dtype=h.dtype)
    for hd in range(H):
        s = (q_plain[:, hd] @ k[:, hd].T + q_rot[:, hd] @ kr.T) * m["scale"]
        out[:, hd] = softmax_with_sink(s, seen) @ v[:, hd]
    gate = torch.sigmoid(h @ w[pre + "g"].T)
    return (out.reshape(T, H * E) * gate) @ w[pre + "o"].T


def attention_keys_values(h, w, pre, m, eps, positions=None):
    """What an attention layer keeps per token: keys after rotation and unit norm, and values."""
    T = h.shape[0]
    pos = torch.arange(T) if positions is None else positions
    G, D, E = m["kv_heads"], m["dim"], m["vdim"]
    k = rotate((h @ w[pre + "k"].T).view(T, G, D), pos, m["rot"]["dims"], m["rot"]["base"], "half")
    return rms_div(k, eps), (h @ w[pre + "v"].T).view(T, G, E)


def chunked_sink_attention(h, w, pre, m, eps, k, v, positions=None):
    T = h.shape[0]
    pos = torch.arange(T) if positions is None else positions
    H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_div(rotate((h @ w[pre + "q"].T).view(T, H, D), pos, m["rot"]["dims"], m["rot"]["base"], "half"), eps)
    seen = causal_mask(T, T, 0, (m.get("mask") or {}).get("size"))
    gate = torch.sigmoid(h @ w[pre + "g"].T)        # [T, H]
    out = torch.zeros(T, H, E, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * m["scale"]
        out[:, hd] = (softmax_with_sink(s, seen, w[pre + "sink"][hd]) @ v[:, g]) * gate[:, hd:hd + 1]
    return out.reshape(T, H * E) @ w[pre + "o"].T


def gla_decay(h, w, pre, m):
    z = (h @ w[pre + "a1"].T) @ w[pre + "a2"].T + w[pre + "a2.b"]
    return torch.sigmoid(z) ** (1.0 / m["tau"])


def gated_linear_attention(h, w, pre, m, eps, state=None):
    """state: [H, D, E] carried in (None: zeros); returns (out, state after the last token)."""
    T = h.shape[0]
    H, D, E = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[pre + "q"].T).view(T, H, D) * D ** -0.5
    k = (h @ w[pre + "k"].T).view(T, H, D)
    v = (h @ w[pre + "v"].T).view(T, H, E)
    alpha = gla_decay(h, w, pre, m).view(T, H, D)
    S = torch.zeros(H, D, E, dtype=h.dtype) if state is None else state.clone()
    o = torch.zeros(T, H, E, dtype=h.dtype)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hde,hd->he", S, q[t])
    o = rms_div(o, eps) * w[pre + "norm"]
    gate = torch.nn.functional.silu(h @ w[pre + "g"].T)
    return (o.reshape(T, H * E) * gate) @ w[pre + "o"].T, S


def forward(config, weights, tokens, layers_out=None):
    """Logits [T, vocab] of one whole sequence. `weights`: {name: tensor}, taken to float64. layers_out: a list that
    gets the residual stream after every layer."""
    w = {k: (v.to(F) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    x = layer_norm(w["embed"][torch.as_tensor(tokens, dtype=torch.long)], w["embed.norm"], w["embed.norm.b"], eps)
    kept = {}
    for i, L in enumerate(config["layers"]):
        pre, m = f"l{i}.", L["mixer"]
        h = layer_norm(x, w[pre + "norm1"], w[pre + "norm1.b"], eps)
        if L["type"] == "latent_attention":
            y = latent_attention(h, w, pre + "mix.", m, eps)
        elif L["type"] == "attention":
            src = m.get("kv_from")
            if src is None:
                kept[i] = attention_keys_values(h, w, pre + "mix.", m, eps)
                src = i
            y = chunked_sink_attention(h, w, pre + "mix.", m, eps, *kept[src])
        elif L["type"] == "gla":
            y, _ = gated_linear_attention(h, w, pre + "mix.", m, eps)
        else:
            raise ValueError(L["type"])
        if L.get("mlp") is not None:
            y = y + dense_ff(h, w, pre + "mlp.")
        x = x + y
        if layers_out is not None:
            layers_out.append(x.clone())
    x = layer_norm(x, w["final.norm"], w["final.norm.b"], eps)
    return x @ w["head"].T


class PlainVegodra:
    """The whole model with a memory of the tokens it was given: forward(tokens) appends them to the sequence, computes
    the whole sequence anew and returns the logits of the new tokens. reset() starts another sequence."""

    def __init__(self, config, weights):
        self.config, self.weights, self.tokens = config, weights, []

    def reset(self):
        self.tokens = []

    def forward(self, tokens):
        n = len(self.tokens)
        self.tokens = self.tokens + [int(t) for t in tokens]
        return forward(self.config, self.weights, self.tokens)[n:]
