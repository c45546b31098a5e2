"""The delta-rule mixer: a linear recurrence with one state matrix per head instead of a cache of keys and values.

For each head, with a state S [dim, dim] (key channel by value channel) that starts at zero and is carried from token
to token in 32-bit:

    r, k, v = Wr h, Wk h, Wv h                                  (heads x dim each)
    w = exp(-decay_scale * sigmoid(W2 tanh(W1 h) + w0))         decay per head and key channel (W1, W2 a low-rank pair)
    a = sigmoid(Wa h + ba)                                      removal rate per head and key channel
    u = k / sqrt(sum(k^2) + unit_eps)                           the head's unit key
    S <- diag(w) S - (a * u) (u^T S) + k v^T                    both terms read the old state
    o = S^T r

then o of each head is divided by its root mean square (eps), the heads are concatenated, multiplied by a weight
vector and by sigmoid(Wg h), and projected by Wo. The five projections that read h and W1 are one product whose
32-bit result feeds the recurrence directly; decays, rates, unit keys, the state and the head norm are 32-bit
(csrc/delta_rule.cu). The state lives in the request's state slot (`state_need`), zeroed at admission.

params: hidden_size, heads, dim, eps (of the head norm), decay_scale (default exp(-1/2)), unit_eps (default 1e-6),
decay_rank (None: read from the W1 tensor's shape), and the tensor names r, k, v, g, a, a_bias, w1, w2, w0, norm, o
(`<key>_name`, relative to the prefix). With `out_scale=` the output projection's result is multiplied by that vector
before it is added into the residual stream.
"""
from __future__ import annotations

import math

import torch

from ..kernels import ops
from ..weights import ParamSpec
from . import planes
from .registry import Mixer, register_part, to_compute

_DEFAULT_NAMES = dict(r="mix.r", k="mix.k", v="mix.v", g="mix.g", a="mix.a", a_bias="mix.a.b", w1="mix.w1", w2="mix.w2",
                      w0="mix.w0", norm="mix.norm", o="mix.o")


class DeltaRuleMixer(Mixer):
    takes_out_scale = True

    def __init__(self, params, ctx, prefix=""):
        super().__init__(params, ctx, prefix)
        p = params
        self.hidden, self.heads, self.dim = int(p["hidden_size"]), int(p["heads"]), int(p["dim"])
        self.eps = float(p["eps"])
        self.decay_scale = float(p.get("decay_scale", math.exp(-0.5)))
        self.unit_eps = float(p.get("unit_eps", 1e-6))
        self.rank = p.get("decay_rank")
        self.names = {k: prefix + p.get(k + "_name", d) for k, d in _DEFAULT_NAMES.items()}
        self.w_in = self.w2 = self.wo = None

    def param_specs(self):
        HD, W, n = self.heads * self.dim, self.hidden, self.names
        rank = int(self.rank) if self.rank else max(8, self.dim // 4)
        free = () if self.rank else (0,)
        return ([ParamSpec(n[k], (HD, W)) for k in ("r", "k", "v", "g", "a")]
                + [ParamSpec(n["a_bias"], (HD,), init="zeros"), ParamSpec(n["w1"], (rank, W), free=free),
                   ParamSpec(n["w2"], (HD, rank), free=(() if self.rank else (1,))), ParamSpec(n["w0"], (HD,), init="zeros"),
                   ParamSpec(n["norm"], (HD,), init="ones"), ParamSpec(n["o"], (W, HD))])

    def load(self, tensors):
        t = {k: to_compute(tensors[n], self.ctx) for k, n in self.names.items()}
        self.rank = int(t["w1"].shape[0])
        if t["w2"].shape[1] != self.rank:
            raise ValueError(f"{self.names['w2']}: {t['w2'].shape[1]} columns do not fit the {self.rank} rows of {self.names['w1']}")
        mats = [t[k] for k in ("r", "k", "v", "a", "g", "w1")]
        dt = mats[0].dtype if all(m.dtype == mats[0].dtype for m in mats) else torch.float32
        self.w_in = ops.Weight(torch.cat([m.to(dt) for m in mats], 0).contiguous())     # rows [r | k | v | a | g | w1]
        self.w2, self.wo = ops.Weight(t["w2"]), ops.Weight(t["o"])
        vec_dt = t["norm"].dtype
        self.w0, self.a_bias, self.norm_w = t["w0"].to(vec_dt), t["a_bias"].to(vec_dt), t["norm"]

    def weight_bytes(self):
        return self.w_in.nbytes + self.w2.nbytes + self.wo.nbytes

    def state_need(self):
        return {"S": ((self.heads, self.dim, self.dim), torch.float32)}

    def forward(self, xn, x, batch, cache, state, out_scale=None):
        T, HD = xn.shape[0], self.heads * self.dim
        proj = torch.empty(T, 5 * HD + self.rank, dtype=torch.float32, device=xn.device)
        ops.linear(xn, self.w_in, proj)
        mid = torch.empty(T, self.rank, dtype=torch.float32, device=xn.device)
        ops.bias_act(proj[:, 5 * HD:], None, mid, "tanh")
        w_raw = torch.empty(T, HD, dtype=torch.float32, device=xn.device)
        ops.linear(mid, self.w2, w_raw)          # rank is small: 32-bit rows of tanh, the plain product
        y = torch.empty(T, HD, dtype=self.ctx.dtype, device=xn.device)
        ops.delta_rule(proj, (0, HD, 2 * HD, 3 * HD, 4 * HD), w_raw, self.w0, self.a_bias, self.norm_w, state["S"], batch, y,
                       self.heads, self.dim, self.decay_scale, self.unit_eps, self.eps)
        planes.record(batch, "attention", y)
        if out_scale is None:
            ops.linear(y, self.wo, x, accumulate=True)
        else:
            ops.linear_scaled_add(y, self.wo, x, out_scale)
        return None


register_part("mixer", "delta_rule", DeltaRuleMixer)
