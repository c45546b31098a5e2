"""Gated linear attention: a linear recurrence with one state matrix per head and a learned decay per key channel.

For each head, with a state S [dim, vdim] (key channel by value channel) that starts at zero and is carried from token to
token in 32-bit:

    q = Wq h / sqrt(dim),  k = Wk h,  v = Wv h                  (heads x dim, heads x dim, heads x vdim)
    alpha = sigmoid(Wa2 (Wa1 h) + b)^(1 / tau)                  decay per head and key channel (Wa1, Wa2 a low-rank pair)
    S <- diag(alpha) S + k v^T                                  the decay acts on the rows of S (key channels)
    o = S^T q

then o of each head is divided by its root mean square over vdim (eps inside the root) and multiplied by a weight vector
(vdim wide, shared by the heads); the heads are concatenated, multiplied by silu(Wg h) and projected by Wo. The four
projections that read h and Wa1 are one product whose 32-bit result feeds the recurrence directly; the decay (through
its logarithm), the state and the head norm are 32-bit (csrc/gla.cu). The state lives in the request's state slot
(`state_need`), zeroed at admission; there is no cache.

params: hidden_size, heads, dim, vdim, tau, eps, decay_rank (None: read from the Wa1 tensor's shape), and the tensor
names q, k, v, g, o, norm, a1, a2, a2_bias (`<key>_name`, relative to the prefix).
"""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights import ParamSpec
from . import planes
from .registry import Mixer, register_part, to_compute

_DEFAULT_NAMES = dict(q="mix.q", k="mix.k", v="mix.v", g="mix.g", o="mix.o", norm="mix.norm", a1="mix.a1", a2="mix.a2",
                      a2_bias="mix.a2.b")


class GatedLinearAttentionMixer(Mixer):
    def __init__(self, params, ctx, prefix=""):
        super().__init__(params, ctx, prefix)
        p = params
        self.hidden, self.heads, self.dim, self.vdim = int(p["hidden_size"]), int(p["heads"]), int(p["dim"]), int(p["vdim"])
        self.tau, self.eps = float(p["tau"]), float(p["eps"])
        if not self.tau > 0:
            raise ValueError("gated linear attention: tau must be positive")
        self.rank = p.get("decay_rank")
        self.names = {k: prefix + p.get(k + "_name", d) for k, d in _DEFAULT_NAMES.items()}
        self.w_in = self.w_a2 = self.wo = None

    def param_specs(self):
        n, W, HD, HE = self.names, self.hidden, self.heads * self.dim, self.heads * self.vdim
        rank = int(self.rank) if self.rank else 16
        free1, free2 = (() if self.rank else (0,)), (() if self.rank else (1,))
        return [ParamSpec(n["q"], (HD, W)), ParamSpec(n["k"], (HD, W)), ParamSpec(n["v"], (HE, W)), ParamSpec(n["g"], (HE, W)),
                ParamSpec(n["o"], (W, HE)), ParamSpec(n["norm"], (self.vdim,), init="ones"),
                ParamSpec(n["a1"], (rank, W), free=free1), ParamSpec(n["a2"], (HD, rank), free=free2),
                ParamSpec(n["a2_bias"], (HD,), init="zeros")]

    def load(self, tensors):
        t = {k: to_compute(tensors[n], self.ctx) for k, n in self.names.items()}
        self.rank = int(t["a1"].shape[0])
        if t["a2"].shape[1] != self.rank:
            raise ValueError(f"{self.names['a2']}: {t['a2'].shape[1]} columns do not fit the {self.rank} rows of {self.names['a1']}")
        mats = [t[k] for k in ("q", "k", "v", "g", "a1")]
        dt = mats[0].dtype if all(m.dtype == mats[0].dtype for m in mats) else torch.float32
        self.w_in = ops.Weight(torch.cat([m.to(dt) for m in mats], 0).contiguous())     # rows [q | k | v | g | a1]
        self.w_a2, self.wo = ops.Weight(t["a2"]), ops.Weight(t["o"])
        self.norm_w, self.a_bias = t["norm"], t["a2_bias"].to(t["norm"].dtype)

    def weight_bytes(self):
        return self.w_in.nbytes + self.w_a2.nbytes + self.wo.nbytes

    def state_need(self):
        return {"S": ((self.heads, self.dim, self.vdim), torch.float32)}

    def forward(self, xn, x, batch, cache, state):
        T, HD, HE = xn.shape[0], self.heads * self.dim, self.heads * self.vdim
        proj = torch.empty(T, 2 * HD + 2 * HE + self.rank, dtype=torch.float32, device=xn.device)
        ops.linear_rows32(xn, self.w_in, proj)
        z = torch.empty(T, HD, dtype=torch.float32, device=xn.device)
        ops.linear(proj[:, 2 * HD + 2 * HE:], self.w_a2, z)      # the rank is small: 32-bit rows, the plain product
        y = torch.empty(T, HE, dtype=self.ctx.dtype, device=xn.device)
        ops.gla(proj, (0, HD, 2 * HD, 2 * HD + HE), z, self.a_bias, self.norm_w, state["S"], batch, y, self.heads, self.dim,
                self.vdim, self.tau, self.eps)
        planes.record(batch, "attention", y)
        ops.linear_into_stream(y, self.wo, x)
        return None


register_part("mixer", "gla", GatedLinearAttentionMixer)
