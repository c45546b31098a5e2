"""Differential attention over the paged cache, with a sliding window that keeps the first tokens.

A head has TWO score maps: its query is [map 1 (dim) | map 2 (dim)] and so are the keys of its kv head (query head h
reads kv head h // (heads / kv_heads)); both maps are ordinary softmax attention over the same values (vdim wide):

    q, k, v = Wq h + bq, Wk h + bk, Wv h + bv          no position encoding: positions enter through the mask alone
    a_m = softmax(scale * q_m k_m^T over the visible keys) v,   m = 1, 2
    o = a_1 - lambda * a_2,   lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff      (one number for the layer)
    o <- o / sqrt(mean(o^2) + eps) * (1 - diff)        over the head's vdim values, no weight
    out = Wo (concat(o) * sigmoid(Wg h))

Key j is visible from position i iff j <= i and (i - j < window or j < keep_first); no window: every j <= i.
The cache keeps, per token and kv head, a key plane 2 * dim wide and a value plane vdim wide. A mixer with
`reads_cache` has no key/value projections: it attends, with its own queries and mask, over the cache of the layer the
model's run order names. What the cache retains is given apart from the mask (`cache_window`, `cache_keep_first`),
because the layers that share a cache may look back differently far: the model gives all of them the widest.

lambda depends on the weights alone and is computed when they are loaded. Scores, softmax, the combination and the
head norm are 32-bit (csrc/attention_window.cu); q, k, v are rounded once, after their bias.

params: hidden_size, heads, kv_heads, dim, vdim, scale, diff, eps, window (None or 0: none), keep_first, cache_window,
cache_keep_first, reads_cache, and tensor names (`<key>_name`): q, k, v, g, o, q_bias, k_bias, v_bias, lq1, lk1, lq2, lk2.
With `out_scale=` the output projection's result is multiplied by that vector before it is added into the residual stream.
"""
from __future__ import annotations

import math

import torch

from ..kernels import ops
from ..weights import ParamSpec
from . import planes
from .registry import CacheNeed, Mixer, register_part, to_compute

_DEFAULT_NAMES = dict(q="mix.q", k="mix.k", v="mix.v", g="mix.g", o="mix.o", q_bias="mix.q.b", k_bias="mix.k.b",
                      v_bias="mix.v.b", lq1="mix.lq1", lk1="mix.lk1", lq2="mix.lq2", lk2="mix.lk2")


class DifferentialAttentionMixer(Mixer):
    takes_out_scale = True
    MAPS = 2

    def __init__(self, params, ctx, prefix=""):
        super().__init__(params, ctx, prefix)
        p = params
        self.hidden = int(p["hidden_size"])
        self.heads, self.kv_heads, self.dim, self.vdim = int(p["heads"]), int(p["kv_heads"]), int(p["dim"]), int(p["vdim"])
        if self.heads % self.kv_heads:
            raise ValueError(f"differential attention: {self.heads} heads are not a multiple of {self.kv_heads} kv heads")
        self.scale, self.diff, self.eps = float(p["scale"]), float(p["diff"]), float(p["eps"])
        self.window, self.keep_first = int(p.get("window") or 0), int(p.get("keep_first") or 0)
        self.cache_window = int(p["cache_window"] or 0) if "cache_window" in p else self.window
        self.cache_keep_first = int(p.get("cache_keep_first", self.keep_first))
        if self.cache_window and (not self.window or self.window > self.cache_window or self.keep_first > self.cache_keep_first):
            raise ValueError("differential attention: the cache retains less than the mask sees")
        self.reads_cache = bool(p.get("reads_cache", False))
        self.names = {k: prefix + p.get(k + "_name", d) for k, d in _DEFAULT_NAMES.items()}
        self.w_in = self.wo = None
        self.lam = 0.0

    @property
    def n_q(self):
        return self.heads * self.MAPS * self.dim

    @property
    def n_k(self):
        return self.kv_heads * self.MAPS * self.dim

    def param_specs(self):
        n, W = self.names, self.hidden
        specs = [ParamSpec(n["q"], (self.n_q, W)), ParamSpec(n["q_bias"], (self.n_q,), init="zeros")]
        if not self.reads_cache:
            specs += [ParamSpec(n["k"], (self.n_k, W)), ParamSpec(n["k_bias"], (self.n_k,), init="zeros"),
                      ParamSpec(n["v"], (self.kv_heads * self.vdim, W)),
                      ParamSpec(n["v_bias"], (self.kv_heads * self.vdim,), init="zeros")]
        specs += [ParamSpec(n[k], (self.dim,)) for k in ("lq1", "lk1", "lq2", "lk2")]
        specs += [ParamSpec(n["g"], (self.heads * self.vdim, W)), ParamSpec(n["o"], (W, self.heads * self.vdim))]
        return specs

    def load(self, tensors):
        t = {k: to_compute(tensors[n], self.ctx) for k, n in self.names.items() if n in tensors}
        mats = [t["q"]] + ([] if self.reads_cache else [t["k"], t["v"]]) + [t["g"]]
        dt = mats[0].dtype if all(m.dtype == mats[0].dtype for m in mats) else torch.float32
        self.w_in = ops.Weight(torch.cat([m.to(dt) for m in mats], 0).contiguous())     # rows [q | k | v | g] or [q | g]
        self.wo = ops.Weight(t["o"])
        bdt = t["q_bias"].dtype
        self.bq = t["q_bias"]
        self.bk = None if self.reads_cache else t["k_bias"].to(bdt)
        self.bv = None if self.reads_cache else t["v_bias"].to(bdt)
        dot = lambda a, b: float((t[a].double().cpu() * t[b].double().cpu()).sum())
        self.lam = math.exp(dot("lq1", "lk1")) - math.exp(dot("lq2", "lk2")) + self.diff

    def weight_bytes(self):
        return self.w_in.nbytes + self.wo.nbytes

    def cache_need(self):
        planes_ = (("k", self.kv_heads, self.MAPS * self.dim), ("v", self.kv_heads, self.vdim))
        if not self.cache_window:
            return CacheNeed("full", self.kv_heads, self.dim, 0, planes_)
        return CacheNeed("window_keep_first", self.kv_heads, self.dim, self.cache_window, planes_,
                         (("keep_first", self.cache_keep_first),))

    def forward(self, xn, x, batch, cache, state, out_scale=None):
        T = xn.shape[0]
        n_kv = 0 if self.reads_cache else self.n_k + self.kv_heads * self.vdim
        proj = torch.empty(T, self.n_q + n_kv + self.heads * self.vdim, dtype=torch.float32, device=xn.device)
        ops.linear(xn, self.w_in, proj)
        q = torch.empty(T, self.n_q, dtype=self.ctx.dtype, device=xn.device)
        write = cache.write and not self.reads_cache
        ops.qkv_bias_store(proj[:, :self.n_q + n_kv], self.bq, self.bk, self.bv, batch.slot_maps[cache.group] if write else None,
                           q, cache.k, cache.v, self.n_q, self.kv_heads, self.MAPS * self.dim, self.vdim, self.ctx.page_size)
        att = torch.empty(T, self.heads * self.vdim, dtype=self.ctx.dtype, device=xn.device)
        ops.attention_window(q, cache.k, cache.v, batch, cache.group, att, self.heads, self.kv_heads, self.dim, self.vdim,
                             self.MAPS, self.ctx.page_size, self.window, self.keep_first, self.scale, self.lam,
                             1.0 - self.diff, self.eps, True, gate=proj, gate_offset=self.n_q + n_kv)
        planes.record(batch, "q", q)
        planes.record(batch, "attention", att)
        if out_scale is None:
            ops.linear(att, self.wo, x, accumulate=True)
        else:
            ops.linear_scaled_add(att, self.wo, x, out_scale)
        return None


register_part("mixer", "differential_attention", DifferentialAttentionMixer)
