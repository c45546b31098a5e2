"""Small Torirax configurations of the tests' own, with weights drawn so that faults show: matrices of unit gain (the
scores spread, the decays move), layer scales and norm weights away from 1, biases and coefficients away from 0."""
from __future__ import annotations

import json
import math
import os

import torch


def delta(heads, dim, ff=None, rank=None):
    m = dict(heads=heads, dim=dim)
    if rank:
        m["decay_rank"] = rank
    return dict(type="general_delta", mixer=m, mlp=None if ff is None else dict(kind="dense", ff=ff))


def attn(heads, kv_heads, dim, vdim, window=None, keep=0, diff=0.5, kv_from=None, ff=None, scale=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, diff=diff, scale=scale or 1.0 / math.sqrt(dim))
    if window is not None:
        m["mask"] = dict(size=window, keep_first=keep)
    if kv_from is not None:
        m["kv_from"] = kv_from
    return dict(type="attention", mixer=m, mlp=None if ff is None else dict(kind="dense", ff=ff))


def model(vocab, width, layers, max_positions=512, scale=2.0, eps=1e-5):
    return dict(architecture="Torirax", vocab=vocab, width=width, max_positions=max_positions, embedding=dict(scale=scale),
                norm=dict(eps=eps), layers=layers)


# P: delta first, attention with a window and kept first tokens, an attention layer that reads the other's cache with a
#    SHORTER window and no kept tokens; heads of 32; ff on one layer only
P = model(160, 64, [delta(2, 32, rank=8), attn(4, 2, 16, 24, window=24, keep=3, ff=96), delta(2, 32, rank=8),
                    attn(4, 2, 16, 24, window=9, keep=0, kv_from=1, diff=0.3)], max_positions=400)
# Q: attention first; no window at all; every head its own kv head; dim == vdim; delta heads of 48 (no register kernel)
#    with a feed-forward; one kept token with a window of 1
Q = model(97, 48, [attn(3, 3, 8, 8, ff=80), delta(1, 48, ff=56, rank=5), attn(2, 1, 8, 40, window=1, keep=1, diff=0.8)],
          max_positions=300, scale=1.0, eps=1e-6)
# R: wider: delta heads of 64 and of 128, a group of 4, windows that cross pages and the attention kernel's key tiles,
#    a reader with a LONGER window and more kept tokens than the layer that writes the cache
#    (heads of 32 with values of 64: in bfloat16 the attention of portions runs on the tensor-core kernel)
R = model(211, 128, [delta(2, 64), attn(8, 2, 32, 64, window=70, keep=2, ff=192), delta(1, 128, rank=24),
                     attn(8, 2, 32, 64, window=130, keep=5, kv_from=1), attn(4, 4, 16, 16, window=64, keep=64, ff=64)],
          max_positions=700, scale=3.0)

# S: delta heads wider together than the model (3 x 64 over a width of 96) and narrower (1 x 32); every attention head its
#    own kv head with maps of 64 and values of 128 (tensor-core kernels with one head a group); no kept tokens; a second
#    cache of the same shape with another window; a reader WITHOUT a window, so the cache it reads keeps everything
S = model(131, 96, [delta(3, 64), attn(4, 4, 64, 128, window=200, keep=0, ff=160, diff=0.1), delta(1, 32, ff=40),
                    attn(4, 4, 64, 128, window=50, keep=7), attn(4, 4, 64, 128, kv_from=1, diff=0.9)],
          max_positions=450, scale=1.5, eps=1e-5)

MODELS = {"p": P, "q": Q, "r": R, "s": S}


def draw_weights(config: dict, seed: int, dtype=torch.bfloat16):
    """{name: tensor} for `config` from the product's own list of tensors, rounded to `dtype` (so that the engine and the
    plain implementation start from the same numbers)."""
    from hipinfer_b200.config import config_from_dict, get_architecture
    from hipinfer_b200.parts.spec import spec_param_specs

    c = config_from_dict(config)
    g = torch.Generator().manual_seed(seed)
    out = {}
    for s in spec_param_specs(get_architecture(c.architecture).build_spec(c)):
        n, shape = s.name, tuple(s.shape)
        rnd = torch.randn(shape, generator=g)
        if len(shape) == 2 and n not in ("embed", "pos"):
            t = rnd * (1.2 / math.sqrt(shape[1]))
        elif n in ("embed", "pos"):
            t = rnd * 0.7
        elif n.endswith(".act"):
            t = torch.tensor([0.7, 0.4, 0.25, 0.1]) + 0.05 * rnd
        elif n.endswith((".ls1", ".ls2")):
            t = 0.6 + 0.3 * torch.rand(shape, generator=g)
        elif "norm" in n:
            t = 1.0 + 0.2 * rnd
        elif n.endswith((".lq1", ".lk1", ".lq2", ".lk2")):
            t = 0.3 * rnd
        else:                      # biases, w0
            t = 0.5 * rnd
        out[n] = t.to(dtype)
    return out


def make_folder(folder, which, seed=1, dtype=torch.bfloat16):
    from hipinfer_b200.weights.safetensors_io import save_safetensors

    cfg = MODELS[which] if isinstance(which, str) else which
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    w = draw_weights(cfg, seed, dtype)
    save_safetensors(w, os.path.join(folder, "model.safetensors"), {"format": "pt"})
    return str(folder), cfg, w
