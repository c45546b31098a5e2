"""Small Vegodra configurations of the tests' own, with weights drawn so that faults show: matrices of unit gain (the
scores spread, the decays move), norm weights away from 1, biases and sinks away from 0."""
from __future__ import annotations

import json
import math
import os

import torch


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, ff=None, dims=None, base=10000.0, scale=None):
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, q_rank=q_rank, kv_rank=kv_rank,
             scale=scale or 1.0 / math.sqrt(dim + rot_dim), rot=dict(base=base, dims=rot_dim if dims is None else dims))
    return dict(type="latent_attention", mixer=m, mlp=None if ff is None else dict(kind="dense", ff=ff))


def attn(heads, kv_heads, dim, vdim, dims, chunk=None, kv_from=None, ff=None, base=50000.0, scale=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale or 4.0 / math.sqrt(dim), rot=dict(base=base, dims=dims))
    if chunk is not None:
        m["mask"] = dict(size=chunk)
    if kv_from is not None:
        m["kv_from"] = kv_from
    return dict(type="attention", mixer=m, mlp=None if ff is None else dict(kind="dense", ff=ff))


def gla(heads, dim, vdim, tau, ff=None, rank=None):
    m = dict(heads=heads, dim=dim, vdim=vdim, tau=tau)
    if rank:
        m["decay_rank"] = rank
    return dict(type="gla", mixer=m, mlp=None if ff is None else dict(kind="dense", ff=ff))


def model(vocab, width, layers, eps=1e-5, max_positions=None):
    d = dict(architecture="Vegodra", vocab=vocab, width=width, norm=dict(eps=eps), layers=layers)
    if max_positions:
        d["max_positions"] = max_positions
    return d


# A: latent first; a recurrent layer without a feed-forward; chunks of 24 (a page and a half); a reader of the same chunks
A = model(160, 64, [latent(3, 16, 8, 24, 40, 56, ff=96), gla(2, 32, 16, 8.0, rank=8), attn(4, 2, 32, 16, 8, chunk=24, ff=64),
                    latent(2, 8, 16, 8, 24, 32), attn(4, 2, 32, 16, 8, chunk=24, kv_from=2, ff=48)], max_positions=700)
# B: attention first with chunks of ONE token (a row sees itself and the sink), every head its own kv head, dim == vdim,
#    rotation over the whole head; a reader with LONGER chunks than its writer and one without a mask (the cache keeps
#    everything); a single recurrent head with dim != vdim and tau 1; a latent rotated on part of its rotated size;
#    a feed-forward whose width is no multiple of 16
B = model(97, 48, [attn(3, 3, 8, 8, 8, chunk=1, ff=80), gla(1, 48, 40, 1.0, ff=56, rank=5), latent(1, 24, 12, 40, 16, 24, dims=8),
                   attn(3, 3, 8, 8, 8, chunk=50, kv_from=0), attn(3, 3, 8, 8, 8, kv_from=0, ff=32)], eps=1e-6, max_positions=600)
# C: wider; chunks that cross pages and key tiles; recurrent heads of 64 and of 128; latent heads of 8 with keys longer
#    than a key split when the prompt is long
C = model(211, 128, [gla(2, 64, 64, 16.0), latent(8, 32, 16, 32, 96, 64, ff=192), attn(8, 2, 64, 64, 32, chunk=70, ff=128),
                     gla(1, 128, 128, 4.0, rank=24), attn(8, 2, 64, 64, 32, chunk=200, kv_from=2),
                     attn(4, 1, 32, 48, 16, chunk=130, ff=64)], max_positions=900)
# D: sizes no vectorised kernel takes: a width that is no multiple of 4, heads of 10 and 6, a latent of 20
D = model(90, 50, [latent(2, 10, 6, 6, 14, 20, ff=30, dims=4), gla(3, 10, 6, 2.0, ff=22, rank=3), attn(3, 1, 10, 6, 6, chunk=5)],
          max_positions=300)

MODELS = {"a": A, "b": B, "c": C, "d": D}


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
        if n == "embed":
            t = rnd * 0.7
        elif len(shape) == 2:
            t = rnd * (1.2 / math.sqrt(shape[1]))
        elif n.endswith(".a2.b"):
            t = 1.0 + rnd                   # decays between nearly 0 and nearly 1
        elif n.endswith(".b") or n.endswith(".sink"):
            t = 0.5 * rnd
        else:                               # norm weights
            t = 1.0 + 0.2 * rnd
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
