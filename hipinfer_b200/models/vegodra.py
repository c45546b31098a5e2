"""The Vegodra decoder as a ModelSpec: a token embedding that goes through a layer norm; layers in the order config.json
lists them, each a parallel block (ONE layer norm whose result both the sequence mixer and the feed-forward read; their
results are added to the residual stream together); the mixer is latent attention (a cached latent and one rotated key
part per token), grouped-query attention with partial rotation, unit-norm queries and keys, a chunked mask, a sink in
the softmax and a gate per head (such a layer may read the keys and values an earlier one cached), or gated linear
attention (a recurrent state per head); the feed-forward is gated with the tanh form of GELU; layer norms with weight
and bias everywhere; an untied head.

Tensor names: embed, embed.norm(.b), head, final.norm(.b), and per layer i under "l<i>.": norm1(.b), mix.*, mlp.*.
"""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.vegodra import VegodraConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunStep


def vegodra_spec(c: VegodraConfig) -> ModelSpec:
    W, eps = c.width, c.norm_eps
    norm = lambda name: PartSpec("layernorm", dict(name=name, bias_name=name + ".b", size=W, eps=eps))
    # what a cache must retain: the chunk sizes of the layer that writes it and of the layers that read it (a reader
    # without a mask makes it keep everything)
    chunks = {}
    for i, L in enumerate(c.layers):
        if L.type == "attention":
            owner = i if L.mixer.kv_from is None else L.mixer.kv_from
            chunks.setdefault(owner, []).append(L.mixer.chunk)
    layers, order, step_of = [], [], {}
    for i, L in enumerate(c.layers):
        m = L.mixer
        if L.type == "latent_attention":
            mixer = PartSpec("latent_attention", dict(
                hidden_size=W, heads=m.heads, dim=m.dim, rot_dim=m.rot_dim, vdim=m.vdim, q_rank=m.q_rank, kv_rank=m.kv_rank,
                scale=m.scale, eps=eps, rot_dims=m.rot.dims, rot_base=m.rot.base))
            order.append(RunStep(i))
        elif L.type == "attention":
            owner = i if m.kv_from is None else m.kv_from
            sizes = chunks[owner]
            mixer = PartSpec("masked_attention", dict(
                hidden_size=W, heads=m.heads, kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim, scale=m.scale, eps=eps,
                rot_dims=m.rot.dims, rot_base=m.rot.base, pairing="half", unit_norm=True,
                mask="chunk" if m.chunk else "causal", chunk=m.chunk or 0, sink=True, gate="head",
                reads_cache=m.kv_from is not None, cache_chunks=() if any(s is None for s in sizes) else tuple(sizes)))
            order.append(RunStep(i, None if m.kv_from is None else step_of[m.kv_from]))
        else:
            mixer = PartSpec("gla", dict(hidden_size=W, heads=m.heads, dim=m.dim, vdim=m.vdim, tau=m.tau, eps=eps,
                                         decay_rank=m.decay_rank))
            order.append(RunStep(i))
        step_of[i] = len(order) - 1
        parts = dict(norm=norm("norm1"), mixer=mixer)
        if L.ff is not None:
            parts["feed_forward"] = PartSpec("gated", dict(hidden_size=W, intermediate_size=L.ff, activation="gelu_tanh"))
        layers.append(LayerSpec(prefix=f"l{i}.", block="parallel", parts=parts))
    return ModelSpec(
        architecture=c.architecture, hidden_size=W, vocab_size=c.vocab, max_position=c.max_positions,
        embedding=PartSpec("token_normed", dict(name="embed", vocab_size=c.vocab, hidden_size=W, norm=norm("embed.norm"))),
        layers=tuple(layers), order=tuple(order), final_norm=norm("final.norm"),
        head=PartSpec("linear", dict(name="head", vocab_size=c.vocab, hidden_size=W)), eos_token_ids=c.eos_token_ids)


register_architecture("Vegodra", VegodraConfig, vegodra_spec)
