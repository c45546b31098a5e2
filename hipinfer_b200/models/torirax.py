"""The Torirax decoder as a ModelSpec: a scaled token embedding plus learned position vectors; layers in the order
config.json lists them, each a pre-norm block with layer scale around one mixer (a delta-rule recurrence or
differential attention with a window that keeps the first tokens; an attention layer may read the keys and values of
an earlier one instead of projecting its own) and, where the layer has one, a dense feed-forward with the PolyNorm
activation; layer norms with a weight and no bias everywhere; an untied head.

Tensor names: embed, pos, head, final.norm, and per layer i under "l<i>.": norm1, norm2, ls1, ls2, mix.*, mlp.*.
"""
from __future__ import annotations

from ..config import ToriraxConfig, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunStep


def torirax_spec(c: ToriraxConfig) -> ModelSpec:
    W, eps = c.width, c.norm_eps
    norm = lambda name: PartSpec("layernorm", dict(name=name, size=W, eps=eps))
    # what a cache must retain: the widest look-back among the layer that writes it and the layers that read it
    retain = {}
    for i, L in enumerate(c.layers):
        if L.type != "attention":
            continue
        owner, win, keep = (i if L.mixer.kv_from is None else L.mixer.kv_from), L.mixer.window, L.mixer.keep_first
        if owner in retain:
            have = retain[owner]
            win = None if (win is None or have[0] is None) else max(win, have[0])
            keep = max(keep, have[1])
        retain[owner] = (win, keep)
    layers, order, step_of = [], [], {}
    for i, L in enumerate(c.layers):
        m = L.mixer
        if L.type == "general_delta":
            mixer = PartSpec("delta_rule", dict(hidden_size=W, heads=m.heads, dim=m.dim, eps=eps, decay_rank=m.decay_rank))
            order.append(RunStep(i))
        else:
            owner = i if m.kv_from is None else m.kv_from
            win, keep = retain[owner]
            mixer = PartSpec("differential_attention", dict(
                hidden_size=W, heads=m.heads, kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim, scale=m.scale, diff=m.diff, eps=eps,
                window=m.window, keep_first=m.keep_first, cache_window=win, cache_keep_first=keep if win else 0,
                reads_cache=m.kv_from is not None))
            order.append(RunStep(i, None if m.kv_from is None else step_of[m.kv_from]))
        step_of[i] = len(order) - 1
        parts = dict(mixer_norm=norm("norm1"), mixer=mixer)
        if L.ff is not None:
            parts.update(feed_forward_norm=norm("norm2"),
                         feed_forward=PartSpec("polynorm", dict(hidden_size=W, intermediate_size=L.ff, eps=eps)))
        layers.append(LayerSpec(prefix=f"l{i}.", block="pre_norm_scaled", parts=parts,
                                params=dict(hidden_size=W, mixer_scale_name="ls1", feed_forward_scale_name="ls2")))
    return ModelSpec(
        architecture=c.architecture, hidden_size=W, vocab_size=c.vocab, max_position=c.max_positions,
        embedding=PartSpec("token_position", dict(name="embed", vocab_size=c.vocab, hidden_size=W, scale=c.embedding_scale,
                                                  position_name="pos", max_position=c.max_positions)),
        layers=tuple(layers), order=tuple(order), final_norm=PartSpec("layernorm", dict(name="final.norm", size=W, eps=eps)),
        head=PartSpec("linear", dict(name="head", vocab_size=c.vocab, hidden_size=W)), eos_token_ids=c.eos_token_ids)


register_architecture("Torirax", ToriraxConfig, torirax_spec)
