"""The Vegodra design without a GPU: its configuration, its description as parts, the cache and state plan the decoder
derives from it, the retention rule of chunked caches, and the plain implementation against itself (a sequence at once
against the same sequence continued token by token; each mask and the sink against hand-made cases)."""
import json
import math

import pytest
import torch

import plain_vegodra as plain
import vegodra_models as tm


def test_config_round_trip_and_refusals():
    from hipinfer_b200.config import ConfigError, config_from_dict

    for name, cfg in tm.MODELS.items():
        c = config_from_dict(cfg)
        assert c.architecture == "Vegodra" and c.to_dict()["layers"] == cfg["layers"], name
        assert config_from_dict(json.loads(json.dumps(c.to_dict()))) == c
    bad = json.loads(json.dumps(tm.A))
    bad["layers"][4]["mixer"]["kv_from"] = 1                      # not an attention layer
    with pytest.raises(ConfigError):
        config_from_dict(bad)
    bad = json.loads(json.dumps(tm.A))
    bad["layers"][4]["mixer"]["dim"] = 16                         # a reader whose keys would not fit
    with pytest.raises(ConfigError):
        config_from_dict(bad)
    bad = json.loads(json.dumps(tm.A))
    bad["layers"][0]["mixer"]["rot"]["dims"] = 10                 # more rotated dimensions than the rotated part has
    with pytest.raises(ConfigError):
        config_from_dict(bad)
    bad = json.loads(json.dumps(tm.A))
    bad["layers"][1]["type"] = "convolution"
    with pytest.raises(ConfigError):
        config_from_dict(bad)


def test_spec_caches_and_states():
    from hipinfer_b200.config import config_from_dict, get_architecture
    from hipinfer_b200.models.decoder import DecoderModel
    from hipinfer_b200.parts.registry import BuildContext

    c = config_from_dict(tm.B)
    spec = get_architecture("Vegodra").build_spec(c)
    m = DecoderModel(spec, BuildContext.meta())
    # B: the attention cache is read by a layer without a mask, so it keeps everything; one latent cache; one state
    kinds = sorted((g.kind, g.n_layers) for g in m.cache_groups)
    assert kinds == [("full", 1), ("full", 1)]
    assert [p.write if p else None for p in m.cache_plan] == [True, None, True, False, False]
    assert list(m.state_specs) == [(1, "S")] and m.state_specs[(1, "S")][0] == (1, 48, 40)
    names = {s.name for s in m.param_specs()}
    assert "l3.mix.k" not in names and "l3.mix.q" in names and "l0.mix.sink" in names and "embed.norm.b" in names
    # C: writer chunks of 70, reader chunks of 200: the cache retains back to the earlier of the two starts
    m = DecoderModel(get_architecture("Vegodra").build_spec(config_from_dict(tm.C)), BuildContext.meta())
    g = [g for g in m.cache_groups if g.kind == "chunks" and g.kv_heads == 2][0]
    assert dict(g.extra)["chunks"] == (70, 200)


def test_chunk_retention_rule():
    from hipinfer_b200.cache import CacheGroupSpec, CacheManager

    spec = CacheGroupSpec("g", "chunks", 1, 1, 8, 0, (("k", 1, 8), ("v", 1, 8)), (("chunks", (32, 48)),))
    cm = CacheManager([spec], 16, 12, 1)
    cm.add_request("x")
    cm.append("x", 100)                # next query at 100: chunk starts 96 and 96 -> positions below 96 are dead
    assert cm.release_behind_window("x") == 6 and cm.block_table("x", 0)[:6] == [-1] * 6
    cm.append("x", 50)                 # next query at 150: starts 128 and 144 -> below 128
    cm.release_behind_window("x")
    assert cm.block_table("x", 0)[:8] == [-1] * 8 and cm.block_table("x", 0)[8] >= 0
    cm.free_request("x")
    cm.check()


@pytest.mark.parametrize("which", ["a", "b", "d"])
def test_plain_model_whole_against_token_by_token(which):
    cfg = tm.MODELS[which]
    w = tm.draw_weights(cfg, 3, torch.float32)
    toks = torch.randint(0, cfg["vocab"], (60,), generator=torch.Generator().manual_seed(1)).tolist()
    whole = plain.forward(cfg, w, toks)
    m = plain.PlainVegodra(cfg, w)
    parts = torch.cat([m.forward(toks[:25])] + [m.forward([t]) for t in toks[25:]])
    assert float((whole - parts).abs().max()) < 1e-9 * float(whole.abs().max())


def test_plain_masks_sink_and_rotation():
    seen = plain.causal_mask(7, 7, 0, 3)
    assert seen.tolist()[5] == [False, False, False, True, True, True, False] and seen.tolist()[3] == [False, False, False, True, False, False, False]
    assert plain.causal_mask(2, 6, 4, None).tolist() == [[True] * 5 + [False], [True] * 6]
    s = torch.tensor([[0.0, 1.0, 2.0]], dtype=torch.float64)
    p = plain.softmax_with_sink(s, torch.tensor([[True, True, False]]), 0.5)
    den = math.exp(0.0) + math.exp(1.0) + math.exp(0.5)
    assert torch.allclose(p, torch.tensor([[1 / den, math.e / den, 0.0]], dtype=torch.float64))
    # a rotation keeps lengths, composes (p then q is p + q) and leaves the unrotated dimensions alone
    t = torch.randn(1, 2, 12, dtype=torch.float64, generator=torch.Generator().manual_seed(0))
    for pairing in ("half", "interleaved"):
        a = plain.rotate(t, torch.tensor([5]), 8, 100.0, pairing)
        assert torch.allclose(a.norm(dim=-1), t.norm(dim=-1)) and torch.equal(a[..., 8:], t[..., 8:])
        b = plain.rotate(plain.rotate(t, torch.tensor([2]), 8, 100.0, pairing), torch.tensor([3]), 8, 100.0, pairing)
        assert torch.allclose(a, b)
    a = plain.rotate(t, torch.tensor([1]), 8, 100.0, "interleaved")
    assert torch.allclose(a[0, 0, 0], t[0, 0, 0] * math.cos(1.0) - t[0, 0, 1] * math.sin(1.0))
    a = plain.rotate(t, torch.tensor([1]), 8, 100.0, "half")
    assert torch.allclose(a[0, 0, 0], t[0, 0, 0] * math.cos(1.0) - t[0, 0, 4] * math.sin(1.0))
    assert torch.allclose(a[0, 0, 5], t[0, 0, 5] * math.cos(100.0 ** -0.25) + t[0, 0, 1] * math.sin(100.0 ** -0.25))


def test_random_weights_mode_writes_a_loadable_folder(tmp_path):
    from hipinfer_b200.config import config_from_dict, load_config
    from hipinfer_b200.weights import write_random_model
    from hipinfer_b200.weights.safetensors_io import ModelFiles

    write_random_model(config_from_dict(tm.D), str(tmp_path / "m"), seed=4)
    assert load_config(str(tmp_path / "m")) == config_from_dict(tm.D)
    files = ModelFiles(str(tmp_path / "m"))
    assert "l1.mix.a2.b" in files.names() and "l2.mix.sink" in files.names() and files.info("l1.mix.a1")[1] == (3, 50)
    files.close()
