"""What of the Torirax design can be checked without a GPU: the configuration reader, the model's list of parts and
tensors, what the cache manager is asked to retain, and the plain implementation against itself (portions against the
whole sequence, the mask's edges)."""
import math

import pytest
import torch

import plain_torirax as plain
import torirax_models as tm
from hipinfer_b200.cache import CacheGroupSpec, CacheManager
from hipinfer_b200.config import ConfigError, config_from_dict, get_architecture
from hipinfer_b200.models.decoder import DecoderModel
from hipinfer_b200.parts.registry import BuildContext
from hipinfer_b200.parts.spec import spec_param_specs
from hipinfer_b200.weights import ParamSpec
from hipinfer_b200.weights.loader import WeightError, check_names


def _spec(cfg):
    c = config_from_dict(cfg)
    return c, get_architecture(c.architecture).build_spec(c)


def test_config_round_trip_and_every_size_from_the_file():
    for name, cfg in tm.MODELS.items():
        c, spec = _spec(cfg)
        assert config_from_dict(c.to_dict()) == c
        assert spec.vocab_size == cfg["vocab"] and spec.hidden_size == cfg["width"] and spec.max_position == cfg["max_positions"]
        assert len(spec.layers) == len(cfg["layers"])
        for L, ls in zip(cfg["layers"], spec.layers):
            assert ("feed_forward" in ls.parts) == (L["mlp"] is not None)
            assert ls.parts["mixer"].kind == ("delta_rule" if L["type"] == "general_delta" else "differential_attention")


@pytest.mark.parametrize("edit, text", [
    (lambda d: d["layers"][1].update(type="conv"), "not known"),
    (lambda d: d["layers"][1]["mixer"].update(kv_heads=3), "multiple"),
    (lambda d: d["layers"][3]["mixer"].update(kv_from=2), "earlier attention layer"),
    (lambda d: d["layers"][3]["mixer"].update(vdim=8), "differ"),
    (lambda d: d["layers"][1].update(mlp=dict(kind="routed", ff=8)), "not known"),
    (lambda d: d.pop("norm"), "norm"),
    (lambda d: d.update(width=-4), "positive"),
])
def test_config_refuses(edit, text):
    import copy

    d = copy.deepcopy(tm.P)
    edit(d)
    with pytest.raises(ConfigError, match=text):
        config_from_dict(d)


def test_tensor_list_and_the_rank_the_file_decides():
    c, spec = _spec(tm.R)           # layer 0 gives no decay_rank, layer 2 does
    specs = {s.name: s for s in spec_param_specs(spec)}
    assert "l3.mix.k" not in specs and "l3.mix.v.b" not in specs and "l3.mix.q" in specs      # the reader has no k/v
    assert "l0.norm2" not in specs and "l0.ls2" not in specs and "l1.ls2" in specs            # no feed-forward, no second norm
    assert specs["l1.mix.q"].shape == (8 * 2 * 32, 128) and specs["l1.mix.k"].shape == (2 * 2 * 32, 128)
    assert specs["l1.mix.v"].shape == (2 * 64, 128) and specs["l1.mix.o"].shape == (128, 8 * 64)
    assert specs["l2.mix.w1"].shape == (24, 128) and specs["l2.mix.w1"].free == ()
    assert specs["l0.mix.w1"].free == (0,) and specs["l0.mix.w2"].free == (1,)
    have = {n: tuple(s.shape) for n, s in specs.items()}
    have["l0.mix.w1"], have["l0.mix.w2"] = (7, 128), (128, 7)                                  # any rank fits layer 0
    check_names("x", list(specs.values()), have)
    have["l2.mix.w1"] = (7, 128)
    with pytest.raises(WeightError, match="l2.mix.w1"):
        check_names("x", list(specs.values()), have)


def test_cache_plan_shares_and_retains_the_widest_look_back():
    c, spec = _spec(tm.R)
    m = DecoderModel(spec, BuildContext.meta())
    plan = m.cache_plan
    assert plan[0] is None and plan[2] is None and m.state_specs[(0, "S")][0] == (2, 64, 64) and m.state_specs[(2, "S")][0] == (1, 128, 128)
    assert plan[1].write and not plan[3].write and (plan[3].group, plan[3].slot) == (plan[1].group, plan[1].slot)
    g = m.cache_groups[plan[1].group]
    assert g.kind == "window_keep_first" and g.window == 130 and dict(g.extra)["keep_first"] == 5      # the reader's, wider
    assert g.planes == (("k", 2, 64), ("v", 2, 64))
    assert [o.reads_cache_of for o in spec.order] == [None, None, None, 1, None]
    # a reader without a window: the cache it reads keeps everything, the other cache of the same shape keeps its window
    c, spec = _spec(tm.S)
    m = DecoderModel(spec, BuildContext.meta())
    kinds = {g.kind: g for g in m.cache_groups}
    assert m.cache_groups[m.cache_plan[1].group].kind == "full" and m.cache_plan[4].group == m.cache_plan[1].group
    assert m.cache_groups[m.cache_plan[3].group].kind == "window_keep_first" and kinds["window_keep_first"].window == 50
    # no window anywhere: everything is kept
    c, spec = _spec(tm.Q)
    m = DecoderModel(spec, BuildContext.meta())
    assert m.cache_groups[m.cache_plan[0].group].kind == "full"
    # a reader without a window makes the writer's cache keep everything
    import copy

    d = copy.deepcopy(tm.P)
    del d["layers"][3]["mixer"]["mask"]
    c, spec = _spec(d)
    m = DecoderModel(spec, BuildContext.meta())
    assert m.cache_groups[m.cache_plan[1].group].kind == "full"


def test_retention_gives_back_pages_between_the_kept_tokens_and_the_window():
    g = CacheGroupSpec("g", "window_keep_first", 1, 1, 8, window=10, planes=(("k", 1, 16), ("v", 1, 4)), extra=(("keep_first", 5),))
    cm = CacheManager([g], 4, 64, 2)
    cm.add_request("a")
    cm.append("a", 40)
    assert cm.release_behind_window("a") == 5          # the next query, at 40, sees 31..40 and 0..4: pages 2..6 (8..27) go
    t = cm.block_table("a", 0)
    assert [p >= 0 for p in t] == [True, True] + [False] * 5 + [True, True, True]
    cm.append("a", 3)
    assert cm.release_behind_window("a") == 1          # the query at 43 sees 34..: page 7 (28..31) goes
    cm.append("a", 1)
    assert cm.release_behind_window("a") == 0          # the query at 44 still sees 35 on page 8 (32..35)
    cm.append("a", 1)
    assert cm.release_behind_window("a") == 1          # the query at 45 sees 36..: page 8 goes
    cm.check()
    cm.free_request("a")
    cm.check()
    assert cm.free_pages() == [64]


def test_plain_portions_equal_the_whole():
    for name in ("p", "q"):
        cfg = tm.MODELS[name]
        w = tm.draw_weights(cfg, 3, torch.float32)
        toks = torch.randint(0, cfg["vocab"], (70,), generator=torch.Generator().manual_seed(5)).tolist()
        m = plain.PlainTorirax(cfg, w)
        whole = m.forward(toks)
        m.reset()
        parts, i = [], 0
        for n in (1, 2, 30, 2, 1, 17, 3, 14):
            parts.append(m.forward(toks[i:i + n]))
            i += n
        assert i == 70
        assert torch.allclose(torch.cat(parts), whole, rtol=0, atol=1e-9 * float(whole.abs().max()))


def test_plain_mask_edges():
    seen = lambda i, j, w, k: plain.visible(i, j, w, k)
    assert seen(9, 9, 1, 0) and not seen(9, 8, 1, 0)
    assert seen(20, 11, 10, 2) and not seen(20, 10, 10, 2) and seen(20, 1, 10, 2) and not seen(20, 2, 10, 2)
    assert not seen(3, 4, None, 0) and seen(300, 0, None, 0)
    s = torch.zeros(3, 30, dtype=torch.float64)
    p = plain.softmax_over_visible(s, 10, 2, first_query=27)
    assert torch.equal(p[0] > 0, torch.tensor([j < 2 or 18 <= j <= 27 for j in range(30)]))
    assert abs(float(p[2].sum()) - 1) < 1e-12 and float(p[2, 19]) == 0 and float(p[2, 20]) > 0
    lam = plain.differential_lambda(torch.ones(4) * 0.5, torch.ones(4), torch.zeros(4), torch.ones(4), 0.25)
    assert abs(lam - (math.exp(2.0) - 1 + 0.25)) < 1e-12


def test_random_model_from_the_command_line_and_back(tmp_path):
    """`random-model` writes a Torirax folder whose config reads back equal and whose tensors fit the model's list (the
    rank the file decides takes the spec's default)."""
    import json
    import os
    import subprocess
    import sys

    from hipinfer_b200.config import load_config
    from hipinfer_b200.weights.safetensors_io import ModelFiles

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = tmp_path / "cfg.json"
    cfg.write_text(json.dumps(tm.R))
    out = tmp_path / "model"
    r = subprocess.run([sys.executable, "-m", "hipinfer_b200", "random-model", "--config", str(cfg), "--out", str(out), "--seed", "3"],
                       capture_output=True, text=True, cwd=root, env=dict(os.environ, PYTHONPATH=root))
    assert r.returncode == 0, r.stderr[-2000:]
    c = load_config(str(out))
    assert c == config_from_dict(tm.R)
    spec = get_architecture(c.architecture).build_spec(c)
    f = ModelFiles(str(out))
    try:
        check_names(str(out), spec_param_specs(spec), {n: f.info(n)[1] for n in f.names()}, [], {n: f.info(n)[0] for n in f.names()})
        assert f.info("l0.mix.w1")[1] == (16, 128) and f.info("l2.mix.w1")[1] == (24, 128)
    finally:
        f.close()
