"""The Vegodra design through the engine: the step function, the cache and state manager, trace replay, the scheduler
and the Python entry point, in 32-bit and in bfloat16, against the plain implementation of tests/plain_vegodra.py, on
four small configurations of the tests' own (tests/vegodra_models.py)."""
import math

import pytest
import torch

import plain_vegodra as plain
import tiny
import vegodra_models as tm

pytestmark = pytest.mark.gpu

LENGTHS = {"a": [1, 2, 5, 40, 90, 130, 33, 64], "b": [3, 1, 70, 16, 17, 100, 48, 2], "c": [600, 7, 129, 64, 200, 65, 1, 150],
           "d": [120, 31, 57, 2, 64, 90, 16, 100]}
TOL = {"float32": 3e-5, "bfloat16": 2.5e-2}


def _close(got, ref, dtype, what):
    scale, err = float(ref.abs().max()), float((got.double() - ref.double()).abs().max())
    assert got.shape == ref.shape and torch.isfinite(got).all(), what
    if err > TOL[dtype] * scale:
        bad = (got.double() - ref.double()).abs().amax(-1)
        raise AssertionError(f"{what}: {err:.3e} > {TOL[dtype]:.0e} * {scale:.3e}; first wrong position "
                             f"{int((bad > TOL[dtype] * scale).nonzero()[0])} of {got.shape[0]}")


@pytest.fixture(scope="module", params=[(m, d) for m in ("a", "b", "c", "d") for d in ("float32", "bfloat16")], ids=lambda p: f"{p[0]}-{p[1]}")
def setup(request, tmp_path_factory):
    from hipinfer_b200.engine.runner import ModelRunner

    which, dtype = request.param
    folder, cfg, w = tm.make_folder(tmp_path_factory.mktemp(f"vegodra_{which}_{dtype}"), which, seed=7,
                                    dtype=torch.float32 if dtype == "float32" else torch.bfloat16)
    requests = {f"r{i}": tiny.random_tokens(n, cfg["vocab"], 300 + i) for i, n in enumerate(LENGTHS[which])}
    model = plain.PlainVegodra(cfg, w)
    ref = {}
    for rid, toks in requests.items():
        model.reset()
        ref[rid] = model.forward(toks)
    longest = -(-max(LENGTHS[which]) // 64) * 64
    # pages for four live requests of the longest kind and four state slots: both are used again
    runner = ModelRunner.from_folder(folder, dtype=dtype, page_size=16, num_pages=4 * longest // 16, max_num_seqs=4)
    yield dict(which=which, dtype=dtype, folder=folder, cfg=cfg, weights=w, requests=requests, ref=ref, runner=runner,
               stepper=tiny.RunnerStepper(runner))
    assert not runner.live_requests()
    runner.cache.check()
    assert runner.cache.free_pages() == [p.num_pages for p in runner.cache.pools]


def _check(setup, plan, what):
    got = tiny.run_plan(setup["stepper"], setup["requests"], plan)
    for rid, ref in setup["ref"].items():
        _close(got[rid], ref, setup["dtype"], f"{what} {setup['which']} {setup['dtype']} {rid}")
    return got


def test_whole_prompts(setup):
    _check(setup, tiny.plan_whole(setup["requests"]), "whole")


def test_last_tokens_one_by_one(setup):
    _check(setup, tiny.plan_tail_decode(setup["requests"], 48), "tail")


def test_every_token_alone(setup):
    short = {r: t for r, t in setup["requests"].items() if len(t) <= 70}
    got = tiny.run_plan(setup["stepper"], short, [[(r, 1)] for r, t in short.items() for _ in t])
    for rid in short:
        _close(got[rid], setup["ref"][rid], setup["dtype"], f"token by token {rid}")


@pytest.mark.parametrize("sizes", [(7, 2, 16, 3, 2, 33, 5, 2, 64, 1, 9), (2,), (15, 17, 1, 31), (64, 2, 63, 66)])
def test_portions(setup, sizes):
    _check(setup, tiny.plan_portions(setup["requests"], sizes), f"portions {sizes}")


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_mixed_batches(setup, seed):
    _check(setup, tiny.plan_mixed(setup["requests"], seed), f"mixed{seed}")


def test_mixed_batches_with_long_portions(setup):
    _check(setup, tiny.plan_mixed_long(setup["requests"], 1, long=(65, 140)), "mixed long")


def test_a_request_in_a_batch_equals_the_request_alone(setup):
    """Beyond rounding nothing of a row depends on the batch: in 32-bit the two agree to a few units of the last place."""
    reqs = setup["requests"]
    alone = tiny.run_plan(setup["stepper"], reqs, tiny.plan_whole(reqs))
    ids = list(reqs)
    together = tiny.run_plan(setup["stepper"], reqs, [[(r, len(reqs[r])) for r in ids[:4]], [(r, len(reqs[r])) for r in ids[4:]]])
    tol = 2e-6 if setup["dtype"] == "float32" else 1e-2
    for rid in ids:
        scale = float(alone[rid].abs().max())
        assert float((alone[rid] - together[rid]).abs().max()) <= tol * scale, rid


def test_a_state_slot_and_pages_used_again_start_clean(setup):
    """The same request after others have used and returned every slot and page gives the same bits as on a fresh engine
    state (the recurrent state is zeroed at admission; pages hold what the request itself wrote)."""
    reqs, st = setup["requests"], setup["stepper"]
    first = tiny.run_plan(st, {"r3": reqs["r3"]}, [[("r3", len(reqs["r3"]))]])["r3"]
    others = {r: reqs[r] for r in ("r4", "r5", "r0", "r2", "r7")}
    tiny.run_plan(st, others, tiny.plan_mixed(others, 5))
    again = tiny.run_plan(st, {"r3": reqs["r3"]}, [[("r3", len(reqs["r3"]))]])["r3"]
    assert torch.equal(first, again)


def test_long_decoding_past_every_window(setup):
    """A short prompt, then hundreds of single tokens: windows pass over decoded tokens, pages are given back while the
    request runs, decode-only steps replay from CUDA graphs."""
    cfg = setup["cfg"]
    n = min(cfg["max_positions"], 330 if setup["which"] != "c" else 560)
    toks = tiny.random_tokens(n, cfg["vocab"], 77)
    model = plain.PlainVegodra(cfg, setup["weights"])
    ref = model.forward(toks)
    got = tiny.run_plan(setup["stepper"], {"long": toks}, [[("long", 6)]] + [[("long", 1)]] * (n - 6))["long"]
    _close(got, ref, setup["dtype"], "long decoding")
    r = setup["runner"]
    if any(g.kind != "full" for g in r.cache.groups):
        assert r.steps_run > 0      # (pages were given back on the way: the pool is smaller than the request only where a window is)


def test_two_requests_decode_together_through_graph_replays(setup):
    reqs = setup["requests"]
    a, b = "r4", "r5"
    ha, hb = len(reqs[a]) // 2, len(reqs[b]) // 3 + 1
    plan = [[(a, ha), (b, hb)]] + [[(a, 1), (b, 1)]] * min(len(reqs[a]) - ha, len(reqs[b]) - hb)
    fed_a, fed_b = ha + len(plan) - 1, hb + len(plan) - 1
    sub = {a: reqs[a][:fed_a], b: reqs[b][:fed_b]}
    got = tiny.run_plan(setup["stepper"], sub, plan)
    _close(got[a], setup["ref"][a][:fed_a], setup["dtype"], "pair a")
    _close(got[b], setup["ref"][b][:fed_b], setup["dtype"], "pair b")


def test_trace_replay_program(setup, tmp_path):
    """bin/trace_run as a child process on the same folder: portions, single tokens, a batch, few pages."""
    reqs = {r: setup["requests"][r] for r in ("r2", "r3", "r6", "r7")}
    tr = tiny.TraceRun(setup["folder"], setup["dtype"], tmp_path / "out", 2 * 64 * -(-max(len(t) for t in reqs.values()) // 64))
    try:
        got = tiny.run_plan(tr, reqs, tiny.plan_mixed(reqs, 3, max_live=2))
    finally:
        tr.close()
    for rid in reqs:
        _close(got[rid], setup["ref"][rid], setup["dtype"], f"trace_run {rid}")


def test_greedy_generation_through_the_entry_point_and_scheduler(setup):
    """Engine.generate and three requests through the scheduler at once, against greedy decoding with the plain model; a
    different token is accepted only where the plain logits nearly tie."""
    from hipinfer_b200 import Engine

    cfg, n_new = setup["cfg"], 12
    model = plain.PlainVegodra(cfg, setup["weights"])

    def plain_greedy(prompt):
        model.reset()
        logits = model.forward(prompt)[-1]
        out, steps = [], []
        for _ in range(n_new):
            steps.append(logits)
            out.append(int(logits.argmax()))
            logits = model.forward([out[-1]])[-1]
        return out, steps

    def same(got, want, steps, what):
        for i, (g, w) in enumerate(zip(got, want)):
            if g != w:
                top = torch.topk(steps[i], 2).values
                gap = float(top[0] - top[1]) / float(steps[i].abs().max())
                assert gap < (0.02 if setup["dtype"] == "bfloat16" else 1e-3), f"{what}: token {i} is {g}, plain {w} (gap {gap:.5f})"
                return
        assert len(got) == len(want)

    eng = Engine(setup["folder"], dtype=setup["dtype"], max_batch=3, max_seq=min(256, cfg["max_positions"]), max_prefill=32)
    try:
        prompts = [tiny.random_tokens(n, cfg["vocab"], 900 + n) for n in (9, 70, 33)]
        want = [plain_greedy(p) for p in prompts]
        same(eng.generate(prompts[0], n_new), want[0][0], want[0][1], "generate")
        ids = [eng.add_request(p, n_new) for p in prompts]        # portions of 32 tokens beside decoding requests
        done = eng.run()
        for i, rid in enumerate(ids):
            same(done[rid], want[i][0], want[i][1], f"scheduler request {i}")
    finally:
        eng.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("layers", ["recurrent only", "attention only", "latent only", "one layer"])
def test_models_of_one_kind_of_layer(layers, dtype, tmp_path):
    """A model without any cache (recurrent layers only), models without any state (attention only, the second layer
    reading the first one's cache; latent attention only) and a single layer: whole, in portions and token by token."""
    from hipinfer_b200.engine.runner import ModelRunner

    cfg = tm.model(90, 64, {"recurrent only": [tm.gla(2, 32, 32, 4.0, ff=48), tm.gla(4, 16, 8, 32.0)],
                            "attention only": [tm.attn(2, 1, 32, 64, 16, chunk=30, ff=48), tm.attn(2, 1, 32, 64, 16, chunk=12, kv_from=0)],
                            "latent only": [tm.latent(2, 16, 16, 16, 32, 32, ff=32), tm.latent(4, 8, 4, 8, 16, 48)],
                            "one layer": [tm.attn(4, 4, 16, 16, 16, ff=32)]}[layers], max_positions=200)
    folder, cfg, w = tm.make_folder(tmp_path / "m", cfg, seed=3, dtype=torch.float32 if dtype == "float32" else torch.bfloat16)
    reqs = {"a": tiny.random_tokens(150, 90, 1), "b": tiny.random_tokens(37, 90, 2)}
    model = plain.PlainVegodra(cfg, w)
    ref = {}
    for rid, toks in reqs.items():
        model.reset()
        ref[rid] = model.forward(toks)
    runner = ModelRunner.from_folder(folder, dtype=dtype, page_size=16, num_pages=24, max_num_seqs=2)
    st = tiny.RunnerStepper(runner)
    for plan in (tiny.plan_whole(reqs), tiny.plan_portions(reqs, (5, 2, 40, 1, 17)), tiny.plan_tail_decode(reqs, 20),
                 tiny.plan_mixed(reqs, 4, max_live=2)):
        got = tiny.run_plan(st, reqs, plan)
        for rid in reqs:
            _close(got[rid], ref[rid], dtype, f"{layers} {rid}")
    assert not runner.live_requests()


def test_pages_behind_every_reader_s_chunk_are_given_back(tmp_path):
    """A cache whose writer and reader look back to the start of chunks of 32 and 48: while a request runs, the pages before
    the earlier of the two starts return to the pool, and the logits stay those of the plain model."""
    from hipinfer_b200.engine.runner import ModelRunner

    cfg = tm.model(90, 64, [tm.attn(2, 1, 32, 32, 16, chunk=32, ff=48), tm.attn(2, 1, 32, 32, 16, chunk=48, kv_from=0)], max_positions=400)
    folder, cfg, w = tm.make_folder(tmp_path / "m", cfg, seed=5, dtype=torch.float32)
    toks = tiny.random_tokens(300, 90, 4)
    ref = plain.PlainVegodra(cfg, w).forward(toks)
    runner = ModelRunner.from_folder(folder, dtype="float32", page_size=16, num_pages=8, max_num_seqs=1)     # 128 tokens of pages
    got = tiny.run_plan(tiny.RunnerStepper(runner), {"x": toks}, [[("x", 50)], [("x", 30)]] + [[("x", 1)]] * 40 + [[("x", 60)]] * 3)
    _close(got["x"], ref, "float32", "300 tokens through 128 tokens of pages")
    assert not runner.live_requests()


def _random_config(seed):
    """A configuration drawn from sizes that resemble real layers in the small: every kind of layer at least once, in a
    random order, a reader where an attention layer precedes it."""
    import random

    rng = random.Random(seed)
    pick = rng.choice
    width = pick([64, 96, 128, 160, 192, 256])
    layers, owners = [], []
    kinds = ["latent", "attn", "gla"] + [pick(["latent", "attn", "gla", "reader"]) for _ in range(rng.randint(1, 4))]
    rng.shuffle(kinds)
    attn_shape = None
    for kind in kinds:
        ff = pick([None, 64, 96, 256, 320])
        if kind == "reader" and not owners:
            kind = "attn"
        if kind == "latent":
            rot_dim = pick([8, 16, 32, 64])
            layers.append(tm.latent(pick([1, 2, 3, 4, 6, 8]), pick([16, 32, 48, 64, 96, 128]), rot_dim, pick([16, 32, 48, 64, 96, 128]),
                                    pick([24, 48, 80, 128]), pick([32, 64, 96, 128, 192, 256]), ff=ff, dims=pick([rot_dim, rot_dim // 2]),
                                    base=pick([100.0, 10000.0, 500000.0])))
        elif kind == "gla":
            layers.append(tm.gla(pick([1, 2, 4]), pick([16, 32, 48, 64, 128]), pick([16, 32, 64, 128]), pick([1.0, 4.0, 16.0]), ff=ff,
                                 rank=pick([4, 16, 24])))
        elif kind == "attn":
            kv = pick([1, 2, 4])
            dim = pick([16, 32, 64, 128])
            attn_shape = dict(heads=kv * pick([1, 2, 3, 4]), kv_heads=kv, dim=dim, vdim=pick([16, 32, 64, 128]), dims=pick([dim, dim // 2, dim // 4]),
                              base=pick([10000.0, 1000000.0]), scale=pick([0.125, 0.3, 1.0 / math.sqrt(dim)]))
            owners.append((len(layers), attn_shape))
            layers.append(tm.attn(chunk=pick([None, 16, 33, 64, 96, 128]), ff=ff, **attn_shape))
        else:
            src, shape = pick(owners)
            layers.append(tm.attn(chunk=pick([None, 16, 33, 64, 96, 128]), kv_from=src, ff=ff, **shape))
    return tm.model(pick([64, 97, 300, 576]), width, layers, eps=pick([1e-5, 1e-6]), max_positions=512)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", list(range(24)))
def test_random_configurations(seed, dtype, tmp_path):
    """Two dozen configurations drawn at random (sizes on either side of every kernel's size steps): whole prompts, the last
    tokens one by one, portions, and a mixed batch, against the plain model."""
    from hipinfer_b200.engine.runner import ModelRunner

    cfg = _random_config(seed)
    folder, cfg, w = tm.make_folder(tmp_path / "m", cfg, seed=seed, dtype=torch.float32 if dtype == "float32" else torch.bfloat16)
    reqs = {"a": tiny.random_tokens(170, cfg["vocab"], 1), "b": tiny.random_tokens(41, cfg["vocab"], 2), "c": tiny.random_tokens(1, cfg["vocab"], 3)}
    model = plain.PlainVegodra(cfg, w)
    ref = {}
    for rid, toks in reqs.items():
        model.reset()
        ref[rid] = model.forward(toks)
    runner = ModelRunner.from_folder(folder, dtype=dtype, page_size=16, num_pages=30, max_num_seqs=3)
    st = tiny.RunnerStepper(runner)
    for plan in (tiny.plan_whole(reqs), tiny.plan_tail_decode(reqs, 24), tiny.plan_portions(reqs, (17, 2, 40, 1, 33)),
                 tiny.plan_mixed(reqs, seed, max_live=3)):
        got = tiny.run_plan(st, reqs, plan)
        for rid in reqs:
            _close(got[rid], ref[rid], dtype, f"random configuration {seed} {rid}")
    assert not runner.live_requests()
