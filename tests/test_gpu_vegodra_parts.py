"""Each mechanism of the Vegodra design alone: the kernel against the plain function of tests/plain_vegodra.py, in 32-bit
and in bfloat16, at sizes the vectorised paths take and at sizes they do not, with inputs made so that a fault shows
(a far key that dominates, a key one position outside the mask with a huge score, a sink that matters)."""
import math
from types import SimpleNamespace

import pytest
import torch

import plain_vegodra as plain

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
TOL = {torch.float32: 2e-5, torch.bfloat16: 1.2e-2}


def rnd(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


def close(got, want, dtype, what=""):
    got, want = got.double().cpu(), want.double()
    err, ref = float((got - want).abs().max()), float(want.abs().max())
    assert torch.isfinite(got).all(), what
    assert err <= TOL[dtype] * ref, f"{what}: {err:.3e} > {TOL[dtype]:.0e} * {ref:.3e}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H", [50, 200, 4104])
def test_layer_norm_with_bias(dtype, H):
    from hipinfer_b200.kernels import ops

    x = rnd(9, H, seed=1) * 3 + 5.0
    w, b = (1 + 0.3 * rnd(H, seed=2)).to(dtype), rnd(H, seed=3).to(dtype)
    out = torch.empty(9, H, dtype=dtype, device=DEV)
    ops.layernorm(x.to(DEV), w.to(DEV), 1e-5, out, bias=b.to(DEV))
    close(out, plain.layer_norm(x.double(), w.double(), b.double(), 1e-5), dtype, "all rows")
    rows = torch.tensor([7, 0, 3], dtype=torch.int32)
    out32 = torch.empty(3, H, dtype=torch.float32, device=DEV)            # a norm inside the 32-bit stream
    ops.layernorm(x.to(DEV), w.to(DEV), 1e-5, out32, rows.to(DEV), bias=b.to(DEV))
    close(out32, plain.layer_norm(x[rows.long()].double(), w.double(), b.double(), 1e-5), torch.float32, "picked rows, 32-bit out")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("I,group", [(64, 16), (56, 56), (7, 7)])
def test_gelu_gate(dtype, I, group):
    from hipinfer_b200.kernels import ops

    g, u = rnd(5, I, seed=1) * 3, rnd(5, I, seed=2)
    gu = torch.stack([g.view(5, I // group, group), u.view(5, I // group, group)], 2).reshape(5, 2 * I)
    out = torch.empty(5, I, dtype=dtype, device=DEV)
    ops.gated_act(gu.to(DEV), out, group, "gelu_tanh")
    close(out, plain.gelu_tanh(g.double()) * u.double(), dtype)
    ops.gated_act(gu.to(DEV), out, group, "silu")
    close(out, torch.nn.functional.silu(g.double()) * u.double(), dtype, "silu")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,D,E,rot,pairing,unit", [(4, 2, 32, 16, 8, "half", True), (3, 3, 10, 6, 10, "half", True),
                                                      (2, 1, 64, 64, 64, "interleaved", False), (5, 1, 24, 40, 0, "half", True),
                                                      (2, 2, 12, 12, 6, "interleaved", True)])
def test_rotation_unit_norm_and_cache_write(dtype, H, G, D, E, rot, pairing, unit):
    from hipinfer_b200.kernels import ops

    T, ps, pages, base, eps = 7, 4, 6, 1000.0, 1e-5
    extra = 3                                                    # other columns behind v (a gate)
    proj = rnd(T, H * D + G * (D + E) + extra, seed=1)
    pos = torch.tensor([0, 1, 2, 77, 500, 3, 4], dtype=torch.int32)
    slots = torch.tensor([17, 3, 0, 19, 8, 9, 23], dtype=torch.int32)
    table = ops.shared_rope_table(rot, base, 512, DEV)
    kc = torch.zeros(pages, G, ps, D, dtype=dtype, device=DEV)
    vc = torch.zeros(pages, G, ps, E, dtype=dtype, device=DEV)
    q = torch.empty(T, H * D, dtype=dtype, device=DEV)
    ops.rope_norm_store(proj.to(DEV), (0, H * D, H * D + G * D), pos.to(DEV), slots.to(DEV), table, rot, pairing, unit, eps, q, kc, vc,
                        H, G, D, E, ps)
    fin = (lambda t: plain.rms_div(t, eps)) if unit else (lambda t: t)
    q_want = fin(plain.rotate(proj[:, :H * D].double().view(T, H, D), pos, rot, base, pairing))
    k_want = fin(plain.rotate(proj[:, H * D:H * D + G * D].double().view(T, G, D), pos, rot, base, pairing))
    v_want = proj[:, H * D + G * D:H * D + G * (D + E)].double().view(T, G, E)
    close(q.view(T, H, D), q_want, dtype, "q")
    for t, s in enumerate(slots.tolist()):
        close(kc[s // ps, :, s % ps], k_want[t], dtype, f"k of row {t}")
        close(vc[s // ps, :, s % ps], v_want[t], dtype, f"v of row {t}")
    assert int((vc.float().abs().sum(-1) > 0).sum()) == T * G              # nothing else was written
    q2 = torch.empty(T, H * D, dtype=dtype, device=DEV)                     # q alone (a layer that reads another's cache)
    ops.rope_norm_store(proj.to(DEV), (0, 0, 0), pos.to(DEV), None, table, rot, pairing, unit, eps, q2, None, None, H, G, D, E, ps)
    assert torch.equal(q2, q)


# ------------------------------------------------------------------------------------------ attention with a mask
def _paged(keys, values, ps, dtype, seed=0, alias=False):
    """keys [R][n_r, G, D], values [R][n_r, G, E] of R requests -> (k plane, v plane, block table) with pages handed out in a
    shuffled order. alias: values are the first columns of the key rows (one plane)."""
    R = len(keys)
    n_pages = [-(-k.shape[0] // ps) for k in keys]
    order = torch.randperm(sum(n_pages) + 3, generator=torch.Generator().manual_seed(seed)).tolist()
    G, D = keys[0].shape[1:]
    E = values[0].shape[2]
    kc = torch.zeros(len(order), G, ps, D, dtype=dtype)
    vc = kc if alias else torch.zeros(len(order), G, ps, E, dtype=dtype)
    bt = torch.full((R, max(n_pages)), -1, dtype=torch.int32)
    it = iter(order)
    for r in range(R):
        for lp in range(n_pages[r]):
            page = next(it)
            bt[r, lp] = page
            n = min(ps, keys[r].shape[0] - lp * ps)
            kc[page, :, :n] = keys[r][lp * ps:lp * ps + n].transpose(0, 1).to(dtype)
            if not alias:
                vc[page, :, :n] = values[r][lp * ps:lp * ps + n].transpose(0, 1).to(dtype)
    return kc.to(DEV), (kc.to(DEV) if alias else vc.to(DEV)), bt.to(DEV)


def _attend_plain(q, k, v, p, H, G, scale, mask, window, keep, chunk, sink, gate, per_head):
    """One row at position p against its request's keys k [n, G, D] and values v [n, G, E]."""
    n = k.shape[0]
    j = torch.arange(n)
    seen = j <= p
    if mask == "window":
        seen = seen & ((p - j < window) | (j < keep))
    elif mask == "chunk":
        seen = seen & (j // chunk == p // chunk)
    out = []
    for h in range(H):
        g = h // (H // G)
        s = (k[:, g] @ q[h]) * scale
        w = plain.softmax_with_sink(s[None], seen[None], None if sink is None else sink[h])[0]
        o = w @ v[:, g]
        if gate is not None:
            o = o * torch.sigmoid(gate[h] if per_head else gate[h * o.numel():(h + 1) * o.numel()])
        out.append(o)
    return torch.cat(out)


CASES = [  # H, G, D, E, mask, window, keep, chunk, sink, gate, lengths
    (8, 2, 64, 64, "chunk", 0, 0, 80, True, "head", [400, 97]),
    (4, 4, 8, 8, "chunk", 0, 0, 1, True, "head", [40, 3]),
    (3, 1, 10, 6, "chunk", 0, 0, 5, False, "none", [33]),
    (8, 2, 32, 48, "chunk", 0, 0, 70, True, "element", [700, 150]),
    (2, 1, 160, 128, "causal", 0, 0, 0, False, "none", [600, 65]),
    (4, 2, 16, 24, "window", 20, 3, 0, True, "head", [130, 64]),
    (16, 1, 40, 40, "causal", 0, 0, 0, False, "element", [90]),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", CASES, ids=lambda c: f"{c[4]}{c[7] or c[5] or ''}-h{c[0]}g{c[1]}-d{c[2]}e{c[3]}")
def test_masked_attention_rows(dtype, case):
    """Every row of two requests (prompt rows and single rows alike are rows to this kernel) over shuffled pages."""
    from hipinfer_b200.kernels import ops

    H, G, D, E, mask, window, keep, chunk, has_sink, gate_kind, lens = case
    ps, scale = 16, 1.7 / math.sqrt(D)
    keys = [rnd(n, G, D, seed=10 + r) for r, n in enumerate(lens)]
    vals = [rnd(n, G, E, seed=20 + r) for r, n in enumerate(lens)]
    kc, vc, bt = _paged(keys, vals, ps, dtype, seed=3)
    rows = [(r, p) for r, n in enumerate(lens) for p in sorted(set([0, 1, n // 2, n - 2, n - 1] + list(range(max(0, n - 70), n, 7))) - {-1})]
    T = len(rows)
    q = rnd(T, H * D, seed=5)
    sink = rnd(H, seed=6) * 2 if has_sink else None
    n_gate = {"none": 0, "head": H, "element": H * E}[gate_kind]
    gate = rnd(T, 5 + n_gate, seed=7) * 2 if n_gate else None
    batch = SimpleNamespace(block_tables=[bt], row_request=torch.tensor([r for r, _ in rows], dtype=torch.int32, device=DEV),
                            positions=torch.tensor([p for _, p in rows], dtype=torch.int32, device=DEV), max_pos=max(lens) - 1)
    for out_dtype in ({dtype, torch.float32}):
        out = torch.empty(T, H * E, dtype=out_dtype, device=DEV)
        ops.attention_masked(q.to(dtype).to(DEV), kc, vc, batch, 0, out, H, G, D, E, ps, scale, mask, window, keep, chunk,
                             None if sink is None else sink.to(DEV), None if gate is None else gate.to(DEV), 5, gate_kind == "head")
        for t, (r, p) in enumerate(rows):
            want = _attend_plain(q[t].to(dtype).double().view(H, D), keys[r].to(dtype).double(), vals[r].to(dtype).double(), p, H, G,
                                 scale, mask, window, keep, chunk, None if sink is None else sink.double(),
                                 None if gate is None else gate[t, 5:].double(), gate_kind == "head")
            close(out[t], want, dtype, f"row {t} (request {r}, position {p}, out {out_dtype})")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_far_key_dominates_and_a_key_outside_the_chunk_does_not_leak(dtype):
    """One key far back is made to carry nearly all the weight of a row: the result is its value. A key one position
    before the row's chunk is given a far larger score still: nothing of its value may show. And a sink far above every
    score takes all the weight: the result is near zero."""
    from hipinfer_b200.kernels import ops

    H, G, D, E, ps, chunk, n = 2, 1, 16, 8, 16, 640, 1300
    k, v = rnd(n, G, D, seed=1) * 0.1, rnd(n, G, E, seed=2)
    qv = rnd(H * D, seed=3)
    unit = qv.view(H, D)[0] / qv.view(H, D)[0].norm()
    far, outside, p = 645, 639, 1270                  # the chunk of p is [640, 1280)
    k[far, 0] = unit * 30
    k[outside, 0] = unit * 300
    qv.view(H, D)[0] = unit * 3
    kc, vc, bt = _paged([k], [v], ps, dtype, seed=9)
    batch = SimpleNamespace(block_tables=[bt], row_request=torch.zeros(1, dtype=torch.int32, device=DEV),
                            positions=torch.tensor([p], dtype=torch.int32, device=DEV), max_pos=n - 1)
    out = torch.empty(1, H * E, dtype=torch.float32, device=DEV)
    ops.attention_masked(qv.view(1, -1).to(dtype).to(DEV), kc, vc, batch, 0, out, H, G, D, E, ps, 1.0, "chunk", chunk=chunk,
                         sink=torch.zeros(H, device=DEV))
    close(out[0, :E], v[far, 0].to(dtype), dtype, "the far key's value")
    # causal instead: the key at 639 is seen and wins
    ops.attention_masked(qv.view(1, -1).to(dtype).to(DEV), kc, vc, batch, 0, out, H, G, D, E, ps, 1.0, "causal")
    close(out[0, :E], v[outside, 0].to(dtype), dtype, "without the chunk mask")
    # the sink: scores of at most a few units (the far key's is -90 now) against a sink of 40
    q2 = -qv.view(1, -1) * 1.0
    ops.attention_masked(q2.to(dtype).to(DEV), kc, vc, batch, 0, out, H, G, D, E, ps, 1.0, "chunk", chunk=chunk,
                         sink=torch.full((H,), 40.0, device=DEV))
    assert float(out[0, :E].abs().max()) < 1e-6
    ops.attention_masked(q2.to(dtype).to(DEV), kc, vc, batch, 0, out, H, G, D, E, ps, 1.0, "chunk", chunk=chunk)
    assert float(out[0, :E].abs().max()) > 1e-2       # without a sink the weights sum to one


# ------------------------------------------------------------------------------------------ latent attention
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("Rq,R,Dr,rot", [(72, 136, 32, 32), (14, 20, 6, 4), (300, 520, 64, 64)])
def test_latents_into_the_cache(dtype, Rq, R, Dr, rot):
    from hipinfer_b200.kernels import ops

    T, ps, pages, base, eps = 6, 4, 5, 10000.0, 1e-5
    proj = rnd(T, 2 + Rq + R + Dr + 7, seed=1) * 2
    wq, wc = (1 + 0.3 * rnd(Rq, seed=2)).to(dtype), (1 + 0.3 * rnd(R, seed=3)).to(dtype)
    pos = torch.tensor([0, 1, 300, 2, 3, 4], dtype=torch.int32)
    slots = torch.tensor([13, 3, 0, 19, 8, 9], dtype=torch.int32)
    table = ops.shared_rope_table(rot, base, 512, DEV)
    cache = torch.zeros(pages, 1, ps, R + Dr, dtype=dtype, device=DEV)
    cq = torch.empty(T, Rq, dtype=dtype, device=DEV)
    ops.latent_prepare(proj.to(DEV), (2, 2 + Rq, 2 + Rq + R), wq.to(DEV), wc.to(DEV), pos.to(DEV), slots.to(DEV), table, rot, eps, cq,
                       cache, Rq, R, Dr, ps)
    p = proj.double()
    close(cq, plain.rms_div(p[:, 2:2 + Rq], eps) * wq.double(), dtype, "query latent")
    c_want = plain.rms_div(p[:, 2 + Rq:2 + Rq + R], eps) * wc.double()
    kr_want = plain.rotate(p[:, 2 + Rq + R:2 + Rq + R + Dr], pos, rot, base, "interleaved")
    for t, s in enumerate(slots.tolist()):
        close(cache[s // ps, 0, s % ps, :R], c_want[t], dtype, f"latent of row {t}")
        close(cache[s // ps, 0, s % ps, R:], kr_want[t], dtype, f"rotated key part of row {t}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T", [1, 9, 70])
def test_products_head_by_head(dtype, T):
    from hipinfer_b200.kernels import ops

    H, K, N, tail, rot, base = 3, 24, 150, 6, 4, 10000.0
    a, wt = rnd(T, 2 + H * (K + tail), seed=1), rnd(H, K, N, seed=2, scale=0.2).to(dtype)
    pos = torch.arange(5, 5 + T, dtype=torch.int32)
    table = ops.shared_rope_table(rot, base, 512, DEV)
    out = torch.empty(T, H * (N + tail), dtype=dtype, device=DEV)
    ops.heads_linear(a[:, 2:].to(DEV), K + tail, wt.to(DEV), out, N + tail, tail=tail, rot=rot, positions=pos.to(DEV), table=table)
    av = a[:, 2:].double().view(T, H, K + tail)
    want = torch.cat([torch.einsum("thk,hkn->thn", av[..., :K], wt.double()), plain.rotate(av[..., K:], pos, rot, base, "interleaved")], -1)
    close(out.view(T, H, N + tail), want, dtype, "with a rotated tail")
    gate = rnd(T, 4 + H * N, seed=3)
    out = torch.empty(T, H * N, dtype=dtype, device=DEV)
    ops.heads_linear(a[:, 2:].to(DEV), K + tail, wt.to(DEV), out, N, gate=gate.to(DEV), gate_offset=4)
    want = torch.einsum("thk,hkn->thn", av[..., :K], wt.double()) * torch.sigmoid(gate[:, 4:].double()).view(T, H, N)
    close(out.view(T, H, N), want, dtype, "with a gate")


# ------------------------------------------------------------------------------------------ gated linear attention
def _gla_plain(proj, z, ab, nw, state, lens, slots, H, D, E, tau, eps):
    """Rows of several requests, one after the other, with the recurrence written out; returns (out, states)."""
    out = torch.zeros(proj.shape[0], H * E, dtype=torch.float64)
    state = state.clone().double()
    t = 0
    HD, HE = H * D, H * E
    for n, s in zip(lens, slots):
        for _ in range(n):
            row = proj[t].double()
            q, k = row[:HD].view(H, D) / math.sqrt(D), row[HD:2 * HD].view(H, D)
            v, g = row[2 * HD:2 * HD + HE].view(H, E), row[2 * HD + HE:2 * HD + 2 * HE]
            alpha = torch.sigmoid(z[t].double() + ab.double()).view(H, D) ** (1.0 / tau)
            state[s] = alpha[:, :, None] * state[s] + k[:, :, None] * v[:, None, :]
            o = torch.einsum("hde,hd->he", state[s], q)
            o = plain.rms_div(o, eps) * nw.double()
            out[t] = o.reshape(-1) * torch.nn.functional.silu(g)
            t += 1
    return out, state


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,D,E,tau", [(4, 48, 24, 8.0), (2, 128, 128, 4.0), (3, 10, 6, 1.0), (1, 64, 256, 2.0), (2, 200, 24, 8.0), (2, 64, 64, 16.0)])
def test_gated_linear_attention(dtype, H, D, E, tau):
    from hipinfer_b200.kernels import ops

    lens, slots, eps = [37, 1, 20], [2, 0, 3], 1e-5
    T, HD, HE = sum(lens), H * D, H * E
    proj, z = rnd(T, 2 * HD + 2 * HE + 3, seed=1), rnd(T, HD, seed=2) * 2
    ab, nw = (1 + rnd(HD, seed=3)).to(dtype), (1 + 0.2 * rnd(E, seed=4)).to(dtype)
    state0 = rnd(4, H, D, E, seed=5) * 0.5              # carried in: the slots are not fresh
    starts = [0, lens[0], lens[0] + lens[1]]
    batch = SimpleNamespace(n_requests=3, req_q_start=torch.tensor(starts, dtype=torch.int32, device=DEV),
                            req_q_len=torch.tensor(lens, dtype=torch.int32, device=DEV),
                            req_state_slot=torch.tensor(slots, dtype=torch.int32, device=DEV))
    state = state0.clone().to(DEV)
    out = torch.empty(T, HE, dtype=dtype, device=DEV)
    ops.gla(proj.to(DEV), (0, HD, 2 * HD, 2 * HD + HE), z.to(DEV), ab.to(DEV), nw.to(DEV), state, batch, out, H, D, E, tau, eps)
    want, state_want = _gla_plain(proj, z, ab, nw, state0, lens, slots, H, D, E, tau, eps)
    close(out, want, dtype, "outputs")
    close(state, state_want, torch.float32, "states")
    assert torch.equal(state[1].cpu(), state0[1])                            # a slot no request uses is left alone
    # the same rows one token a launch: the same bits (a token's arithmetic does not depend on where a portion starts)
    state2 = state0.clone().to(DEV)
    out2 = torch.empty(T, HE, dtype=dtype, device=DEV)
    t = 0
    for n, s in zip(lens, slots):
        for _ in range(n):
            b1 = SimpleNamespace(n_requests=1, req_q_start=torch.tensor([t], dtype=torch.int32, device=DEV),
                                 req_q_len=torch.tensor([1], dtype=torch.int32, device=DEV),
                                 req_state_slot=torch.tensor([s], dtype=torch.int32, device=DEV))
            ops.gla(proj.to(DEV), (0, HD, 2 * HD, 2 * HD + HE), z.to(DEV), ab.to(DEV), nw.to(DEV), state2, b1, out2, H, D, E, tau, eps)
            t += 1
    assert torch.equal(out2, out) and torch.equal(state2, state)


def test_a_decay_of_one_keeps_and_a_decay_of_zero_forgets():
    """With a large positive pre-activation the state keeps everything (o is the running sum of k v^T applied to q); with a
    large negative one only the current token is left."""
    from hipinfer_b200.kernels import ops

    H, D, E, T = 1, 8, 4, 5
    proj = rnd(T, 2 * D + 2 * E, seed=1)
    proj[:, 2 * D + E:] = 30.0                          # silu(30) = 30: the gate is a constant factor
    nw, eps = torch.ones(E), 0.0
    batch = SimpleNamespace(n_requests=1, req_q_start=torch.zeros(1, dtype=torch.int32, device=DEV),
                            req_q_len=torch.tensor([T], dtype=torch.int32, device=DEV),
                            req_state_slot=torch.zeros(1, dtype=torch.int32, device=DEV))
    for zval, keep in ((40.0, True), (-40.0, False)):
        state = torch.zeros(1, H, D, E, device=DEV)
        out = torch.empty(T, E, dtype=torch.float32, device=DEV)
        ops.gla(proj.to(DEV), (0, D, 2 * D, 2 * D + E), torch.full((T, D), zval, device=DEV), torch.zeros(D, device=DEV), nw.to(DEV),
                state, batch, out, H, D, E, 1.0, eps)
        q, k, v = proj[:, :D].double() / math.sqrt(D), proj[:, D:2 * D].double(), proj[:, 2 * D:2 * D + E].double()
        S = torch.zeros(D, E, dtype=torch.float64)
        for t in range(T):
            S = (S if keep else 0 * S) + k[t][:, None] * v[t][None, :]
            o = S.T @ q[t]
            close(out[t], o / o.pow(2).mean().sqrt() * 30.0, torch.float32, f"token {t}, z = {zval}")


@pytest.mark.parametrize("case", [(12, 4, 64, 64, "chunk", 0, 0, 112, True, "head"), (8, 2, 128, 128, "chunk", 0, 0, 200, True, "element"),
                                  (4, 4, 64, 48, "causal", 0, 0, 0, False, "element"), (4, 1, 32, 32, "window", 70, 5, 0, True, "head"),
                                  (2, 2, 48, 32, "chunk", 0, 0, 64, False, "none")],
                         ids=lambda c: f"{c[4]}{c[7] or c[5] or ''}-h{c[0]}g{c[1]}-d{c[2]}e{c[3]}")
def test_masked_attention_portions_on_tensor_cores(case):
    """Portions of 16 rows and more run on the tensor-core kernel, the other rows of the same step on the row kernel:
    a portion behind a long context (its first rows look back into other chunks and pages), a portion from position 0
    whose last tile is ragged, and two single rows."""
    from hipinfer_b200.kernels import ops

    H, G, D, E, mask, window, keep, chunk, has_sink, gate_kind = case
    dtype, ps, scale = torch.bfloat16, 16, 1.7 / math.sqrt(D)
    ctx, new = [300, 0, 77, 5], [150, 83, 1, 1]
    lens = [c + n for c, n in zip(ctx, new)]
    keys = [rnd(n, G, D, seed=10 + r) for r, n in enumerate(lens)]
    vals = [rnd(n, G, E, seed=20 + r) for r, n in enumerate(lens)]
    kc, vc, bt = _paged(keys, vals, ps, dtype, seed=3)
    rows = [(r, p) for r in range(4) for p in range(ctx[r], lens[r])]
    T = len(rows)
    q = rnd(T, H * D, seed=5)
    sink = rnd(H, seed=6) * 2 if has_sink else None
    n_gate = {"none": 0, "head": H, "element": H * E}[gate_kind]
    gate = rnd(T, 8 + n_gate, seed=7) * 2 if n_gate else None
    starts = [sum(new[:r]) for r in range(4)]
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    batch = SimpleNamespace(block_tables=[bt], row_request=i32([r for r, _ in rows]), positions=i32([p for _, p in rows]),
                            max_pos=max(lens) - 1, n_requests=4, max_q_len=max(new), h_q_len=new, req_q_start=i32(starts),
                            req_q_len=i32(new), req_ctx_len=i32(ctx))
    out = torch.full((T, H * E), float("nan"), dtype=dtype, device=DEV)
    ops.attention_masked(q.to(dtype).to(DEV), kc, vc, batch, 0, out, H, G, D, E, ps, scale, mask, window, keep, chunk,
                         None if sink is None else sink.to(DEV), None if gate is None else gate.to(DEV), 8, gate_kind == "head")
    rows_only = torch.empty_like(out)
    ops.attention_masked(q.to(dtype).to(DEV), kc, vc, batch, 0, rows_only, H, G, D, E, ps, scale, mask, window, keep, chunk,
                         None if sink is None else sink.to(DEV), None if gate is None else gate.to(DEV), 8, gate_kind == "head",
                         force_rows=True)
    for t, (r, p) in enumerate(rows):
        want = _attend_plain(q[t].to(dtype).double().view(H, D), keys[r].to(dtype).double(), vals[r].to(dtype).double(), p, H, G, scale,
                             mask, window, keep, chunk, None if sink is None else sink.double(),
                             None if gate is None else gate[t, 8:].double(), gate_kind == "head")
        close(out[t], want, dtype, f"row {t} (request {r}, position {p})")
        close(rows_only[t], want, dtype, f"row kernel, row {t}")


@pytest.mark.parametrize("H,D,E", [(5, 160, 64), (32, 288, 256), (3, 48, 32), (16, 80, 64), (1, 32, 16), (40, 96, 64), (9, 176, 128)])
def test_single_rows_whose_values_are_a_prefix_of_the_key_rows(H, D, E):
    """Latent attention's pass over the cache: one kv head, keys D wide, values their first E columns (one plane), 32-bit
    result; rows at the first positions, at tile and split borders and far in; sizes on both sides of the kernels'
    shared-memory steps and head tiles."""
    from hipinfer_b200.kernels import ops

    dtype, ps, scale = torch.bfloat16, 16, 1.3 / math.sqrt(D)
    lens = [530, 70]
    keys = [rnd(n, 1, D, seed=10 + r) for r, n in enumerate(lens)]
    kc, _, bt = _paged(keys, [k[..., :E] for k in keys], ps, dtype, seed=3, alias=True)
    rows = [(0, p) for p in (0, 1, 63, 64, 255, 256, 257, 511, 512, 529)] + [(1, p) for p in (0, 15, 16, 69)]
    T = len(rows)
    q = rnd(T, H * D, seed=5)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    batch = SimpleNamespace(block_tables=[bt], row_request=i32([r for r, _ in rows]), positions=i32([p for _, p in rows]), max_pos=max(lens) - 1)
    for plain_kernel in (False, True):
        out = torch.empty(T, H * E, dtype=torch.float32, device=DEV)
        ops.attention_masked(q.to(dtype).to(DEV), kc, kc, batch, 0, out, H, 1, D, E, ps, scale, "causal", force_plain=plain_kernel)
        for t, (r, p) in enumerate(rows):
            kk = keys[r].to(dtype).double()
            want = _attend_plain(q[t].to(dtype).double().view(H, D), kk, kk[..., :E], p, H, 1, scale, "causal", 0, 0, 0, None, None, False)
            close(out[t], want, dtype, f"row {t} (request {r}, position {p}, plain kernel {plain_kernel})")
