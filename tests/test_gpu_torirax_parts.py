"""Each mechanism of the Torirax design alone: the kernel against the plain function of tests/plain_torirax.py, in
32-bit and in bfloat16, at sizes the vectorised and register paths take and at sizes they do not."""
import math
from types import SimpleNamespace

import pytest
import torch

import plain_torirax as plain

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
def test_layer_norm(dtype, H):
    from hipinfer_b200.kernels import ops

    x = rnd(9, H, seed=1) * 3 + 5.0                      # a mean far from zero: the variance is of the deviations
    w = (1 + 0.3 * rnd(H, seed=2)).to(dtype)
    out = torch.empty(9, H, dtype=dtype, device=DEV)
    ops.layernorm(x.to(DEV), w.to(DEV), 1e-5, out)
    close(out, plain.layer_norm(x.double(), w.double(), 1e-5), dtype, "all rows")
    rows = torch.tensor([7, 0, 3], dtype=torch.int32)
    out = torch.empty(3, H, dtype=dtype, device=DEV)
    ops.layernorm(x.to(DEV), w.to(DEV), 1e-5, out, rows.to(DEV))
    close(out, plain.layer_norm(x[rows.long()].double(), w.double(), 1e-5), dtype, "picked rows")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_scaled_embedding_with_positions(dtype):
    from hipinfer_b200.kernels import ops

    table, ptab = rnd(30, 40, seed=1).to(dtype), rnd(64, 40, seed=2).to(dtype)
    tok = torch.tensor([3, 29, 0, 3, 7], dtype=torch.int32)
    pos = torch.tensor([0, 63, 5, 6, 1], dtype=torch.int32)
    x = torch.empty(5, 40, dtype=torch.float32, device=DEV)
    ops.embedding_scaled(table.to(DEV), tok.to(DEV), x, 2.5, ptab.to(DEV), pos.to(DEV))
    want = table.double()[tok.long()] * 2.5 + ptab.double()[pos.long()]
    close(x, want, torch.float32, "scaled, with positions")
    ops.embedding_scaled(table.to(DEV), tok.to(DEV), x, 1.0)
    close(x, table.double()[tok.long()], torch.float32, "plain gather")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_polynorm(dtype):
    from hipinfer_b200.kernels import ops

    z = rnd(6, 333, seed=3) * 2
    coef = [0.7, -0.4, 0.25, 0.1]
    out = torch.empty(6, 333, dtype=dtype, device=DEV)
    ops.polynorm(z.to(DEV), coef, 1e-6, out)
    close(out, plain.polynorm(z.double(), coef, 1e-6), dtype)
    # every term matters: with one coefficient alone the result is that term
    for i in range(3):
        c = [0.0] * 4
        c[i] = 1.0
        ops.polynorm(z.to(DEV), c, 1e-6, out)
        close(out, plain.rms_div(z.double() ** (i + 1), 1e-6), dtype, f"term {i + 1}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M", [3, 70])
def test_product_with_a_scale_vector_added_into_the_stream(dtype, M):
    from hipinfer_b200.kernels import ops

    a, w, s = rnd(M, 72, seed=1).to(dtype), rnd(40, 72, seed=2, scale=0.2).to(dtype), (0.5 + torch.rand(40)).to(dtype)
    x0 = rnd(M, 40, seed=3)
    x = x0.clone().to(DEV)
    ops.linear_scaled_add(a.to(DEV), ops.Weight(w.to(DEV)), x, s.to(DEV))
    close(x, x0.double() + s.double() * (a.double() @ w.double().T), torch.float32 if dtype == torch.float32 else dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_bias_and_cache_write_without_rotation(dtype):
    from hipinfer_b200.kernels import ops

    T, nq, G, kw, vw, ps, pages = 7, 24, 2, 10, 6, 4, 5
    qkv = rnd(T, nq + G * (kw + vw), seed=1)
    bq, bk, bv = (rnd(n, seed=s).to(dtype) for n, s in ((nq, 2), (G * kw, 3), (G * vw, 4)))
    slots = torch.tensor([17, 3, 0, 19, 8, 9, 10], dtype=torch.int32)
    kc = torch.zeros(pages, G, ps, kw, dtype=dtype, device=DEV)
    vc = torch.zeros(pages, G, ps, vw, dtype=dtype, device=DEV)
    q = torch.empty(T, nq, dtype=dtype, device=DEV)
    ops.qkv_bias_store(qkv.to(DEV), bq.to(DEV), bk.to(DEV), bv.to(DEV), slots.to(DEV), q, kc, vc, nq, G, kw, vw, ps)
    close(q, qkv[:, :nq].double() + bq.double(), dtype, "q")
    k_want = (qkv[:, nq:nq + G * kw].double() + bk.double()).view(T, G, kw)
    v_want = (qkv[:, nq + G * kw:].double() + bv.double()).view(T, G, vw)
    for t, s in enumerate(slots.tolist()):
        close(kc[s // ps, :, s % ps], k_want[t], dtype, f"k of row {t}")
        close(vc[s // ps, :, s % ps], v_want[t], dtype, f"v of row {t}")
    assert int((kc.float().abs().sum(-1) > 0).sum()) == T * G              # nothing else was written
    # q alone (a layer that reads another layer's cache)
    q2 = torch.empty(T, nq, dtype=dtype, device=DEV)
    ops.qkv_bias_store(qkv[:, :nq].to(DEV).contiguous(), bq.to(DEV), None, None, None, q2, None, None, nq, G, kw, vw, ps)
    assert torch.equal(q2, q)


# ------------------------------------------------------------------------------------------ the delta rule
def _delta_reference(proj, w_raw, w0, ab, nw, state, lens, slots, heads, D, eps):
    """Rows of several requests, one after the other, with the plain one-token function; returns (out, states)."""
    HD = heads * D
    out = torch.zeros(proj.shape[0], HD, dtype=torch.float64)
    state = state.clone().double()
    t = 0
    for n, s in zip(lens, slots):
        for _ in range(n):
            row = proj[t].double()
            r, k, v, a_raw, g = (row[i * HD:(i + 1) * HD].view(heads, D) for i in range(5))
            w = torch.exp(-math.exp(-0.5) * torch.sigmoid(w_raw[t].double() + w0.double())).view(heads, D)
            a = torch.sigmoid(a_raw + ab.double().view(heads, D))
            o = torch.zeros(heads, D, dtype=torch.float64)
            for h in range(heads):
                state[s, h], o[h] = plain.delta_rule_step(state[s, h], r[h], k[h], v[h], w[h], a[h])
            out[t] = (plain.rms_div(o, eps).reshape(HD) * nw.double() * torch.sigmoid(g.reshape(HD)))
            t += 1
    return out, state


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads, D, force_any", [(2, 32, False), (3, 64, False), (1, 128, False), (2, 48, False), (3, 20, False),
                                                 (2, 64, True)])
def test_delta_rule_against_token_by_token(dtype, heads, D, force_any):
    from hipinfer_b200.kernels import ops

    HD, lens, slots = heads * D, [5, 1, 23, 2], [3, 0, 2, 5]
    T = sum(lens)
    proj = rnd(T, 5 * HD + 4, seed=1)                       # four more columns behind, as a fused projection leaves them
    w_raw = rnd(T, HD, seed=2) * 2
    w0, ab, nw = (rnd(HD, seed=s).to(dtype) for s in (3, 4, 5))
    state0 = rnd(6, heads, D, D, seed=6) * 0.3               # the requests continue from states that are not zero
    state = state0.clone().to(DEV)
    starts = [sum(lens[:i]) for i in range(len(lens))]
    batch = SimpleNamespace(req_q_start=torch.tensor(starts, dtype=torch.int32, device=DEV),
                            req_q_len=torch.tensor(lens, dtype=torch.int32, device=DEV),
                            req_state_slot=torch.tensor(slots, dtype=torch.int32, device=DEV), n_requests=len(lens))
    out = torch.empty(T, HD, dtype=dtype, device=DEV)
    ops.delta_rule(proj.to(DEV), (0, HD, 2 * HD, 3 * HD, 4 * HD), w_raw.to(DEV), w0.to(DEV), ab.to(DEV), nw.to(DEV), state,
                   batch, out, heads, D, math.exp(-0.5), 1e-6, 1e-5, force_any=force_any)
    want, state_want = _delta_reference(proj, w_raw, w0, ab, nw, state0, lens, slots, heads, D, 1e-5)
    close(out, want, dtype, "outputs")
    close(state, state_want, torch.float32, "states")
    assert torch.equal(state[1].cpu(), state0[1]) and torch.equal(state[4].cpu(), state0[4])        # slots of no request

    # the same rows one token a launch give the same bits: the state carries everything
    state = state0.clone().to(DEV)
    out1 = torch.empty(T, HD, dtype=dtype, device=DEV)
    t = 0
    for n, s, st in zip(lens, slots, starts):
        for i in range(n):
            b = SimpleNamespace(req_q_start=torch.tensor([st + i], dtype=torch.int32, device=DEV),
                                req_q_len=torch.tensor([1], dtype=torch.int32, device=DEV),
                                req_state_slot=torch.tensor([s], dtype=torch.int32, device=DEV), n_requests=1)
            ops.delta_rule(proj.to(DEV), (0, HD, 2 * HD, 3 * HD, 4 * HD), w_raw.to(DEV), w0.to(DEV), ab.to(DEV), nw.to(DEV),
                           state, b, out1, heads, D, math.exp(-0.5), 1e-6, 1e-5, force_any=force_any)
    assert torch.equal(out1, out)


def test_delta_rule_register_and_shared_memory_kernels_agree():
    from hipinfer_b200.kernels import ops

    heads, D, T = 2, 64, 40
    HD = heads * D
    proj, w_raw = rnd(T, 5 * HD, seed=1).to(DEV), rnd(T, HD, seed=2).to(DEV)
    vec = [rnd(HD, seed=s).to(DEV) for s in (3, 4, 5)]
    batch = SimpleNamespace(req_q_start=torch.tensor([0], dtype=torch.int32, device=DEV),
                            req_q_len=torch.tensor([T], dtype=torch.int32, device=DEV),
                            req_state_slot=torch.tensor([0], dtype=torch.int32, device=DEV), n_requests=1)
    res = []
    for any_ in (False, True):
        st = torch.zeros(1, heads, D, D, device=DEV)
        out = torch.empty(T, HD, device=DEV)
        ops.delta_rule(proj, (0, HD, 2 * HD, 3 * HD, 4 * HD), w_raw, *vec, st, batch, out, heads, D, 0.6, 1e-6, 1e-5, force_any=any_)
        res.append((out, st))
    close(res[0][0], res[1][0].double().cpu(), torch.float32)
    close(res[0][1], res[1][1].double().cpu(), torch.float32)


# ------------------------------------------------------------------------------------------ attention with a window
def _paged(k, v, G, ps, seed):
    """k [n, G, kw], v [n, G, vw] of one request into scrambled pages; returns (k cache, v cache, block table row)."""
    n = k.shape[0]
    n_pages = -(-n // ps)
    perm = torch.randperm(n_pages + 3, generator=torch.Generator().manual_seed(seed))[:n_pages]
    kc = torch.zeros(n_pages + 3, G, ps, k.shape[-1], dtype=k.dtype)
    vc = torch.zeros(n_pages + 3, G, ps, v.shape[-1], dtype=v.dtype)
    for p in range(n):
        kc[perm[p // ps], :, p % ps] = k[p]
        vc[perm[p // ps], :, p % ps] = v[p]
    return kc, vc, perm.to(torch.int32)


def _attend(dtype, H, G, D, E, M, n_keys, q_pos, window, keep, ps, plant=(), lam=0.7, c=0.4, gate=True, seed=0, drop_dead=True,
            portion=False, force_plain=False, force_simt=False):
    """Rows at positions q_pos over n_keys keys; `plant`: (row, key position) whose score is made to stand out in BOTH maps.
    Pages that no row can see are taken out of the block table (-1), as the cache manager does. Returns (got, want)."""
    from hipinfer_b200.kernels import ops

    T = len(q_pos)
    q, k, v = rnd(T, H, M, D, seed=seed + 1), rnd(n_keys, G, M, D, seed=seed + 2), rnd(n_keys, G, E, seed=seed + 3)
    for row, j in plant:
        for h in range(H):
            k[j, h // (H // G)] = q[row, h] * 6.0            # this key's score towers over the others (for the group's last head)
    g_raw = rnd(T, 5 + H * E, seed=seed + 4)
    q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
    kc, vc, bt = _paged(k.reshape(n_keys, G, M * D), v, G, ps, seed)
    if drop_dead and window:
        for lp in range(bt.numel()):
            if all(not any(plain.visible(p, j, window, keep) for j in range(lp * ps, min(n_keys, (lp + 1) * ps))) for p in q_pos):
                kc[bt[lp]] = float("nan")                    # a read of a page that was given back would show
                vc[bt[lp]] = float("nan")
                bt[lp] = -1
    batch = SimpleNamespace(block_tables=[bt.view(1, -1).to(DEV)], row_request=torch.zeros(T, dtype=torch.int32, device=DEV),
                            positions=torch.tensor(q_pos, dtype=torch.int32, device=DEV))
    if portion:        # the rows are one request's portion: what the tensor-core kernel is told about it
        assert list(q_pos) == list(range(q_pos[0], q_pos[0] + T))
        i32 = lambda v: torch.tensor([v], dtype=torch.int32, device=DEV)
        batch.req_q_start, batch.req_q_len, batch.req_ctx_len = i32(0), i32(T), i32(q_pos[0])
        batch.h_q_len, batch.max_q_len, batch.n_requests = [T], T, 1
    out = torch.empty(T, H * E, dtype=dtype, device=DEV)
    scale = 1.0 / math.sqrt(D)
    ops.attention_window(q.reshape(T, -1).to(DEV), kc.to(DEV), vc.to(DEV), batch, 0, out, H, G, D, E, M, ps, window or 0, keep,
                         scale, lam, 1.0 - c, 1e-5, M == 2, gate=g_raw.to(DEV) if gate else None, gate_offset=5,
                         force_plain=force_plain, force_simt=force_simt)
    qd, kd, vd = q.double(), k.double(), v.double()
    want = torch.zeros(T, H, E, dtype=torch.float64)
    for t, p in enumerate(q_pos):
        for h in range(H):
            gi = h // (H // G)
            maps = [plain.softmax_over_visible((qd[t:t + 1, h, m] @ kd[:, gi, m].T) * scale, window, keep, p) @ vd[:, gi]
                    for m in range(M)]
            o = maps[0] * (1.0 - c) if M == 1 else plain.rms_div(maps[0] - lam * maps[1], 1e-5) * (1.0 - c)
            want[t, h] = o[0]
    want = want.reshape(T, H * E)
    if gate:
        want = want * torch.sigmoid(g_raw[:, 5:].double())
    return out, want


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H, G, D, E, M", [(4, 2, 16, 24, 2), (3, 3, 8, 8, 2), (8, 2, 32, 48, 2), (2, 1, 40, 12, 1), (6, 1, 16, 16, 2)])
def test_window_attention_shapes(dtype, H, G, D, E, M):
    got, want = _attend(dtype, H, G, D, E, M, 200, [0, 1, 5, 63, 64, 65, 130, 199], 50, 3, 16)
    close(got, want, dtype)
    got, want = _attend(dtype, H, G, D, E, M, 90, [0, 17, 89], None, 0, 8, gate=False)
    close(got, want, dtype, "no window, no gate")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window, keep, ps", [(40, 4, 16), (64, 1, 16), (1, 1, 4), (16, 0, 16), (130, 70, 32), (7, 9, 8)])
def test_a_key_that_stands_out_at_every_edge(dtype, window, keep, ps):
    """One key's score towers in a row of hundreds: just inside and just outside the window, the last kept token and the
    first that is not, on both sides of a page's and of a key tile's border, and the row's own position."""
    n = 600
    for p in (599, 300, 64 + window, window, window - 1 if window > 1 else 0, 63, 64):
        if p >= n:
            continue
        edges = {p - window + 1, p - window, p - window - 1, keep - 1, keep, 0, p, p - 1, (p // ps) * ps, (p // ps) * ps - 1,
                 (p // 64) * 64, (p // 64) * 64 - 1, 1}
        for j in sorted(e for e in edges if 0 <= e <= p):
            got, want = _attend(dtype, 4, 2, 16, 24, 2, n, [p], window, keep, ps, plant=[(0, j)], seed=p + j)
            close(got, want, dtype, f"row at {p}, key at {j}")


def test_a_planted_key_decides_the_result_when_seen_only():
    """The construction of the test above does what it claims: with one map, the result is the planted key's value when the
    key is visible, and far from it when it lies one step outside."""
    for j, seen in ((560, True), (559, False), (2, True), (3, False)):
        got, want = _attend(torch.float32, 1, 1, 16, 8, 1, 600, [599], 40, 3, 16, plant=[(0, j)], gate=False, seed=j)
        close(got, want, torch.float32)
        v = rnd(600, 1, 8, seed=j + 3)[j, 0].double()
        dist = float((got.double().cpu().view(8) / 0.6 - v).abs().max())
        assert (dist < 1e-3) == seen, (j, dist)


@pytest.mark.parametrize("D, E", [(32, 64), (64, 128), (128, 64), (32, 128), (64, 64), (128, 128)])
@pytest.mark.parametrize("window, keep, ctx, n", [(70, 3, 0, 200), (100, 5, 333, 130), (64, 64, 200, 64), (1, 1, 10, 17),
                                                  (None, 0, 50, 100), (500, 2, 600, 16)])
def test_window_attention_portions_on_tensor_cores(D, E, window, keep, ctx, n):
    """A portion of n rows behind ctx cached tokens through the flash kernel (bfloat16): windows shorter and longer than a
    key tile, kept tokens within and beyond the first tile, a portion that ends inside a query tile, planted keys at the
    window's edge of the first, a middle and the last row."""
    rows = (0, n // 2, n - 1)
    plant = [(r, ctx + r - window + 1) for r in rows if window and ctx + r - window + 1 >= 0]
    plant += [(r, ctx + r - window) for r in rows[1:] if window and ctx + r - window >= keep]
    got, want = _attend(torch.bfloat16, 4, 2, D, E, 2, ctx + n, list(range(ctx, ctx + n)), window, keep, 16, plant=plant,
                        seed=D + E + n, portion=True)
    close(got, want, torch.bfloat16)
    # and the row kernel on the same rows: the two paths differ by rounding only
    got_rows, _ = _attend(torch.bfloat16, 4, 2, D, E, 2, ctx + n, list(range(ctx, ctx + n)), window, keep, 16, plant=plant,
                          seed=D + E + n)
    close(got, got_rows.double().cpu(), torch.bfloat16, "flash against rows")


@pytest.mark.parametrize("H, G, D, E, M", [(4, 2, 16, 24, 2), (8, 2, 32, 64, 2), (4, 1, 64, 128, 2), (2, 1, 40, 16, 1)])
def test_row_kernels_with_and_without_shared_memory_tiles_give_the_same_bits(H, G, D, E, M):
    args = (torch.bfloat16, H, G, D, E, M, 300, [0, 5, 63, 64, 200, 299], 90, 3, 16)
    a, _ = _attend(*args, seed=4, force_simt=True)
    b, _ = _attend(*args, seed=4, force_plain=True)
    assert torch.equal(a, b)


@pytest.mark.parametrize("window, keep", [(700, 3), (None, 0), (300, 130)])
def test_rows_whose_keys_are_split_over_several_blocks(window, keep):
    """Windows of many key tiles: the bfloat16 rows kernel walks them in several blocks that meet in a workspace; planted
    keys in the first, a middle and the last split and at the window's edge."""
    n = 1500
    rows = [1499, 900, 256, 255, 700, 40]
    plant = [(0, 1499 - (window or 1500) + 1 if window else 0), (0, 1498), (1, 600), (4, 2)]
    got, want = _attend(torch.bfloat16, 4, 2, 32, 64, 2, n, rows, window, keep, 16, plant=plant, seed=9)
    close(got, want, torch.bfloat16)
    plain_rows, _ = _attend(torch.bfloat16, 4, 2, 32, 64, 2, n, rows, window, keep, 16, plant=plant, seed=9, force_plain=True)
    close(got, plain_rows.double().cpu(), torch.bfloat16, "split against one walk")
    again, _ = _attend(torch.bfloat16, 4, 2, 32, 64, 2, n, rows, window, keep, 16, plant=plant, seed=9)
    assert torch.equal(got, again)          # whichever block arrives last, the splits are joined in their order
    simt, _ = _attend(torch.bfloat16, 4, 2, 32, 64, 2, n, rows, window, keep, 16, plant=plant, seed=9, force_simt=True)
    close(simt, want, torch.bfloat16, "the kernel without warp MMAs")
    close(got, simt.double().cpu(), torch.bfloat16, "warp MMAs against FFMA")


@pytest.mark.parametrize("H, G, D, E", [(4, 1, 32, 64), (16, 1, 64, 128), (32, 8, 32, 64), (3, 3, 128, 64), (12, 2, 64, 64),
                                        (5, 1, 32, 128), (2, 1, 128, 128)])
@pytest.mark.parametrize("window, keep", [(100, 2), (None, 0), (64, 64), (1, 1)])
def test_single_rows_on_warp_mmas(H, G, D, E, window, keep):
    """Groups of 1 to 16 heads as the rows of an MMA tile, every size the kernel takes; rows at the first positions, at tile
    and page borders and far out; planted keys at the window's edge and among the kept tokens."""
    rows = [0, 1, 15, 16, 63, 64, 65, 500, 999]
    plant = [(7, 500 - window + 1), (8, 999 - window)] if window and window > 1 else [(7, 3)]
    if keep:
        plant.append((8, keep - 1))
    got, want = _attend(torch.bfloat16, H, G, D, E, 2, 1000, rows, window, keep, 16, plant=plant, seed=H + D)
    close(got, want, torch.bfloat16)
