"""The Vobusun kernels alone against the plain functions, with inputs made so that a fault shows: one key whose score
stands out just inside and just outside the window and at page borders (over NaN-poisoned pages), one far key under a slow
decay among hundreds, the first tokens, pair-table rows across step cuts, streams joined in one pass, the clamp's edges."""

import math

import pytest
import torch

import plain_vobusun as P
from dryft_b200.ops import kernels as K

pytestmark = pytest.mark.gpu
DEV = "cuda"


def i32(v):
    return torch.tensor(v, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("streams, width", [(1, 40), (3, 72), (8, 257)])
def test_streams_joined_and_normed_in_one_pass(dtype, streams, width):
    n = 5
    x = torch.randn(n, streams, width, device=DEV)
    y = torch.randn(n, width, device=DEV).to(dtype)
    mix, outw, inw = torch.randn(streams, streams, device=DEV), torch.randn(streams, device=DEV), torch.randn(streams, device=DEV)
    w = torch.rand(width, device=DEV) + 0.5
    want_x = torch.einsum("st,nsw->ntw", mix.double(), x.double()) + 0.7 * outw.double()[None, :, None] * y.double()[:, None, :]
    want_h = P.rms_norm(torch.einsum("t,ntw->nw", inw.double(), want_x), w.double(), 1e-5)
    h = torch.empty(n, width, device=DEV, dtype=dtype)
    got_x = x.clone()
    K.hc_step(got_x, streams, x_out=got_x, y=y, mix=mix, outw=outw, mult=0.7, inw=inw, norm_w=w, eps=1e-5, h=h)
    assert torch.allclose(got_x.double(), want_x, atol=1e-5, rtol=1e-5)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert torch.allclose(h.double(), want_h, atol=tol * 4, rtol=tol)
    # gathered rows: nothing written back, the same values
    rows = i32([4, 0, 2])
    h2 = torch.empty(3, width, device=DEV, dtype=dtype)
    x2 = x.clone()
    K.hc_step(x2, streams, y=y, mix=mix, outw=outw, mult=0.7, inw=inw, norm_w=w, eps=1e-5, rows=rows, h=h2)
    assert torch.equal(x2, x) and torch.equal(h2, h[[4, 0, 2]])
    # the start: one copy stands for all streams
    x0 = torch.randn(n, width, device=DEV)
    out = torch.empty(n, streams, width, device=DEV)
    K.hc_step(x0, streams, x_out=out, inw=inw, norm_w=w, eps=1e-5, h=h)
    assert torch.equal(out, x0[:, None, :].expand(-1, streams, -1))
    assert torch.allclose(h.double(), P.rms_norm(inw.double().sum() * x0.double(), w.double(), 1e-5), atol=tol * 4, rtol=tol)


@pytest.mark.parametrize("table_dtype", [torch.float32, torch.bfloat16])
def test_pair_rows_across_step_cuts_and_first_tokens(table_dtype):
    vocab, width, buckets, mp, mc = 50, 24, 11, 7, 3
    table = torch.randn(vocab, width, device=DEV).to(table_dtype)
    pairs = torch.randn(buckets + 1, width, device=DEV).to(table_dtype)
    w = torch.rand(width, device=DEV) + 0.5
    seqs = {0: [3, 9, 9, 41, 0, 17], 2: [8, 8, 30]}
    state = torch.full((4,), 12345, dtype=torch.int32, device=DEV)    # what the slots' last holders left
    state[[0, 2]] = 0
    want = {s: P.rms_norm(table.double()[t] * 1.5 + pairs.double()[P.bigram_rows(t, buckets, mp, mc)], w.double(), 1e-6) for s, t in seqs.items()}
    # step 1: slot 0 brings 2 tokens, slot 2 brings 1; step 2: slot 2 brings 2, slot 0 brings 1 (and padding); step 3: the rest
    plan = [[(0, 0, 2), (2, 0, 1)], [(2, 1, 2), (0, 2, 1), (-1, 0, 1)], [(0, 3, 3)]]
    for step in plan:
        toks, slots, pos, where = [], [], [], []
        for slot, p0, cnt in step:
            for j in range(cnt):
                toks.append(seqs[slot][p0 + j] if slot >= 0 else 0)
                slots.append(slot)
                pos.append(p0 + j if slot >= 0 else 0)
                where.append((slot, p0 + j))
        x = torch.empty(len(toks), width, device=DEV)
        K.embed_pair_norm(i32(toks), i32(slots), i32(pos), table, x, scale=1.5, pair_table=pairs, buckets=buckets, mul_prev=mp,
                          mul_cur=mc, prev_state=state, norm_w=w, eps=1e-6)
        K.seq_last_token(i32(toks), i32(slots), len(toks), state)
        for r, (slot, p) in enumerate(where):
            if slot < 0:
                assert float(x[r].abs().max()) == 0.0
            else:
                assert torch.allclose(x[r].double(), want[slot][p], atol=2e-6, rtol=2e-6), (slot, p)
    assert state.tolist() == [17, 12345, 30, 12345]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_clamped_gate_at_its_edges(dtype):
    g = torch.tensor([[-9.0, -0.3, 0.0, 0.79, 0.8, 0.81, 5.0]], device=DEV)
    u = torch.tensor([[-5.0, -0.8, -0.79, 0.0, 0.8, 0.81, 9.0]], device=DEV)
    gu = torch.cat([g, u], dim=1).to(dtype)
    out = torch.empty(1, 7, device=DEV, dtype=dtype)
    K.glu_clamp(gu, out, 0.8, 1.702, 1.0)
    gd, ud = gu[:, :7].double().clamp(max=0.8), gu[:, 7:].double().clamp(-0.8, 0.8)
    want = gd * torch.sigmoid(1.702 * gd) * (ud + 1.0)
    assert torch.allclose(out.double(), want, atol=1e-6 if dtype == torch.float32 else 1e-2)
    K.glu_clamp(gu, out, None, 1.0, 0.0)     # no clamp, another constant pair
    want = gu[:, :7].double() * torch.sigmoid(gu[:, :7].double()) * gu[:, 7:].double()
    assert torch.allclose(out.double(), want, rtol=1e-5 if dtype == torch.float32 else 1e-2, atol=1e-6)


def _retention_plain(q, k, v, g, decay, rot, base, eps):
    """o [T, H*dv] from projections [T, H, .] in float64, token by token."""
    T, H, d = q.shape
    pos = torch.arange(T)
    if rot:
        q, k = P.rotate(q, pos, rot, base, False), P.rotate(k, pos, rot, base, False)
    k = k * d ** -0.5
    S = torch.zeros(H, d, v.shape[-1], dtype=torch.float64)
    o = torch.zeros(T, H, v.shape[-1], dtype=torch.float64)
    for t in range(T):
        S = torch.tensor(decay, dtype=torch.float64)[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return (P.unit_rms(o, eps) * g * torch.sigmoid(g)).reshape(T, -1)


@pytest.mark.parametrize("H, d, dv, rot", [(2, 16, 24, 8), (1, 7, 5, 0), (3, 64, 48, 64), (2, 40, 300, 40)])
def test_retention_keeps_one_far_key_among_hundreds_and_splits_anywhere(H, d, dv, rot):
    T, base, eps = 700, 1000.0, 1e-6
    decay = [0.9992] + [0.9] * (H - 1)                    # the first head still holds 57 % of a key 700 tokens back
    q, k = torch.randn(T, H, d, dtype=torch.float64) * 0.3, torch.randn(T, H, d, dtype=torch.float64) * 0.3
    v, g = torch.randn(T, H, dv, dtype=torch.float64), torch.randn(T, H, dv, dtype=torch.float64)
    k[0] *= 40.0                                           # the far key: without it the last outputs are others entirely
    v[0] += 3.0
    want = _retention_plain(q, k, v, g, decay, rot, base, eps)
    without = _retention_plain(q[1:], k[1:], v[1:], g[1:], decay, 0, base, eps)
    if rot == 0:
        assert float((want[-1] - without[-1]).abs().max()) > 0.1
    proj = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1), g.reshape(T, -1)], dim=1).float().to(DEV).contiguous()
    offs = (0, H * d, 2 * H * d, 2 * H * d + H * dv)
    inv = inv_lo = None
    if rot:     # the frequencies as a 32-bit value and what it drops: angles of hundreds of radians stay exact
        exact = torch.tensor([base ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float64)
        inv = exact.float().to(DEV)
        inv_lo = (exact - exact.float().double()).float().to(DEV)
    dec = torch.tensor(decay, dtype=torch.float64, device=DEV)
    # whole, and in pieces (one token, two, across any edge); token by token and in the chunked form
    for cuts, chunked in (([T], False), ([T], True), ([1, 2, 64, 65, 300, T], False), ([1, 3, 64, 129, 131, 300, T], True)):
        state = torch.full((3, H, d, dv), float("nan"), device=DEV)
        state[1] = 0.0                                     # the sequence's slot starts at zero; the others hold rubbish
        out = torch.empty(T, H * dv, device=DEV)
        lo = 0
        for hi in cuts:
            pos = torch.arange(lo, hi, dtype=torch.int32, device=DEV)
            piece = torch.empty(hi - lo, H * dv, device=DEV)
            K.retention_scan(proj[lo:hi].contiguous(), offs, i32([0, hi - lo]), i32([1]), pos, inv, rot, dec, state, piece, 1, H, d, dv,
                             d ** -0.5, eps, inv_freq_lo=inv_lo, chunked=chunked)
            out[lo:hi] = piece
            lo = hi
        err = (out.double().cpu() - want).abs().max() / want.abs().max()
        assert float(err) < 2e-5, (cuts, chunked, float(err))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kv_rank, rot, interleaved, window, H", [(24, 4, True, 20, 3), (40, 16, False, 64, 3), (70, 2, True, 97, 1),
                                                                 (17, 0, True, 0, 5), (512, 64, True, 130, 3), (32, 8, True, 50, 18)])
def test_latent_attention_one_key_stands_out_at_every_edge(dtype, kv_rank, rot, interleaved, window, H):
    """Query positions around the window's edge and the page borders; the key at ``mark`` has a score far above all
    others, so the output is that key's latent exactly while it is visible and something else once it is not."""
    page, Dk = 64, kv_rank + rot      # 18 heads: two blocks of heads, the second with a warp of two heads and two warps of none
    n_pos = 300
    pages = 8
    k_pages = torch.full((pages, 1, page, Dk), float("nan"), device=DEV, dtype=dtype)      # poisoned: unread rows stay NaN
    table = torch.zeros(2, 6, dtype=torch.int32, device=DEV)
    table[1, :5] = i32([5, 2, 7, 0, 3])
    rows = (torch.randn(n_pos, Dk, device=DEV) * 0.2).to(dtype)
    inv = torch.tensor([50.0 ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float32, device=DEV) if rot else None
    for mark in (0, 63, 64, 100):
        r = rows.clone()
        r[mark, :kv_rank] = 0.0
        r[mark, 0] = 6.0                                   # the marked key: a large first latent entry
        for p in range(n_pos):
            k_pages[int(table[1, p // page]), 0, p % page] = r[p]
        ends = [mark, mark + 1]
        if window:
            ends += [mark + window - 1, mark + window, mark + window + 1]
        ends = [e for e in ends if e < n_pos] + [n_pos - 1]
        q_lat = torch.randn(H, len(ends), kv_rank, device=DEV) * 0.1
        q_lat[:, :, 0] = 8.0                               # every query looks for the marked key
        q = (torch.randn(len(ends), H, 5 + rot, device=DEV) * 0.1).to(dtype)
        o_lat = torch.empty(H, len(ends), kv_rank, device=DEV, dtype=dtype)
        K.latent_attn_rows(q_lat, q, 5, k_pages, table, i32([1] * len(ends)), i32(ends), inv, interleaved, o_lat, kv_rank, rot, 1.3,
                           window or None)
        for n_splits in (2, 5):    # the keys of every query shared by several blocks: the same result
            split = torch.empty_like(o_lat)
            K.latent_attn_rows(q_lat, q, 5, k_pages, table, i32([1] * len(ends)), i32(ends), inv, interleaved, split, kv_rank, rot, 1.3,
                               window or None, n_splits=n_splits)
            assert torch.allclose(split.float(), o_lat.float(), atol=1e-5 if dtype == torch.float32 else 1e-2), (mark, n_splits)
        # plain: the same scores in float64
        c, kr = r[:, :kv_rank].double().cpu(), r[:, kv_rank:].double().cpu()
        for e_i, e in enumerate(ends):
            lo = max(0, e - window + 1) if window else 0
            for hd in range(H):
                s = c[lo:e + 1] @ q_lat[hd, e_i].double().cpu()
                if rot:
                    qr = P.rotate(q[e_i:e_i + 1, hd, 5:].double().cpu(), torch.tensor([e]), rot, 50.0, interleaved)[0]
                    # the cache holds rotated keys already (rows are taken as cached); only the query is rotated here
                    s = s + kr[lo:e + 1] @ qr
                w = torch.softmax(s * 1.3, dim=0)
                want = w @ c[lo:e + 1]
                got = o_lat[hd, e_i].double().cpu()
                tol = 2e-5 if dtype == torch.float32 else 2e-2
                assert torch.allclose(got, want, atol=tol, rtol=tol), (mark, e, hd)
                seen = lo <= mark <= e
                assert (float(got[0]) > 5.5) == seen, (mark, e, hd, float(got[0]))


def test_gated_recurrence_tail_across_cuts_shorter_than_the_taps():
    """Five taps and pieces of one and two tokens: the tail is shifted, not rebuilt; two sequences side by side."""
    C, taps, blocks, T = 20, 5, 2, 23
    nb = C // blocks
    g = torch.Generator().manual_seed(3)
    t = {"y": torch.zeros(C, 4), "y.b": torch.randn(C, generator=g), "x": torch.zeros(C, 4), "x.b": torch.zeros(C),
         "conv": torch.randn(C, taps, generator=g), "conv.b": torch.randn(C, generator=g) * 0.1,
         "ra": torch.randn(blocks, nb, nb, generator=g), "ra.b": torch.randn(blocks, nb, generator=g),
         "ri": torch.randn(blocks, nb, nb, generator=g), "ri.b": torch.randn(blocks, nb, generator=g),
         "lam": torch.randn(C, generator=g) - 2.0, "o": torch.eye(C)}
    t = {"m." + k: v for k, v in t.items()}
    seqs = [torch.randn(T, 2 * C, generator=g, dtype=torch.float64), torch.randn(T - 6, 2 * C, generator=g, dtype=torch.float64)]

    def plain(pr):      # the projections are given: feed them through identity "weights" of the plain function
        tt = dict(t)
        tt["m.y"], tt["m.x"] = torch.cat([torch.eye(C), torch.zeros(C, C)], 1), torch.cat([torch.zeros(C, C), torch.eye(C)], 1)
        return P.rglru({"width": C, "conv": taps, "blocks": blocks}, "m.", tt, pr)

    want = [plain(s) for s in seqs]
    f = lambda k: t["m." + k].float().to(DEV).contiguous()
    w_gates = torch.stack([f("ra").transpose(1, 2), f("ri").transpose(1, 2)], dim=2).contiguous()
    sp = torch.nn.functional.softplus(t["m.lam"].double()).float().to(DEV)
    state, tail = torch.zeros(4, C, device=DEV), torch.zeros(4, taps - 1, C, device=DEV)
    state[[0, 2]] = float("nan")
    got = [torch.empty(s.shape[0], C, device=DEV) for s in seqs]
    at, slots = [0, 0], [3, 1]
    for cnt in (1, 2, 1, 3, 2, 5, 1, 8):                   # both sequences advance by cnt (the shorter one until it ends)
        live = [b for b in range(2) if at[b] < seqs[b].shape[0]]
        lens = [min(cnt, seqs[b].shape[0] - at[b]) for b in live]
        proj = torch.cat([seqs[b][at[b]:at[b] + n] for b, n in zip(live, lens)]).float().to(DEV).contiguous()
        cu = [0]
        for n in lens:
            cu.append(cu[-1] + n)
        tok_slot = i32([slots[b] for b, n in zip(live, lens) for _ in range(n)])
        out = torch.empty(proj.shape[0], C, device=DEV)
        K.rglru(proj, 0, C, f("y.b"), f("x.b"), i32(cu), i32([slots[b] for b in live]), tok_slot, f("conv"), f("conv.b"), w_gates,
                f("ra.b").reshape(C), f("ri.b").reshape(C), sp, 8.0, state, tail, out, len(live), blocks)
        for i, (b, n) in enumerate(zip(live, lens)):
            got[b][at[b]:at[b] + n] = out[cu[i]:cu[i + 1]]
            at[b] += n
    for b in range(2):
        err = (got[b].double().cpu() - want[b]).abs().max() / want[b].abs().max()
        assert float(err) < 1e-5, (b, float(err))


def test_retention_chunked_with_several_sequences_of_unequal_lengths():
    """Three sequences in one step (one of a single token, one that ends on a chunk's edge) from states of their own."""
    H, d, dv, rot, eps = 2, 24, 40, 12, 1e-6
    decay = [0.97, 0.9995]
    lens, starts = [1, 128, 77], [5, 0, 300]
    inv = torch.tensor([100.0 ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float64)
    rows, pos, cu = [], [], [0]
    for n, s0 in zip(lens, starts):
        rows.append(torch.randn(n, 2 * H * d + 2 * H * dv, dtype=torch.float64) * 0.5)
        pos += list(range(s0, s0 + n))
        cu.append(cu[-1] + n)
    proj = torch.cat(rows).float().to(DEV).contiguous()
    state0 = torch.randn(4, H, d, dv, device=DEV)
    args = dict(inv_freq_lo=(inv - inv.float().double()).float().to(DEV))
    offs = (0, H * d, 2 * H * d, 2 * H * d + H * dv)
    outs = []
    for chunked in (False, True):
        state = state0.clone()
        out = torch.empty(proj.shape[0], H * dv, device=DEV)
        K.retention_scan(proj, offs, i32(cu), i32([2, 0, 3]), i32(pos), inv.float().to(DEV), rot, torch.tensor(decay, dtype=torch.float64, device=DEV),
                         state, out, 3, H, d, dv, d ** -0.5, eps, chunked=chunked, **args)
        outs.append((out, state))
    assert torch.equal(outs[0][1][1], state0[1])                       # a slot no sequence of the step holds
    assert torch.allclose(outs[0][0], outs[1][0], atol=2e-5, rtol=2e-5)
    assert torch.allclose(outs[0][1], outs[1][1], atol=2e-5, rtol=2e-5)
