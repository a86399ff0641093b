"""Every mechanism of the Tevovik decoder alone, kernel against the plain function of ``plain_tevovik.py``: the sinusoid
embedding, the offset norms around the 32-bit stream, the per-map q/k norm with the cache write, differential attention
(row-wise in both precisions, tensor-core prompts in bfloat16) with one dominating key at every edge of a chunk, a
window and a page, over poisoned pages, the router's choice, and the experts (assignment by assignment, and grouped)."""

import math

import pytest
import torch

import plain_tevovik as P

pytestmark = pytest.mark.gpu
DEV = "cuda"
PAGE = 64


def K():
    from dryft_b200.ops import kernels

    return kernels


def close(got, want, tol, what):
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    assert torch.isfinite(got).all(), what
    err = float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))
    assert err <= tol, f"{what}: off by {err:.3g} (allowed {tol:.3g})"


# ----------------------------------------------------------------------------------------- stream kernels
@pytest.mark.parametrize("act", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [48, 101, 640])
def test_sinusoid_embedding(act, width):
    vocab, n, scale = 37, 50, 0.37
    table = torch.randn(vocab, width).to(torch.bfloat16)
    toks = torch.randint(0, vocab, (n,))
    pos = torch.randint(0, 6000, (n,))
    pos[:3] = torch.tensor([0, 1, 5999])
    freq = torch.pow(torch.tensor(10000.0, dtype=torch.float64), -2.0 * torch.arange((width + 1) // 2, dtype=torch.float64) / width)
    x = torch.empty(n, width, dtype=torch.float32, device=DEV)
    h = torch.empty(n, width, dtype=act, device=DEV)
    tab = table.to(DEV) if act == torch.bfloat16 else table.float().to(DEV)
    K().embed_sinusoid(toks.int().to(DEV), pos.int().to(DEV), tab, freq.float().to(DEV), scale, x, h)
    want = P.embed(toks, table.double(), scale, pos)
    # the angle is a 32-bit product: at position 6000 its rounding alone moves a sine by 3e-4
    close(x, want, 2e-4, "stream")
    close(h, want, 2e-4 if act == torch.float32 else 5e-3, "rounded stream")


@pytest.mark.parametrize("act", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,top", [(48, 0), (101, 3), (1024, 1)])
def test_norm_of_the_output_added_to_the_32_bit_stream(act, width, top):
    n, eps, off = 9, 1e-5, 1.0
    w = (torch.randn(width) * 0.3)
    x = torch.randn(n, width) * 5
    y = (torch.randn(n * max(top, 1), width) * 3).to(act)
    wts = torch.rand(n, top) if top else None
    xd = x.clone().to(DEV)
    h = torch.empty(n, width, dtype=act, device=DEV)
    K().stream_norm_add(y.to(DEV), w.to(DEV), off, eps, xd, h, wts=wts.to(DEV) if top else None, top=top)
    yy = y.double()
    if top:
        yy = (yy.reshape(n, top, width) * wts.double()[:, :, None]).sum(1)
    want = x.double() + P.norm_one_plus(yy, w.double(), eps)
    close(xd, want, 2e-6, "stream")
    close(h, want, 2e-6 if act == torch.float32 else 5e-3, "rounded stream")
    rows = torch.tensor([4, 0, 7], dtype=torch.int32)
    out = torch.empty(3, width, dtype=act, device=DEV)
    K().stream_norm_rows(xd, w.to(DEV), off, eps, out, rows=rows.to(DEV))
    close(out, P.norm_one_plus(xd.double().cpu()[rows.long()], w.double(), eps), 2e-6 if act == torch.float32 else 5e-3, "gathered norm")


# ----------------------------------------------------------------------------------------- attention
def paged(k, v, n_pages, perm_seed, act):
    """Keys ``[T, G, KW]`` and values ``[T, G, DV]`` of one sequence in shuffled pages of a poisoned cache."""
    T, G, KW = k.shape
    DV = v.shape[2]
    g = torch.Generator().manual_seed(perm_seed)
    used = (T + PAGE - 1) // PAGE
    phys = torch.randperm(n_pages, generator=g)[:used]
    kp = torch.full((n_pages, G, PAGE, KW), float("nan"), dtype=act)
    vp = torch.full((n_pages, G, PAGE, DV), float("nan"), dtype=act)
    for p in range(T):
        kp[phys[p // PAGE], :, p % PAGE] = k[p].to(act)
        vp[phys[p // PAGE], :, p % PAGE] = v[p].to(act)
    table = torch.zeros(3, used + 2, dtype=torch.int32)
    table[1, :used] = phys.int()
    return kp.to(DEV), vp.to(DEV), table.to(DEV)


def attention_case(T, H, G, d, dv, act, boost):
    q = torch.randn(T, H, 2, d).to(act)
    k = torch.randn(T, G, 2, d).to(act)
    v = torch.randn(T, G, dv).to(act)
    if boost is not None:
        qp, kp = boost
        u = torch.randn(d)
        u = u / u.norm() * 6.0
        q[qp] = u.to(act)            # every head and map of this query points at ...
        k[kp] = u.to(act)            # ... this key: its score stands out by exp(36 * scale)
        k[kp, :, 1] = -u.to(act)     # but not in the second map
    gate = torch.randn(T, H + 3).to(act)
    return q, k, v, gate


EDGES = [  # (chunk, window, [(query position, boosted key position)])
    (None, None, [(199, 0), (130, 63), (130, 64), (64, 64)]),
    (7, None, [(20, 14), (20, 13), (6, 0), (7, 6), (199, 196)]),
    (64, None, [(127, 64), (127, 63), (128, 127), (190, 128)]),
    (96, None, [(191, 96), (191, 95), (95, 0), (96, 95), (150, 128), (150, 127)]),
    (150, None, [(149, 0), (150, 149), (199, 150), (199, 149)]),
    (None, 40, [(100, 61), (100, 60), (199, 160), (199, 159)]),
    (96, 50, [(100, 96), (100, 95), (180, 131), (180, 130)]),
]


@pytest.mark.parametrize("act", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kernel", ["rows", "rows_split", "prefill"])
@pytest.mark.parametrize("sizes", [(4, 2, 16, 24), (6, 1, 32, 48), (2, 2, 48, 16)])
def test_differential_attention_sees_exactly_the_keys_it_may(act, kernel, sizes):
    H, G, d, dv = sizes
    kern = K()
    if kernel == "prefill" and (act != torch.bfloat16 or not kern.diff_attention_prefill_supported(d, dv, H // G, PAGE)):
        pytest.skip("the tensor-core prompt kernel is bfloat16 only")
    T, scale, lam, diff, eps = 200, 1.0 / math.sqrt(d) * 1.5, 0.37, 0.3, 1e-5
    pos = torch.arange(T)
    tok_slot = torch.full((T,), 1, dtype=torch.int32, device=DEV)
    tok_pos = pos.int().to(DEV)
    for chunk, window, pairs in EDGES:
        for boost in [None] + pairs:
            q, k, v, gate = attention_case(T, H, G, d, dv, act, boost)
            kp, vp, table = paged(k.reshape(T, G, 2 * d), v, 9, 5, act)
            out = torch.empty(T, H * dv, dtype=act, device=DEV)
            qd = q.reshape(T, H, 2 * d).contiguous().to(DEV)
            gd = gate.to(DEV)
            if kernel == "prefill":
                t0 = torch.arange(0, T, 64, dtype=torch.int32)
                tn = torch.tensor([min(64, T - int(a)) for a in t0], dtype=torch.int32)
                kern.diff_attn_prefill(qd, kp, vp, table, t0.to(DEV), tn.to(DEV), tok_slot, tok_pos, out, t0.numel(), scale, lam, eps,
                                       1.0 - diff, window=window, chunk=chunk, gate=gd, gate_col=2)
            else:
                s = 3 if kernel == "rows_split" else 1
                po = torch.empty(T * H * 2 * s * dv, dtype=torch.float32, device=DEV) if s > 1 else None
                pm = torch.empty(T * H * 2 * s * 2, dtype=torch.float32, device=DEV) if s > 1 else None
                kern.diff_attn_rows(qd, kp, vp, table, tok_slot, tok_pos, out, scale, lam, eps, 1.0 - diff, window=window, chunk=chunk,
                                    gate=gd, gate_col=2, n_splits=s, part_o=po, part_ml=pm)
            want = P.diff_attention_core(q.double(), k.double(), v.double(), gate.double()[:, 2:2 + H], pos, scale=scale, lam=lam,
                                         diff=diff, eps=eps, chunk=chunk, window=window).reshape(T, H * dv)
            close(out, want, 3e-5 if act == torch.float32 else 2.5e-2, f"{kernel} chunk {chunk} window {window} boost {boost}")


@pytest.mark.parametrize("act", [torch.float32, torch.bfloat16])
def test_per_map_norm_and_cache_write(act):
    kern = K()
    H, G, d, dv, n, eps = 4, 2, 16, 24, 11, 1e-5
    extra = 5
    width = H * 2 * d + G * 2 * d + G * dv + extra
    proj = (torch.randn(n, width) * 2).to(act)
    qw, kw = torch.rand(d) + 0.5, torch.rand(d) + 0.5
    slots = torch.tensor([0, 0, 0, 2, 2, -1, 1, 1, 1, 1, 2], dtype=torch.int32)
    pos = torch.tensor([62, 63, 64, 0, 1, 0, 130, 131, 132, 133, 2], dtype=torch.int32)
    table = torch.tensor([[3, 1, 7], [0, 2, 4], [5, 6, 8]], dtype=torch.int32)
    kp = torch.zeros(9, G, PAGE, 2 * d, dtype=act, device=DEV)
    vp = torch.zeros(9, G, PAGE, dv, dtype=act, device=DEV)
    q = torch.empty(n, H, 2 * d, dtype=act, device=DEV)
    kern.kv_maps_store(proj.to(DEV), qw.to(DEV), kw.to(DEV), slots.to(DEV), pos.to(DEV), q, kp, vp, table.to(DEV), H, G, 2, d, dv, eps)
    tol = 2e-6 if act == torch.float32 else 5e-3
    pq = proj.double()[:, :H * 2 * d].reshape(n, H, 2, d)
    want_q = (P.rms_unit(pq, eps) * qw.double()).reshape(n, H, 2 * d)
    want_q[5] = 0
    close(q, want_q, tol, "queries")
    pk = proj.double()[:, H * 2 * d:H * 2 * d + G * 2 * d].reshape(n, G, 2, d)
    want_k = (P.rms_unit(pk, eps) * kw.double()).reshape(n, G, 2 * d)
    want_v = proj.double()[:, H * 2 * d + G * 2 * d:H * 2 * d + G * 2 * d + G * dv].reshape(n, G, dv)
    written = torch.zeros(9, PAGE, dtype=torch.bool)
    for i in range(n):
        if slots[i] < 0:
            continue
        page = int(table[slots[i], pos[i] // PAGE])
        written[page, pos[i] % PAGE] = True
        close(kp[page, :, pos[i] % PAGE], want_k[i], tol, f"key of token {i}")
        close(vp[page, :, pos[i] % PAGE], want_v[i], tol, f"value of token {i}")
    assert float(kp.float().abs().sum(dim=(1, 3)).cpu()[~written].sum()) == 0.0   # nothing else was touched


# ----------------------------------------------------------------------------------------- mixture of experts
@pytest.mark.parametrize("E,groups,keep,top", [(8, 4, 2, 2), (16, 4, 3, 4), (6, 1, 1, 1), (12, 3, 3, 4), (16, 8, 5, 5), (40, 5, 2, 6),
                                               (64, 8, 4, 8), (7, 7, 3, 3)])
def test_router_choice(E, groups, keep, top):
    n = 333
    logits = torch.randn(n, E) * 2.5
    idx = torch.empty(n, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(n, top, dtype=torch.float32, device=DEV)
    K().moe_route(logits.to(DEV), groups, keep, top, idx, wts)
    s = torch.softmax(logits.double(), -1)
    # the plain router with the logits as its input and the identity as its weight
    want_idx, _ = P.route(logits.double(), torch.eye(E, dtype=torch.float64), {"experts": E, "top": top, "groups": {"count": groups, "keep": keep}})
    got = idx.cpu().long()
    assert (got.sort(-1).values == want_idx.sort(-1).values).all()
    close(wts, s.gather(1, got), 2e-6, "weights are the chosen experts' own scores")
    assert (wts.cpu()[:, :-1] >= wts.cpu()[:, 1:]).all()   # largest first


@pytest.mark.parametrize("act", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("E,groups,keep,top,width", [(8, 4, 2, 2, 48), (6, 1, 1, 1, 72), (64, 8, 4, 8, 1024), (12, 3, 3, 4, 101)])
def test_router_product_and_choice_in_one_launch(act, E, groups, keep, top, width):
    n = 13
    h = torch.randn(n, width).to(act)
    w = (torch.randn(E, width) / math.sqrt(width) * 3).to(act)
    idx = torch.empty(n, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(n, top, dtype=torch.float32, device=DEV)
    K().moe_route_rows(h.to(DEV), w.to(DEV), groups, keep, top, idx, wts)
    want_idx, want_w = P.route(h.double(), w.double(), {"experts": E, "top": top, "groups": {"count": groups, "keep": keep}})
    assert (idx.cpu().long().sort(-1).values == want_idx.sort(-1).values).all()
    close(wts.sort(-1).values, want_w.sort(-1).values, 1e-5, "weights")


@pytest.mark.parametrize("act", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,width,ff,E,top", [(5, 48, 40, 8, 2), (1, 72, 24, 6, 1), (70, 64, 56, 12, 4), (300, 128, 96, 16, 3)])
def test_experts_assignment_by_assignment_and_grouped(act, n, width, ff, E, top):
    kern = K()
    h = torch.randn(n, width).to(act)
    wgu = (torch.randn(E, 2 * ff, width) / math.sqrt(width) * 2).to(act)
    wd = (torch.randn(E, width, ff) / math.sqrt(ff) * 2).to(act)
    idx = torch.stack([torch.randperm(E)[:top] for _ in range(n)]).int()
    if n > 20:
        idx[:, 0] = 3          # a crowded expert and (E > top + 1) idle ones
    t = {}
    for e in range(E):
        t[f"e{e}.gate"], t[f"e{e}.up"], t[f"e{e}.down"] = wgu[e, :ff].double(), wgu[e, ff:].double(), wd[e].double()
    want = torch.stack([P.expert(h[i:i + 1].double(), t, f"e{int(idx[i, j])}.")[0] for i in range(n) for j in range(top)])
    hd, wgud, wdd, idxd = h.to(DEV), wgu.to(DEV), wd.to(DEV), idx.to(DEV)
    act_buf = torch.empty(n * top, ff, dtype=act, device=DEV)
    y = torch.empty(n * top, width, dtype=act, device=DEV)
    kern.moe_rows(hd, wgud, idxd, act_buf, "gate_up")
    kern.moe_rows(act_buf, wdd, idxd, y, "down")
    tol = 2e-5 if act == torch.float32 else 2e-2
    close(y, want, tol, "assignment by assignment")
    wts = torch.rand(n, top)
    out = torch.empty(n, width, dtype=act, device=DEV)
    kern.moe_combine(y, wts.to(DEV), out)
    close(out, (y.double().cpu().reshape(n, top, width) * wts.double()[:, :, None]).sum(1), 1e-6 if act == torch.float32 else 5e-3, "weighted sum")
    if act == torch.bfloat16 and kern.moe_grouped_supported(width, ff):
        y2 = torch.full((n * top, width), float("nan"), dtype=act, device=DEV)
        kern.moe_grouped(hd, wgud, wdd, idxd, y2)
        close(y2, want, tol, "grouped by expert")
