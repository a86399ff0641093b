"""Small Vobusun models for the tests: configurations of the tests' own (none of them a published model's sizes), weights
drawn here (not by the product's random-weights code), written as a model folder the engine loads."""

from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from tevovik_models import prompts, row_errors, write_model  # noqa: F401  (shared helpers of the tests)


def retention(heads=3, dim=16, vdim=24, rot_dims: Optional[int] = 8, base=500.0, decay=None, ff: Optional[int] = 40, limit=0.8, **kw) -> dict:
    mixer = {"heads": heads, "dim": dim, "vdim": vdim,
             "decay": decay if decay is not None else [1.0 - 0.3 ** (h + 1.5) for h in range(heads)]}
    if rot_dims:
        mixer["rot"] = {"dims": rot_dims, "base": base}
    return _layer("retention", mixer, ff, limit, **kw)


def latent(heads=3, dim=8, rot_dim=4, vdim=12, q_rank=20, kv_rank=24, window: Optional[int] = 20, base=300.0, scale=None,
           ff: Optional[int] = 40, limit=0.8, **kw) -> dict:
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
             "scale": scale if scale is not None else 1.4 / math.sqrt(dim + rot_dim)}
    if rot_dim:
        mixer["rot"] = {"dims": rot_dim, "base": base}
    if window is not None:
        mixer["mask"] = {"size": window}
    return _layer("latent_attention", mixer, ff, limit, **kw)


def rglru(width=36, conv=3, blocks=3, ff: Optional[int] = 40, limit=0.8, **kw) -> dict:
    return _layer("rglru", {"width": width, "conv": conv, "blocks": blocks}, ff, limit, **kw)


def _layer(kind: str, mixer: dict, ff, limit, weights_of: Optional[int] = None) -> dict:
    out = {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff, "limit": limit}}
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


def again(layers: List[dict], j: int) -> dict:
    """A layer that runs layer ``j``'s weights."""
    d = dict(layers[j])
    d["weights_of"] = j
    return d


def config(layers: List[dict], width=48, vocab=101, emb_scale=3.0, eps=1e-5, mult=0.6, streams: Optional[int] = 2,
           bigram: Optional[tuple] = (37, 11, 5)) -> dict:
    cfg = {"architecture": "Vobusun", "vocab": vocab, "width": width, "embedding": {"scale": emb_scale}, "norm": {"eps": eps},
           "residual_mult": mult, "layers": layers}
    if bigram is not None:
        cfg["embedding"]["bigram"] = {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}
    if streams is not None:
        cfg["streams"] = streams
    return cfg


def _mixed() -> List[dict]:
    ls = [rglru(), retention(), latent(), retention(heads=2, dim=8, vdim=8, rot_dims=8, ff=None)]
    return ls + [again(ls, 0), again(ls, 2)]


# Sizes chosen to differ from one another in everything a kernel could take for granted: sizes that are no multiple of a
# vector or a warp, a rotation over part of the key / all of it / none, a window below / equal to / above the 64-token page
# and none at all, one group of gate matrices and several, one convolution tap and five, one stream / several / none, no
# pair table, no feed-forward, no clamp, layers that run another layer's weights (also twice over).
CONFIGS: Dict[str, dict] = {
    "ret": config([retention()], streams=None),
    "ret_wide": config([retention(heads=2, dim=24, vdim=40, rot_dims=24, decay=[0.999, 0.9], ff=None),
                        retention(heads=5, dim=6, vdim=5, rot_dims=None, limit=None)], width=40, streams=1, bigram=None),
    "lat": config([latent()], streams=None),
    "lat_page": config([latent(heads=2, dim=16, rot_dim=16, vdim=8, q_rank=12, kv_rank=40, window=64, ff=None),
                        latent(heads=5, dim=6, rot_dim=0, vdim=10, q_rank=33, kv_rank=17, window=None),
                        latent(heads=1, dim=10, rot_dim=2, vdim=3, q_rank=9, kv_rank=70, window=97, limit=None)],
                       width=56, vocab=211, streams=3, mult=1.0),
    # head sizes in steps of 16: in bfloat16 a prompt from position 0 takes the tensor-core prompt attention (values narrower
    # than the head, as wide as it, no rotated part), every later piece and token the kernel over the cached latents
    "lat_tc": config([latent(heads=3, dim=24, rot_dim=8, vdim=16, q_rank=20, kv_rank=40, window=70),
                      latent(heads=2, dim=16, rot_dim=0, vdim=16, q_rank=24, kv_rank=32, window=None, ff=None),
                      latent(heads=4, dim=8, rot_dim=8, vdim=8, q_rank=16, kv_rank=16, window=130)], width=64, vocab=173, streams=2),
    "rec": config([rglru()], streams=None),
    "rec_taps": config([rglru(width=40, conv=1, blocks=1, ff=None), rglru(width=35, conv=5, blocks=5), rglru(width=64, conv=2, blocks=2)],
                       width=40, streams=4, bigram=(13, 3, 1), emb_scale=1.0),
    "mixed": config(_mixed(), width=64, vocab=157, streams=3, mult=0.8),
}


def draw_weights(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    """bfloat16 tensors with spreads that make every stage matter (flat logits hide faults)."""
    g = torch.Generator().manual_seed(seed)
    w = cfg["width"]

    def mat(rows, cols, gain=1.0):
        return (torch.randn(rows, cols, generator=g) * gain / math.sqrt(cols)).to(torch.bfloat16)

    def vec(n, mean, spread):
        return (mean + torch.randn(n, generator=g) * spread).to(torch.bfloat16)

    t = {"embed": torch.randn(cfg["vocab"], w, generator=g).to(torch.bfloat16), "head": mat(cfg["vocab"], w, 2.0),
         "embed.norm": vec(w, 1.0, 0.2), "final.norm": vec(w, 1.0, 0.2)}
    bg = cfg["embedding"].get("bigram")
    if bg:
        t["bigram"] = (torch.randn(bg["buckets"] + 1, w, generator=g) * 2.0).to(torch.bfloat16)
    s = cfg.get("streams")
    for i, ly in enumerate(cfg["layers"]):
        if ly.get("weights_of") is not None:
            continue
        m, p = ly["mixer"], f"l{i}."
        t[p + "norm1"] = vec(w, 1.0, 0.2)
        if ly["type"] == "retention":
            t[p + "mix.q"] = mat(m["heads"] * m["dim"], w, 2.0)
            t[p + "mix.k"] = mat(m["heads"] * m["dim"], w, 2.0)
            t[p + "mix.v"] = mat(m["heads"] * m["vdim"], w, 1.5)
            t[p + "mix.g"] = mat(m["heads"] * m["vdim"], w, 2.0)
            t[p + "mix.o"] = mat(w, m["heads"] * m["vdim"], 1.5)
        elif ly["type"] == "latent_attention":
            r = m["rot_dim"]
            t[p + "mix.dq"] = mat(m["q_rank"], w, 1.5)
            t[p + "mix.dq.norm"] = vec(m["q_rank"], 1.0, 0.2)
            t[p + "mix.uq"] = mat(m["heads"] * (m["dim"] + r), m["q_rank"], 1.5)
            t[p + "mix.dkv"] = mat(m["kv_rank"] + r, w, 1.5)
            t[p + "mix.dkv.norm"] = vec(m["kv_rank"], 1.0, 0.2)
            t[p + "mix.uk"] = mat(m["heads"] * m["dim"], m["kv_rank"], 1.5)
            t[p + "mix.uv"] = mat(m["heads"] * m["vdim"], m["kv_rank"], 1.5)
            t[p + "mix.g"] = mat(m["heads"], w, 2.0)
            t[p + "mix.o"] = mat(w, m["heads"] * m["vdim"], 1.5)
        else:
            c, nb = m["width"], m["width"] // m["blocks"]
            t[p + "mix.y"] = mat(c, w, 1.5)
            t[p + "mix.y.b"] = vec(c, 0.0, 0.3)
            t[p + "mix.x"] = mat(c, w, 1.5)
            t[p + "mix.x.b"] = vec(c, 0.0, 0.3)
            t[p + "mix.conv"] = (torch.randn(c, m["conv"], generator=g) * 0.6).to(torch.bfloat16)
            t[p + "mix.conv.b"] = vec(c, 0.0, 0.2)
            for nm in ("ra", "ri"):
                t[p + "mix." + nm] = (torch.randn(m["blocks"], nb, nb, generator=g) * 1.5 / math.sqrt(nb)).to(torch.bfloat16)
                t[p + "mix." + nm + ".b"] = (torch.randn(m["blocks"], nb, generator=g) * 0.5).to(torch.bfloat16)
            t[p + "mix.lam"] = vec(c, -2.0, 1.5)      # decays from short to hundreds of tokens
            t[p + "mix.o"] = mat(w, c, 1.5)
        if ly["mlp"] is not None:
            ff = ly["mlp"]["ff"]
            t[p + "norm2"] = vec(w, 1.0, 0.2)
            t[p + "mlp.gate"] = mat(ff, w, 2.5)
            t[p + "mlp.up"] = mat(ff, w, 2.5)
            t[p + "mlp.down"] = mat(w, ff, 2.0)
        if s:
            for q in (1, 2) if ly["mlp"] is not None else (1,):
                t[p + f"hc{q}.in"] = vec(s, 1.0 / s, 0.2)
                t[p + f"hc{q}.out"] = vec(s, 1.0, 0.3)
                t[p + f"hc{q}.mix"] = (torch.eye(s) + torch.randn(s, s, generator=g) * 0.2).to(torch.bfloat16)
    return {k: v.contiguous() for k, v in t.items()}


FP32_TOL = 5e-5     # sums in another order, device sin / exp, recurrences of hundreds of steps in 32-bit
BF16_TOL = 0.08     # what rounding at every stage does to logits of these narrow models, with room (32-bit is the sharp test)


def assert_close(got: torch.Tensor, want: torch.Tensor, dtype: str, what: str) -> None:
    assert torch.isfinite(got).all(), f"{what}: not finite"
    e = row_errors(got, want)
    if dtype == "float32":
        assert float(e.max()) <= FP32_TOL, f"{what}: row {int(e.argmax())} off by {float(e.max()):.3g}"
    else:
        over = int((e > BF16_TOL).sum())
        allowed = 0 if e.numel() < 8 else max(1, e.numel() // 12)
        assert over <= allowed and float(e.max()) <= 4 * BF16_TOL, \
            f"{what}: {over} of {e.numel()} rows off by more than {BF16_TOL} ({allowed} allowed), worst {float(e.max()):.3g}"
