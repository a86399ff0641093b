"""Small Tevovik models for the tests: configurations of the tests' own (none of them a published model's sizes),
weights drawn here (not by the product's random-weights code), written as a model folder the engine loads."""

from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional

import torch
from safetensors.torch import save_file


def layer(heads=4, kv_heads=2, dim=16, vdim=24, chunk: Optional[int] = 20, diff=0.3, scale=None, kv_from=None,
          ff=40, experts=8, top=2, groups=4, keep=2, mlp=True) -> dict:
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff,
             "scale": scale if scale is not None else 1.3 / math.sqrt(dim)}
    if chunk is not None:
        mixer["mask"] = {"size": chunk}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    out = {"type": "attention", "mixer": mixer, "mlp": None}
    if mlp:
        out["mlp"] = {"kind": "moe", "expert": {"ff": ff},
                      "router": {"experts": experts, "top": top, "groups": {"count": groups, "keep": keep}}}
    return out


def config(layers: List[dict], width=48, vocab=101, emb_scale=0.7, eps=1e-5) -> dict:
    return {"architecture": "Tevovik", "vocab": vocab, "width": width, "embedding": {"scale": emb_scale},
            "norm": {"eps": eps}, "layers": layers}


# Sizes chosen to differ from one another in everything a kernel could take for granted: a value size that is not
# twice the map size, one kv head and several, groups of one, a chunk below / equal to / above the 64-token page and not
# a divisor of it, layers without a feed-forward, layers that read another layer's keys and values, a single expert
# chosen, no groups, every group kept, widths that are not powers of two.
CONFIGS: Dict[str, dict] = {
    "a": config([layer(), layer(kv_from=0, top=3, keep=3), layer(chunk=64, heads=2, kv_heads=2, vdim=16, mlp=False)]),
    "b": config([layer(heads=6, kv_heads=1, dim=32, vdim=48, chunk=96, experts=6, groups=1, keep=1, top=1, ff=24),
                 layer(heads=6, kv_heads=1, dim=32, vdim=48, chunk=33, kv_from=0, experts=12, groups=3, keep=3, top=4, ff=56)],
                width=72, vocab=257, emb_scale=1.4, eps=3e-6),
    "c": config([layer(heads=4, kv_heads=4, dim=8, vdim=40, chunk=None, experts=4, groups=2, keep=1, top=2),
                 layer(heads=8, kv_heads=2, dim=16, vdim=16, chunk=7, diff=0.55),
                 layer(heads=8, kv_heads=2, dim=16, vdim=16, chunk=150, kv_from=1, diff=0.1, experts=16, groups=8, keep=5, top=5)],
                width=64, vocab=130),
    # every size a multiple of 16: the tensor-core prompt attention and the grouped expert products run here
    "d": config([layer(heads=8, kv_heads=2, dim=16, vdim=32, chunk=80, ff=48, experts=16, groups=4, keep=3, top=4),
                 layer(heads=8, kv_heads=2, dim=16, vdim=32, chunk=80, kv_from=0, ff=32, experts=8, groups=2, keep=2, top=2),
                 layer(heads=4, kv_heads=1, dim=32, vdim=16, chunk=128, ff=64, experts=4, groups=1, keep=1, top=3)],
                width=96, vocab=211, emb_scale=0.9),
    # a width of 256 (the decode products compiled per inner size), and every expert chosen: no router's close call can
    # move a logit here, so bfloat16 is compared as sharply as rounding allows
    "e": config([layer(heads=8, kv_heads=2, dim=32, vdim=48, chunk=128, ff=128, experts=4, groups=1, keep=1, top=4),
                 layer(heads=8, kv_heads=2, dim=32, vdim=48, chunk=128, kv_from=0, ff=128, experts=4, groups=2, keep=2, top=4),
                 layer(heads=4, kv_heads=4, dim=64, vdim=64, chunk=50, mlp=False),
                 layer(heads=4, kv_heads=4, dim=64, vdim=64, chunk=200, kv_from=2, ff=256, experts=2, groups=1, keep=1, top=2)],
                width=256, vocab=1000),
    # sizes that fit no vector, tile or tensor-core step (odd map and value sizes, three query heads on one kv head, a width
    # of 100): every kernel's element-by-element form and the library's products at unaligned sizes
    "f": config([layer(heads=3, kv_heads=1, dim=24, vdim=20, chunk=10, ff=36, experts=5, groups=1, keep=1, top=5),
                 layer(heads=3, kv_heads=1, dim=5, vdim=7, chunk=70, ff=9, experts=5, groups=5, keep=5, top=5),
                 layer(heads=5, kv_heads=5, dim=6, vdim=10, chunk=None, ff=18, experts=3, groups=1, keep=1, top=3)],
                width=100, vocab=99),
}


def draw_weights(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    """bfloat16 tensors with spreads that make every stage matter (flat logits hide faults)."""
    g = torch.Generator().manual_seed(seed)
    w = cfg["width"]

    def mat(rows, cols, gain=1.0):
        return (torch.randn(rows, cols, generator=g) * gain / math.sqrt(cols)).to(torch.bfloat16)

    def vec(n, mean, spread):
        return (mean + torch.randn(n, generator=g) * spread).to(torch.bfloat16)

    t = {"embed": (torch.randn(cfg["vocab"], w, generator=g)).to(torch.bfloat16), "head": mat(cfg["vocab"], w, 2.0),
         "final.norm": vec(w, 0.0, 0.2)}
    for i, ly in enumerate(cfg["layers"]):
        m = ly["mixer"]
        p = f"l{i}."
        t[p + "norm1"] = vec(w, 0.0, 0.2)
        t[p + "mix.q"] = mat(m["heads"] * 2 * m["dim"], w, 2.0)
        t[p + "mix.q.norm"] = vec(m["dim"], 1.0, 0.2)
        if m.get("kv_from") is None:
            t[p + "mix.k"] = mat(m["kv_heads"] * 2 * m["dim"], w, 2.0)
            t[p + "mix.v"] = mat(m["kv_heads"] * m["vdim"], w, 1.5)
            t[p + "mix.k.norm"] = vec(m["dim"], 1.0, 0.2)
        for nm in ("lq1", "lk1", "lq2", "lk2"):
            t[p + "mix." + nm] = vec(m["dim"], 0.0, 0.35)
        t[p + "mix.g"] = mat(m["heads"], w, 2.0)
        t[p + "mix.o"] = mat(w, m["heads"] * m["vdim"], 1.5)
        if ly["mlp"] is not None:
            t[p + "norm2"] = vec(w, 0.0, 0.2)
            r = ly["mlp"]["router"]
            ff = ly["mlp"]["expert"]["ff"]
            t[p + "mlp.router"] = mat(r["experts"], w, 3.0)
            for e in range(r["experts"]):
                t[p + f"mlp.e{e}.gate"] = mat(ff, w, 2.0)
                t[p + f"mlp.e{e}.up"] = mat(ff, w, 2.0)
                t[p + f"mlp.e{e}.down"] = mat(w, ff, 2.0)
    return {k: v.contiguous() for k, v in t.items()}


def write_model(cfg: dict, tensors: Dict[str, torch.Tensor], out_dir: str) -> str:
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg, f)
    save_file(tensors, os.path.join(out_dir, "model.safetensors"))
    return out_dir


def prompts(cfg: dict, lengths, seed: int = 0) -> List[List[int]]:
    g = torch.Generator().manual_seed(7000 + seed)
    return [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in lengths]


def row_errors(got: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    """Per row: rms of the difference (means taken off) over the rms of the wanted row (mean taken off)."""
    got = got.detach().to(torch.float64).cpu()
    want = want.detach().to(torch.float64).cpu()
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    ref = want - want.mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / ref.pow(2).mean(-1).sqrt().clamp_min(1e-30)


FP32_TOL = 3e-5     # sums in another order, device sin / exp
BF16_TOL = 0.05     # what rounding at every stage does to logits of these models, with room
BF16_MOST = 0.9     # share of rows that must be within BF16_TOL (one row may always be off when there are two or more):
                    # bfloat16 noise can flip a router's close call, which moves that token's logits by far more than
                    # rounding does (the 32-bit path is the sharp test)


def assert_close(got: torch.Tensor, want: torch.Tensor, dtype: str, what: str) -> None:
    assert torch.isfinite(got).all(), f"{what}: not finite"
    e = row_errors(got, want)
    if dtype == "float32":
        assert float(e.max()) <= FP32_TOL, f"{what}: row {int(e.argmax())} off by {float(e.max()):.3g}"
    else:
        over = int((e > BF16_TOL).sum())
        allowed = 0 if e.numel() < 2 else max(1, int((1.0 - BF16_MOST) * e.numel()))
        assert over <= allowed and float(e.median()) <= BF16_TOL / 2, \
            f"{what}: {over} of {e.numel()} rows off by more than {BF16_TOL} ({allowed} allowed), median {float(e.median()):.3g}"


def assert_all_close(pairs, dtype: str, what: str) -> None:
    """``pairs``: (got, want, label).  In 32-bit every pair is held to the sharp tolerance on its own; in bfloat16 the rows
    of all pairs are judged together (a single row, a one-token request say, cannot be judged statistically)."""
    if dtype == "float32":
        for got, want, label in pairs:
            assert_close(got, want, dtype, f"{what}: {label}")
    else:
        assert_close(torch.cat([g.detach().float().cpu() for g, _, _ in pairs]), torch.cat([w for _, w, _ in pairs]), dtype, what)
