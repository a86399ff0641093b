"""A plain, slow evaluation of the Tevovik decoder on the CPU, one function per mechanism, written from the
design's equations and sharing no code with ``dryft_b200``.  It reads the raw ``config.json`` mapping and a
``{name: tensor}`` dictionary, works in one floating type throughout (float64 by default) and processes one
whole sequence at a time, so it has no cache, no batch and no step.

Notation: ``x`` is the residual stream ``[T, W]``; ``p`` the positions ``0..T-1``; ``H`` query heads,
``G`` key/value heads, ``d`` the query/key size of one score map, ``dv`` the value size, ``C`` the chunk
size, ``E`` experts, ``R`` experts a token uses.
"""

from __future__ import annotations

import math
from typing import Dict, List, Mapping, Optional

import torch


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """``x / sqrt(mean(x^2) + eps)`` over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_one_plus(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The layer norm of the design: unit RMS, then ``(1 + w)``."""
    return rms_unit(x, eps) * (1.0 + w)


def sinusoid_positions(pos: torch.Tensor, width: int, dtype) -> torch.Tensor:
    """``out[p, 2i] = sin(p / 10000^(2i/W))``, ``out[p, 2i+1] = cos`` of the same angle."""
    out = torch.zeros(pos.numel(), width, dtype=dtype)
    for i in range((width + 1) // 2):
        ang = pos.to(dtype) * (10000.0 ** (-2.0 * i / width))
        out[:, 2 * i] = torch.sin(ang)
        if 2 * i + 1 < width:
            out[:, 2 * i + 1] = torch.cos(ang)
    return out


def embed(tokens: torch.Tensor, table: torch.Tensor, scale: float, pos: torch.Tensor) -> torch.Tensor:
    return table[tokens] * scale + sinusoid_positions(pos, table.shape[1], table.dtype)


def diff_lambda(lq1, lk1, lq2, lk2, diff: float) -> float:
    return math.exp(float((lq1 * lk1).sum())) - math.exp(float((lq2 * lk2).sum())) + diff


def project_keys_values(h: torch.Tensor, t: Mapping[str, torch.Tensor], pre: str, m: Mapping, eps: float):
    """Keys after their per-map norm ``[T, G, 2, d]`` and values ``[T, G, dv]`` of one layer."""
    G, d, dv = m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    k = (h @ t[pre + "k"].T).reshape(T, G, 2, d)
    k = rms_unit(k, eps) * t[pre + "k.norm"]
    v = (h @ t[pre + "v"].T).reshape(T, G, dv)
    return k, v


def diff_attention_core(q, k, v, gate, pos, *, scale: float, lam: float, diff: float, eps: float,
                        chunk: Optional[int] = None, window: Optional[int] = None, key_pos: Optional[torch.Tensor] = None):
    """Heads' outputs ``[T, H, dv]`` from normalised queries ``q [T, H, 2, d]``, keys ``k [S, G, 2, d]``, values
    ``v [S, G, dv]`` and gate logits ``gate [T, H]`` (or None).  ``key_pos`` are the keys' positions (default: the
    queries' own, ``S = T``)."""
    T, H = q.shape[0], q.shape[1]
    G = k.shape[1]
    kp = pos if key_pos is None else key_pos
    i, j = pos[:, None], kp[None, :]
    mask = j <= i
    if chunk:
        mask = mask & (torch.div(i, chunk, rounding_mode="floor") == torch.div(j, chunk, rounding_mode="floor"))
    if window:
        mask = mask & (i - j < window)
    out = []
    for hd in range(H):
        g = hd // (H // G)
        maps = []
        for mp in range(2):
            s = (q[:, hd, mp] @ k[:, g, mp].T) * scale
            s = s.masked_fill(~mask, float("-inf"))
            maps.append(torch.softmax(s, dim=-1) @ v[:, g])
        o = maps[0] - lam * maps[1]
        o = rms_unit(o, eps) * (1.0 - diff)
        if gate is not None:
            o = o * torch.sigmoid(gate[:, hd:hd + 1])
        out.append(o)
    return torch.stack(out, dim=1)


def diff_attention(h: torch.Tensor, pos: torch.Tensor, t: Mapping[str, torch.Tensor], pre: str, m: Mapping, eps: float,
                   k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """The mixer's output ``[T, W]`` given the keys and values it reads (its own or another layer's)."""
    H, d = m["heads"], m["dim"]
    diff = float(m["diff"])
    T = h.shape[0]
    q = (h @ t[pre + "q"].T).reshape(T, H, 2, d)
    q = rms_unit(q, eps) * t[pre + "q.norm"]
    lam = diff_lambda(t[pre + "lq1"], t[pre + "lk1"], t[pre + "lq2"], t[pre + "lk2"], diff)
    o = diff_attention_core(q, k, v, h @ t[pre + "g"].T, pos, scale=float(m["scale"]), lam=lam, diff=diff, eps=eps,
                            chunk=(m.get("mask") or {}).get("size"))
    return o.reshape(T, -1) @ t[pre + "o"].T


def route(h: torch.Tensor, w_router: torch.Tensor, r: Mapping):
    """Chosen experts ``[T, R]`` and their weights: ``s = softmax(z)`` over all ``E`` experts; group ``g`` holds experts
    ``g * E/count .. (g+1) * E/count - 1`` and is ranked by ``max s`` inside it; among the ``keep`` highest-ranked groups the
    ``R`` largest ``s`` are chosen and used as weights without rescaling."""
    E, R = r["experts"], r["top"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    n_g, keep = groups["count"], groups["keep"]
    s = torch.softmax(h @ w_router.T, dim=-1)
    T = s.shape[0]
    gs = s.reshape(T, n_g, E // n_g).max(-1).values
    best = gs.topk(keep, dim=-1).indices
    allowed = torch.zeros(T, n_g, dtype=torch.bool)
    allowed.scatter_(1, best, True)
    allowed = allowed[:, :, None].expand(T, n_g, E // n_g).reshape(T, E)
    masked = torch.where(allowed, s, torch.full_like(s, -1.0))
    idx = masked.topk(R, dim=-1).indices
    return idx, s.gather(1, idx)


def expert(h: torch.Tensor, t: Mapping[str, torch.Tensor], pre: str) -> torch.Tensor:
    z = h @ t[pre + "gate"].T
    return ((z * torch.sigmoid(z)) * (h @ t[pre + "up"].T)) @ t[pre + "down"].T


def moe(h: torch.Tensor, t: Mapping[str, torch.Tensor], pre: str, cfg: Mapping) -> torch.Tensor:
    idx, w = route(h, t[pre + "router"], cfg["router"])
    out = torch.zeros_like(h)
    for tok in range(h.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[tok, j])
            out[tok] += w[tok, j] * expert(h[tok:tok + 1], t, f"{pre}e{e}.")[0]
    return out


def forward(config: Mapping, tensors: Mapping[str, torch.Tensor], tokens, dtype=torch.float64, layers_out: Optional[list] = None):
    """Logits ``[T, vocab]`` of one whole sequence.  ``layers_out`` receives the stream after every layer."""
    t = {k: v.to(dtype) for k, v in tensors.items() if v.is_floating_point()}
    eps = float(config["norm"]["eps"])
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    pos = torch.arange(tokens.numel())
    x = embed(tokens, t["embed"], float(config["embedding"]["scale"]), pos)
    kept: Dict[int, tuple] = {}
    for i, layer in enumerate(config["layers"]):
        if layer["type"] != "attention":
            raise ValueError(f"layer {i}: unknown type {layer['type']!r}")
        m = layer["mixer"]
        src = m.get("kv_from")
        if src is None:
            kept[i] = project_keys_values(x, t, f"l{i}.mix.", m, eps)
            src = i
        k, v = kept[src]
        x = x + norm_one_plus(diff_attention(x, pos, t, f"l{i}.mix.", m, eps, k, v), t[f"l{i}.norm1"], eps)
        if layer.get("mlp") is not None:
            x = x + norm_one_plus(moe(x, t, f"l{i}.mlp.", layer["mlp"]), t[f"l{i}.norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return norm_one_plus(x, t["final.norm"], eps) @ t["head"].T


def greedy(config: Mapping, tensors: Mapping[str, torch.Tensor], prompt, n_new: int, dtype=torch.float64) -> List[int]:
    """``n_new`` tokens chosen greedily (first index on ties), the whole sequence evaluated anew each time."""
    toks = list(prompt)
    out = []
    for _ in range(n_new):
        nxt = int(forward(config, tensors, toks, dtype)[-1].argmax())
        out.append(nxt)
        toks.append(nxt)
    return out
