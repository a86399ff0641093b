"""A plain, slow evaluation of the Vobusun decoder: one function per mechanism, whole sequences, token-by-token
recurrences, no cache, float64 on the CPU.  It shares no code with ``dryft_b200``: it reads ``config.json`` as a
mapping and the tensors by name, and is what the tests compare the engine with.

Notation: ``h [T, W]`` is a sublayer's input for the ``T`` tokens of one sequence, positions ``0..T-1``; weights are
``[out, in]`` and applied as ``h @ W.T``.
"""

from __future__ import annotations

import math
from typing import Dict, List, Mapping, Optional

import torch

F64 = torch.float64


def _t(tensors: Mapping[str, torch.Tensor], name: str) -> torch.Tensor:
    return tensors[name].to(F64)


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """``x / sqrt(mean(x^2) + eps)`` over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * w


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.log1p(torch.exp(-z.abs())) + z.clamp(min=0.0)


# ----------------------------------------------------------------------------- embedding
def bigram_rows(tokens: List[int], buckets: int, mul_prev: int, mul_cur: int) -> List[int]:
    """Row of the bigram table per token: a hash of (previous token, token); the table's last row for a first token."""
    rows = []
    for i, t in enumerate(tokens):
        rows.append(buckets if i == 0 else (tokens[i - 1] * mul_prev + t * mul_cur) % buckets)
    return rows


def embedding(cfg: Mapping, tensors: Mapping[str, torch.Tensor], tokens: List[int]) -> torch.Tensor:
    emb = cfg.get("embedding") or {}
    x = _t(tensors, "embed")[tokens] * float(emb.get("scale", 1.0))
    bg = emb.get("bigram")
    if bg:
        x = x + _t(tensors, "bigram")[bigram_rows(tokens, bg["buckets"], bg["mul_prev"], bg["mul_cur"])]
    return rms_norm(x, _t(tensors, "embed.norm"), cfg["norm"]["eps"])


# ----------------------------------------------------------------------------- rotations
def rotate(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float, interleaved: bool) -> torch.Tensor:
    """Rotary positions on the first ``dims`` entries of the last axis of ``x [T, ..., D]``; pair ``i`` turns by
    ``p * base^(-2i/dims)``.  Pairs are ``(i, i + dims/2)`` or, interleaved, ``(2i, 2i+1)``."""
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    ang = positions.to(F64)[:, None] * f[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    c, s = torch.cos(ang).reshape(shape), torch.sin(ang).reshape(shape)
    out = x.clone()
    if interleaved:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * c - v * s
        out[..., 1:dims:2] = v * c + u * s
    else:
        u, v = x[..., :half], x[..., half:dims]
        out[..., :half] = u * c - v * s
        out[..., half:dims] = v * c + u * s
    return out


# ----------------------------------------------------------------------------- mixers
def retention(m: Mapping, p: str, tensors, h: torch.Tensor, eps: float) -> torch.Tensor:
    """Linear attention with one fixed decay per head: ``S_t = decay S_(t-1) + k_t v_t^T``, ``o_t = S_t^T q_t``."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = (h @ _t(tensors, p + "q").T).reshape(T, H, d)
    k = (h @ _t(tensors, p + "k").T).reshape(T, H, d)
    v = (h @ _t(tensors, p + "v").T).reshape(T, H, dv)
    rot = m.get("rot")
    if rot:
        q = rotate(q, pos, rot["dims"], rot["base"], interleaved=False)
        k = rotate(k, pos, rot["dims"], rot["base"], interleaved=False)
    k = k * d ** -0.5
    decay = torch.tensor(m["decay"], dtype=F64)
    S = torch.zeros(H, d, dv, dtype=F64)
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = unit_rms(o, eps).reshape(T, H * dv)
    g = h @ _t(tensors, p + "g").T
    return (o * g * torch.sigmoid(g)) @ _t(tensors, p + "o").T


def latent_attention(m: Mapping, p: str, tensors, h: torch.Tensor, eps: float) -> torch.Tensor:
    """Softmax attention whose queries, keys and values come from low-rank latents; one rotated key part is shared by
    all heads; position ``i`` sees ``j`` with ``0 <= i - j < window``; a sigmoid gate per head."""
    T = h.shape[0]
    H, d, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    cq = rms_norm(h @ _t(tensors, p + "dq").T, _t(tensors, p + "dq.norm"), eps)
    q = (cq @ _t(tensors, p + "uq").T).reshape(T, H, d + dr)
    q_plain, q_rot = q[..., :d], q[..., d:]
    dkv = h @ _t(tensors, p + "dkv").T
    c = rms_norm(dkv[:, :r], _t(tensors, p + "dkv.norm"), eps)
    k_rot = dkv[:, r:]
    rot = m.get("rot")
    if rot and dr:
        q_rot = rotate(q_rot, pos, rot["dims"], rot["base"], interleaved=True)
        k_rot = rotate(k_rot, pos, rot["dims"], rot["base"], interleaved=True)
    k_plain = (c @ _t(tensors, p + "uk").T).reshape(T, H, d)
    v = (c @ _t(tensors, p + "uv").T).reshape(T, H, dv)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * m["scale"]
    diff = pos[:, None] - pos[None, :]
    seen = diff >= 0
    if m.get("mask"):
        seen = seen & (diff < m["mask"]["size"])
    scores = scores.masked_fill(~seen[None], float("-inf"))
    o = torch.einsum("hij,jhv->ihv", torch.softmax(scores, dim=-1), v)
    gate = torch.sigmoid(h @ _t(tensors, p + "g").T)          # [T, H]
    return (o * gate[:, :, None]).reshape(T, H * dv) @ _t(tensors, p + "o").T


def rglru(m: Mapping, p: str, tensors, h: torch.Tensor) -> torch.Tensor:
    """Two branches: a gelu branch, and a short causal convolution followed by a gated linear recurrence per channel."""
    T = h.shape[0]
    C, taps, B = m["width"], m["conv"], m["blocks"]
    y = gelu_tanh(h @ _t(tensors, p + "y").T + _t(tensors, p + "y.b"))
    xin = h @ _t(tensors, p + "x").T + _t(tensors, p + "x.b")
    cw, cb = _t(tensors, p + "conv"), _t(tensors, p + "conv.b")
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=F64), xin])
    u = cb + sum(padded[j:j + T] * cw[:, j] for j in range(taps))       # the last column meets the current token
    n = C // B
    ub = u.reshape(T, B, n)
    r = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, _t(tensors, p + "ra")) + _t(tensors, p + "ra.b")).reshape(T, C)
    i = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, _t(tensors, p + "ri")) + _t(tensors, p + "ri.b")).reshape(T, C)
    log_a = -8.0 * r * softplus(_t(tensors, p + "lam"))
    a = torch.exp(log_a)
    S = torch.zeros(C, dtype=F64)
    out = torch.zeros(T, C, dtype=F64)
    for t in range(T):
        S = a[t] * S + torch.sqrt(1.0 - a[t] ** 2) * i[t] * u[t]
        out[t] = S
    return (out * y) @ _t(tensors, p + "o").T


def dense_mlp(f: Mapping, p: str, tensors, h: torch.Tensor) -> torch.Tensor:
    g = h @ _t(tensors, p + "gate").T
    u = h @ _t(tensors, p + "up").T
    limit = f.get("limit")
    if limit is not None:
        g = g.clamp(max=limit)
        u = u.clamp(min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ _t(tensors, p + "down").T


def mixer(layer: Mapping, p: str, tensors, h: torch.Tensor, eps: float) -> torch.Tensor:
    kind = layer["type"]
    if kind == "retention":
        return retention(layer["mixer"], p, tensors, h, eps)
    if kind == "latent_attention":
        return latent_attention(layer["mixer"], p, tensors, h, eps)
    if kind == "rglru":
        return rglru(layer["mixer"], p, tensors, h)
    raise ValueError(f"unknown layer type {kind!r}")


# ----------------------------------------------------------------------------- the stack
def weights_layer(cfg: Mapping, i: int) -> int:
    """The layer whose tensors layer ``i`` uses."""
    while cfg["layers"][i].get("weights_of") is not None:
        i = cfg["layers"][i]["weights_of"]
    return i


def forward(cfg: Mapping, tensors: Mapping[str, torch.Tensor], tokens: List[int], layer_outputs: Optional[list] = None) -> torch.Tensor:
    """Logits ``[T, vocab]`` (float64) of one sequence.  ``layer_outputs`` (a list) receives the residual stream -- the
    sum of the streams where there are several -- after every layer."""
    eps = cfg["norm"]["eps"]
    mult = float(cfg.get("residual_mult", 1.0))
    x0 = embedding(cfg, tensors, tokens)
    streams = cfg.get("streams")
    xs = [x0.clone() for _ in range(streams or 1)]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{weights_layer(cfg, i)}."
        subs = [(1, lambda hh: mixer(layer, p + "mix.", tensors, hh, eps))]
        if layer.get("mlp") is not None:
            subs.append((2, lambda hh: dense_mlp(layer["mlp"], p + "mlp.", tensors, hh)))
        for q, fn in subs:
            norm_w = _t(tensors, f"{p}norm{q}")
            if streams and (p + f"hc{q}.in") in tensors:
                w_in, w_out, w_mix = _t(tensors, f"{p}hc{q}.in"), _t(tensors, f"{p}hc{q}.out"), _t(tensors, f"{p}hc{q}.mix")
                u = sum(w_in[s] * xs[s] for s in range(len(xs)))
                y = fn(rms_norm(u, norm_w, eps))
                xs = [sum(w_mix[s, t] * xs[s] for s in range(len(xs))) + mult * w_out[t] * y for t in range(len(xs))]
            else:
                xs = [x + mult * fn(rms_norm(x, norm_w, eps)) for x in xs]
        if layer_outputs is not None:
            layer_outputs.append(sum(xs))
    x = sum(xs)
    return rms_norm(x, _t(tensors, "final.norm"), eps) @ _t(tensors, "head").T


def greedy(cfg: Mapping, tensors, prompt: List[int], n_new: int) -> List[int]:
    ids, out = list(prompt), []
    for _ in range(n_new):
        t = int(torch.argmax(forward(cfg, tensors, ids)[-1]))
        out.append(t)
        ids.append(t)
    return out
