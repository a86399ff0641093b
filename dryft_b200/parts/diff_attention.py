"""Differential attention over the paged cache: every head has two score maps over one set of values, and
the head's output is the difference of the two maps' results, re-normalised and gated.

Per step, with ``H`` query heads, ``G`` key/value heads, ``d`` the size of one map's queries and keys, ``dv`` the
value size and ``h`` the mixer's input:

  ``[q | k | v | g] = h @ W.T`` -- one product; q is ``H x 2 x d`` (head by head: map 1, map 2), k is ``G x 2 x d``,
  v is ``G x dv``, g is one gate logit per head.  A layer that reads another layer's cache has no k and v.
  -> every (head, map) vector of q and k gets an RMS norm over ``d`` (one weight vector for all queries, one for
  all keys); no rotation -> k and v are written into the cache at the token's position (``csrc/kv_maps.cu``)
  -> per map, softmax attention with ``score = q . k * scale`` over the keys the query may see: ``j <= i``, inside
  the last ``window`` keys if there is a window, and inside the query's own block of ``chunk`` positions (blocks
  ``[m chunk, (m+1) chunk)`` of the sequence's positions, however the prompt was fed) if there is a chunk size
  -> ``o = a1 - lambda * a2`` with ``lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff`` (one number per layer),
  ``o <- o / sqrt(mean(o^2) + eps) * (1 - diff)`` over the head's ``dv`` values, ``o <- o * sigmoid(g_head)``
  -> ``@ W_o.T``.

Scores, softmax, lambda, the combination, its norm and the gate are 32-bit in both precisions.  Attention is
``csrc/diff_attn_prefill.cu`` (bfloat16 prompts, tensor cores) or ``csrc/diff_attn_rows.cu`` (decode, and everything
in 32-bit).  Every size and constant is a parameter; ``params["names"]`` maps the tensors' roles to their names behind
the prefix.
"""

from __future__ import annotations

import math
from typing import Dict, Mapping, Optional

import torch

from ..cache.store import CacheEntry, KVNeed, StateNeed
from ..ops import kernels as K
from .base import Runtime, StepContext, TensorInfo, register_mixer
from .linear import linear

PREFILL_TILE = 64   # query rows per block of the tensor-core prefill kernel

_ROLES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight", "gate": "g_proj.weight",
          "q_norm": "q_norm.weight", "k_norm": "k_norm.weight", "lq1": "lambda_q1", "lk1": "lambda_k1", "lq2": "lambda_q2",
          "lk2": "lambda_k2"}


def _names(params: Mapping, prefix: str) -> Dict[str, str]:
    given = params.get("names") or {}
    return {role: prefix + given.get(role, default) for role, default in _ROLES.items()}


@register_mixer("diff_attention")
class DiffAttention:
    MAPS = 2

    @staticmethod
    def tensors(params: Mapping, prefix: str) -> Dict[str, TensorInfo]:
        w, nh, nkv, d, dv = (params["hidden_size"], params["num_heads"], params["num_kv_heads"], params["qk_dim"], params["v_dim"])
        nm = _names(params, prefix)
        t = {
            nm["q"]: TensorInfo((nh * 2 * d, w), "matrix"),
            nm["o"]: TensorInfo((w, nh * dv), "matrix"),
            nm["q_norm"]: TensorInfo((d,), "vector"),
        }
        for role in ("lq1", "lk1", "lq2", "lk2"):
            t[nm[role]] = TensorInfo((d,), "vector", False, 0.0)   # drawn around zero: lambda stays near `diff`
        if params.get("gate", True):
            t[nm["gate"]] = TensorInfo((nh, w), "matrix")
        if params.get("own_kv", True):
            t[nm["k"]] = TensorInfo((nkv * 2 * d, w), "matrix")
            t[nm["v"]] = TensorInfo((nkv * dv, w), "matrix")
            t[nm["k_norm"]] = TensorInfo((d,), "vector")
        return t

    def __init__(self, params: Mapping, prefix: str, weights, rt: Runtime):
        self.rt = rt
        self.hidden = int(params["hidden_size"])
        self.n_heads = int(params["num_heads"])
        self.n_kv = int(params["num_kv_heads"])
        self.qk_dim = int(params["qk_dim"])
        self.v_dim = int(params["v_dim"])
        self.scale = float(params["scale"])
        self.diff = float(params["diff"])
        self.eps = float(params["eps"])
        self.window: Optional[int] = params.get("window")
        self.chunk: Optional[int] = params.get("chunk")
        self.own_kv = bool(params.get("own_kv", True))
        self.has_gate = bool(params.get("gate", True))
        if self.n_heads % self.n_kv:
            raise ValueError(f"diff_attention: {self.n_heads} heads are not a multiple of {self.n_kv} kv heads")
        self.group = self.n_heads // self.n_kv
        self.q_cols = self.n_heads * self.MAPS * self.qk_dim
        self.k_cols = self.n_kv * self.MAPS * self.qk_dim if self.own_kv else 0
        self.v_cols = self.n_kv * self.v_dim if self.own_kv else 0
        self.o_cols = self.n_heads * self.v_dim
        nm = _names(params, prefix)
        names, rows = [nm["q"]], [self.q_cols]
        if self.own_kv:
            names += [nm["k"], nm["v"]]
            rows += [self.k_cols, self.v_cols]
        if self.has_gate:
            names.append(nm["gate"])
            rows.append(self.n_heads)
        # one product for everything that reads the mixer's input; the gate logits ride behind q, k and v
        self.gate_col = self.q_cols + self.k_cols + self.v_cols
        self.w_in = weights.load_fused(names, rows, self.hidden)
        self.w_o = weights.load(nm["o"], "matrix")
        self.q_norm_w = weights.load(nm["q_norm"], "vector")
        self.k_norm_w = weights.load(nm["k_norm"], "vector") if self.own_kv else None
        lam = [weights.load(nm[r], "vector").to(torch.float32) for r in ("lq1", "lk1", "lq2", "lk2")]
        # one number per layer, evaluated once in 32-bit
        self.lam = float(torch.exp((lam[0] * lam[1]).sum()) - torch.exp((lam[2] * lam[3]).sum())) + self.diff
        self.out_scale = 1.0 - self.diff
        K.diff_attention_rows_lib(self.qk_dim, self.v_dim, self.group, rt.page_size)
        self.use_prefill_kernel = rt.is_bf16 and K.diff_attention_prefill_supported(self.qk_dim, self.v_dim, self.group, rt.page_size)
        self.prefill_tile = PREFILL_TILE
        if self.use_prefill_kernel:
            K.diff_attention_prefill_lib(self.qk_dim, self.v_dim, self.group, rt.page_size)

    def kv_need(self) -> Optional[KVNeed]:
        return KVNeed(self.n_kv, self.MAPS * self.qk_dim, self.window, self.v_dim, self.chunk)

    def state_need(self) -> Optional[StateNeed]:
        return None

    def _n_splits(self, n_rows: int, max_kv: int) -> int:
        """Split a row's visible keys over blocks until the device is filled, two pages per block at least and at most 16
        splits (the block that finishes last combines them: measured, more and shorter splits lengthen that tail by more
        than they shorten the walk)."""
        span = max(1, max_kv)
        for bound in (self.window, self.chunk):
            if bound:
                span = min(span, bound)
        pages = (span + self.rt.page_size - 1) // self.rt.page_size + (1 if (self.window or self.chunk) else 0)
        want = math.ceil(2 * self.rt.sm_count / max(1, n_rows * self.n_kv))
        return max(1, min(16, want, (pages + 1) // 2))

    def forward(self, h: torch.Tensor, ctx: StepContext, cache: CacheEntry, state, owns_cache: bool = True) -> torch.Tensor:
        if owns_cache != self.own_kv:
            raise ValueError("diff_attention: a layer without key/value projections must read another layer's cache "
                             "(and a layer with them owns its cache)")
        n = h.shape[0]
        dev = h.device
        proj = linear(h, self.w_in, self.rt)
        o = torch.empty((n, self.o_cols), dtype=h.dtype, device=dev)
        gate = proj if self.has_gate else None
        if ctx.decode:
            # every row is its sequence's one new token: per-map norms, the cache write and attention in one launch
            s = self._n_splits(n, ctx.max_kv)
            part_o = part_ml = None
            if s > 1:
                part_o = torch.empty((n, self.n_heads, self.MAPS, s, self.v_dim), dtype=torch.float32, device=dev)
                part_ml = torch.empty((n, self.n_heads, self.MAPS, s, 2), dtype=torch.float32, device=dev)
            K.diff_attn_rows(None, cache.k, cache.v, cache.page_table, ctx.tok_slot, ctx.tok_pos, o, self.scale, self.lam, self.eps,
                             self.out_scale, window=self.window, chunk=self.chunk, gate=gate, gate_col=self.gate_col, n_splits=s,
                             part_o=part_o, part_ml=part_ml, proj=proj, n_heads=self.n_heads, q_norm_w=self.q_norm_w,
                             k_norm_w=self.k_norm_w, qk_eps=self.eps, write_kv=self.own_kv)
            return linear(o, self.w_o, self.rt)
        q = torch.empty((n, self.n_heads, self.MAPS * self.qk_dim), dtype=h.dtype, device=dev)
        K.kv_maps_store(proj, self.q_norm_w, self.k_norm_w, ctx.tok_slot, ctx.tok_pos, q, cache.k, cache.v, cache.page_table,
                        self.n_heads, self.n_kv, self.MAPS, self.qk_dim, self.v_dim, self.eps, write_kv=self.own_kv)
        if self.use_prefill_kernel and not ctx.decode and ctx.n_tiles > 0 and ctx.tile_size <= PREFILL_TILE:
            K.diff_attn_prefill(q, cache.k, cache.v, cache.page_table, ctx.tile_tok0, ctx.tile_rows, ctx.tok_slot, ctx.tok_pos, o,
                                ctx.n_tiles, self.scale, self.lam, self.eps, self.out_scale, window=self.window, chunk=self.chunk,
                                gate=gate, gate_col=self.gate_col)
        else:
            s = self._n_splits(n, ctx.max_kv)
            part_o = part_ml = None
            if s > 1:
                part_o = torch.empty((n, self.n_heads, self.MAPS, s, self.v_dim), dtype=torch.float32, device=dev)
                part_ml = torch.empty((n, self.n_heads, self.MAPS, s, 2), dtype=torch.float32, device=dev)
            K.diff_attn_rows(q, cache.k, cache.v, cache.page_table, ctx.tok_slot, ctx.tok_pos, o, self.scale, self.lam, self.eps,
                             self.out_scale, window=self.window, chunk=self.chunk, gate=gate, gate_col=self.gate_col,
                             n_splits=s, part_o=part_o, part_ml=part_ml)
        return linear(o, self.w_o, self.rt)
