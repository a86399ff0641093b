"""Retention: linear attention with one fixed decay per head, no softmax and no denominator.

Per head, with ``q_t``, ``k_t`` (both rotated at the token's position; ``k_t`` then times ``k_scale``) and ``v_t``:

    S_t = decay * S_(t-1) + k_t v_t^T            (``S [dim, vdim]``, 32-bit, zero at a sequence's start)
    o_t = S_t^T q_t ;   o_t <- o_t / sqrt(mean(o_t^2) + eps) ;   out_t = o_t * silu(g_t)  ->  @ W_o.T

``q | k | v | g`` are one product of the mixer's input.  The state is per-sequence state of fixed size (``state_need``), so
a prompt, a piece of a prompt and a single token are the same operation: the step's tokens are walked from the state the
step before left (``csrc/recurrent.cu``).  The rotation, the state, the sums and the norm are 32-bit in both precisions.
Every size and constant is a parameter; ``params["names"]`` maps ``q k v g o`` to the tensors' names behind the prefix.
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..cache.store import KVNeed, StateNeed
from ..config.spec import PartSpec
from ..ops import kernels as K
from .base import POSITIONS, Runtime, StepContext, TensorInfo, register_mixer
from .linear import linear

_ROLES = ("q", "k", "v", "g", "o")


def _names(params: Mapping, prefix: str) -> Dict[str, str]:
    given = params.get("names") or {}
    return {r: prefix + given.get(r, r + "_proj.weight") for r in _ROLES}


@register_mixer("retention")
class Retention:
    @staticmethod
    def tensors(params: Mapping, prefix: str) -> Dict[str, TensorInfo]:
        w, h, d, dv = params["hidden_size"], params["num_heads"], params["qk_dim"], params["v_dim"]
        nm = _names(params, prefix)
        return {nm["q"]: TensorInfo((h * d, w), "matrix"), nm["k"]: TensorInfo((h * d, w), "matrix"),
                nm["v"]: TensorInfo((h * dv, w), "matrix"), nm["g"]: TensorInfo((h * dv, w), "matrix"),
                nm["o"]: TensorInfo((w, h * dv), "matrix")}

    def __init__(self, params: Mapping, prefix: str, weights, rt: Runtime):
        self.rt = rt
        self.hidden = int(params["hidden_size"])
        self.n_heads = int(params["num_heads"])
        self.qk_dim = int(params["qk_dim"])
        self.v_dim = int(params["v_dim"])
        self.eps = float(params["eps"])
        self.k_scale = float(params.get("k_scale", self.qk_dim ** -0.5))
        decay = [float(d) for d in params["decay"]]
        if len(decay) != self.n_heads:
            raise ValueError(f"retention: {len(decay)} decays for {self.n_heads} heads")
        self.decay = torch.tensor(decay, dtype=torch.float64).to(rt.device)   # 64-bit: the kernels split it into a pair
        pos: PartSpec = params.get("position") or PartSpec("none")
        self.position = POSITIONS.get(pos.kind)(pos.params, self.qk_dim, rt)
        if getattr(self.position, "interleaved", False):
            raise ValueError("retention: the rotation pairs dims j and j + R/2; an interleaved layout is not served")
        nm = _names(params, prefix)
        hd, hv = self.n_heads * self.qk_dim, self.n_heads * self.v_dim
        self.w_in = weights.load_fused([nm["q"], nm["k"], nm["v"], nm["g"]], [hd, hd, hv, hv], self.hidden)
        self.offsets = (0, hd, 2 * hd, 2 * hd + hv)
        self.w_o = weights.load(nm["o"], "matrix")
        K.recurrent_lib()   # build (or find) the kernels now, not at the first step

    def kv_need(self) -> Optional[KVNeed]:
        return None

    def state_need(self) -> StateNeed:
        return StateNeed((self.n_heads, self.qk_dim, self.v_dim), torch.float32)

    def forward(self, h: torch.Tensor, ctx: StepContext, cache, state: torch.Tensor, owns_cache: bool = True) -> torch.Tensor:
        proj = linear(h, self.w_in, self.rt)
        o = torch.empty((h.shape[0], self.n_heads * self.v_dim), dtype=h.dtype, device=h.device)
        K.retention_scan(proj, self.offsets, ctx.cu_q, ctx.seq_slot, ctx.tok_pos, self.position.inv_freq, self.position.rotary_dim,
                         self.decay, state, o, ctx.n_seqs, self.n_heads, self.qk_dim, self.v_dim, self.k_scale, self.eps,
                         inv_freq_lo=getattr(self.position, "inv_freq_lo", None), chunked=not ctx.decode)
        return linear(o, self.w_o, self.rt)
