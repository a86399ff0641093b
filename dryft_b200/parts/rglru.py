"""A recurrent block around a real-gated linear recurrent unit over ``C`` channels.

Two branches of the mixer's input ``h`` (one product): ``y = gelu_tanh(W_y h + b_y)`` and ``x = W_x h + b_x``; then

    u_t = conv_b + sum_j conv_w[:, j] * x_(t - (taps-1) + j)          (causal, per channel; zeros before the start)
    r_t = sigmoid(Wa[b] u_t,b + ba) ;  i_t = sigmoid(Wi[b] u_t,b + bi)   (the channels in ``blocks`` equal groups, square
                                                                        matrices ``[out, in]`` per group)
    log a_t = -c * r_t * softplus(lam) ;  a_t = exp(log a_t)
    S_t = a_t * S_(t-1) + sqrt(1 - a_t^2) * i_t * u_t                  (32-bit, zero at a sequence's start)
    out_t = W_o (S_t * y_t)

The recurrent state and the convolution's tail (its last ``taps - 1`` inputs) are per-sequence state of fixed size, so a
prompt, a piece of one and a single token are the same operation (``csrc/recurrent.cu``).  Gates, decays, softplus, the
state and the convolution run in 32-bit in both precisions.  ``params["names"]`` maps the tensors' roles to their names.
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..cache.store import KVNeed, StateNeed
from ..ops import kernels as K
from .base import Runtime, StepContext, TensorInfo, register_mixer
from .linear import linear

_ROLES = {"y": "y_proj.weight", "y_bias": "y_proj.bias", "x": "x_proj.weight", "x_bias": "x_proj.bias", "conv": "conv.weight",
          "conv_bias": "conv.bias", "gate_a": "gate_a.weight", "gate_a_bias": "gate_a.bias", "gate_i": "gate_i.weight",
          "gate_i_bias": "gate_i.bias", "lam": "lambda", "o": "o_proj.weight"}


def _names(params: Mapping, prefix: str) -> Dict[str, str]:
    given = params.get("names") or {}
    return {role: prefix + given.get(role, default) for role, default in _ROLES.items()}


@register_mixer("rglru")
class RGLRU:
    @staticmethod
    def tensors(params: Mapping, prefix: str) -> Dict[str, TensorInfo]:
        w, c, taps, blocks = params["hidden_size"], params["channels"], params["taps"], params["blocks"]
        nb = c // blocks
        nm = _names(params, prefix)
        return {
            nm["y"]: TensorInfo((c, w), "matrix"), nm["y_bias"]: TensorInfo((c,), "vector", False, 0.0),
            nm["x"]: TensorInfo((c, w), "matrix"), nm["x_bias"]: TensorInfo((c,), "vector", False, 0.0),
            nm["conv"]: TensorInfo((c, taps), "vector", False, 1.0 / taps), nm["conv_bias"]: TensorInfo((c,), "vector", False, 0.0),
            nm["gate_a"]: TensorInfo((blocks, nb, nb), "vector", False, 0.0), nm["gate_a_bias"]: TensorInfo((blocks, nb), "vector", False, 0.0),
            nm["gate_i"]: TensorInfo((blocks, nb, nb), "vector", False, 0.0), nm["gate_i_bias"]: TensorInfo((blocks, nb), "vector", False, 0.0),
            nm["lam"]: TensorInfo((c,), "vector", False, 0.0), nm["o"]: TensorInfo((w, c), "matrix"),
        }

    def __init__(self, params: Mapping, prefix: str, weights, rt: Runtime):
        self.rt = rt
        self.hidden = int(params["hidden_size"])
        self.channels = int(params["channels"])
        self.taps = int(params["taps"])
        self.blocks = int(params["blocks"])
        self.c_mult = float(params.get("c", 8.0))
        if self.taps < 1 or self.blocks < 1 or self.channels % self.blocks:
            raise ValueError(f"rglru: {self.channels} channels in {self.blocks} groups with {self.taps} taps")
        nm = _names(params, prefix)
        c = self.channels
        self.w_in = weights.load_fused([nm["y"], nm["x"]], [c, c], self.hidden)
        self.w_o = weights.load(nm["o"], "matrix")
        f32 = lambda role: weights.load(nm[role], "vector").to(torch.float32).contiguous()
        self.y_bias, self.x_bias, self.conv_w, self.conv_b = f32("y_bias"), f32("x_bias"), f32("conv"), f32("conv_bias")
        # both gates' matrices side by side with the input index first: a thread per output channel reads along them
        ga, gi = f32("gate_a"), f32("gate_i")                                    # [blocks, out, in]
        self.w_gates = torch.stack([ga.transpose(1, 2), gi.transpose(1, 2)], dim=2).contiguous()   # [blocks, in, 2, out]
        self.b_a, self.b_i = f32("gate_a_bias").reshape(c), f32("gate_i_bias").reshape(c)
        # softplus of the decay parameter: a constant of the layer, evaluated once (in 64-bit, rounded once)
        self.sp_lam = torch.nn.functional.softplus(f32("lam").to(torch.float64)).to(torch.float32)
        K.recurrent_lib()

    def kv_need(self) -> Optional[KVNeed]:
        return None

    def state_need(self):
        need = {"s": StateNeed((self.channels,), torch.float32)}
        if self.taps > 1:
            need["tail"] = StateNeed((self.taps - 1, self.channels), torch.float32)
        return need

    def forward(self, h: torch.Tensor, ctx: StepContext, cache, state, owns_cache: bool = True) -> torch.Tensor:
        proj = linear(h, self.w_in, self.rt)
        out = torch.empty((h.shape[0], self.channels), dtype=h.dtype, device=h.device)
        K.rglru(proj, 0, self.channels, self.y_bias, self.x_bias, ctx.cu_q, ctx.seq_slot, ctx.tok_slot, self.conv_w, self.conv_b,
                self.w_gates, self.b_a, self.b_i, self.sp_lam, self.c_mult, state["s"], state.get("tail"), out, ctx.n_seqs, self.blocks)
        return linear(out, self.w_o, self.rt)
