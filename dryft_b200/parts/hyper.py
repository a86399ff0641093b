"""A residual stream kept as several 32-bit copies ("streams") that small learned matrices join (hyper-connections),
and the block arrangement around it.

For a sublayer ``f`` with its connection's weights ``in [S]``, ``out [S]``, ``mix [S, S]`` (indexed ``[from, to]``) and
the streams ``x_1 .. x_S`` (all equal to the embedding's output at the start):

    u = sum_s in[s] x_s ;   y = f(norm(u)) ;   x_t <- sum_s mix[s, t] x_s + mult * out[t] * y     (all t from the old x)

and the rows the last norm reads are the sum of the streams.  ``S = 1`` with all three weights 1 is the plain pre-norm
residual ``x += mult * f(norm(x))``; a connection built without streams is exactly that and has no tensors.

One kernel (``csrc/stream_hc.cu:hc_step``) applies the update a sublayer left pending and forms the next sublayer's normed
input in the same pass over the streams, so a layer of two sublayers costs two such launches; the update of the last
sublayer is folded into the gather of the rows the head wants.  Sums and norms are 32-bit in both precisions; the
sublayers read and write the activation type.
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..ops import kernels as K
from .base import Residual, Runtime, StepContext, TensorInfo, fused_rms, register_block, register_connection


@register_connection("hyper_connection")
class HyperConnection:
    """``params``: ``streams`` (None: one stream and no tensors), ``mult``; tensors ``in``, ``out``, ``mix`` behind the
    prefix.  With one stream the tensors may be absent (all ones)."""

    @staticmethod
    def tensors(params: Mapping, prefix: str) -> Dict[str, TensorInfo]:
        s = params.get("streams")
        if s is None:
            return {}
        opt = int(s) == 1
        return {prefix + "in": TensorInfo((s,), "vector", opt), prefix + "out": TensorInfo((s,), "vector", opt),
                prefix + "mix": TensorInfo((s, s), "vector", opt, 0.0, 1.0)}

    def __init__(self, params: Mapping, prefix: str, weights, rt: Runtime):
        s = params.get("streams")
        self.streams = int(s) if s is not None else 1
        if not 1 <= self.streams <= K.HC_MAX_STREAMS:
            raise ValueError(f"hyper_connection: 1..{K.HC_MAX_STREAMS} streams are served, got {self.streams}")
        self.mult = float(params.get("mult", 1.0))
        names = [prefix + n for n in ("in", "out", "mix")]
        if s is not None and all(weights.has(n) for n in names):
            self.inw, self.outw, self.mix = (weights.load(n, "vector").to(torch.float32).contiguous() for n in names)
        elif self.streams == 1:
            ones = torch.ones(1, dtype=torch.float32, device=rt.device)
            self.inw, self.outw, self.mix = ones, ones.clone(), ones.clone().reshape(1, 1)
        else:
            raise ValueError(f"hyper_connection: {self.streams} streams need the tensors {names}")


@register_block("hyper")
class HyperBlock:
    """``norm_mixer`` / ``norm_ffn`` must be plain RMS norms (they are folded into the joint's kernel); ``extra`` holds the
    two connections as ``conn_mixer`` and ``conn_ffn``.  A layer without a feed-forward stops after the mixer."""

    def __init__(self, norm_mixer, mixer, norm_ffn, ffn, extra: Optional[Mapping] = None):
        extra = extra or {}
        self.norm_mixer, self.mixer, self.norm_ffn, self.ffn = norm_mixer, mixer, norm_ffn, ffn
        self.conn_mixer, self.conn_ffn = extra.get("conn_mixer"), extra.get("conn_ffn")
        if self.conn_mixer is None or (ffn is not None and self.conn_ffn is None):
            raise ValueError("the 'hyper' arrangement needs a connection per sublayer (extra parts conn_mixer, conn_ffn)")
        for nm in (norm_mixer, norm_ffn):
            if nm is not None and fused_rms(nm) is None:
                raise ValueError("the 'hyper' arrangement folds plain RMS norms into its joints; this norm is of another kind")
        self.extra = dict(extra)
        self.streams = self.conn_mixer.streams
        self._ones = torch.ones(self.streams, dtype=torch.float32, device=self.conn_mixer.inw.device)

    def _joint(self, res: Residual, conn: HyperConnection, norm) -> tuple:
        """Apply the pending update (if any) to the streams and form ``conn``'s normed input.  Returns (streams, h)."""
        x = res.x
        if x.dtype != torch.float32:
            raise ValueError("the 'hyper' arrangement keeps its streams in float32; the embedding must start them")
        n, width = x.shape[0], x.shape[-1]
        act = self.mixer.rt.dtype
        w, eps = fused_rms(norm)
        h = torch.empty((n, width), dtype=act, device=x.device)
        pend = res.conn
        if x.dim() == 2 and self.streams > 1:
            out = torch.empty((n, self.streams, width), dtype=torch.float32, device=x.device)   # the start: one copy for all
        else:
            out = x if x.dim() == 3 else x.view(n, 1, width)
        write = res.delta is not None or out.data_ptr() != x.data_ptr()
        K.hc_step(x, self.streams, x_out=out if write else None, y=res.delta, mix=pend.mix if pend is not None else None,
                  outw=pend.outw if pend is not None else None, mult=pend.mult if pend is not None else 1.0, inw=conn.inw,
                  norm_w=w, eps=eps, h=h)
        return out, h

    def forward(self, res: Residual, ctx: StepContext, cache, state, owns_cache: bool = True) -> Residual:
        if res.delta is not None and res.conn is None:
            raise ValueError("the 'hyper' arrangement follows an embedding or another 'hyper' block")
        x, h = self._joint(res, self.conn_mixer, self.norm_mixer)
        y = self.mixer.forward(h, ctx, cache, state, owns_cache)
        res = Residual(x, y, conn=self.conn_mixer, closer=self)
        if self.ffn is None:
            return res
        x, h = self._joint(res, self.conn_ffn, self.norm_ffn)
        return Residual(x, self.ffn.forward(h, ctx), conn=self.conn_ffn, closer=self)

    def final_rows(self, res: Residual, norm, rows: Optional[torch.Tensor], n_rows: int) -> torch.Tensor:
        """The rows the head reads: the pending update applied, the streams summed, ``norm`` applied (one launch, only
        the wanted rows)."""
        rms = fused_rms(norm)
        if rms is None:
            raise ValueError("the 'hyper' arrangement folds a plain RMS norm into its last joint; the final norm is of another kind")
        x = res.x
        h = torch.empty((n_rows, x.shape[-1]), dtype=self.mixer.rt.dtype, device=x.device)
        pend = res.conn
        K.hc_step(x, self.streams, y=res.delta, mix=pend.mix if pend is not None else None,
                  outw=pend.outw if pend is not None else None, mult=pend.mult if pend is not None else 1.0, inw=self._ones,
                  norm_w=rms[0], eps=rms[1], rows=rows, h=h)
        return h

    def stream_sum(self, res: Residual) -> torch.Tensor:
        """The sum of the streams with the pending update applied, ``[n, W]`` float32 (for tests and bring-up; plain
        tensor operations, not on the product path)."""
        x = res.x if res.x.dim() == 3 else res.x[:, None, :].expand(-1, self.streams, -1)
        if res.delta is not None:
            c = res.conn
            x = torch.einsum("st,nsw->ntw", c.mix, x) + c.mult * c.outw[None, :, None] * res.delta.to(torch.float32)[:, None, :]
        return x.sum(dim=1)
