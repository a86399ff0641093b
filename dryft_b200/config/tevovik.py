"""Typed configuration of the Tevovik decoder, read from its own ``config.json`` keys.

The design: token embedding times a constant plus a sinusoidal position vector; layers that add the
*normalised output* of each sublayer to a 32-bit residual stream (``x += norm(f(x))``, the sublayer reading ``x``
itself); a differential-attention mixer (two score maps per head over one set of values, per-map q/k RMS norm, no
rotation, keys visible only inside the query's own block of positions, a per-head output gate), whose keys and
values a layer may take from an earlier layer's cache; and a mixture-of-experts feed-forward with group-limited
top-k routing.  ``config.json`` gives every size and every constant that can differ between models:

    architecture        "Tevovik"
    vocab, width
    embedding.scale
    norm.eps
    layers[i].type      "attention"
    layers[i].mixer     heads, kv_heads, dim, vdim, scale, diff, mask.size, kv_from (optional)
    layers[i].mlp       null, or kind "moe" with expert.ff and router.{experts, top, groups.{count, keep}}

Tensors: ``embed``, ``head``, ``final.norm``, and per layer ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``,
``l<i>.mlp.*`` (see the parts for their local names).  No size or constant that ``config.json`` gives appears as a
literal below; what the design fixes (the sinusoid's base 10000, the norms' ``1 + w`` weight) does.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Optional, Tuple

from .qwen3 import ConfigError
from .spec import LayerSpec, ModelSpec, PartSpec, RunStep

SINUSOID_BASE = 10000.0       # fixed by the design
NORM_WEIGHT_OFFSET = 1.0      # layer norms and the final norm multiply by (1 + w)
DEFAULT_MAX_POSITIONS = 1 << 20   # the design has no longest sequence; the engine's own limits apply


def _pos_int(d: Mapping[str, Any], key: str, where: str) -> int:
    if key not in d:
        raise ConfigError(f"config.json: {where}.{key} is missing")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {where}.{key} must be a positive integer, got {v!r}")
    return v


def _number(d: Mapping[str, Any], key: str, where: str) -> float:
    if key not in d:
        raise ConfigError(f"config.json: {where}.{key} is missing")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {where}.{key} must be a number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class TevovikMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    diff: float
    chunk: Optional[int]
    kv_from: Optional[int]


@dataclass(frozen=True)
class TevovikMoE:
    ff: int
    experts: int
    top: int
    groups: int
    keep: int


@dataclass(frozen=True)
class TevovikConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    mixers: Tuple[TevovikMixer, ...]
    mlps: Tuple[Optional[TevovikMoE], ...]
    architecture: str = "Tevovik"

    @property
    def num_layers(self) -> int:
        return len(self.mixers)

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "TevovikConfig":
        vocab = _pos_int(raw, "vocab", "config")
        width = _pos_int(raw, "width", "config")
        if not isinstance(raw.get("embedding"), Mapping):
            raise ConfigError("config.json: embedding is missing")
        if not isinstance(raw.get("norm"), Mapping):
            raise ConfigError("config.json: norm is missing")
        emb_scale = _number(raw["embedding"], "scale", "embedding")
        eps = _number(raw["norm"], "eps", "norm")
        if not eps > 0.0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps!r}")
        layers = raw.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: layers must be a non-empty list")
        mixers: List[TevovikMixer] = []
        mlps: List[Optional[TevovikMoE]] = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            if not isinstance(layer, Mapping):
                raise ConfigError(f"config.json: {where} must be a mapping")
            if layer.get("type") != "attention":
                raise ConfigError(f"config.json: {where}.type {layer.get('type')!r} is not a mixer of this design (known: 'attention')")
            m = layer.get("mixer")
            if not isinstance(m, Mapping):
                raise ConfigError(f"config.json: {where}.mixer is missing")
            mw = where + ".mixer"
            heads, kv_heads = _pos_int(m, "heads", mw), _pos_int(m, "kv_heads", mw)
            if heads % kv_heads:
                raise ConfigError(f"config.json: {mw}.heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
            chunk = None
            mask = m.get("mask")
            if mask is not None:
                if not isinstance(mask, Mapping):
                    raise ConfigError(f"config.json: {mw}.mask must be a mapping or null")
                chunk = _pos_int(mask, "size", mw + ".mask")
            kv_from = m.get("kv_from")
            if kv_from is not None:
                if isinstance(kv_from, bool) or not isinstance(kv_from, int) or not 0 <= kv_from < i:
                    raise ConfigError(f"config.json: {mw}.kv_from must name an earlier layer, got {kv_from!r}")
                src = mixers[kv_from]
                if src.kv_from is not None:
                    raise ConfigError(f"config.json: {mw}.kv_from names layer {kv_from}, which has no keys and values of its own")
            mix = TevovikMixer(heads, kv_heads, _pos_int(m, "dim", mw), _pos_int(m, "vdim", mw), _number(m, "scale", mw),
                               _number(m, "diff", mw), chunk, kv_from)
            if kv_from is not None:
                src = mixers[kv_from]
                if (src.kv_heads, src.dim, src.vdim) != (mix.kv_heads, mix.dim, mix.vdim):
                    raise ConfigError(f"config.json: {mw}.kv_from names layer {kv_from}, which differs from this layer in kv_heads, dim or vdim")
            mixers.append(mix)
            mlp = layer.get("mlp")
            if mlp is None:
                mlps.append(None)
                continue
            lw = where + ".mlp"
            if not isinstance(mlp, Mapping) or mlp.get("kind") != "moe":
                raise ConfigError(f"config.json: {lw}.kind {mlp.get('kind') if isinstance(mlp, Mapping) else mlp!r} is not a feed-forward of this design (known: 'moe')")
            if not isinstance(mlp.get("expert"), Mapping) or not isinstance(mlp.get("router"), Mapping):
                raise ConfigError(f"config.json: {lw} needs 'expert' and 'router'")
            r = mlp["router"]
            experts, top = _pos_int(r, "experts", lw + ".router"), _pos_int(r, "top", lw + ".router")
            groups, keep = 1, 1
            if r.get("groups") is not None:
                groups = _pos_int(r["groups"], "count", lw + ".router.groups")
                keep = _pos_int(r["groups"], "keep", lw + ".router.groups")
            if experts % groups:
                raise ConfigError(f"config.json: {lw}.router: {experts} experts do not form {groups} equal groups")
            if keep > groups:
                raise ConfigError(f"config.json: {lw}.router.groups.keep ({keep}) exceeds count ({groups})")
            if top > keep * (experts // groups):
                raise ConfigError(f"config.json: {lw}.router.top ({top}) exceeds the experts of the kept groups ({keep * (experts // groups)})")
            mlps.append(TevovikMoE(_pos_int(mlp["expert"], "ff", lw + ".expert"), experts, top, groups, keep))
        arch = raw.get("architecture") or (raw.get("architectures") or ["Tevovik"])[0]
        return cls(vocab, width, emb_scale, eps, tuple(mixers), tuple(mlps), str(arch))

    def to_dict(self) -> dict:
        """The ``config.json`` this configuration is read back from."""
        layers = []
        for m, f in zip(self.mixers, self.mlps):
            mixer: Dict[str, Any] = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale,
                                     "diff": m.diff}
            if m.chunk is not None:
                mixer["mask"] = {"size": m.chunk}
            if m.kv_from is not None:
                mixer["kv_from"] = m.kv_from
            mlp = None
            if f is not None:
                mlp = {"kind": "moe", "expert": {"ff": f.ff},
                       "router": {"experts": f.experts, "top": f.top, "groups": {"count": f.groups, "keep": f.keep}}}
            layers.append({"type": "attention", "mixer": mixer, "mlp": mlp})
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps}, "layers": layers}

    # ------------------------------------------------------------------ accounting (benchmarks)
    def weight_bytes_per_decode_step(self, itemsize: int, batch: int = 1) -> int:
        """Bytes of weights one decode step of ``batch`` tokens reads at least: the projections, the experts the tokens
        choose (at most ``batch * top`` distinct ones per layer) and the output head."""
        total = self.vocab * self.width
        for m, f in zip(self.mixers, self.mlps):
            total += (m.heads * 2 * m.dim + m.heads) * self.width + self.width * m.heads * m.vdim
            if m.kv_from is None:
                total += (m.kv_heads * 2 * m.dim + m.kv_heads * m.vdim) * self.width
            if f is not None:
                total += f.experts * self.width + min(f.experts, batch * f.top) * 3 * f.ff * self.width
        return itemsize * total

    def matmul_flops_per_token(self) -> int:
        """Multiply-add flops of the weight matrices one token passes through, output head excluded."""
        total = 0
        for m, f in zip(self.mixers, self.mlps):
            total += (m.heads * 2 * m.dim + m.heads) * self.width + self.width * m.heads * m.vdim
            if m.kv_from is None:
                total += (m.kv_heads * 2 * m.dim + m.kv_heads * m.vdim) * self.width
            if f is not None:
                total += f.experts * self.width + f.top * 3 * f.ff * self.width
        return 2 * total

    # ------------------------------------------------------------------ the parts of each layer
    def model_spec(self) -> ModelSpec:
        def norm(name: str) -> PartSpec:
            return PartSpec("rmsnorm_offset", {"size": self.width, "eps": self.norm_eps, "offset": NORM_WEIGHT_OFFSET, "name": name})

        layers = []
        for i, (m, f) in enumerate(zip(self.mixers, self.mlps)):
            mixer = PartSpec("diff_attention", {
                "hidden_size": self.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "qk_dim": m.dim, "v_dim": m.vdim,
                "scale": m.scale, "diff": m.diff, "chunk": m.chunk, "window": None, "eps": self.norm_eps,
                "own_kv": m.kv_from is None, "gate": True,
                "names": {"q": "q", "k": "k", "v": "v", "o": "o", "gate": "g", "q_norm": "q.norm", "k_norm": "k.norm",
                          "lq1": "lq1", "lk1": "lk1", "lq2": "lq2", "lk2": "lk2"},
            })
            ffn = None
            if f is not None:
                ffn = PartSpec("moe", {
                    "hidden_size": self.width, "intermediate_size": f.ff, "experts": f.experts, "top": f.top,
                    "groups": f.groups, "keep": f.keep, "renormalize": False,
                    "names": {"router": "router", "expert": "e{}.", "gate": "gate", "up": "up", "down": "down"},
                })
            layers.append(LayerSpec(
                block="outnorm", mixer=mixer, ffn=ffn, norm_mixer=norm("norm1"), norm_ffn=norm("norm2") if f is not None else None,
                mixer_prefix=f"l{i}.mix.", ffn_prefix=f"l{i}.mlp.", norm_mixer_prefix=f"l{i}.", norm_ffn_prefix=f"l{i}.",
            ))
        spec = ModelSpec(
            architecture=self.architecture,
            vocab_size=self.vocab,
            hidden_size=self.width,
            max_positions=DEFAULT_MAX_POSITIONS,
            embedding=PartSpec("sinusoid_embedding", {"vocab_size": self.vocab, "hidden_size": self.width,
                                                      "scale": self.embedding_scale, "base": SINUSOID_BASE, "name": "embed"}),
            layers=tuple(layers),
            schedule=tuple(RunStep(layer=i, cache_from=m.kv_from) for i, m in enumerate(self.mixers)),
            final_norm=norm("norm"),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": self.width, "tied": False, "name": "head"}),
            embedding_prefix="",
            final_norm_prefix="final.",
            head_prefix="",
        )
        spec.validate()
        return spec
