"""Typed configuration of the Vobusun decoder, read from its own ``config.json`` keys.

The design: a token embedding times a constant plus a hashed token-pair (bigram) embedding, normalised; a 32-bit residual
stream kept as several copies joined by small matrices (hyper-connections) around pre-norm sublayers whose outputs are
scaled by a constant; three kinds of mixer -- retention (linear attention with a fixed decay per head), latent attention
(low-rank queries, keys and values, a sliding window, a gate per head) and a gated linear recurrence behind a short
convolution; a gated feed-forward with clamped branches; layers that run another layer's weights with a state of their own.

    architecture        "Vobusun"
    vocab, width, residual_mult, streams (absent: one plain residual stream)
    embedding           scale, bigram.{buckets, mul_prev, mul_cur} (absent: no pair table)
    norm.eps
    layers[i].type      "retention" | "latent_attention" | "rglru"
    layers[i].mixer     retention: heads, dim, vdim, decay[heads], rot.{dims, base}
                        latent_attention: heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, rot.{dims, base}, mask.size
                        rglru: width, conv, blocks
    layers[i].mlp       null, or kind "dense" with ff and limit
    layers[i].weights_of   the layer whose tensors this layer runs (it has none of its own)

Tensors: ``embed``, ``bigram``, ``embed.norm``, ``final.norm``, ``head`` and per layer with weights ``l<i>.norm1``,
``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``l<i>.hc1.*``, ``l<i>.hc2.*``.  What the design fixes is a constant below;
everything ``config.json`` gives is read from there.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Optional, Tuple

from .qwen3 import ConfigError
from .spec import ExtraPart, LayerSpec, ModelSpec, PartSpec, RunStep

# fixed by the design
GLU_ALPHA = 1.702          # the feed-forward's gate is g * sigmoid(1.702 g)
GLU_UP_OFFSET = 1.0        # ... times (u + 1)
RGLRU_C = 8.0              # log a = -8 r softplus(lam)
DEFAULT_MAX_POSITIONS = 1 << 20   # the design has no longest sequence; the engine's own limits apply

MIXER_TYPES = ("retention", "latent_attention", "rglru")


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


def _rot(m: Mapping[str, Any], where: str, limit: int) -> Optional[Tuple[int, float]]:
    rot = m.get("rot")
    if rot is None:
        return None
    if not isinstance(rot, Mapping):
        raise ConfigError(f"config.json: {where}.rot must be a mapping or null")
    dims, base = _pos_int(rot, "dims", where + ".rot"), _number(rot, "base", where + ".rot")
    if dims % 2 or dims > limit:
        raise ConfigError(f"config.json: {where}.rot.dims must be even and at most {limit}, got {dims}")
    if not base > 0.0:
        raise ConfigError(f"config.json: {where}.rot.base must be positive, got {base!r}")
    return dims, base


@dataclass(frozen=True)
class VobusunLayer:
    type: str
    mixer: Mapping[str, Any]               # the validated mixer sizes, as config.json gives them
    ff: Optional[int]
    limit: Optional[float]
    weights_of: Optional[int]


@dataclass(frozen=True)
class VobusunConfig:
    vocab: int
    width: int
    embedding_scale: float
    bigram: Optional[Tuple[int, int, int]]     # buckets, mul_prev, mul_cur
    norm_eps: float
    residual_mult: float
    streams: Optional[int]
    layers: Tuple[VobusunLayer, ...]
    architecture: str = "Vobusun"

    @property
    def num_layers(self) -> int:
        return len(self.layers)

    def weights_layer(self, i: int) -> int:
        """The layer whose tensors layer ``i`` runs."""
        while self.layers[i].weights_of is not None:
            i = self.layers[i].weights_of
        return i

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "VobusunConfig":
        vocab, width = _pos_int(raw, "vocab", "config"), _pos_int(raw, "width", "config")
        if not isinstance(raw.get("norm"), Mapping):
            raise ConfigError("config.json: norm is missing")
        eps = _number(raw["norm"], "eps", "norm")
        if not eps > 0.0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps!r}")
        emb = raw.get("embedding") or {}
        if not isinstance(emb, Mapping):
            raise ConfigError("config.json: embedding must be a mapping")
        scale = _number(emb, "scale", "embedding") if "scale" in emb else 1.0
        bigram = None
        if emb.get("bigram") is not None:
            bg = emb["bigram"]
            if not isinstance(bg, Mapping):
                raise ConfigError("config.json: embedding.bigram must be a mapping or null")
            bigram = (_pos_int(bg, "buckets", "embedding.bigram"), int(_number(bg, "mul_prev", "embedding.bigram")),
                      int(_number(bg, "mul_cur", "embedding.bigram")))
        mult = _number(raw, "residual_mult", "config") if "residual_mult" in raw else 1.0
        streams = None
        if raw.get("streams") is not None:
            streams = _pos_int(raw, "streams", "config")
        layers = raw.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: layers must be a non-empty list")
        out: List[VobusunLayer] = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            if not isinstance(layer, Mapping):
                raise ConfigError(f"config.json: {where} must be a mapping")
            kind = layer.get("type")
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of this design (known: {', '.join(MIXER_TYPES)})")
            m = layer.get("mixer")
            if not isinstance(m, Mapping):
                raise ConfigError(f"config.json: {where}.mixer is missing")
            mw = where + ".mixer"
            if kind == "retention":
                heads, dim = _pos_int(m, "heads", mw), _pos_int(m, "dim", mw)
                _pos_int(m, "vdim", mw)
                decay = m.get("decay")
                if not isinstance(decay, (list, tuple)) or len(decay) != heads or any(isinstance(d, bool) or not isinstance(d, (int, float)) for d in decay):
                    raise ConfigError(f"config.json: {mw}.decay must list one number per head ({heads})")
                _rot(m, mw, dim)
            elif kind == "latent_attention":
                for key in ("heads", "dim", "vdim", "q_rank", "kv_rank"):
                    _pos_int(m, key, mw)
                rot_dim = m.get("rot_dim", 0)
                if isinstance(rot_dim, bool) or not isinstance(rot_dim, int) or rot_dim < 0 or rot_dim % 2:
                    raise ConfigError(f"config.json: {mw}.rot_dim must be an even integer >= 0, got {rot_dim!r}")
                _number(m, "scale", mw)
                rot = _rot(m, mw, max(rot_dim, 2))
                if rot_dim and (rot is None or rot[0] != rot_dim):
                    raise ConfigError(f"config.json: {mw}.rot.dims must equal rot_dim ({rot_dim})")
                if m.get("mask") is not None:
                    if not isinstance(m["mask"], Mapping):
                        raise ConfigError(f"config.json: {mw}.mask must be a mapping or null")
                    _pos_int(m["mask"], "size", mw + ".mask")
            else:
                c, blocks = _pos_int(m, "width", mw), _pos_int(m, "blocks", mw)
                _pos_int(m, "conv", mw)
                if c % blocks:
                    raise ConfigError(f"config.json: {mw}.width ({c}) must be a multiple of blocks ({blocks})")
            ff = limit = None
            mlp = layer.get("mlp")
            if mlp is not None:
                lw = where + ".mlp"
                if not isinstance(mlp, Mapping) or mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: {lw}.kind {mlp.get('kind') if isinstance(mlp, Mapping) else mlp!r} is not a feed-forward of this design (known: 'dense')")
                ff = _pos_int(mlp, "ff", lw)
                limit = _number(mlp, "limit", lw) if mlp.get("limit") is not None else None
            src = layer.get("weights_of")
            if src is not None:
                if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < len(layers) or src == i:
                    raise ConfigError(f"config.json: {where}.weights_of must name another layer, got {src!r}")
            out.append(VobusunLayer(kind, dict(m), ff, limit, src))
        for i, layer in enumerate(out):
            seen, j = {i}, layer.weights_of
            while j is not None:
                if j in seen:
                    raise ConfigError(f"config.json: layers[{i}].weights_of runs in a circle")
                seen.add(j)
                j = out[j].weights_of
            if layer.weights_of is not None:
                src = out[cls._resolve(out, i)]
                if (src.type, dict(src.mixer), src.ff, src.limit) != (layer.type, dict(layer.mixer), layer.ff, layer.limit):
                    raise ConfigError(f"config.json: layers[{i}] runs the weights of layers[{layer.weights_of}] but differs from it in type or sizes")
        arch = raw.get("architecture") or (raw.get("architectures") or ["Vobusun"])[0]
        return cls(vocab, width, scale, bigram, eps, mult, streams, tuple(out), str(arch))

    @staticmethod
    def _resolve(layers: List[VobusunLayer], i: int) -> int:
        while layers[i].weights_of is not None:
            i = layers[i].weights_of
        return i

    def to_dict(self) -> dict:
        """The ``config.json`` this configuration is read back from."""
        layers = []
        for l in self.layers:
            d: Dict[str, Any] = {"type": l.type, "mixer": dict(l.mixer),
                                 "mlp": None if l.ff is None else {"kind": "dense", "ff": l.ff, "limit": l.limit}}
            if l.weights_of is not None:
                d["weights_of"] = l.weights_of
            layers.append(d)
        emb: Dict[str, Any] = {"scale": self.embedding_scale}
        if self.bigram is not None:
            emb["bigram"] = {"buckets": self.bigram[0], "mul_prev": self.bigram[1], "mul_cur": self.bigram[2]}
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "embedding": emb,
               "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult, "layers": layers}
        if self.streams is not None:
            out["streams"] = self.streams
        return out

    # ------------------------------------------------------------------ accounting (benchmarks)
    def _layer_weights(self, l: VobusunLayer) -> int:
        w, m = self.width, l.mixer
        if l.type == "retention":
            n = 2 * m["heads"] * m["dim"] * w + 3 * m["heads"] * m["vdim"] * w
        elif l.type == "latent_attention":
            r = m.get("rot_dim", 0)
            n = (m["q_rank"] + m["kv_rank"] + r + m["heads"]) * w + m["heads"] * (m["dim"] + r) * m["q_rank"] \
                + m["heads"] * (m["dim"] + m["vdim"]) * m["kv_rank"] + w * m["heads"] * m["vdim"]
        else:
            n = 3 * m["width"] * w + 2 * m["width"] * (m["width"] // m["blocks"])
        if l.ff is not None:
            n += 3 * l.ff * w
        return n

    def weight_bytes_per_decode_step(self, itemsize: int, batch: int = 1) -> int:
        """Bytes of weights one decode step reads at least: every run layer's matrices and the output head."""
        return itemsize * (self.vocab * self.width + sum(self._layer_weights(l) for l in self.layers))

    def matmul_flops_per_token(self) -> int:
        """Multiply-add flops of the weight matrices one token passes through, output head excluded."""
        return 2 * sum(self._layer_weights(l) for l in self.layers)

    # ------------------------------------------------------------------ the parts of each layer
    def _mixer_spec(self, l: VobusunLayer) -> PartSpec:
        m, w = l.mixer, self.width

        def rope(layout: str) -> Optional[PartSpec]:
            rot = m.get("rot")
            if rot is None:
                return None
            return PartSpec("rope", {"theta": float(rot["base"]), "rotary_dim": int(rot["dims"]), "layout": layout, "freq": "rounded_once"})

        if l.type == "retention":
            return PartSpec("retention", {
                "hidden_size": w, "num_heads": m["heads"], "qk_dim": m["dim"], "v_dim": m["vdim"], "decay": tuple(m["decay"]),
                "k_scale": m["dim"] ** -0.5, "eps": self.norm_eps, "position": rope("half"),
                "names": {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o"}})
        if l.type == "latent_attention":
            return PartSpec("latent_attention", {
                "hidden_size": w, "num_heads": m["heads"], "qk_dim": m["dim"], "rot_dim": m.get("rot_dim", 0), "v_dim": m["vdim"],
                "q_rank": m["q_rank"], "kv_rank": m["kv_rank"], "scale": float(m["scale"]), "eps": self.norm_eps,
                "window": m["mask"]["size"] if m.get("mask") else None, "gate": True, "position": rope("interleaved"),
                "names": {"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv",
                          "gate": "g", "o": "o"}})
        return PartSpec("rglru", {
            "hidden_size": w, "channels": m["width"], "taps": m["conv"], "blocks": m["blocks"], "c": RGLRU_C,
            "names": {"y": "y", "y_bias": "y.b", "x": "x", "x_bias": "x.b", "conv": "conv", "conv_bias": "conv.b", "gate_a": "ra",
                      "gate_a_bias": "ra.b", "gate_i": "ri", "gate_i_bias": "ri.b", "lam": "lam", "o": "o"}})

    def model_spec(self) -> ModelSpec:
        def norm(name: str) -> PartSpec:
            return PartSpec("rmsnorm", {"size": self.width, "eps": self.norm_eps, "name": name})

        conn = PartSpec("hyper_connection", {"streams": self.streams, "mult": self.residual_mult})
        own = [i for i, l in enumerate(self.layers) if l.weights_of is None]     # layers with tensors of their own
        index = {i: k for k, i in enumerate(own)}
        specs = []
        for i in own:
            l = self.layers[i]
            ffn = None
            extra = [ExtraPart("conn_mixer", "connection", conn, f"l{i}.hc1.")]
            if l.ff is not None:
                ffn = PartSpec("clamped_glu", {"hidden_size": self.width, "intermediate_size": l.ff, "limit": l.limit,
                                               "alpha": GLU_ALPHA, "up_offset": GLU_UP_OFFSET,
                                               "names": {"gate": "gate", "up": "up", "down": "down"}})
                extra.append(ExtraPart("conn_ffn", "connection", conn, f"l{i}.hc2."))
            specs.append(LayerSpec(
                block="hyper", mixer=self._mixer_spec(l), ffn=ffn, norm_mixer=norm("norm1"), norm_ffn=norm("norm2") if ffn is not None else None,
                mixer_prefix=f"l{i}.mix.", ffn_prefix=f"l{i}.mlp.", norm_mixer_prefix=f"l{i}.", norm_ffn_prefix=f"l{i}.", extra=tuple(extra)))
        pair = None
        if self.bigram is not None:
            pair = {"buckets": self.bigram[0], "mul_prev": self.bigram[1], "mul_cur": self.bigram[2], "name": "bigram"}
        spec = ModelSpec(
            architecture=self.architecture,
            vocab_size=self.vocab,
            hidden_size=self.width,
            max_positions=DEFAULT_MAX_POSITIONS,
            embedding=PartSpec("pair_embedding", {"vocab_size": self.vocab, "hidden_size": self.width, "scale": self.embedding_scale,
                                                  "pair": pair, "norm": {"eps": self.norm_eps, "name": "embed.norm"}, "name": "embed"}),
            layers=tuple(specs),
            # every layer of config.json is a run step; one that runs another's weights names that layer and keeps a state of its own
            schedule=tuple(RunStep(layer=index[self.weights_layer(i)]) for i in range(len(self.layers))),
            final_norm=norm("final.norm"),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": self.width, "tied": False, "name": "head"}),
            embedding_prefix="",
            final_norm_prefix="",
            head_prefix="",
        )
        spec.validate()
        return spec
