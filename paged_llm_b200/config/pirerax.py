"""Typed configuration of the Pirerax decoder, read from a checkpoint's config.json.

config.json gives every size and every constant that may differ between models of the design:

    architecture     "Pirerax"
    vocab, width     vocabulary and width of the residual stream
    norm.eps         epsilon of every RMS norm
    layers           one entry per layer: `type` (the mixer), `mixer` (its sizes and constants) and `mlp`
                     ({"kind": "moe", "expert": {ff, limit}, "router": {experts, top, groups {count, keep}}}, or
                     null for none)

Mixers by `type`:

    "attention"         heads, kv_heads, dim (query/key head), vdim (value head), scale,
                        q_temp {coef, every} (optional: queries grow with the logarithm of their position)
    "latent_attention"  heads, dim (unrotated query/key part), rot_dim (rotated part), vdim, kv_rank (the cached
                        latent), scale, rot {dims, base}
    "parallel"          two mixers on the same input, each output RMS-normed, then their mean
                        left:   heads, kv_heads, dim, vdim, scale, rot {dims, base}
                        right:  heads (value heads), kv_heads (query/key heads), dim, vdim, conv (taps)

What the engine does not compute is refused here with a message, never computed wrongly.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any

from .model import ConfigError, ModelConfig
from .rokarax import RokaraxRotary as RotaryConfig
from .rokarax import _need, _positive_int

MIXER_TYPES = ("attention", "latent_attention", "parallel")


def _heads(d: dict, where: str) -> tuple[int, int]:
    heads, kv = _positive_int(d, "heads", where), _positive_int(d, "kv_heads", where)
    if heads % kv:
        raise ConfigError(f"{where}: heads={heads} is not a multiple of kv_heads={kv}")
    return heads, kv


def _scale(d: dict, where: str) -> float:
    scale = float(_need(d, "scale", where))
    if not (scale > 0 and math.isfinite(scale)):
        raise ConfigError(f"{where}: scale={scale} must be positive")
    return scale


@dataclass(frozen=True)
class PireraxAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    q_temp: tuple | None = None         # (coef, every)
    rot: RotaryConfig | None = None

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "PireraxAttention":
        heads, kv = _heads(d, where)
        dim = _positive_int(d, "dim", where)
        vdim = int(d.get("vdim", dim))
        if vdim < 1:
            raise ConfigError(f"{where}: vdim={vdim} must be positive")
        qt = d.get("q_temp")
        if qt is not None:
            qt = (float(_need(qt, "coef", where + ".q_temp")), _positive_int(qt, "every", where + ".q_temp"))
        rot = d.get("rot")
        if rot is not None:
            rot = RotaryConfig.from_dict(rot, dim, where + ".rot")
            if rot.scaling is not None:
                raise ConfigError(f"{where}.rot: a scaling of the frequencies is not part of this design")
        return cls(heads, kv, dim, vdim, _scale(d, where), qt, rot)

    def to_dict(self) -> dict:
        d: dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                             "scale": self.scale}
        if self.q_temp is not None:
            d["q_temp"] = {"coef": self.q_temp[0], "every": self.q_temp[1]}
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        return d


@dataclass(frozen=True)
class PireraxLatentAttention:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot: RotaryConfig

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "PireraxLatentAttention":
        rot_dim = _positive_int(d, "rot_dim", where)
        rot = RotaryConfig.from_dict(_need(d, "rot", where), rot_dim, where + ".rot")
        if rot.scaling is not None:
            raise ConfigError(f"{where}.rot: a scaling of the frequencies is not part of this design")
        dim = _positive_int(d, "dim", where)
        return cls(_positive_int(d, "heads", where), dim, rot_dim, int(d.get("vdim", dim)),
                   _positive_int(d, "kv_rank", where), _scale(d, where), rot)

    def to_dict(self) -> dict:
        return {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "kv_rank": self.kv_rank,
                "scale": self.scale, "rot": self.rot.to_dict()}


@dataclass(frozen=True)
class PireraxDeltaRule:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "PireraxDeltaRule":
        heads, kv = _heads(d, where)
        dim = _positive_int(d, "dim", where)
        return cls(heads, kv, dim, int(d.get("vdim", dim)), _positive_int(d, "conv", where))

    def to_dict(self) -> dict:
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "conv": self.conv}


@dataclass(frozen=True)
class PireraxParallel:
    left: PireraxAttention
    right: PireraxDeltaRule

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "PireraxParallel":
        left = PireraxAttention.from_dict(_need(d, "left", where), where + ".left")
        if left.rot is None:
            raise ConfigError(f"config.json: {where}.left lacks the key 'rot'")
        return cls(left, PireraxDeltaRule.from_dict(_need(d, "right", where), where + ".right"))

    def to_dict(self) -> dict:
        return {"left": self.left.to_dict(), "right": self.right.to_dict()}


_MIXERS = {"attention": PireraxAttention, "latent_attention": PireraxLatentAttention, "parallel": PireraxParallel}


@dataclass(frozen=True)
class PireraxMLP:
    ff: int
    limit: float
    experts: int
    top: int
    groups: tuple | None = None         # (count, keep)

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "PireraxMLP":
        kind = _need(d, "kind", where)
        if kind != "moe":
            raise ConfigError(f"{where}: kind={kind!r} is not implemented (moe only)")
        ex, ro = _need(d, "expert", where), _need(d, "router", where)
        limit = float(_need(ex, "limit", where + ".expert"))
        if not limit > 0:
            raise ConfigError(f"{where}.expert: limit={limit} must be positive")
        experts, top = _positive_int(ro, "experts", where + ".router"), _positive_int(ro, "top", where + ".router")
        groups = ro.get("groups")
        allowed = experts
        if groups is not None:
            count, keep = _positive_int(groups, "count", where + ".router.groups"), _positive_int(groups, "keep", where + ".router.groups")
            if experts % count or keep > count:
                raise ConfigError(f"{where}.router.groups: {experts} experts in {count} groups of which {keep} are kept")
            groups, allowed = (count, keep), experts // count * keep
        if top > allowed:
            raise ConfigError(f"{where}.router: top={top} of {allowed} experts that may be chosen")
        return cls(_positive_int(ex, "ff", where + ".expert"), limit, experts, top, groups)

    def to_dict(self) -> dict:
        router: dict[str, Any] = {"experts": self.experts, "top": self.top}
        if self.groups is not None:
            router["groups"] = {"count": self.groups[0], "keep": self.groups[1]}
        return {"kind": "moe", "expert": {"ff": self.ff, "limit": self.limit}, "router": router}


@dataclass(frozen=True)
class PireraxLayer:
    type: str
    mixer: Any
    mlp: PireraxMLP | None


@dataclass(frozen=True)
class PireraxConfig(ModelConfig):
    norm_eps: float = 1e-6
    layers: tuple = ()
    extra: dict = field(default_factory=dict, compare=False, hash=False)

    @classmethod
    def from_hf_dict(cls, cfg: dict[str, Any], architecture: str = "Pirerax") -> "PireraxConfig":
        top = "the top level"
        vocab, width = _positive_int(cfg, "vocab", top), _positive_int(cfg, "width", top)
        eps = float(_need(_need(cfg, "norm", top), "eps", "norm"))
        if not (eps > 0 and math.isfinite(eps)):
            raise ConfigError(f"norm.eps must be positive, got {eps}")
        raw = _need(cfg, "layers", top)
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, lay in enumerate(raw):
            where = f"layers[{i}]"
            kind = _need(lay, "type", where)
            if kind not in _MIXERS:
                raise ConfigError(f"{where}: type={kind!r} is not implemented ({', '.join(MIXER_TYPES)} only)")
            mixer = _MIXERS[kind].from_dict(_need(lay, "mixer", where), where + ".mixer")
            if kind == "attention" and mixer.rot is not None:
                raise ConfigError(f"{where}.mixer: this mixer rotates nothing; 'rot' belongs to latent_attention and parallel")
            mlp = lay.get("mlp")
            layers.append(PireraxLayer(kind, mixer, PireraxMLP.from_dict(mlp, where + ".mlp") if mlp is not None else None))
        return cls(architecture=architecture, vocab_size=vocab, hidden_size=width, num_hidden_layers=len(layers),
                   max_position_embeddings=int(cfg.get("max_positions", 1 << 20)),
                   torch_dtype=str(cfg.get("torch_dtype") or cfg.get("dtype") or "bfloat16"),
                   norm_eps=eps, layers=tuple(layers))

    def to_hf_dict(self) -> dict:
        return {
            "architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
            "norm": {"eps": self.norm_eps},
            "layers": [{"type": lay.type, "mixer": lay.mixer.to_dict(),
                        "mlp": lay.mlp.to_dict() if lay.mlp is not None else None} for lay in self.layers],
            "torch_dtype": self.torch_dtype,
        }

    @property
    def num_parameters(self) -> int:
        from ..models.causal_lm import build_model
        from ..models.pirerax import pirerax_spec

        total = 0
        for spec in build_model(pirerax_spec(self)).tensor_specs().values():
            n = 1
            for e in spec.draw_shape or spec.shape:
                n *= e
            total += n
        return total
