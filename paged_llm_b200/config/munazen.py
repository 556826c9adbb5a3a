"""Typed configuration of the Munazen decoder, read from a checkpoint's config.json.

config.json gives every size and every constant that may differ between models of the design:

    architecture     "Munazen"
    vocab, width     vocabulary and width of the residual stream
    norm.eps         epsilon of every RMS norm
    norm.groups      equal consecutive parts of the stream that the layers' norms divide by their own root mean square
    streams          copies of the residual stream that the hyper-connections keep (absent: one stream and plain
                     residual sums, no `hc` tensors)
    loop             {start, stop, times}: layers start .. stop-1 run `times` times in a row with the same weights,
                     each run with a cache and state of its own (absent: every layer once)
    layers           one entry per layer: `type` (the mixer), `mixer` (its sizes and constants) and `mlp`
                     ({"kind": "dense", "ff": n}, or null for none)

Mixers by `type`:

    "parallel"  two mixers on the same input, summed as left_scale * left + right_scale * right
                left:   heads, kv_heads, dim (query/key head), vdim (value head), scale,
                        rot {dims, base, scaling {factor, original, fast, slow} (optional)}
                right:  width (channels of the recurrence), blocks (of the block-diagonal gates), conv (taps)
    "gla"       heads, dim (query/key head), vdim (value head), tau (the decay is sigmoid(z)^(1/tau))

What the engine does not compute is refused here with a message, never computed wrongly.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any

from .model import ConfigError, ModelConfig
from .rokarax import RokaraxRotary as RotaryConfig
from .rokarax import _need, _positive_int

MIXER_TYPES = ("parallel", "gla")


@dataclass(frozen=True)
class MunazenAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: RotaryConfig

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "MunazenAttention":
        heads, kv = _positive_int(d, "heads", where), _positive_int(d, "kv_heads", where)
        if heads % kv:
            raise ConfigError(f"{where}: heads={heads} is not a multiple of kv_heads={kv}")
        dim = _positive_int(d, "dim", where)
        vdim = int(d.get("vdim", dim))
        if vdim < 2 or vdim % 2:
            raise ConfigError(f"{where}: vdim={vdim} must be even (values are rotated in pairs)")
        return cls(heads, kv, dim, vdim, float(_need(d, "scale", where)),
                   RotaryConfig.from_dict(_need(d, "rot", where), dim, where + ".rot"))

    def to_dict(self) -> dict:
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale,
                "rot": self.rot.to_dict()}


@dataclass(frozen=True)
class MunazenRecurrence:
    width: int
    blocks: int
    conv: int

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "MunazenRecurrence":
        m = cls(*(_positive_int(d, k, where) for k in ("width", "blocks", "conv")))
        if m.width % m.blocks:
            raise ConfigError(f"{where}: width={m.width} is not a multiple of blocks={m.blocks}")
        return m

    def to_dict(self) -> dict:
        return {"width": self.width, "blocks": self.blocks, "conv": self.conv}


@dataclass(frozen=True)
class MunazenParallel:
    left: MunazenAttention
    right: MunazenRecurrence
    left_scale: float
    right_scale: float

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "MunazenParallel":
        return cls(MunazenAttention.from_dict(_need(d, "left", where), where + ".left"),
                   MunazenRecurrence.from_dict(_need(d, "right", where), where + ".right"),
                   float(d.get("left_scale", 1.0)), float(d.get("right_scale", 1.0)))

    def to_dict(self) -> dict:
        return {"left": self.left.to_dict(), "right": self.right.to_dict(), "left_scale": self.left_scale,
                "right_scale": self.right_scale}


@dataclass(frozen=True)
class MunazenLinearAttention:
    heads: int
    dim: int
    vdim: int
    tau: float

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "MunazenLinearAttention":
        dim = _positive_int(d, "dim", where)
        tau = float(_need(d, "tau", where))
        if not (tau > 0 and math.isfinite(tau)):
            raise ConfigError(f"{where}: tau={tau} must be positive")
        return cls(_positive_int(d, "heads", where), dim, int(d.get("vdim", dim)), tau)

    def to_dict(self) -> dict:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "tau": self.tau}


_MIXERS = {"parallel": MunazenParallel, "gla": MunazenLinearAttention}


@dataclass(frozen=True)
class MunazenLayer:
    type: str
    mixer: Any
    ff: int | None                      # inner size of the dense feed-forward, None for none


@dataclass(frozen=True)
class MunazenConfig(ModelConfig):
    norm_eps: float = 1e-6
    norm_groups: int = 1
    streams: int | None = None          # None: no hyper-connections
    loop: tuple | None = None           # (start, stop, times)
    layers: tuple = ()
    extra: dict = field(default_factory=dict, compare=False, hash=False)

    @classmethod
    def from_hf_dict(cls, cfg: dict[str, Any], architecture: str = "Munazen") -> "MunazenConfig":
        top = "the top level"
        vocab, width = _positive_int(cfg, "vocab", top), _positive_int(cfg, "width", top)
        norm = _need(cfg, "norm", top)
        eps = float(_need(norm, "eps", "norm"))
        if not (eps > 0 and math.isfinite(eps)):
            raise ConfigError(f"norm.eps must be positive, got {eps}")
        groups = int(norm.get("groups") or 1)
        if groups < 1 or width % groups:
            raise ConfigError(f"norm.groups={groups} must divide width={width}")
        streams = cfg.get("streams")
        if streams is not None:
            streams = int(streams)
            if not 1 <= streams <= 8:
                raise ConfigError(f"streams={streams}: the hyper-connection kernels take 1 to 8 streams")
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
            mlp, ff = lay.get("mlp"), None
            if mlp is not None:
                if _need(mlp, "kind", where + ".mlp") != "dense":
                    raise ConfigError(f"{where}.mlp: kind={mlp['kind']!r} is not implemented (dense only)")
                ff = _positive_int(mlp, "ff", where + ".mlp")
            layers.append(MunazenLayer(kind, mixer, ff))
        loop = cfg.get("loop")
        if loop is not None:
            start, stop, times = (int(_need(loop, k, "loop")) for k in ("start", "stop", "times"))
            if not (0 <= start <= stop <= len(layers)) or times < 1:
                raise ConfigError(f"loop: start={start}, stop={stop}, times={times} do not fit {len(layers)} layers")
            loop = (start, stop, times)
        return cls(architecture=architecture, vocab_size=vocab, hidden_size=width, num_hidden_layers=len(layers),
                   max_position_embeddings=int(cfg.get("max_positions", 1 << 20)),
                   torch_dtype=str(cfg.get("torch_dtype") or cfg.get("dtype") or "bfloat16"),
                   norm_eps=eps, norm_groups=groups, streams=streams, loop=loop, layers=tuple(layers))

    def to_hf_dict(self) -> dict:
        d = {
            "architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
            "norm": {"eps": self.norm_eps, "groups": self.norm_groups},
            "layers": [{"type": lay.type, "mixer": lay.mixer.to_dict(),
                        "mlp": {"kind": "dense", "ff": lay.ff} if lay.ff is not None else None} for lay in self.layers],
            "torch_dtype": self.torch_dtype,
        }
        if self.streams is not None:
            d["streams"] = self.streams
        if self.loop is not None:
            d["loop"] = dict(zip(("start", "stop", "times"), self.loop))
        return d

    def layer_runs(self) -> list[int]:
        """The layers in the order they run: the looped span `times` times in a row, the others once."""
        n = len(self.layers)
        if self.loop is None:
            return list(range(n))
        start, stop, times = self.loop
        return list(range(start)) + list(range(start, stop)) * times + list(range(stop, n))

    @property
    def num_parameters(self) -> int:
        from ..models.causal_lm import build_model
        from ..models.munazen import munazen_spec

        total = 0
        for spec in build_model(munazen_spec(self)).tensor_specs().values():
            n = 1
            for e in spec.draw_shape or spec.shape:
                n *= e
            total += n
        return total
