"""Interfaces of the parts a model is put together from, and their registries.

A model is data: a `ModelSpec` lists layers, each layer names a block
arrangement, a mixer, a feed-forward and a norm by registry key with their
sizes and constants as parameters, and a schedule lists the order in which
layers run.  `build_model` (models/causal_lm.py) turns the data into objects by
looking the keys up here.  A part never learns which architecture it belongs
to: it gets its own sizes, the names of its tensors, and at run time a
`StepContext`.

Adding a part = subclass the interface, decorate with `register_*`, and name
the key in a spec.  Nothing else in the package has to change.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable

import torch


# --------------------------------------------------------------------------- specs (data)

@dataclass
class PartSpec:
    """One part as data: registry key, parameters, and tensor names.

    `weights` maps the part's own short names (e.g. "q_proj") to the tensor
    names of the checkpoint (e.g. "model.layers.3.self_attn.q_proj.weight").
    """

    kind: str
    params: dict[str, Any] = field(default_factory=dict)
    weights: dict[str, str] = field(default_factory=dict)


@dataclass
class LayerSpec:
    """One layer: how mixer, feed-forward and norms are arranged (`block`: the registry key of the arrangement,
    or a `PartSpec` if the arrangement has parameters and tensors of its own)."""

    block: "str | PartSpec"
    mixer: PartSpec
    feed_forward: PartSpec | None          # None: the layer has no feed-forward
    norms: dict[str, PartSpec]


@dataclass
class ScheduleEntry:
    """One run of a layer.  `layer` indexes `ModelSpec.layers`, so a layer may be
    named twice (its weights are shared, each run has a cache of its own).
    `cache_from` names an earlier schedule entry whose cache this run reads
    instead of keeping one itself.  `add_embedding`: before this run the output
    of the embedding (the stream as it was in front of the first run) is added
    to the stream once more."""

    layer: int
    cache_from: int | None = None
    add_embedding: bool = False


@dataclass
class ModelSpec:
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    layers: list[LayerSpec]
    schedule: list[ScheduleEntry]
    final_norm: PartSpec
    head: PartSpec
    positions: dict[str, PartSpec] = field(default_factory=dict)   # position encodings by name
    ignored_tensors: tuple[str, ...] = ()                          # name suffixes a checkpoint may carry


@dataclass(frozen=True)
class TensorSpec:
    """What a part expects of one checkpoint tensor.

    role: "matrix" (a GEMM operand: kept in the compute dtype), "vector" (norm
    weights and the like: a tensor stored in 32-bit stays 32-bit, else compute
    dtype), "table_int" (integer tables: int32).
    init: how the random-weights mode draws it: "normal", "norm" (1 or 1+noise), "norm_zero" (0 or noise:
    a norm weight stored as its deviation from 1), "identity" (a matrix: the identity, or that plus noise).
    optional: may be absent from the checkpoint (e.g. a tied head).
    shape: an entry of -1 stands for a size that only the checkpoint gives (the rows of a table that
    config.json does not state); `draw_shape` is then what the random-weights mode draws.
    """

    shape: tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"
    optional: bool = False
    alias_of: str | None = None      # optional tensor that, when absent, is this other tensor
    draw_shape: tuple[int, ...] | None = None

    def fits(self, shape) -> bool:
        shape = tuple(shape)
        return len(shape) == len(self.shape) and all(e == -1 or e == g for e, g in zip(self.shape, shape))


# --------------------------------------------------------------------------- cache needs

@dataclass(frozen=True)
class PagedKV:
    """The mixer keeps a key and a value vector per token, in pages.
    `window`: only the last `window` tokens are ever read (None: all).
    `chunk`: positions are cut into chunks of this many, counted from 0, and a query reads
    only the keys of its own chunk (None: no such cut)."""

    num_kv_heads: int
    head_dim: int
    window: int | None = None
    chunk: int | None = None


@dataclass(frozen=True)
class FixedState:
    """The mixer keeps a state of fixed size per request (float32 by default)."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


def cache_leaves(requirement) -> list:
    """The single needs (`PagedKV`, `FixedState`) of a mixer's cache requirement, which may be one need, None, or a
    tuple of requirements (a mixer made of several mixers: each part gets a view of its own)."""
    if requirement is None:
        return []
    if isinstance(requirement, tuple):
        return [leaf for r in requirement for leaf in cache_leaves(r)]
    return [requirement]


# --------------------------------------------------------------------------- lazy branch outputs

@dataclass
class LazyLinear:
    """A branch output `input @ weight^T` that has not been computed yet.

    A mixer or feed-forward whose last operation is a projection may return this
    instead of a tensor.  The norm that consumes the branch can then let one
    kernel do projection + residual sum + normalisation; anything else calls
    `materialize`.  A part that returns a plain tensor works everywhere too.
    `bias` (float32 [out] or None) is added to the product."""

    input: torch.Tensor
    weight: torch.Tensor
    bias: torch.Tensor | None = None

    def materialize(self, ops) -> torch.Tensor:
        y = ops.linear(self.input, self.weight)
        return y if self.bias is None else ops.add_bias(y, self.bias)

    def rows(self, ops, idx: torch.Tensor) -> "LazyLinear":
        """The same branch for the rows `idx` only."""
        return LazyLinear(ops.gather_rows(self.input, idx), self.weight, self.bias)


@dataclass
class LazyNormed:
    """A branch output whose own norm (`norm`, applied to the branch before it joins the stream) has not been
    carried out yet.  The norm that consumes the branch may fuse it with the residual sum; anything else calls
    `materialize`.  `branch` is a tensor or a `LazyLinear`."""

    branch: object
    norm: object

    def materialize(self, ops) -> torch.Tensor:
        return self.norm.apply(materialize(self.branch, ops), ops)

    def rows(self, ops, idx: torch.Tensor) -> "LazyNormed":
        b = self.branch
        return LazyNormed(b.rows(ops, idx) if hasattr(b, "rows") else ops.gather_rows(b, idx), self.norm)


@dataclass
class LazyPair:
    """A branch output that is the weighted sum of two tensors which has not been formed yet:
    scales[0] * (a + biases[0]) + scales[1] * (b + biases[1]) in float32 (a mixer of two mixers side by side).  A norm
    over the copies of the stream takes both in its own kernel (`branch_args`); anything else calls `materialize`."""

    a: torch.Tensor
    b: torch.Tensor
    scales: tuple
    biases: tuple

    def materialize(self, ops) -> torch.Tensor:
        return ops.scaled_sum(self.a, self.scales[0], self.biases[0], self.b, self.scales[1], self.biases[1])

    def rows(self, ops, idx: torch.Tensor) -> "LazyPair":
        return LazyPair(ops.gather_rows(self.a, idx), ops.gather_rows(self.b, idx), self.scales, self.biases)


@dataclass
class LazyNormedPair:
    """A branch output that is the weighted sum of two tensors, each first divided by its own root mean square over
    the row and multiplied by a weight: scales[0] * rms_norm(a) * weights[0] + scales[1] * rms_norm(b) * weights[1],
    in float32 (a mixer of two mixers side by side whose outputs are normed before they meet).  The RMS norm that
    consumes the branch does both norms, the residual sum and its own norm in one kernel; anything else calls
    `materialize`."""

    a: torch.Tensor
    b: torch.Tensor
    weights: tuple
    scales: tuple
    eps: float

    def materialize(self, ops) -> torch.Tensor:
        return ops.normed_pair_sum(self.a, self.b, self.weights[0], self.weights[1], self.scales[0], self.scales[1], self.eps)

    def rows(self, ops, idx: torch.Tensor) -> "LazyNormedPair":
        return LazyNormedPair(ops.gather_rows(self.a, idx), ops.gather_rows(self.b, idx), self.weights, self.scales, self.eps)


def branch_args(branch, ops):
    """(branch tensor, keyword arguments) for `ops.stream_norm`: a pair travels as two branches with their scales and
    biases, everything else as one tensor."""
    if isinstance(branch, LazyPair):
        return branch.a, dict(branch2=branch.b, scales=branch.scales, biases=branch.biases)
    return materialize(branch, ops), {}


@dataclass
class StreamBranch:
    """A branch output that several copies of the residual stream are waiting for (hyper-connections): the copies
    become x_t <- sum_s mix[s, t] x_s + out[t] * branch, all at once from the old ones.  `mix` [streams, streams]
    and `out` [streams] are float32 tensors on the device; `branch` is a tensor or a `LazyLinear`.  The norm that
    follows carries the update out in the kernel that also forms its own input."""

    branch: object
    mix: torch.Tensor
    out: torch.Tensor

    def rows(self, ops, idx: torch.Tensor) -> "StreamBranch":
        b = self.branch
        return StreamBranch(b.rows(ops, idx) if hasattr(b, "rows") else ops.gather_rows(b, idx), self.mix, self.out)


def materialize(branch, ops):
    return branch.materialize(ops) if isinstance(branch, (LazyLinear, LazyNormed, LazyPair, LazyNormedPair)) else branch


# --------------------------------------------------------------------------- interfaces

class Part:
    """Common to all parts: which tensors it wants and how it takes them."""

    # True if `forward` hands its input straight to the kernel library's products, which
    # also take a normalisation that has not been carried out yet (ops.materialize turns
    # one into a tensor).  Parts that look at their input themselves leave this False.
    accepts_lazy_input = False

    # True if `forward` only launches work on the step's stream from the step's device
    # metadata, so that a decode step may be captured once and replayed.  A part that reads
    # `ctx.host`, waits for the device (e.g. to count rows) or allocates by data sets it
    # False; a model with one such part runs every step eagerly.
    capturable = True

    def tensor_specs(self) -> dict[str, TensorSpec]:
        """Checkpoint tensor name -> expectation."""
        return {}

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        """Take (already cast, on device) tensors by checkpoint name.  A part may
        fuse them into its own layout here; names on disk stay the checkpoint's."""

    def bytes_read_per_step(self) -> int:
        """Weight bytes one step has to read (for roofline arithmetic)."""
        return 0


class Norm(Part):
    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        """Normalise rows of `x` (residual stream dtype) -> compute dtype."""
        raise NotImplementedError

    def add_forward(self, x: torch.Tensor, branch, ctx) -> torch.Tensor:
        """x += branch (in place, in the residual dtype), then normalise.  With
        branch None this is `forward`.  `branch` is a tensor or a `LazyLinear`."""
        raise NotImplementedError


class PositionEncoding(Part):
    """Owns what positions turn into (for rotary: the cos/sin table)."""

    def prepare(self, max_positions: int, device, ops) -> None:
        raise NotImplementedError


class Embedding(Part):
    """Turns the step's token ids into the residual stream."""

    def forward(self, ids: torch.Tensor, ctx) -> torch.Tensor:
        """ids: [T] int32 -> [T, hidden] float32 (the residual dtype).  A spec may give the
        part a `position` parameter naming a position encoding; it arrives as the object."""
        raise NotImplementedError


class Head(Part):
    """Turns normalised rows into logits."""

    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:
        """h: [rows, hidden] in the compute dtype -> [rows, vocab] float32."""
        raise NotImplementedError


class Mixer(Part):
    """Mixes information between the tokens of a request (attention here)."""

    def cache_requirement(self) -> "PagedKV | FixedState | tuple | None":
        """What the mixer keeps per request: pages of keys and values, a state of fixed size, nothing, or, for a
        mixer made of several, a tuple with the requirement of each part (`cache.parts` holds their views)."""
        return None

    def forward(self, h: torch.Tensor, ctx, cache) -> torch.Tensor:
        """h: [T, hidden] in the compute dtype, token-major over all requests of
        the step.  `cache` is a `LayerCache` view (cache/storage.py) for this run
        of the layer, or None if the mixer keeps nothing.  Returns [T, hidden]
        (a tensor, or a `LazyLinear` if the last operation is a projection)."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    """Arrangement of norms, mixer and feed-forward around the residual stream.

    The stream is a pair (x, pending): `x` in the residual dtype and a branch
    output not yet added, so that the sum can be fused with the next norm.
    """

    def __init__(self, mixer: Mixer, feed_forward: FeedForward | None, norms: dict[str, Norm]):
        self.mixer, self.feed_forward, self.norms = mixer, feed_forward, norms

    def _parts(self):
        return [p for p in (self.mixer, self.feed_forward, *self.norms.values()) if p is not None]

    def forward(self, x, pending, ctx, cache):
        raise NotImplementedError

    def tensor_specs(self):
        out = {}
        for part in self._parts():
            out.update(part.tensor_specs())
        return out

    def load(self, tensors):
        for part in self._parts():
            part.load(tensors)

    def bytes_read_per_step(self):
        return sum(p.bytes_read_per_step() for p in self._parts())

    @property
    def capturable(self):
        return all(p.capturable for p in self._parts())


# --------------------------------------------------------------------------- registries

MIXERS: dict[str, Callable[..., Mixer]] = {}
FEED_FORWARDS: dict[str, Callable[..., FeedForward]] = {}
NORMS: dict[str, Callable[..., Norm]] = {}
POSITION_ENCODINGS: dict[str, Callable[..., PositionEncoding]] = {}
BLOCKS: dict[str, Callable[..., Block]] = {}
EMBEDDINGS: dict[str, Callable[..., Embedding]] = {}
HEADS: dict[str, Callable[..., Head]] = {}


def _register(table: dict, what: str):
    def outer(name: str):
        def inner(cls):
            if name in table and table[name] is not cls:
                raise ValueError(f"{what} {name!r} is already registered")
            table[name] = cls
            return cls
        return inner
    return outer


register_mixer = _register(MIXERS, "mixer")
register_feed_forward = _register(FEED_FORWARDS, "feed-forward")
register_norm = _register(NORMS, "norm")
register_position_encoding = _register(POSITION_ENCODINGS, "position encoding")
register_block = _register(BLOCKS, "block")
register_embedding = _register(EMBEDDINGS, "embedding")
register_head = _register(HEADS, "head")


def make_part(table: dict, what: str, spec: PartSpec, **extra):
    """Look a part up by its key and construct it from its spec."""
    try:
        cls = table[spec.kind]
    except KeyError:
        raise KeyError(f"unknown {what} {spec.kind!r}; registered: {sorted(table)}") from None
    return cls(weights=spec.weights, **spec.params, **extra)
