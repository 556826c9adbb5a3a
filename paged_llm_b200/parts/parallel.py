"""Two mixers side by side on the same input: out = left_scale * left(h) + right_scale * right(h).

The parts are ordinary mixers named by registry key; each keeps whatever it keeps (pages of keys and values, a state
of fixed size, nothing), so the cache requirement is the pair of theirs and each part gets its own view
(`cache.parts`).  The weighted sum of the two branch outputs, with a bias either output projection may have, is
float32 and is formed by one kernel.

With `out_norm_eps` each output is first RMS-normed over the model width with a weight of its own (tensors
`left_norm`, `right_norm`): out = left_scale * rms_norm(left(h)) * w_l + right_scale * rms_norm(right(h)) * w_r.  The
pair then travels unsummed (`LazyNormedPair`) to the norm that follows, whose kernel does all of it.
"""

from __future__ import annotations

from .base import MIXERS, LazyLinear, LazyNormedPair, LazyPair, Mixer, PartSpec, TensorSpec, make_part, register_mixer


@register_mixer("parallel")
class ParallelMixer(Mixer):
    accepts_lazy_input = False

    def __init__(self, weights: dict[str, str], left: PartSpec, right: PartSpec, left_scale: float = 1.0,
                 right_scale: float = 1.0, out_norm_eps: float | None = None):
        self.parts = (make_part(MIXERS, "mixer", left), make_part(MIXERS, "mixer", right))
        self.scales = (float(left_scale), float(right_scale))
        self.out_norm_eps = float(out_norm_eps) if out_norm_eps is not None else None
        self.names = weights
        self.out_weights = None

    @property
    def capturable(self):
        return all(p.capturable for p in self.parts)

    def cache_requirement(self):
        return tuple(p.cache_requirement() for p in self.parts)

    def attention_plan_key(self):
        keys = {k for k in (getattr(p, "attention_plan_key", lambda: None)() for p in self.parts) if k is not None}
        if len(keys) > 1:
            raise ValueError(f"the two parts of a parallel mixer plan attention differently: {sorted(keys)}")
        return next(iter(keys), None)

    def tensor_specs(self):
        out = {}
        for p in self.parts:
            out.update(p.tensor_specs())
        if self.out_norm_eps is not None:
            width = self.parts[0].hidden_size
            for key in ("left_norm", "right_norm"):
                out[self.names[key]] = TensorSpec((width,), role="vector", init="norm")
        return out

    def load(self, tensors):
        for p in self.parts:
            p.load(tensors)
        if self.out_norm_eps is not None:
            self.out_weights = tuple(tensors[self.names[k]].float().contiguous() for k in ("left_norm", "right_norm"))

    def bytes_read_per_step(self):
        return sum(p.bytes_read_per_step() for p in self.parts)

    def forward(self, h, ctx, cache):
        ops = ctx.ops
        outs = []
        for part, view in zip(self.parts, cache.parts):
            y = part.forward(h, ctx, view)
            bias = None
            if isinstance(y, LazyLinear):
                y, bias = ops.linear(y.input, y.weight), y.bias
            outs.append((y, bias))
        (a, bias_a), (b, bias_b) = outs
        if self.out_norm_eps is not None:
            if bias_a is not None or bias_b is not None:
                a, b = (y if bias is None else ops.add_bias(y, bias) for y, bias in outs)
            return LazyNormedPair(a, b, self.out_weights, self.scales, self.out_norm_eps)
        return LazyPair(a, b, (self.scales[0], self.scales[1]), (bias_a, bias_b))
