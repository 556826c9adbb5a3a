"""Pre-norm arrangement: x += mixer(norm_in(x)); x += ffn(norm_post(x))
(reference: pagedllm/model/llama.py:174-185).  Each residual sum is handed to
the following norm as a pending branch so that one kernel does both.  A layer
without a feed-forward (`feed_forward` None, no "post_mixer" norm) is
x += mixer(norm_in(x)) alone."""

from __future__ import annotations

import torch

from .base import Block, LazyNormed, StreamBranch, TensorSpec, branch_args, materialize, register_block


@register_block("pre_norm")
class PreNormBlock(Block):
    NORM_NAMES = ("input", "post_mixer")

    def forward(self, x, pending, ctx, cache):
        h = self.norms["input"].add_forward(x, pending, ctx)
        if not self.mixer.accepts_lazy_input:
            h = ctx.ops.materialize(h)
        a = self.mixer.forward(h, ctx, cache)
        if self.feed_forward is None:
            return x, a
        h = self.norms["post_mixer"].add_forward(x, a, ctx)
        if not self.feed_forward.accepts_lazy_input:
            h = ctx.ops.materialize(h)
        f = self.feed_forward.forward(h, ctx)
        return x, f


@register_block("sandwich_norm")
class SandwichNormBlock(Block):
    """A norm in front of and behind each part: x += behind_mixer(mixer(input(x))), then
    x += behind_ffn(ffn(post_mixer(x))).  The norm behind a part travels with the branch (`LazyNormed`), so the
    norm that follows can do both norms and the sum in one kernel."""

    NORM_NAMES = ("input", "behind_mixer", "post_mixer", "behind_ffn")

    def forward(self, x, pending, ctx, cache):
        h = self.norms["input"].add_forward(x, pending, ctx)
        if not self.mixer.accepts_lazy_input:
            h = ctx.ops.materialize(h)
        a = LazyNormed(self.mixer.forward(h, ctx, cache), self.norms["behind_mixer"])
        if self.feed_forward is None:
            return x, a
        h = self.norms["post_mixer"].add_forward(x, a, ctx)
        if not self.feed_forward.accepts_lazy_input:
            h = ctx.ops.materialize(h)
        return x, LazyNormed(self.feed_forward.forward(h, ctx), self.norms["behind_ffn"])


@register_block("hyper_connections")
class HyperConnectionBlock(Block):
    """Pre-norm layer over `streams` copies x_1 .. x_s of the residual stream (a row of the stream tensor holds them
    side by side, [rows, streams * width]).  For sublayer q (the mixer, then the feed-forward) with its learned
    vectors `in`, `out` [streams] and matrix `mix` [streams, streams] (indexed [from, to]):

        u = sum_s in[s] x_s;   y = sublayer(norm(u));   x_t <- sum_s mix[s, t] x_s + out[t] y   (all t from the old x)

    The update travels as a `StreamBranch` to whatever norm comes next, so that one kernel mixes the copies, adds the
    branch, forms the next u and norms it.  `weights`: {"mixer": (in, out, mix), "ffn": (in, out, mix)} tensor names."""

    NORM_NAMES = ("input", "post_mixer")

    def __init__(self, mixer, feed_forward, norms, weights: dict, streams: int):
        super().__init__(mixer, feed_forward, norms)
        self.streams = int(streams)
        self.names = {k: tuple(v) for k, v in weights.items() if k == "mixer" or feed_forward is not None}
        self.hc: dict[str, tuple] = {}

    def tensor_specs(self):
        out = super().tensor_specs()
        s = self.streams
        # a single copy may come without connections in the checkpoint: they are then all 1, the plain residual sum
        opt = s == 1
        for w_in, w_out, w_mix in self.names.values():
            out[w_in] = TensorSpec((s,), role="vector", init="norm", optional=opt)
            out[w_out] = TensorSpec((s,), role="vector", init="norm", optional=opt)
            out[w_mix] = TensorSpec((s, s), role="vector", init="identity", optional=opt)
        return out

    def load(self, tensors):
        super().load(tensors)
        like = next(iter(tensors.values()))
        for key, names in self.names.items():
            shapes = ((self.streams,), (self.streams,), (self.streams, self.streams))
            self.hc[key] = tuple(tensors[n].float().contiguous() if n in tensors
                                 else torch.ones(shape, dtype=torch.float32, device=like.device)
                                 for n, shape in zip(names, shapes))

    def _sublayer(self, key, norm, part, x, pending, ctx, *args):
        ops = ctx.ops
        w_in, w_out, w_mix = self.hc[key]
        if pending is None:
            h = ops.stream_norm(x, self.streams, None, None, None, w_in, norm.weight, norm.groups, norm.eps)
        elif isinstance(pending, StreamBranch):
            y, pair = branch_args(pending.branch, ops)
            h = ops.stream_norm(x, self.streams, y, pending.mix, pending.out, w_in, norm.weight, norm.groups, norm.eps, **pair)
        else:
            raise TypeError("a layer of several streams follows a layer of one")
        return StreamBranch(part.forward(h, ctx, *args), w_mix, w_out)

    def forward(self, x, pending, ctx, cache):
        pending = self._sublayer("mixer", self.norms["input"], self.mixer, x, pending, ctx, cache)
        if self.feed_forward is not None:
            pending = self._sublayer("ffn", self.norms["post_mixer"], self.feed_forward, x, pending, ctx)
        return x, pending
