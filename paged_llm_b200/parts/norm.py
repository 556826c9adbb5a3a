"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w, all in 32-bit, eps inside the
root, the weight multiplied before the down-cast (reference:
pagedllm/model/llama.py:74-83).  With `unit_offset` the checkpoint stores the
weight around zero and the factor is 1 + w; it is formed once, in float32, when
the weights are taken.

`groups` g > 1: the row is cut into g equal consecutive parts and each part is divided by its own root mean
square (the weight still spans the row).  `streams` s > 1: the residual stream arrives as s copies per token
([rows, s * dim], hyper-connections); the norm sees their sum, after a pending `StreamBranch` has been mixed in."""

from __future__ import annotations

import torch

from .base import LazyLinear, LazyNormed, LazyNormedPair, LazyPair, Norm, StreamBranch, TensorSpec, branch_args, materialize, register_norm


@register_norm("rms_norm")
class RMSNorm(Norm):
    def __init__(self, weights: dict[str, str], dim: int, eps: float, unit_offset: bool = False, groups: int = 1,
                 streams: int = 1):
        self.dim, self.eps, self.unit_offset = dim, float(eps), bool(unit_offset)
        if groups < 1 or dim % groups:
            raise ValueError(f"a norm over {dim} values does not divide into {groups} equal parts")
        self.groups, self.streams = int(groups), int(streams)
        self.name = weights["weight"]
        self.weight = None

    def tensor_specs(self):
        return {self.name: TensorSpec((self.dim,), role="vector", init="norm_zero" if self.unit_offset else "norm")}

    def load(self, tensors):
        w = tensors[self.name]
        self.weight = (w.float() + 1.0).contiguous() if self.unit_offset else w.contiguous()

    def bytes_read_per_step(self):
        return self.weight.numel() * self.weight.element_size()

    def forward(self, x, ctx):
        return self.add_forward(x, None, ctx)

    def add_forward(self, x, branch, ctx):
        if self.groups > 1 or self.streams > 1 or isinstance(branch, StreamBranch):
            # one kernel: the copies of the stream take the branch in, are summed, and the sum is normed in parts
            ops = ctx.ops
            if isinstance(branch, StreamBranch):
                y, pair = branch_args(branch.branch, ops)
                return ops.stream_norm(x, self.streams, y, branch.mix, branch.out, None, self.weight, self.groups, self.eps,
                                       **pair)
            y, pair = branch_args(branch, ops) if branch is not None else (None, {})
            return ops.stream_norm(x, self.streams, y, None, None, None, self.weight, self.groups, self.eps, **pair)
        if branch is None:
            return ctx.ops.rms_norm(x, self.weight, self.eps)
        if isinstance(branch, LazyNormedPair):
            # both norms of the pair, the residual sum and this norm in one kernel
            return ctx.ops.normed_pair_add_rms_norm(x, branch.a, branch.b, branch.weights[0], branch.weights[1],
                                                    branch.scales[0], branch.scales[1], branch.eps, self.weight, self.eps)
        if isinstance(branch, LazyPair) or (isinstance(branch, LazyLinear) and branch.bias is not None):
            branch = branch.materialize(ctx.ops)
        if isinstance(branch, LazyLinear):
            return ctx.ops.linear_add_rms_norm(branch.input, branch.weight, x, self.weight, self.eps)
        return ctx.ops.add_rms_norm(x, branch, self.weight, self.eps)


@register_norm("dynamic_tanh")
class DynamicTanh(Norm):
    """y = tanh(alpha x) * w + b: a norm that takes no mean and no variance of x.  `alpha` is one learned
    number, w and b are vectors; all of it is elementwise and float32.  As the norm in front of a part it fuses
    with the residual sum; as the norm behind a part (`LazyNormed`) it fuses in front of that sum, so that
    x += behind(branch); h = front(x) is one kernel."""

    def __init__(self, weights: dict[str, str], dim: int):
        self.dim = dim
        self.names = weights                  # weight, bias, alpha
        self.params = None                    # (alpha [1], weight [dim], bias [dim]) float32

    def tensor_specs(self):
        return {self.names["weight"]: TensorSpec((self.dim,), role="vector", init="norm"),
                self.names["bias"]: TensorSpec((self.dim,), role="vector", init="norm_zero"),
                self.names["alpha"]: TensorSpec((), role="vector", init="norm")}

    def load(self, tensors):
        self.params = (tensors[self.names["alpha"]].float().reshape(1).contiguous(),
                       tensors[self.names["weight"]].float().contiguous(),
                       tensors[self.names["bias"]].float().contiguous())

    def bytes_read_per_step(self):
        return sum(t.numel() * 4 for t in self.params)

    def apply(self, t: torch.Tensor, ops) -> torch.Tensor:
        """The norm of a tensor that is not the stream, in the compute dtype."""
        return ops.dyt(None, t, None, self.params)

    def forward(self, x, ctx):
        return ctx.ops.dyt(x, None, None, self.params)

    def add_forward(self, x, branch, ctx):
        if branch is None:
            return self.forward(x, ctx)
        ops = ctx.ops
        if isinstance(branch, LazyNormed) and isinstance(branch.norm, DynamicTanh):
            return ops.dyt(x, materialize(branch.branch, ops), branch.norm.params, self.params)
        return ops.dyt(x, materialize(branch, ops), None, self.params)
