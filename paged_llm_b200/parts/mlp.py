"""Gated feed-forward: down(act(gate(x)) * up(x)), no bias, act = SiLU
(reference: pagedllm/model/llama.py:163-171) or the tanh form of GELU,
0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))).  Gate and up are stacked into
one matrix [2*intermediate, hidden] when the weights are taken."""

from __future__ import annotations

import torch

from .base import FeedForward, LazyLinear, TensorSpec, register_feed_forward


ACTIVATIONS = ("silu", "gelu_tanh")


@register_feed_forward("gated_mlp")
class GatedMLP(FeedForward):
    accepts_lazy_input = True

    def __init__(self, weights: dict[str, str], hidden_size: int, intermediate_size: int, activation: str = "silu"):
        if activation not in ACTIVATIONS:
            raise ValueError(f"activation {activation!r} is not implemented ({', '.join(ACTIVATIONS)} only)")
        self.hidden_size, self.intermediate_size, self.activation = hidden_size, intermediate_size, activation
        self.names = weights
        self.w_gate_up = None
        self.w_down = None

    def tensor_specs(self):
        h, i = self.hidden_size, self.intermediate_size
        return {
            self.names["gate_proj"]: TensorSpec((i, h)),
            self.names["up_proj"]: TensorSpec((i, h)),
            self.names["down_proj"]: TensorSpec((h, i)),
        }

    def load(self, tensors):
        self.w_gate_up = torch.cat([tensors[self.names["gate_proj"]], tensors[self.names["up_proj"]]], dim=0).contiguous()
        self.w_down = tensors[self.names["down_proj"]].contiguous()

    def bytes_read_per_step(self):
        return sum(w.numel() * w.element_size() for w in (self.w_gate_up, self.w_down))

    def forward(self, h, ctx):
        ops = ctx.ops
        if self.activation == "silu":
            return LazyLinear(ops.gated_silu_linear(h, self.w_gate_up), self.w_down)
        return LazyLinear(ops.gated_act_linear(h, self.w_gate_up, self.activation), self.w_down)


@register_feed_forward("poly_norm_mlp")
class PolyNormMLP(FeedForward):
    """down(act(up(x))) with no gate and no bias, where the activation is a polynomial of unit-norm powers:

        act(z) = a N(z) + b N(z^2) + c N(z^3) + e,   N(v) = v / sqrt(mean(v^2) + eps) over the token's inner values,

    powers element by element; a, b, c, e are the four numbers of the checkpoint tensor `act`.  The sums and the
    polynomial are float32."""

    accepts_lazy_input = True

    def __init__(self, weights: dict[str, str], hidden_size: int, intermediate_size: int, eps: float):
        self.hidden_size, self.intermediate_size, self.eps = hidden_size, intermediate_size, float(eps)
        self.names = weights
        self.w_up = self.w_down = self.coef = None

    def tensor_specs(self):
        h, i = self.hidden_size, self.intermediate_size
        return {self.names["up_proj"]: TensorSpec((i, h)), self.names["down_proj"]: TensorSpec((h, i)),
                self.names["act"]: TensorSpec((4,), role="vector", init="norm")}

    def load(self, tensors):
        self.w_up = tensors[self.names["up_proj"]].contiguous()
        self.w_down = tensors[self.names["down_proj"]].contiguous()
        self.coef = tensors[self.names["act"]].float().contiguous()

    def bytes_read_per_step(self):
        return sum(w.numel() * w.element_size() for w in (self.w_up, self.w_down))

    def forward(self, h, ctx):
        ops = ctx.ops
        return LazyLinear(ops.poly_norm(ops.linear(h, self.w_up), self.coef, self.eps), self.w_down)
