"""A recurrent block with a real-gated linear recurrence (the recurrent block of Griffin: De et al., "Griffin: Mixing
Gated Linear Recurrences with Local Attention for Efficient Language Models").

    y = gelu_tanh(W_y h + b_y)                                     [width]
    u = conv(W_x h + b_x)                 causal convolution per channel, `taps` wide, bias, no activation
    r = sigmoid(A_r[b] u_b + c_r[b]),  i = sigmoid(A_i[b] u_b + c_i[b])       per block b of `blocks` equal parts of u
    a = exp(-decay_scale * r * softplus(lam))                                 per channel
    S_t = a_t S_(t-1) + sqrt(1 - a_t^2) * i_t * u_t               from S = 0, the first token like every other
    out = W_o (S_t * y_t)

The state per request is float32 and of fixed size: the convolution's last taps-1 inputs, then S.  It starts at zero
and is carried from token to token, so a request's tokens may arrive in portions of any size.  The gates, the decay,
the square root and the recurrence are float32 in both precisions.
"""

from __future__ import annotations

import torch

from .base import FixedState, LazyLinear, Mixer, TensorSpec, register_mixer


@register_mixer("gated_linear_recurrence")
class GatedLinearRecurrence(Mixer):
    accepts_lazy_input = False

    def __init__(self, weights: dict[str, str], hidden_size: int, width: int, blocks: int, conv_taps: int,
                 decay_scale: float = 8.0):
        if width % blocks:
            raise ValueError(f"{width} channels do not divide into {blocks} blocks")
        if conv_taps < 1:
            raise ValueError(f"conv_taps={conv_taps}")
        self.hidden_size, self.width, self.blocks, self.conv_taps = hidden_size, width, blocks, conv_taps
        self.decay_scale = float(decay_scale)
        self.names = weights
        self.w_in = self.b_in = self.conv_w = self.conv_b = self.w_gates = self.b_gates = self.rate = self.w_o = None

    def cache_requirement(self):
        return FixedState((self.conv_taps * self.width,))          # taps-1 rows of inputs, then S

    def tensor_specs(self):
        n, c, b = self.names, self.width, self.blocks
        bw = c // b
        return {
            n["y_proj"]: TensorSpec((c, self.hidden_size)), n["y_bias"]: TensorSpec((c,), role="vector", init="norm_zero"),
            n["x_proj"]: TensorSpec((c, self.hidden_size)), n["x_bias"]: TensorSpec((c,), role="vector", init="norm_zero"),
            n["conv"]: TensorSpec((c, self.conv_taps), role="vector"),
            n["conv_bias"]: TensorSpec((c,), role="vector", init="norm_zero"),
            n["recurrence_gate"]: TensorSpec((b, bw, bw)),
            n["recurrence_gate_bias"]: TensorSpec((b, bw), role="vector", init="norm_zero"),
            n["input_gate"]: TensorSpec((b, bw, bw)),
            n["input_gate_bias"]: TensorSpec((b, bw), role="vector", init="norm_zero"),
            n["lam"]: TensorSpec((c,), role="vector"),
            n["o_proj"]: TensorSpec((self.hidden_size, c)),
        }

    def load(self, tensors):
        n = self.names
        self.w_in = torch.cat([tensors[n["y_proj"]], tensors[n["x_proj"]]], dim=0).contiguous()
        self.b_in = torch.cat([tensors[n["y_bias"]].float(), tensors[n["x_bias"]].float()]).contiguous()
        self.conv_w = tensors[n["conv"]].float().contiguous()
        self.conv_b = tensors[n["conv_bias"]].float().contiguous()
        # per block the rows of the recurrence gate over the rows of the input gate: one product per block gives both
        self.w_gates = torch.cat([tensors[n["recurrence_gate"]], tensors[n["input_gate"]]], dim=1).contiguous()
        self.b_gates = torch.cat([tensors[n["recurrence_gate_bias"]].float(), tensors[n["input_gate_bias"]].float()],
                                 dim=1).contiguous()
        # a = exp(rate * r) with rate = -decay_scale * softplus(lam), formed once in float32
        self.rate = (-self.decay_scale * torch.nn.functional.softplus(tensors[n["lam"]].float())).contiguous()
        self.w_o = tensors[n["o_proj"]].contiguous()

    def bytes_read_per_step(self):
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_gates, self.w_o))

    def forward(self, h, ctx, cache):
        ops = ctx.ops
        if any(slot < 0 for slot in ctx.host.state_slots):
            raise RuntimeError("a request of a model with per-request state runs without a state slot "
                               "(CacheManager.acquire_state_slot at its admission)")
        c = self.width
        yx = ops.linear(h, self.w_in)                                           # [T, y | x]
        u, u_low = ops.causal_conv(yx, c, c, self.b_in, self.conv_w, self.conv_b, cache.state, ctx)
        gates = ops.heads_linear(u_low, 0, c // self.blocks, self.w_gates, out_float32=True)
        out = ops.gated_recurrence(gates, self.b_gates, u, yx, self.b_in, self.rate, self.blocks, self.conv_taps,
                                   cache.state, ctx)
        return LazyLinear(out, self.w_o)
