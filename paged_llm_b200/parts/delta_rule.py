"""The gated delta rule: a matrix state per head that is decayed, corrected towards the new value along the new key, and
read with the query (Yang et al., "Gated Delta Networks: Improving Mamba2 with Delta Rule").

    q = W_q h, k = W_k h   [kv_heads, dim];   v = W_v h   [heads, vdim];   head i uses q/k head i // (heads // kv_heads)
    each of q, k, v: causal convolution over time per channel (`taps` wide, no bias, zeros before the start), then silu
    q <- q / sqrt(sum(q^2) + 1e-6) * dim^-1/2,   k <- k / sqrt(sum(k^2) + 1e-6)              per head
    beta = sigmoid(W_b h),   g = exp(-exp(A_log) * softplus(W_a h + dt_bias))                one number per head
    S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q                          S: [dim, vdim] per head
    out = W_o (concat_heads(rms_norm(o) * w) * silu(W_g h))          the norm over vdim, one weight for all heads

The state per request is float32 and of fixed size: the convolutions' last taps-1 inputs, then S of every head.  It
starts at zero and is carried from token to token, so a request's tokens may arrive in portions of any size.  Unit
norms, beta, softplus, the decay, the recurrence and the norm behind it are float32 in both precisions.
"""

from __future__ import annotations

import torch

from .base import FixedState, LazyLinear, Mixer, TensorSpec, register_mixer

# added under the root when q and k are made unit vectors: the design fixes it
UNIT_NORM_EPS = 1e-6


@register_mixer("gated_delta_rule")
class GatedDeltaRule(Mixer):
    accepts_lazy_input = False

    def __init__(self, weights: dict[str, str], hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 value_dim: int, conv_taps: int, eps: float, unit_eps: float = UNIT_NORM_EPS):
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads={num_heads} is not a multiple of num_kv_heads={num_kv_heads}")
        if conv_taps < 1:
            raise ValueError(f"conv_taps={conv_taps}")
        self.hidden_size, self.num_heads, self.num_kv_heads = hidden_size, num_heads, num_kv_heads
        self.head_dim, self.value_dim, self.conv_taps = head_dim, value_dim, conv_taps
        self.eps, self.unit_eps = float(eps), float(unit_eps)
        self.channels = 2 * num_kv_heads * head_dim + num_heads * value_dim          # what the convolution runs over
        self.names = weights
        self.w_in = self.conv_w = self.decay_rate = self.decay_bias = self.norm_w = self.w_o = None

    def cache_requirement(self):
        return FixedState(((self.conv_taps - 1) * self.channels + self.num_heads * self.head_dim * self.value_dim,))

    def tensor_specs(self):
        n, hid, H, G, d, dv = self.names, self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim
        return {
            n["q_proj"]: TensorSpec((G * d, hid)), n["k_proj"]: TensorSpec((G * d, hid)), n["v_proj"]: TensorSpec((H * dv, hid)),
            n["q_conv"]: TensorSpec((G * d, self.conv_taps), role="vector"),
            n["k_conv"]: TensorSpec((G * d, self.conv_taps), role="vector"),
            n["v_conv"]: TensorSpec((H * dv, self.conv_taps), role="vector"),
            n["beta_proj"]: TensorSpec((H, hid)), n["decay_proj"]: TensorSpec((H, hid)),
            n["decay_log"]: TensorSpec((H,), role="vector", init="norm_zero"),
            n["decay_bias"]: TensorSpec((H,), role="vector", init="norm_zero"),
            n["norm"]: TensorSpec((dv,), role="vector", init="norm"),
            n["g_proj"]: TensorSpec((H * dv, hid)), n["o_proj"]: TensorSpec((hid, H * dv)),
        }

    def load(self, tensors):
        n = self.names
        # one product for everything that reads the input: [q | k | v | output gate | beta | decay] and zero rows up to a multiple of 8
        stack = [tensors[n[k]] for k in ("q_proj", "k_proj", "v_proj", "g_proj", "beta_proj", "decay_proj")]
        rows = sum(t.shape[0] for t in stack)
        if rows % 8:
            stack.append(torch.zeros((8 - rows % 8, self.hidden_size), dtype=stack[0].dtype, device=stack[0].device))
        self.w_in = torch.cat(stack, dim=0).contiguous()
        self.conv_w = torch.cat([tensors[n[k]].float() for k in ("q_conv", "k_conv", "v_conv")], dim=0).contiguous()
        # g = exp(rate * softplus(a + bias)) with rate = -exp(A_log), formed once in float32
        self.decay_rate = (-torch.exp(tensors[n["decay_log"]].float())).contiguous()
        self.decay_bias = tensors[n["decay_bias"]].float().contiguous()
        self.norm_w = tensors[n["norm"]].float().contiguous()
        self.w_o = tensors[n["o_proj"]].contiguous()

    def bytes_read_per_step(self):
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_o))

    def forward(self, h, ctx, cache):
        ops = ctx.ops
        if any(slot < 0 for slot in ctx.host.state_slots):
            raise RuntimeError("a request of a model with per-request state runs without a state slot "
                               "(CacheManager.acquire_state_slot at its admission)")
        H, G, d, dv, C = self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim, self.channels
        proj = ops.linear(h, self.w_in)                                # [T, q | k | v | g | beta | a | padding]
        u, _ = ops.causal_conv(proj, 0, C, None, self.conv_w, None, cache.state, ctx, activation="silu", low=False)
        o = ops.delta_rule_scan(u, proj, C + H * dv, self.decay_rate, self.decay_bias, H, G, d, dv, self.unit_eps,
                                d ** -0.5, (self.conv_taps - 1) * C, cache.state, ctx)           # float32 [T, H * dv]
        out = ops.head_norm_gate(o, proj, C, H, dv, self.norm_w, self.eps)
        return LazyLinear(out, self.w_o)
