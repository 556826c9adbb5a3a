"""Gated linear attention: a matrix state per head with a decay per key channel (Yang et al., "Gated Linear Attention
Transformers with Hardware-Efficient Training").

    q = W_q h * dim^-1/2,  k = W_k h      [heads, dim];      v = W_v h      [heads, vdim]
    alpha = sigmoid(W_a2 (W_a1 h) + b)^(1/tau)              [heads, dim], through a low rank (the rows of W_a1)
    S_t = diag(alpha_t) S_(t-1) + k_t v_t^T                 S: [dim, vdim] per head, float32, carried per request
    o_t = S_t^T q_t
    out = W_o (concat_heads(rms_norm(o_t) * w) * silu(W_g h))          the norm over vdim, one weight for all heads

The decay (log-sigmoid, division by tau, exponential), the recurrence and the norm are float32 in both precisions.  The
state starts at zero, so a request's tokens may arrive in portions of any size.
"""

from __future__ import annotations

import torch

from .base import FixedState, LazyLinear, Mixer, TensorSpec, register_mixer


@register_mixer("gated_linear_attention")
class GatedLinearAttention(Mixer):
    accepts_lazy_input = False

    def __init__(self, weights: dict[str, str], hidden_size: int, num_heads: int, head_dim: int, value_dim: int,
                 tau: float, eps: float, decay_rank: int = 16):
        self.hidden_size, self.num_heads, self.head_dim, self.value_dim = hidden_size, num_heads, head_dim, value_dim
        self.tau, self.eps = float(tau), float(eps)
        self.decay_rank = int(decay_rank)           # what random weights are drawn with; a checkpoint's own shape rules
        self.names = weights
        self.w_in = self.w_a1 = self.w_a2 = self.b_a2 = self.norm_w = self.w_o = None

    def cache_requirement(self):
        return FixedState((self.num_heads * self.head_dim * self.value_dim,))

    def tensor_specs(self):
        n, hid = self.names, self.hidden_size
        hk, hv, r = self.num_heads * self.head_dim, self.num_heads * self.value_dim, self.decay_rank
        return {
            n["q_proj"]: TensorSpec((hk, hid)), n["k_proj"]: TensorSpec((hk, hid)), n["v_proj"]: TensorSpec((hv, hid)),
            n["g_proj"]: TensorSpec((hv, hid)), n["o_proj"]: TensorSpec((hid, hv)),
            n["norm"]: TensorSpec((self.value_dim,), role="vector", init="norm"),
            n["decay_down"]: TensorSpec((-1, hid), draw_shape=(r, hid)),
            n["decay_up"]: TensorSpec((hk, -1), draw_shape=(hk, r)),
            n["decay_bias"]: TensorSpec((hk,), role="vector", init="norm_zero"),
        }

    def load(self, tensors):
        n = self.names
        self.w_in = torch.cat([tensors[n[k]] for k in ("q_proj", "k_proj", "v_proj", "g_proj")], dim=0).contiguous()
        self.w_a1, self.w_a2 = tensors[n["decay_down"]].contiguous(), tensors[n["decay_up"]].contiguous()
        if self.w_a1.shape[0] != self.w_a2.shape[1]:
            raise ValueError(f"{n['decay_down']} has {self.w_a1.shape[0]} rows, {n['decay_up']} {self.w_a2.shape[1]} columns")
        self.b_a2 = tensors[n["decay_bias"]].float().contiguous()
        self.norm_w = tensors[n["norm"]].float().contiguous()
        self.w_o = tensors[n["o_proj"]].contiguous()

    def bytes_read_per_step(self):
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_a1, self.w_a2, self.w_o))

    def forward(self, h, ctx, cache):
        ops = ctx.ops
        if any(slot < 0 for slot in ctx.host.state_slots):
            raise RuntimeError("a request of a model with per-request state runs without a state slot "
                               "(CacheManager.acquire_state_slot at its admission)")
        H, d, dv = self.num_heads, self.head_dim, self.value_dim
        proj = ops.linear(h, self.w_in)                                          # [T, q | k | v | g]
        z = ops.linear(ops.linear(h, self.w_a1), self.w_a2, out_float32=True)    # [T, H * d] float32
        o = ops.linear_attention_scan(proj, z, self.b_a2, H, d, dv, self.tau, d ** -0.5, cache.state, ctx)
        out = ops.head_norm_gate(o, proj, 2 * H * d + H * dv, H, dv, self.norm_w, self.eps)
        return LazyLinear(out, self.w_o)
