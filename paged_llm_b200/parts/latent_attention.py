"""Attention through low-rank latents.

With h the mixer's input and RMS the root-mean-square norm (float32, a weight each):

    cq = RMS(W_dq h)                       query latent
    q  = W_uq cq                           per head [unrotated: head_dim | rotated: rot_dim]
    [c_raw | kr] = W_dkv h,  c = RMS(c_raw)   key/value latent; kr: one rotated key part shared by all heads
    k_h = [W_uk,h c | rot(kr)],  v_h = W_uv,h c
    score = (q_unrot . W_uk,h c + rot(q_rot) . rot(kr)) * scale

Only c and rot(kr) are cached: one key/value head of size kv_rank + rot_dim (rounded up to 16) whose key is
[c | rot(kr)] and whose value is [c].  The key up-projection is multiplied into the query instead of into
every cached key (q_unrot . W_uk,h c = (W_uk,h^T q_unrot) . c), so the attention kernel runs as
multi-query attention of `num_heads` heads over that one head, and the value up-projection is applied to the
kernel's output (sum_j p_j W_uv,h c_j = W_uv,h sum_j p_j c_j).  A decode step then reads kv_rank + rot_dim
numbers per cached token instead of num_heads * (head_dim + rot_dim + value_dim).

Rotation: the pairs of the position encoding named by `position` ((2i, 2i+1), or i with i + rotary_dim/2), over its
`rotary_dim` leading elements of the rotated part.  `window` as in the other attention parts.

Options: `q_rank` None: there is no query latent, q = W_q h straight from the input (tensor `q_proj`).  `sink`: one
learned number per head whose exponential joins the softmax's denominator (no key, no value, not scaled).
`head_gate`: head h's output is multiplied by sigmoid(w_g[h] . h), one number per head and token; being a scalar per
head it is applied to the kernel's latent output, in front of the value up-projection.
"""

from __future__ import annotations

import torch

from .attention import MAX_HEAD_DIM, pad16
from .base import LazyLinear, Mixer, PagedKV, TensorSpec, register_mixer


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    accepts_lazy_input = False

    def __init__(self, weights: dict[str, str], hidden_size: int, num_heads: int, head_dim: int, rot_dim: int,
                 value_dim: int, q_rank: int | None, kv_rank: int, scale: float, eps: float, window: int | None = None,
                 position=None, sink: bool = False, head_gate: bool = False):
        self.hidden_size, self.num_heads, self.head_dim, self.rot_dim = hidden_size, num_heads, head_dim, rot_dim
        self.value_dim, self.q_rank, self.kv_rank = value_dim, q_rank, kv_rank
        self.scale, self.eps = float(scale), float(eps)
        self.window = int(window) if window else None
        self.position = position
        if position is not None and position.rotary_dim > rot_dim:
            raise ValueError(f"latent attention rotates at most rot_dim={rot_dim} elements, not {position.rotary_dim}")
        self.has_sink, self.head_gate = bool(sink), bool(head_gate)
        self.sink = None
        self.cache_dim = pad16(kv_rank + rot_dim)
        if self.cache_dim > MAX_HEAD_DIM:
            raise ValueError(f"kv_rank + rot_dim = {kv_rank + rot_dim}: the latent is cached as one head, and the attention "
                             f"kernels take heads of at most {MAX_HEAD_DIM}")
        self.names = weights
        self.w_down = self.w_uq = self.w_uk_t = self.w_uv = self.w_o = self.q_weight = self.c_weight = None

    def cache_requirement(self):
        return PagedKV(1, self.cache_dim, self.window)

    def attention_plan_key(self):
        return (self.num_heads, 1, self.window, self.cache_dim)

    def tensor_specs(self):
        w, nh, d, r, dv = self.hidden_size, self.num_heads, self.head_dim, self.rot_dim, self.value_dim
        if self.q_rank is None:
            out = {self.names["q_proj"]: TensorSpec((nh * (d + r), w))}
        else:
            out = {self.names["dq"]: TensorSpec((self.q_rank, w)),
                   self.names["dq_norm"]: TensorSpec((self.q_rank,), role="vector", init="norm"),
                   self.names["uq"]: TensorSpec((nh * (d + r), self.q_rank))}
        if self.has_sink:
            out[self.names["sink"]] = TensorSpec((nh,), role="vector", init="norm_zero")
        if self.head_gate:
            out[self.names["g_proj"]] = TensorSpec((nh, w))
        out.update({
            self.names["dkv"]: TensorSpec((self.kv_rank + r, w)),
            self.names["dkv_norm"]: TensorSpec((self.kv_rank,), role="vector", init="norm"),
            self.names["uk"]: TensorSpec((nh * d, self.kv_rank)),
            self.names["uv"]: TensorSpec((nh * dv, self.kv_rank)),
            self.names["o_proj"]: TensorSpec((w, nh * dv)),
        })
        return out

    def load(self, tensors):
        nh, d, dv, kr = self.num_heads, self.head_dim, self.value_dim, self.kv_rank
        # one product for everything that reads the mixer's input: [query latent or queries | kv latent + rotated key | gates]
        first = "dq" if self.q_rank is not None else "q_proj"
        stack = [tensors[self.names[first]], tensors[self.names["dkv"]]]
        if self.head_gate:
            stack.append(tensors[self.names["g_proj"]])
        self.w_down = torch.cat(stack, dim=0).contiguous()
        self.w_uq = tensors[self.names["uq"]].contiguous() if self.q_rank is not None else None
        if self.has_sink:
            self.sink = tensors[self.names["sink"]].float().contiguous()
        # [heads, kv_rank, head_dim]: the transposed key up-projection of each head, a product's [out, in] operand
        self.w_uk_t = tensors[self.names["uk"]].view(nh, d, kr).transpose(1, 2).contiguous()
        self.w_uv = tensors[self.names["uv"]].view(nh, dv, kr).contiguous()
        self.w_o = tensors[self.names["o_proj"]].contiguous()
        self.q_weight = tensors[self.names["dq_norm"]].float().contiguous() if self.q_rank is not None else None
        self.c_weight = tensors[self.names["dkv_norm"]].float().contiguous()

    def bytes_read_per_step(self):
        return sum(w.numel() * w.element_size() for w in (self.w_down, self.w_uq, self.w_uk_t, self.w_uv, self.w_o)
                   if w is not None)

    def forward(self, h, ctx, cache):
        ops = ctx.ops
        nh, d, r, dv, kr, D = self.num_heads, self.head_dim, self.rot_dim, self.value_dim, self.kv_rank, self.cache_dim
        block_table = ctx.block_tables[cache.group]
        down = ops.linear(h, self.w_down)
        q_cols = self.q_rank if self.q_rank is not None else nh * (d + r)         # the columns in front of the kv latent
        cq = ops.latent_kv_write(down, q_cols, kr, r, D, self.q_weight, self.c_weight, self.eps, self.position, ctx,
                                 cache.kv, block_table, write=cache.owner, norm_q=self.q_rank is not None)
        q = ops.linear(cq, self.w_uq) if self.q_rank is not None else down        # heads at stride d + r from column 0
        q_abs = ops.heads_linear(q, 0, d + r, self.w_uk_t)                        # [T, heads * kv_rank]
        qk = ops.latent_queries(q_abs, q, nh, d, r, kr, D, self.position, ctx)
        o = ops.paged_attention(qk, nh, 1, D, cache.kv, block_table, ctx, self.scale, self.window, sink=self.sink)
        if self.head_gate:
            g0 = q_cols + kr + r
            o = ops.head_unrotate_gate(o, nh, D, kr, None, ctx, down[:, g0:g0 + nh])   # [T, heads * kv_rank], gated
            v = ops.heads_linear(o, 0, kr, self.w_uv)
        else:
            v = ops.heads_linear(o, 0, D, self.w_uv)                              # [T, heads * value_dim]
        return LazyLinear(v, self.w_o)
