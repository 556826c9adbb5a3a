"""Grouped-query attention over the paged cache.

q, k, v = h Wq^T, h Wk^T, h Wv^T (no bias), rotary on q and k, k and v written to
their slots of the cache, attention through the block table with query head h
reading kv head h // (heads // kv_heads), then the output projection
(reference: pagedllm/model/llama.py:131-160; the attention itself:
pagedllm/attention/reference.py:23-55).  The three projections are stacked into
one matrix when the weights are taken, so a step runs one product for them.

`scale` and `window` are parameters: the reference fixes scale = head_dim^-0.5
(llama.py:138) and has no window; a window w keeps, for the query at position p,
the keys at positions p-w+1 .. p.  Two score modifiers, off unless a spec asks
for them (the reference has neither): `score_cap` c turns a scaled score s into
c * tanh(s / c), and `position_slopes` (one number per query head) adds
slope * (key position - query position) to it, a bias by distance that needs no
rotation of q and k.  `chunk` c cuts the positions of a request into chunks of c,
counted from position 0, and lets a query see only the keys of its own chunk;
the cache gives the pages of finished chunks back.  `value_from_key`: there is
no value projection; the value of a token is its key as projected, before the
rotation (the cache still keeps both, since the stored key is rotated).
"""

from __future__ import annotations

import math

import torch

from .base import LazyLinear, Mixer, PagedKV, TensorSpec, register_mixer


@register_mixer("paged_attention")
class PagedAttention(Mixer):
    accepts_lazy_input = True

    def __init__(self, weights: dict[str, str], hidden_size: int, num_heads: int, num_kv_heads: int,
                 head_dim: int, scale: float | None = None, window: int | None = None, position=None,
                 score_cap: float | None = None, position_slopes=None, chunk: int | None = None,
                 value_from_key: bool = False):
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads={num_heads} is not a multiple of num_kv_heads={num_kv_heads}")
        self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim = hidden_size, num_heads, num_kv_heads, head_dim
        self.scale = float(scale) if scale is not None else head_dim ** -0.5
        self.window = window
        if chunk is not None and not chunk > 0:
            raise ValueError(f"chunk={chunk} must be positive")
        self.chunk = int(chunk) if chunk else None
        self.value_from_key = bool(value_from_key)
        self.position = position
        if score_cap is not None and not score_cap > 0:
            raise ValueError(f"score_cap={score_cap} must be positive")
        if position_slopes is not None and len(position_slopes) != num_heads:
            raise ValueError(f"position_slopes has {len(position_slopes)} entries for {num_heads} heads")
        self.score_cap = score_cap
        self.position_slopes = [float(x) for x in position_slopes] if position_slopes is not None else None
        self._slopes = None              # the same on the device, made at the first step
        self.names = weights
        self.w_qkv = None
        self.w_o = None

    def cache_requirement(self):
        return PagedKV(self.num_kv_heads, self.head_dim, self.window, self.chunk)

    def attention_plan_key(self):
        """(query heads per kv head, kv heads, window, head size[, chunk]): what the step's work lists depend on."""
        key = (self.num_heads // self.num_kv_heads, self.num_kv_heads, self.window, self.head_dim)
        return key + (self.chunk,) if self.chunk else key

    def tensor_specs(self):
        h, d = self.hidden_size, self.head_dim
        out = {
            self.names["q_proj"]: TensorSpec((self.num_heads * d, h)),
            self.names["k_proj"]: TensorSpec((self.num_kv_heads * d, h)),
            self.names["o_proj"]: TensorSpec((h, self.num_heads * d)),
        }
        if not self.value_from_key:
            out[self.names["v_proj"]] = TensorSpec((self.num_kv_heads * d, h))
        return out

    def load(self, tensors):
        stacked = ("q_proj", "k_proj") if self.value_from_key else ("q_proj", "k_proj", "v_proj")
        self.w_qkv = torch.cat([tensors[self.names[k]] for k in stacked], dim=0).contiguous()
        self.w_o = tensors[self.names["o_proj"]].contiguous()

    def bytes_read_per_step(self):
        return sum(w.numel() * w.element_size() for w in (self.w_qkv, self.w_o))

    def forward(self, h, ctx, cache):
        ops = ctx.ops
        block_table = ctx.block_tables[cache.group]
        if self.position_slopes is not None and self._slopes is None:
            self._slopes = torch.tensor(self.position_slopes, dtype=torch.float32, device=cache.kv.device)
        extra = {}
        if self.chunk:
            extra["chunk"] = self.chunk
        if self.value_from_key:
            extra["value_from_key"] = True
        o = ops.qkv_attention(h, self.w_qkv, self.num_heads, self.num_kv_heads, self.head_dim, self.position, ctx,
                              cache.kv, block_table, self.scale, self.window, write=cache.owner,
                              softcap=self.score_cap, slopes=self._slopes, **extra)
        return LazyLinear(o, self.w_o)


def log_distance_buckets(rows: int, far: float, length: int) -> list[int]:
    """Row of a bias table for each distance 0 .. length-1: distances below rows // 2 have a row each; from there
    on rows - rows // 2 rows are spaced evenly in the logarithm of the distance up to `far`; every distance whose
    row would lie beyond the table shares the last row.  With h = rows // 2:
    row(n) = n for n < h, else min(rows - 1, h + floor(ln(n / h) / ln(far / h) * (rows - h)))."""
    half = rows // 2
    out = []
    for n in range(length):
        if n < half:
            out.append(n)
        else:
            out.append(min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half)))))
    return out


def pad16(n: int) -> int:
    return -(-n // 16) * 16


MAX_HEAD_DIM = 256      # the largest build of the attention kernels


@register_mixer("gated_attention")
class GatedAttention(Mixer):
    """Grouped-query attention over the paged cache with four things the plain part does not have:

    * keys and values of different sizes (`head_dim`, `value_dim`); the cache and the attention kernel run at
      the larger of the two rounded up to 16, the shorter vectors padded with zeros;
    * a norm over the whole projection: q (all heads together) is divided by its root mean square and multiplied
      by a weight of its size, and so is k; nothing is rotated;
    * a learned bias by distance: the table `rel` [rows, heads] (as many rows as the checkpoint holds) is read at the row of `log_distance_buckets` and
      added to the scaled score; it is laid out by distance once (`[heads, L]`) and the kernels read that;
    * a sigmoid gate, computed from the mixer's input, on the concatenated heads in front of the output projection.

    Further options, all off by default: `position` (a rotary table: q and k are rotated after their norms),
    `query_temperature` (coef, every): the normed query at position p is multiplied by
    1 + coef * ln(floor((p + 1) / every) + 1), so that late queries look harder; `sink`: one learned number per query
    head (tensor `sink`) whose exponential joins the softmax's denominator, a term without key or value that is
    neither scaled nor masked and counts once.

    `window` w: the query at position p sees keys p-w+1 .. p.  `keep_window`: what the cache has to keep (the
    largest window of the layers that read it; a layer with `shares_cache` has no key and value projections and
    reads the cache of another layer, written with that layer's norm).
    """

    accepts_lazy_input = False

    def __init__(self, weights: dict[str, str], hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 value_dim: int, scale: float, eps: float, window: int | None = None, keep_window: int | None = 0,
                 distance_bias: bool = False, bias_far: float = 0.0, bias_rows: int = 32, gate: bool = True,
                 shares_cache: bool = False, sink: bool = False, position=None, query_temperature=None):
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads={num_heads} is not a multiple of num_kv_heads={num_kv_heads}")
        self.hidden_size, self.num_heads, self.num_kv_heads = hidden_size, num_heads, num_kv_heads
        self.head_dim, self.value_dim, self.scale, self.eps = head_dim, value_dim, float(scale), float(eps)
        self.window = int(window) if window else None
        # (a layer without a window of its own keeps everything; else the larger of its window and what is asked)
        self.keep_window = None if self.window is None or keep_window is None else max(int(keep_window), self.window)
        # the table's number of rows is the checkpoint's (`bias_rows` only says how many the random-weights mode draws)
        self.distance_bias, self.bias_far, self.bias_rows = bool(distance_bias), float(bias_far), int(bias_rows)
        self.gate, self.shares_cache = bool(gate), bool(shares_cache)
        self.has_sink, self.position = bool(sink), position
        if position is not None and position.rotary_dim > head_dim:
            raise ValueError(f"a rotation of {position.rotary_dim} elements in heads of {head_dim}")
        self.query_temperature = None
        if query_temperature is not None:
            coef, every = query_temperature
            if not int(every) >= 1:
                raise ValueError(f"query_temperature: every={every} must be at least 1")
            self.query_temperature = (float(coef), int(every))
        self.sink = None
        self.cache_dim = pad16(max(head_dim, value_dim))
        if self.cache_dim > MAX_HEAD_DIM:
            raise ValueError(f"head sizes {head_dim} / {value_dim}: the attention kernels take heads of at most {MAX_HEAD_DIM}")
        self.names = weights
        self.w_in = self.w_o = self.q_weight = self.k_weight = self.bias_by_distance = None

    def cache_requirement(self):
        return PagedKV(self.num_kv_heads, self.cache_dim, self.keep_window)

    def attention_plan_key(self):
        return (self.num_heads // self.num_kv_heads, self.num_kv_heads, self.window, self.cache_dim)

    def tensor_specs(self):
        h, d, dv = self.hidden_size, self.head_dim, self.value_dim
        out = {self.names["q_proj"]: TensorSpec((self.num_heads * d, h)),
               self.names["q_norm"]: TensorSpec((self.num_heads * d,), role="vector", init="norm"),
               self.names["o_proj"]: TensorSpec((h, self.num_heads * dv))}
        if not self.shares_cache:
            out[self.names["k_proj"]] = TensorSpec((self.num_kv_heads * d, h))
            out[self.names["v_proj"]] = TensorSpec((self.num_kv_heads * dv, h))
            out[self.names["k_norm"]] = TensorSpec((self.num_kv_heads * d,), role="vector", init="norm")
        if self.distance_bias:
            out[self.names["rel"]] = TensorSpec((-1, self.num_heads), role="vector", draw_shape=(self.bias_rows, self.num_heads))
        if self.gate:
            out[self.names["g_proj"]] = TensorSpec((self.num_heads * dv, h))
        if self.has_sink:
            out[self.names["sink"]] = TensorSpec((self.num_heads,), role="vector", init="norm_zero")
        return out

    def load(self, tensors):
        if self.has_sink:
            self.sink = tensors[self.names["sink"]].float().contiguous()
        stack = ["q_proj"] + ([] if self.shares_cache else ["k_proj", "v_proj"]) + (["g_proj"] if self.gate else [])
        self.w_in = torch.cat([tensors[self.names[k]] for k in stack], dim=0).contiguous()
        self.w_o = tensors[self.names["o_proj"]].contiguous()
        self.q_weight = tensors[self.names["q_norm"]].float().contiguous()
        self.k_weight = None if self.shares_cache else tensors[self.names["k_norm"]].float().contiguous()
        if self.distance_bias:
            rel = tensors[self.names["rel"]].float()
            if rel.shape[0] < 2 or not self.bias_far > rel.shape[0] // 2:
                raise ValueError(f"a bias table of {rel.shape[0]} rows needs at least two rows and a farthest distance "
                                 f"above {rel.shape[0] // 2}, not {self.bias_far}")
            # all distances from the farthest on share a row; no query reaches further back than its window
            far = int(math.ceil(self.bias_far)) + 1
            length = min(self.window, far) if self.window else far
            rows = log_distance_buckets(rel.shape[0], self.bias_far, length)
            self.bias_by_distance = rel[torch.tensor(rows, device=rel.device)].t().contiguous()      # [heads, length]

    def bytes_read_per_step(self):
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_o))

    def forward(self, h, ctx, cache):
        ops = ctx.ops
        nh, nkv, d, dv, D = self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim, self.cache_dim
        block_table = ctx.block_tables[cache.group]
        proj = ops.linear(h, self.w_in)
        q = ops.normed_qkv_write(proj, nh, nkv, d, dv, D, self.q_weight, self.k_weight, self.eps, ctx, cache.kv,
                                 block_table, has_kv=not self.shares_cache, write=cache.owner and not self.shares_cache,
                                 position=self.position, query_temperature=self.query_temperature)
        o = ops.paged_attention(q, nh, nkv, D, cache.kv, block_table, ctx, self.scale, self.window,
                                dist_bias=self.bias_by_distance, sink=self.sink)
        g0 = nh * d + (0 if self.shares_cache else nkv * (d + dv))
        o = ops.head_gate(o, nh, D, dv, proj[:, g0:g0 + nh * dv] if self.gate else None)
        return LazyLinear(o, self.w_o)


@register_mixer("rotated_value_attention")
class RotatedValueAttention(Mixer):
    """Grouped-query softmax attention over the paged cache whose values carry their position too:

    * q, k, v and the output projection have biases (`bias`);
    * q and k are rotated by `position` (any table of this package: partial rotation, either pairing, YaRN);
    * the value of position j is rotated by j over all its `value_dim` elements with the angles of `value_position`
      and cached so; a head's output at position i (the weighted sum of rotated values) is turned back by -i, so that
      what the output sees of a value depends on the distance i - j only;
    * with `head_gate`, head h's output is multiplied by sigmoid(w_g[h] . input), one number per head, after the
      turn back and in front of the output projection;
    * keys and values may differ in size; the cache and the attention kernel run at the larger of the two rounded
      up to 16, the shorter vectors padded with zeros.
    """

    accepts_lazy_input = False

    def __init__(self, weights: dict[str, str], hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 value_dim: int, scale: float, position=None, value_position=None, bias: bool = True,
                 head_gate: bool = True, window: int | None = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads={num_heads} is not a multiple of num_kv_heads={num_kv_heads}")
        self.hidden_size, self.num_heads, self.num_kv_heads = hidden_size, num_heads, num_kv_heads
        self.head_dim, self.value_dim, self.scale = head_dim, value_dim, float(scale)
        self.position, self.value_position = position, value_position
        if value_position is not None and (value_position.rotary_dim != value_dim or value_dim % 2):
            raise ValueError(f"values of {value_dim} elements are rotated as a whole; the table turns "
                             f"{value_position.rotary_dim}")
        self.bias, self.head_gate = bool(bias), bool(head_gate)
        self.window = int(window) if window else None
        self.cache_dim = pad16(max(head_dim, value_dim))
        if self.cache_dim > MAX_HEAD_DIM:
            raise ValueError(f"head sizes {head_dim} / {value_dim}: the attention kernels take heads of at most {MAX_HEAD_DIM}")
        self.names = weights
        self.w_in = self.b_in = self.w_o = self.b_o = None

    def cache_requirement(self):
        return PagedKV(self.num_kv_heads, self.cache_dim, self.window)

    def attention_plan_key(self):
        return (self.num_heads // self.num_kv_heads, self.num_kv_heads, self.window, self.cache_dim)

    def _stack(self):
        return ["q_proj", "k_proj", "v_proj"] + (["g_proj"] if self.head_gate else [])

    def tensor_specs(self):
        h, d, dv, n = self.hidden_size, self.head_dim, self.value_dim, self.names
        out = {n["q_proj"]: TensorSpec((self.num_heads * d, h)), n["k_proj"]: TensorSpec((self.num_kv_heads * d, h)),
               n["v_proj"]: TensorSpec((self.num_kv_heads * dv, h)), n["o_proj"]: TensorSpec((h, self.num_heads * dv))}
        if self.head_gate:
            out[n["g_proj"]] = TensorSpec((self.num_heads, h))
        if self.bias:
            for k in ("q_proj", "k_proj", "v_proj", "o_proj"):
                out[n[k + "_bias"]] = TensorSpec((out[n[k]].shape[0],), role="vector", init="norm_zero")
        return out

    def load(self, tensors):
        n = self.names
        self.w_in = torch.cat([tensors[n[k]] for k in self._stack()], dim=0).contiguous()
        self.w_o = tensors[n["o_proj"]].contiguous()
        if self.bias:
            self.b_in = torch.cat([tensors[n[k + "_bias"]].float() for k in ("q_proj", "k_proj", "v_proj")]).contiguous()
            self.b_o = tensors[n["o_proj_bias"]].float().contiguous()

    def bytes_read_per_step(self):
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_o))

    def forward(self, h, ctx, cache):
        ops = ctx.ops
        nh, nkv, d, dv, D = self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim, self.cache_dim
        block_table = ctx.block_tables[cache.group]
        proj = ops.linear(h, self.w_in)                                     # [T, q | k | v | gate]
        q = ops.rotated_qkv_write(proj, self.b_in, nh, nkv, d, dv, D, self.position, self.value_position, ctx, cache.kv,
                                  block_table, write=cache.owner)
        o = ops.paged_attention(q, nh, nkv, D, cache.kv, block_table, ctx, self.scale, self.window)
        g0 = nh * d + nkv * (d + dv)
        o = ops.head_unrotate_gate(o, nh, D, dv, self.value_position, ctx,
                                   proj[:, g0:g0 + nh] if self.head_gate else None)
        return LazyLinear(o, self.w_o, self.b_o)
