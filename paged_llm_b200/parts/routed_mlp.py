"""A feed-forward of routed experts.

z = W_r h in float32; the `top_k` experts with the largest z take the token, weighted by the
softmax over those top_k logits only; y = sum of weight * expert(h), each expert a gated
feed-forward down(act(gate h) * up h) without bias.  With `shared_size`, a shared expert of the
same form runs for every token and is added times sigmoid(w_s . h), one number per token.

Options: `scoring` "sigmoid": every expert scores s = sigmoid(z) by itself, the `top_k` largest scores choose, and the
weights are those scores as they are (not renormalised).  `groups` (count, keep): the experts form `count` equal groups
of neighbours, a group scores the sum of its `group_score_top` largest scores, and only experts of the `keep` best
groups can be chosen.  `activation` "swish_clamped" with `activation_limit` L: g = min(gate, L), u = clamp(up, -L, L),
the expert's inner vector is g * sigmoid(1.702 g) * (u + 1).

The experts' matrices are stacked when the weights are taken ([E, 2F, D] gate over up, and
[E, D, F]), the shared gate's row rides behind the router's, and the kernel library does the
rest on the device: no count per expert ever reaches the host, so a step may be captured.
"""

from __future__ import annotations

import torch

from .base import FeedForward, TensorSpec, register_feed_forward
from .mlp import ACTIVATIONS

EXPERT_ACTIVATIONS = ACTIVATIONS + ("swish_clamped",)


@register_feed_forward("routed_mlp")
class RoutedMLP(FeedForward):
    def __init__(self, weights: dict[str, str], hidden_size: int, expert_size: int, num_experts: int, top_k: int,
                 activation: str = "silu", shared_size: int | None = None, shared_activation: str | None = None,
                 activation_limit: float | None = None, scoring: str = "softmax_top", groups=None,
                 group_score_top: int = 2):
        if not 1 <= top_k <= num_experts:
            raise ValueError(f"top_k={top_k} of {num_experts} experts")
        for a in (activation, shared_activation or activation):
            if a not in EXPERT_ACTIVATIONS:
                raise ValueError(f"activation {a!r} is not implemented ({', '.join(EXPERT_ACTIVATIONS)} only)")
        if activation == "swish_clamped" and not (activation_limit is not None and activation_limit > 0):
            raise ValueError("the clamped activation needs a positive activation_limit")
        if shared_size is not None and (shared_activation or activation) not in ACTIVATIONS:
            raise ValueError(f"a shared expert takes the activations {', '.join(ACTIVATIONS)} only")
        if scoring not in ("softmax_top", "sigmoid"):
            raise ValueError(f"scoring {scoring!r} is not implemented (softmax_top and sigmoid only)")
        if groups is not None:
            count, keep = (int(g) for g in groups)
            if count < 1 or num_experts % count or not 1 <= keep <= count or top_k > num_experts // count * keep:
                raise ValueError(f"{num_experts} experts in {count} groups of which {keep} are kept, top_k={top_k}")
            if scoring != "sigmoid":
                raise ValueError("groups of experts are chosen by sigmoid scores")
            groups = (count, keep, int(group_score_top))
        self.activation_limit = float(activation_limit) if activation_limit is not None else 0.0
        self.scoring, self.groups = scoring, groups
        self.hidden_size, self.expert_size, self.num_experts, self.top_k = hidden_size, expert_size, num_experts, top_k
        self.activation, self.shared_size = activation, shared_size
        self.shared_activation = shared_activation or activation
        self.names = weights
        self.w_router = None          # [E (+1) and padding, D]: the router's rows, then the shared expert's gate
        self.w_gate_up = None         # [E, 2F, D]
        self.w_down = None            # [E, D, F]
        self.shared = None            # (gate over up [2Fs, D], down [D, Fs])

    def tensor_specs(self):
        d, f = self.hidden_size, self.expert_size
        out = {self.names["router"]: TensorSpec((self.num_experts, d))}
        for e in range(self.num_experts):
            out[self.names[f"e{e}.gate"]] = TensorSpec((f, d))
            out[self.names[f"e{e}.up"]] = TensorSpec((f, d))
            out[self.names[f"e{e}.down"]] = TensorSpec((d, f))
        if self.shared_size is not None:
            s = self.shared_size
            out[self.names["shared.gate"]] = TensorSpec((s, d))
            out[self.names["shared.up"]] = TensorSpec((s, d))
            out[self.names["shared.down"]] = TensorSpec((d, s))
            out[self.names["shared.sg"]] = TensorSpec((1, d))
        return out

    def load(self, tensors):
        t, n, E = tensors, self.names, self.num_experts
        self.w_gate_up = torch.stack([torch.cat([t[n[f"e{e}.gate"]], t[n[f"e{e}.up"]]], dim=0) for e in range(E)]).contiguous()
        self.w_down = torch.stack([t[n[f"e{e}.down"]] for e in range(E)]).contiguous()
        router = [t[n["router"]]]
        if self.shared_size is not None:
            router.append(t[n["shared.sg"]])
            self.shared = (torch.cat([t[n["shared.gate"]], t[n["shared.up"]]], dim=0).contiguous(),
                           t[n["shared.down"]].contiguous())
        rows = sum(r.shape[0] for r in router)
        if rows % 8:
            # rows of zeros up to a multiple of 8: the library's product of the logits then takes an aligned form
            router.append(torch.zeros((8 - rows % 8, self.hidden_size), dtype=router[0].dtype, device=router[0].device))
        self.w_router = torch.cat(router, dim=0).contiguous()

    def bytes_read_per_step(self):
        """A step of one token: the router, its top_k experts and the shared expert."""
        per_expert = (self.w_gate_up[0].numel() + self.w_down[0].numel()) * self.w_down.element_size()
        total = self.w_router.numel() * self.w_router.element_size() + self.top_k * per_expert
        if self.shared is not None:
            total += sum(w.numel() * w.element_size() for w in self.shared)
        return total

    def forward(self, h, ctx):
        return ctx.ops.routed_experts(h, self.w_router, self.w_gate_up, self.w_down, self.top_k, self.activation,
                                      shared=self.shared, shared_activation=self.shared_activation,
                                      activation_limit=self.activation_limit, scoring=self.scoring, groups=self.groups)
