"""The Pirerax decoder as data: `PireraxConfig` -> `ModelSpec`.

Tensor names: `embed`, `head`, `final.norm`, and per layer i the norms `l<i>.norm1` / `l<i>.norm2`, the mixer under
`l<i>.mix.` and the feed-forward under `l<i>.mlp.` (`router`, and per expert `e<j>.{gate,up,down}`).  Matrices are
stored [out, in].

A layer is pre-norm: x += mixer(norm1(x)), then (unless the layer has no feed-forward) x += ff(norm2(x)).  The mixer is
one of three.  "attention" (`mix.{q,k,v,g,o,q.norm,k.norm,sink}`): grouped-query attention without rotation, q and k
each normed over the whole projection, queries scaled by a temperature that grows with the logarithm of the position,
a learned sink in the softmax's denominator, an elementwise sigmoid gate.  "latent_attention"
(`mix.{q,dkv,dkv.norm,uk,uv,sink,g,o}`): keys and values from a normed latent plus a rotated key part shared by the
heads, a sink, one sigmoid gate per head.  "parallel": `mix.left.*`, the first kind of attention with rotary positions
and neither sink nor temperature, beside `mix.right.*`, the gated delta rule
(`{q,k,v}` with `{q,k,v}.conv`, `b`, `a`, `A_log`, `dt_bias`, `norm`, `g`, `o`); each output is RMS-normed over the width
(`mix.left.out`, `mix.right.out`) and the result is their mean.  The feed-forward routes each token to `top` experts by
sigmoid scores inside the best groups of experts.
"""

from __future__ import annotations

from ..config.pirerax import PireraxConfig
from ..parts.base import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

# The design fixes these: a group of experts scores the sum of its two best; both outputs of a parallel mixer count half.
GROUP_SCORE_TOP = 2
PARALLEL_SHARE = 0.5


def _shared(positions: dict, spec: PartSpec) -> str:
    """The name of a position table with these parameters (layers with the same rotation share one)."""
    for name, ps in positions.items():
        if ps.params == spec.params:
            return name
    name = f"rotary{len(positions)}"
    positions[name] = spec
    return name


def _attention(w: int, eps: float, m, prefix: str, positions: dict, sink: bool) -> PartSpec:
    position = None
    if m.rot is not None:
        position = _shared(positions, PartSpec("rotary", dict(head_dim=m.dim, theta=m.rot.base, pairing="half",
                                                              rotary_dim=m.rot.dims, scaling=None)))
    names = {"q_proj": prefix + "q", "k_proj": prefix + "k", "v_proj": prefix + "v", "g_proj": prefix + "g",
             "o_proj": prefix + "o", "q_norm": prefix + "q.norm", "k_norm": prefix + "k.norm"}
    if sink:
        names["sink"] = prefix + "sink"
    return PartSpec("gated_attention", dict(
        hidden_size=w, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, value_dim=m.vdim, scale=m.scale, eps=eps,
        gate=True, sink=sink, position=position, query_temperature=m.q_temp), names)


def pirerax_spec(cfg: PireraxConfig) -> ModelSpec:
    w, eps = cfg.hidden_size, cfg.norm_eps
    positions: dict[str, PartSpec] = {}
    layers = []

    def norm(name: str) -> PartSpec:
        return PartSpec("rms_norm", dict(dim=w, eps=eps), {"weight": name})

    for i, lay in enumerate(cfg.layers):
        p, m = f"l{i}.", lay.mixer
        mp = p + "mix."
        if lay.type == "attention":
            mixer = _attention(w, eps, m, mp, positions, sink=True)
        elif lay.type == "latent_attention":
            table = _shared(positions, PartSpec("rotary", dict(head_dim=m.rot_dim, theta=m.rot.base, pairing="half",
                                                               rotary_dim=m.rot.dims, scaling=None)))
            mixer = PartSpec("latent_attention", dict(
                hidden_size=w, num_heads=m.heads, head_dim=m.dim, rot_dim=m.rot_dim, value_dim=m.vdim, q_rank=None,
                kv_rank=m.kv_rank, scale=m.scale, eps=eps, position=table, sink=True, head_gate=True),
                {"q_proj": mp + "q", "dkv": mp + "dkv", "dkv_norm": mp + "dkv.norm", "uk": mp + "uk", "uv": mp + "uv",
                 "sink": mp + "sink", "g_proj": mp + "g", "o_proj": mp + "o"})
        else:
            r, rp = m.right, mp + "right."
            left = _attention(w, eps, m.left, mp + "left.", positions, sink=False)
            right = PartSpec("gated_delta_rule", dict(
                hidden_size=w, num_heads=r.heads, num_kv_heads=r.kv_heads, head_dim=r.dim, value_dim=r.vdim,
                conv_taps=r.conv, eps=eps),
                {"q_proj": rp + "q", "k_proj": rp + "k", "v_proj": rp + "v", "q_conv": rp + "q.conv", "k_conv": rp + "k.conv",
                 "v_conv": rp + "v.conv", "beta_proj": rp + "b", "decay_proj": rp + "a", "decay_log": rp + "A_log",
                 "decay_bias": rp + "dt_bias", "norm": rp + "norm", "g_proj": rp + "g", "o_proj": rp + "o"})
            mixer = PartSpec("parallel", dict(left=left, right=right, left_scale=PARALLEL_SHARE, right_scale=PARALLEL_SHARE,
                                              out_norm_eps=eps),
                             {"left_norm": mp + "left.out", "right_norm": mp + "right.out"})
        norms = {"input": norm(p + "norm1")}
        ffn = None
        if lay.mlp is not None:
            norms["post_mixer"] = norm(p + "norm2")
            f = lay.mlp
            names = {"router": p + "mlp.router"}
            for e in range(f.experts):
                for x in ("gate", "up", "down"):
                    names[f"e{e}.{x}"] = f"{p}mlp.e{e}.{x}"
            ffn = PartSpec("routed_mlp", dict(
                hidden_size=w, expert_size=f.ff, num_experts=f.experts, top_k=f.top, activation="swish_clamped",
                activation_limit=f.limit, scoring="sigmoid", groups=f.groups, group_score_top=GROUP_SCORE_TOP), names)
        layers.append(LayerSpec("pre_norm", mixer, ffn, norms))
    return ModelSpec(
        hidden_size=w,
        vocab_size=cfg.vocab_size,
        embedding=PartSpec("embedding", dict(vocab_size=cfg.vocab_size, hidden_size=w), {"weight": "embed"}),
        layers=layers,
        schedule=[ScheduleEntry(i) for i in range(len(layers))],
        final_norm=norm("final.norm"),
        head=PartSpec("lm_head", dict(vocab_size=cfg.vocab_size, hidden_size=w), {"weight": "head"}),
        positions=positions,
    )
