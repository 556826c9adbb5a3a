"""The Munazen decoder as data: `MunazenConfig` -> `ModelSpec`.

Tensor names: `embed`, `head`, `final.norm`, and per layer i the norms `l<i>.norm1` / `l<i>.norm2`, the
hyper-connections `l<i>.hc1.{in,out,mix}` / `l<i>.hc2.{in,out,mix}` (sublayer 1 is the mixer, 2 the feed-forward; only
with `streams`), the mixer under `l<i>.mix.` and the feed-forward `l<i>.mlp.{up,down,act}`.  Matrices are stored
[out, in]; a bias has its matrix's name with `.b` added.

A layer is pre-norm over the copies of the residual stream; every norm is an RMS norm in `norm.groups` parts.  The
mixer is one of: two mixers side by side (`mix.left.*`: softmax attention with biases, rotated queries and keys
(interleaved pairs, YaRN), values rotated by their position and turned back at the query's, a sigmoid gate per head;
`mix.right.*`: a convolution and a real-gated linear recurrence), summed with the configuration's two scales; or gated
linear attention (`mix.{q,k,v,g,o,norm,a1,a2,a2.b}`).  The feed-forward is up -> PolyNorm -> down.  A span of layers
may run several times in a row: the schedule names those layers again and every run keeps a cache and state of its own.
"""

from __future__ import annotations

from ..config.munazen import MunazenConfig
from ..parts.base import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

# The decay of the recurrence is exp(-8 r softplus(lam)): the design fixes the 8.
RECURRENCE_DECAY_SCALE = 8.0


def _shared(positions: dict, spec: PartSpec) -> str:
    """The name of a position table with these parameters (layers with the same rotation share one)."""
    for name, ps in positions.items():
        if ps.params == spec.params:
            return name
    name = f"rotary{len(positions)}"
    positions[name] = spec
    return name


def munazen_spec(cfg: MunazenConfig) -> ModelSpec:
    w, eps, groups = cfg.hidden_size, cfg.norm_eps, cfg.norm_groups
    streams = cfg.streams
    positions: dict[str, PartSpec] = {}
    layers = []

    def norm(name: str, final: bool = False) -> PartSpec:
        return PartSpec("rms_norm", dict(dim=w, eps=eps, groups=groups, streams=(streams or 1) if final else 1),
                        {"weight": name})

    for i, lay in enumerate(cfg.layers):
        p, m = f"l{i}.", lay.mixer
        if lay.type == "parallel":
            a, r = m.left, m.right
            scaling = dict(a.rot.scaling, type="yarn") if a.rot.scaling else None
            qk_table = _shared(positions, PartSpec("rotary", dict(head_dim=a.dim, theta=a.rot.base, pairing="interleaved",
                                                                  rotary_dim=a.rot.dims, scaling=scaling)))
            v_table = _shared(positions, PartSpec("rotary", dict(head_dim=a.vdim, theta=a.rot.base, pairing="interleaved",
                                                                 rotary_dim=a.vdim, scaling=None)))
            lp, rp = p + "mix.left.", p + "mix.right."
            left = PartSpec("rotated_value_attention", dict(
                hidden_size=w, num_heads=a.heads, num_kv_heads=a.kv_heads, head_dim=a.dim, value_dim=a.vdim, scale=a.scale,
                position=qk_table, value_position=v_table, bias=True, head_gate=True),
                {"q_proj": lp + "q", "k_proj": lp + "k", "v_proj": lp + "v", "g_proj": lp + "g", "o_proj": lp + "o",
                 "q_proj_bias": lp + "q.b", "k_proj_bias": lp + "k.b", "v_proj_bias": lp + "v.b", "o_proj_bias": lp + "o.b"})
            right = PartSpec("gated_linear_recurrence", dict(
                hidden_size=w, width=r.width, blocks=r.blocks, conv_taps=r.conv, decay_scale=RECURRENCE_DECAY_SCALE),
                {"y_proj": rp + "y", "y_bias": rp + "y.b", "x_proj": rp + "x", "x_bias": rp + "x.b", "conv": rp + "conv",
                 "conv_bias": rp + "conv.b", "recurrence_gate": rp + "ra", "recurrence_gate_bias": rp + "ra.b",
                 "input_gate": rp + "ri", "input_gate_bias": rp + "ri.b", "lam": rp + "lam", "o_proj": rp + "o"})
            mixer = PartSpec("parallel", dict(left=left, right=right, left_scale=m.left_scale, right_scale=m.right_scale))
        else:
            mp = p + "mix."
            mixer = PartSpec("gated_linear_attention", dict(
                hidden_size=w, num_heads=m.heads, head_dim=m.dim, value_dim=m.vdim, tau=m.tau, eps=eps),
                {"q_proj": mp + "q", "k_proj": mp + "k", "v_proj": mp + "v", "g_proj": mp + "g", "o_proj": mp + "o",
                 "norm": mp + "norm", "decay_down": mp + "a1", "decay_up": mp + "a2", "decay_bias": mp + "a2.b"})
        norms = {"input": norm(p + "norm1")}
        ffn = None
        if lay.ff is not None:
            norms["post_mixer"] = norm(p + "norm2")
            ffn = PartSpec("poly_norm_mlp", dict(hidden_size=w, intermediate_size=lay.ff, eps=eps),
                           {"up_proj": p + "mlp.up", "down_proj": p + "mlp.down", "act": p + "mlp.act"})
        if streams is None:
            block: str | PartSpec = "pre_norm"
        else:
            block = PartSpec("hyper_connections", dict(streams=streams),
                             {"mixer": (p + "hc1.in", p + "hc1.out", p + "hc1.mix"),
                              "ffn": (p + "hc2.in", p + "hc2.out", p + "hc2.mix")})
        layers.append(LayerSpec(block, mixer, ffn, norms))
    return ModelSpec(
        hidden_size=w,
        vocab_size=cfg.vocab_size,
        embedding=PartSpec("embedding", dict(vocab_size=cfg.vocab_size, hidden_size=w, streams=streams or 1),
                           {"weight": "embed"}),
        layers=layers,
        schedule=[ScheduleEntry(i) for i in cfg.layer_runs()],
        final_norm=norm("final.norm", final=True),
        head=PartSpec("lm_head", dict(vocab_size=cfg.vocab_size, hidden_size=w), {"weight": "head"}),
        positions=positions,
    )
