"""The Pirerax mechanisms one at a time, against the plain functions, for any kernel library: the host tests run these
checks with the tensor-code stand-in on the CPU, the GPU tests with the CUDA kernels in both precisions.

Every check builds one part of the package with weights of its own, feeds requests of unequal length through it several
ways (whole; in portions; a portion and then token by token; portions of two tokens; all requests in one batch) and
compares each with the plain function on the whole sequence."""

from __future__ import annotations

import numpy as np
import torch

from paged_llm_b200.parts.base import MIXERS, PartSpec, make_part
from tests import plain_pirerax as plain
from tests.munazen_parts import load, rand, run_mixer, tol  # noqa: F401  (the harness is the same for every design)

F64 = torch.float64
WAYS = ("whole", (0.6, 0.4), (0.25, 0.05, 0.7), "decode", ("every", 2))


def rotary(head_dim, dims, base, ops, device, length=4096):
    from paged_llm_b200.parts.rope import RotaryEncoding
    enc = RotaryEncoding({}, head_dim=head_dim, theta=base, rotary_dim=dims, pairing="half")
    enc.prepare(length, device, ops)
    return enc


def _mat(rows, cols, seed):
    return rand(rows, cols, seed=seed, std=1.2 / np.sqrt(cols))


# ---------------------------------------------------------------- attention with a norm over whole projections
def attention_weights(W, m, seed, sink=True):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    w = {"a.q": _mat(H * d, W, seed), "a.k": _mat(G * d, W, seed + 1), "a.v": _mat(G * dv, W, seed + 2),
         "a.g": _mat(H * dv, W, seed + 3), "a.o": _mat(W, H * dv, seed + 4),
         "a.q.norm": 1.0 + rand(H * d, seed=seed + 5, std=0.2), "a.k.norm": 1.0 + rand(G * d, seed=seed + 6, std=0.2)}
    if sink:
        w["a.sink"] = 1.0 + rand(H, seed=seed + 7)
    return w


def attention_part(W, m, w, eps, dtype, ops, device, sink=True):
    rot = m.get("rot")
    qt = m.get("q_temp")
    names = {"q_proj": "a.q", "k_proj": "a.k", "v_proj": "a.v", "g_proj": "a.g", "o_proj": "a.o", "q_norm": "a.q.norm",
             "k_norm": "a.k.norm", "sink": "a.sink"}
    part = MIXERS["gated_attention"](
        weights=names, hidden_size=W, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"], value_dim=m["vdim"],
        scale=m["scale"], eps=eps, gate=True, sink=sink,
        position=rotary(m["dim"], rot["dims"], rot["base"], ops, device) if rot else None,
        query_temperature=(qt["coef"], qt["every"]) if qt else None)
    return load(part, w, dtype, device)


def check_attention(ops, device, dtype, W, m, lens, seed=0, eps=1e-5, sink=True, weights=None, hs=None, ways=WAYS, ps=8,
                    scale_tol=3.0):
    w = weights if weights is not None else attention_weights(W, m, seed, sink)
    hs = hs if hs is not None else [rand(n, W, seed=seed + 20 + i) for i, n in enumerate(lens)]
    part = attention_part(W, m, w, eps, dtype, ops, device, sink)
    wd = {k: v.double() for k, v in w.items()}
    want = torch.cat([plain.grouped_attention(h.double(), wd, "a.", m, eps, sink, m.get("q_temp"), m.get("rot")) for h in hs])
    for way, got in zip(ways, run_mixer(ops, device, part, hs, dtype, ps=ps, ways=ways)):
        err = (got.double() - want).abs().max().item()
        assert err <= tol(dtype, scale_tol) * max(1.0, want.abs().max().item()), (way, err)
    return want


def loud_key(W, m, n, loud, seed=0, sink=True):
    """Weights and inputs on which position `loud` holds the one key that every later query of every head answers to:
    hidden unit 0 is on at `loud` only and feeds one key element, unit 1 is on everywhere and feeds the matching
    query element; the value at `loud` is marked through unit 0 as well."""
    w = attention_weights(W, m, seed, sink)
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    h = rand(n, W, seed=seed + 31, std=0.05)
    h[:, 0], h[:, 1] = 0.0, 1.0
    h[loud, 0] = 6.0
    for name in ("a.q", "a.k", "a.v"):
        w[name] = w[name] * 0.05
        w[name][:, :2] = 0.0
    for g in range(G):
        w["a.k"][g * d, 0] = 8.0
        w["a.v"][g * dv, 0] = 4.0
    for hh in range(H):
        w["a.q"][hh * d, 1] = 8.0
    w["a.q.norm"][:], w["a.k.norm"][:] = 1.0, 1.0
    return w, h


# ---------------------------------------------------------------- latent attention
def latent_weights(W, m, seed):
    H, d, r, dv, kr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    return {"l.q": _mat(H * (d + r), W, seed), "l.dkv": _mat(kr + r, W, seed + 1), "l.dkv.norm": 1.0 + rand(kr, seed=seed + 2, std=0.2),
            "l.uk": _mat(H * d, kr, seed + 3), "l.uv": _mat(H * dv, kr, seed + 4), "l.sink": 1.0 + rand(H, seed=seed + 5),
            "l.g": _mat(H, W, seed + 6), "l.o": _mat(W, H * dv, seed + 7)}


def latent_part(W, m, w, eps, dtype, ops, device):
    part = MIXERS["latent_attention"](
        weights={"q_proj": "l.q", "dkv": "l.dkv", "dkv_norm": "l.dkv.norm", "uk": "l.uk", "uv": "l.uv", "sink": "l.sink",
                 "g_proj": "l.g", "o_proj": "l.o"},
        hidden_size=W, num_heads=m["heads"], head_dim=m["dim"], rot_dim=m["rot_dim"], value_dim=m["vdim"], q_rank=None,
        kv_rank=m["kv_rank"], scale=m["scale"], eps=eps, sink=True, head_gate=True,
        position=rotary(m["rot_dim"], m["rot"]["dims"], m["rot"]["base"], ops, device))
    return load(part, w, dtype, device)


def check_latent(ops, device, dtype, W, m, lens, seed=0, eps=1e-5, weights=None, hs=None, ways=WAYS, ps=8, scale_tol=3.0):
    w = weights if weights is not None else latent_weights(W, m, seed)
    hs = hs if hs is not None else [rand(n, W, seed=seed + 20 + i) for i, n in enumerate(lens)]
    part = latent_part(W, m, w, eps, dtype, ops, device)
    wd = {k: v.double() for k, v in w.items()}
    want = torch.cat([plain.latent_attention(h.double(), wd, "l.", m, eps) for h in hs])
    for way, got in zip(ways, run_mixer(ops, device, part, hs, dtype, ps=ps, ways=ways)):
        err = (got.double() - want).abs().max().item()
        assert err <= tol(dtype, scale_tol) * max(1.0, want.abs().max().item()), (way, err)
    return want


# ---------------------------------------------------------------- the gated delta rule
def delta_weights(W, m, seed, a_log=None):
    H, G, d, dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
    g = torch.Generator().manual_seed(seed + 99)
    return {"d.q": _mat(G * d, W, seed), "d.k": _mat(G * d, W, seed + 1), "d.v": _mat(H * dv, W, seed + 2),
            "d.q.conv": rand(G * d, taps, seed=seed + 3, std=0.5), "d.k.conv": rand(G * d, taps, seed=seed + 4, std=0.5),
            "d.v.conv": rand(H * dv, taps, seed=seed + 5, std=0.5), "d.b": _mat(H, W, seed + 6), "d.a": _mat(H, W, seed + 7),
            "d.A_log": (-3.0 + 3.0 * torch.rand(H, generator=g)).to(torch.bfloat16).float() if a_log is None else torch.full((H,), float(a_log)),
            "d.dt_bias": rand(H, seed=seed + 8, std=0.5), "d.norm": 1.0 + rand(dv, seed=seed + 9, std=0.2),
            "d.g": _mat(H * dv, W, seed + 10), "d.o": _mat(W, H * dv, seed + 11)}


def delta_part(W, m, w, eps, dtype, device):
    part = MIXERS["gated_delta_rule"](
        weights={"q_proj": "d.q", "k_proj": "d.k", "v_proj": "d.v", "q_conv": "d.q.conv", "k_conv": "d.k.conv", "v_conv": "d.v.conv",
                 "beta_proj": "d.b", "decay_proj": "d.a", "decay_log": "d.A_log", "decay_bias": "d.dt_bias", "norm": "d.norm",
                 "g_proj": "d.g", "o_proj": "d.o"},
        hidden_size=W, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"], value_dim=m["vdim"],
        conv_taps=m["conv"], eps=eps)
    return load(part, w, dtype, device)


def check_delta(ops, device, dtype, W, m, lens, seed=0, eps=1e-5, weights=None, hs=None, ways=WAYS, scale_tol=3.0, a_log=None):
    w = weights if weights is not None else delta_weights(W, m, seed, a_log)
    hs = hs if hs is not None else [rand(n, W, seed=seed + 20 + i) for i, n in enumerate(lens)]
    part = delta_part(W, m, w, eps, dtype, device)
    wd = {k: v.double() for k, v in w.items()}
    want = torch.cat([plain.gated_delta(h.double(), wd, "d.", m, eps) for h in hs])
    for way, got in zip(ways, run_mixer(ops, device, part, hs, dtype, ways=ways)):
        err = (got.double() - want).abs().max().item()
        assert err <= tol(dtype, scale_tol) * max(1.0, want.abs().max().item()), (way, err)
    return want


# ---------------------------------------------------------------- two mixers side by side, each output normed
def check_parallel(ops, device, dtype, W, m, lens, seed=0, eps=1e-5, ways=WAYS, scale_tol=3.0):
    aw = {k.replace("a.", "p.left.", 1): v for k, v in attention_weights(W, m["left"], seed, sink=False).items()}
    dw = {k.replace("d.", "p.right.", 1): v for k, v in delta_weights(W, m["right"], seed + 50).items()}
    w = {**aw, **dw, "p.left.out": 1.0 + rand(W, seed=seed + 70, std=0.2), "p.right.out": 1.0 + rand(W, seed=seed + 71, std=0.2)}
    lm, rm = m["left"], m["right"]
    left = PartSpec("gated_attention", dict(
        hidden_size=W, num_heads=lm["heads"], num_kv_heads=lm["kv_heads"], head_dim=lm["dim"], value_dim=lm["vdim"], scale=lm["scale"],
        eps=eps, gate=True, sink=False, position=rotary(lm["dim"], lm["rot"]["dims"], lm["rot"]["base"], ops, device)),
        {k: "p.left." + v for k, v in {"q_proj": "q", "k_proj": "k", "v_proj": "v", "g_proj": "g", "o_proj": "o", "q_norm": "q.norm",
                                      "k_norm": "k.norm"}.items()})
    right = PartSpec("gated_delta_rule", dict(
        hidden_size=W, num_heads=rm["heads"], num_kv_heads=rm["kv_heads"], head_dim=rm["dim"], value_dim=rm["vdim"],
        conv_taps=rm["conv"], eps=eps),
        {k: "p.right." + v for k, v in {"q_proj": "q", "k_proj": "k", "v_proj": "v", "q_conv": "q.conv", "k_conv": "k.conv",
                                       "v_conv": "v.conv", "beta_proj": "b", "decay_proj": "a", "decay_log": "A_log",
                                       "decay_bias": "dt_bias", "norm": "norm", "g_proj": "g", "o_proj": "o"}.items()})
    part = make_part(MIXERS, "mixer", PartSpec("parallel", dict(left=left, right=right, left_scale=0.5, right_scale=0.5,
                                                                out_norm_eps=eps),
                                               {"left_norm": "p.left.out", "right_norm": "p.right.out"}))
    load(part, w, dtype, device)
    hs = [rand(n, W, seed=seed + 20 + i) for i, n in enumerate(lens)]
    wd = {k: v.double() for k, v in w.items()}
    want = torch.cat([plain.parallel_mixer(h.double(), wd, "p.", m, eps) for h in hs])
    for way, got in zip(ways, run_mixer(ops, device, part, hs, dtype, ways=ways)):
        err = (got.double() - want).abs().max().item()
        assert err <= tol(dtype, scale_tol) * max(1.0, want.abs().max().item()), (way, err)


# ---------------------------------------------------------------- routed experts
def experts_weights(W, mlp, seed):
    E, F = mlp["router"]["experts"], mlp["expert"]["ff"]
    w = {"m.router": rand(E, W, seed=seed, std=2.0 / np.sqrt(W))}
    for e in range(E):
        w[f"m.e{e}.gate"], w[f"m.e{e}.up"] = _mat(F, W, seed + 3 * e + 1), _mat(F, W, seed + 3 * e + 2)
        w[f"m.e{e}.down"] = _mat(W, F, seed + 3 * e + 3)
    return w


def experts_part(W, mlp, w, dtype, device):
    from paged_llm_b200.parts.base import FEED_FORWARDS
    E = mlp["router"]["experts"]
    names = {"router": "m.router"}
    for e in range(E):
        for x in ("gate", "up", "down"):
            names[f"e{e}.{x}"] = f"m.e{e}.{x}"
    g = mlp["router"].get("groups")
    part = FEED_FORWARDS["routed_mlp"](weights=names, hidden_size=W, expert_size=mlp["expert"]["ff"], num_experts=E,
                                       top_k=mlp["router"]["top"], activation="swish_clamped",
                                       activation_limit=mlp["expert"]["limit"], scoring="sigmoid",
                                       groups=(g["count"], g["keep"]) if g else None, group_score_top=2)
    return load(part, w, dtype, device)


def clear_rows(W, mlp, w, rows, seed, margin=0.03):
    """Inputs on which the router has no close call (the plain router's smallest gap is at least `margin`)."""
    keep = []
    s = seed
    while len(keep) < rows:
        h = rand(4 * rows, W, seed=s)
        s += 1
        for i in range(h.shape[0]):
            margins: list[float] = []
            plain.router(h[i:i + 1].double(), w["m.router"].double(), mlp["router"], margins)
            if min(margins, default=1.0) >= margin and len(keep) < rows:
                keep.append(h[i])
    return torch.stack(keep)


def check_experts(ops, device, dtype, W, mlp, rows, seed=0, scale_tol=3.0):
    import types
    w = experts_weights(W, mlp, seed)
    part = experts_part(W, mlp, w, dtype, device)
    h = clear_rows(W, mlp, w, rows, seed + 500)
    ops.set_compute_dtype(dtype)
    got = part.forward(h.to(dtype).to(device).contiguous(), types.SimpleNamespace(ops=ops)).float().cpu()
    want = plain.routed_experts(h.double(), {k: v.double() for k, v in w.items()}, "m.", mlp)
    err = (got.double() - want).abs().max().item()
    assert err <= tol(dtype, scale_tol) * max(1.0, want.abs().max().item()), err
