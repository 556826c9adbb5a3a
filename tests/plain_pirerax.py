"""A plain, slow Pirerax: whole sequences in float64, one function per mechanism, straight from the equations.

It shares nothing with the package: it reads the dictionary of `config.json` itself, takes the weights as a
dictionary of tensors by checkpoint name, and keeps no cache: every function sees a whole sequence [n, ...].
`forward(cfg, w, tokens)` returns (logits [n, vocab], the stream after every layer [layers, n, width]).
"""

from __future__ import annotations

import contextlib
import math

import torch

F = torch.float64


@contextlib.contextmanager
def precision(dtype):
    """Runs the plain model in another precision (float32: what rounding alone does to a given model)."""
    global F
    old, F = F, dtype
    try:
        yield
    finally:
        F = old


def rms(x, weight, eps):
    """Rows of x divided by sqrt(mean(x^2) + eps), times weight (None: no weight)."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def silu(z):
    return z * torch.sigmoid(z)


def rotate_half(x, base, dims):
    """x [n, heads, d]: element i < dims/2 is paired with element i + dims/2 and the pair at position p is turned
    by the angle p * base^(-2i/dims); elements from `dims` on pass."""
    n = x.shape[0]
    half = dims // 2
    i = torch.arange(half, dtype=F)
    ang = torch.arange(n, dtype=F)[:, None] * base ** (-2.0 * i / dims)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def causal_softmax(scores, sink=None):
    """scores [heads, n, n] (query, key): softmax over the keys j <= i; with `sink` [heads] the denominator holds
    exp(sink) as well, a term without a value."""
    H, n, _ = scores.shape
    mask = torch.ones(n, n, dtype=torch.bool).tril()
    s = scores.masked_fill(~mask, -math.inf)
    if sink is None:
        return torch.softmax(s, dim=-1)
    s = torch.cat([s, sink.to(F)[:, None, None].expand(H, n, 1)], dim=-1)
    return torch.softmax(s, dim=-1)[..., :n]


def grouped_attention(h, w, p, m, eps, sink, q_temp=None, rot=None):
    """Grouped-query attention with a norm over the whole q and k projections, an elementwise sigmoid gate on the
    concatenated heads, optionally a sink, a query temperature by position, or rotary positions."""
    n = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms(h @ w[p + "q"].T, w[p + "q.norm"], eps).view(n, H, d)
    k = rms(h @ w[p + "k"].T, w[p + "k.norm"], eps).view(n, G, d)
    v = (h @ w[p + "v"].T).view(n, G, dv)
    if rot is not None:
        q, k = rotate_half(q, rot["base"], rot["dims"]), rotate_half(k, rot["base"], rot["dims"])
    if q_temp is not None:
        pos = torch.arange(n, dtype=F)
        q = q * (1.0 + q_temp["coef"] * torch.log(torch.floor((pos + 1.0) / q_temp["every"]) + 1.0))[:, None, None]
    rep = H // G
    k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    pr = causal_softmax(scores, w[p + "sink"] if sink else None)
    o = torch.einsum("hij,jhd->ihd", pr, v).reshape(n, H * dv)
    return (o * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def latent_attention(h, w, p, m, eps):
    """Keys and values from one normed latent per token plus one rotated key part that all heads share."""
    n = h.shape[0]
    H, d, r, dv, kr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = (h @ w[p + "q"].T).view(n, H, d + r)
    down = h @ w[p + "dkv"].T
    c = rms(down[:, :kr], w[p + "dkv.norm"], eps)
    k_rot = rotate_half(down[:, None, kr:], m["rot"]["base"], m["rot"]["dims"])          # [n, 1, r]
    q_rot = rotate_half(q[..., d:], m["rot"]["base"], m["rot"]["dims"])
    k = (c @ w[p + "uk"].T).view(n, H, d)
    v = (c @ w[p + "uv"].T).view(n, H, dv)
    scores = (torch.einsum("ihd,jhd->hij", q[..., :d], k) + torch.einsum("ihd,jd->hij", q_rot, k_rot[:, 0])) * m["scale"]
    pr = causal_softmax(scores, w[p + "sink"])
    o = torch.einsum("hij,jhd->ihd", pr, v)
    o = o * torch.sigmoid(h @ w[p + "g"].T)[:, :, None]
    return o.reshape(n, H * dv) @ w[p + "o"].T


def short_conv(x, taps_w):
    """x [n, c], taps_w [c, taps]: y_t = sum_j taps_w[:, taps-1-j] x_(t-j), zeros before the start; then silu."""
    n, c = x.shape
    taps = taps_w.shape[1]
    xp = torch.cat([torch.zeros(taps - 1, c, dtype=F), x])
    y = sum(xp[j:j + n] * taps_w[:, j] for j in range(taps))
    return silu(y)


def gated_delta(h, w, p, m, eps):
    """The gated delta rule, token by token."""
    n = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = short_conv(h @ w[p + "q"].T, w[p + "q.conv"]).view(n, G, d)
    k = short_conv(h @ w[p + "k"].T, w[p + "k.conv"]).view(n, G, d)
    v = short_conv(h @ w[p + "v"].T, w[p + "v.conv"]).view(n, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].T)                                               # [n, H]
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    rep = H // G
    out = torch.zeros(n, H, dv, dtype=F)
    for hd in range(H):
        S = torch.zeros(d, dv, dtype=F)
        for t in range(n):
            kt, qt = k[t, hd // rep], q[t, hd // rep]
            S = decay[t, hd] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ kt)
            S = S + torch.outer(kt, u)
            out[t, hd] = S.T @ qt
    out = rms(out, w[p + "norm"], eps) * silu(h @ w[p + "g"].T).view(n, H, dv)
    return out.reshape(n, H * dv) @ w[p + "o"].T


def parallel_mixer(h, w, p, m, eps):
    a = grouped_attention(h, w, p + "left.", m["left"], eps, sink=False, rot=m["left"]["rot"])
    b = gated_delta(h, w, p + "right.", m["right"], eps)
    return 0.5 * (rms(a, w[p + "left.out"], eps) + rms(b, w[p + "right.out"], eps))


def router(h, w_router, r, margins=None):
    """(chosen experts [n, top], their weights [n, top]): sigmoid scores; the experts form `groups.count` equal
    groups of neighbours, a group scores the sum of its two best, only the `groups.keep` best groups may be chosen.
    `margins` (a list) collects how far the closest call was: the smallest gap between what was kept or chosen and
    what came next."""
    s = torch.sigmoid(h @ w_router.T)
    n, E = s.shape
    allowed = torch.ones(n, E, dtype=torch.bool)
    groups = r.get("groups")
    if groups:
        size = E // groups["count"]
        gs = s.view(n, groups["count"], size)
        score = gs.topk(min(2, size), dim=-1).values.sum(-1)
        best = score.topk(groups["keep"], dim=-1).indices
        if margins is not None and groups["keep"] < groups["count"]:
            ranked = score.sort(dim=-1, descending=True).values
            margins.append(float((ranked[:, groups["keep"] - 1] - ranked[:, groups["keep"]]).min()))
        keep = torch.zeros(n, groups["count"], dtype=torch.bool).scatter_(1, best, True)
        allowed = keep[:, :, None].expand(n, groups["count"], size).reshape(n, E)
    masked = s.masked_fill(~allowed, -1.0)
    idx = masked.topk(r["top"], dim=-1).indices
    if margins is not None and r["top"] < E:
        ranked = masked.sort(dim=-1, descending=True).values
        gap = ranked[:, r["top"] - 1] - ranked[:, r["top"]]
        margins.append(float(gap[ranked[:, r["top"]] >= 0].min()) if (ranked[:, r["top"]] >= 0).any() else 1.0)
    return idx, s.gather(1, idx)


def expert(h, w, p, limit):
    g = torch.clamp(h @ w[p + "gate"].T, max=limit)
    u = torch.clamp(h @ w[p + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def routed_experts(h, w, p, mlp, margins=None):
    idx, wt = router(h, w[p + "router"], mlp["router"], margins)
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=F)
    for e in range(mlp["router"]["experts"]):
        tok, slot = (idx == e).nonzero(as_tuple=True)
        if tok.numel():
            out[tok] += wt[tok, slot, None] * expert(h[tok], w, f"{p}e{e}.", mlp["expert"]["limit"])
    return out


def forward(cfg, weights, tokens, margins=None):
    w = {k: (v.to(F) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    after = []
    for i, lay in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = rms(x, w[p + "norm1"], eps)
        m = lay["mixer"]
        if lay["type"] == "latent_attention":
            y = latent_attention(h, w, p + "mix.", m, eps)
        elif lay["type"] == "attention":
            y = grouped_attention(h, w, p + "mix.", m, eps, sink=True, q_temp=m.get("q_temp"))
        elif lay["type"] == "parallel":
            y = parallel_mixer(h, w, p + "mix.", m, eps)
        else:
            raise ValueError(lay["type"])
        x = x + y
        if lay.get("mlp") is not None:
            x = x + routed_experts(rms(x, w[p + "norm2"], eps), w, p + "mlp.", lay["mlp"], margins)
        after.append(x)
    logits = rms(x, w["final.norm"], eps) @ w["head"].T
    return logits, torch.stack(after)


def greedy_generate(cfg, weights, prompt, n):
    """`n` tokens after `prompt`, each the arg-max of the whole sequence's last logits."""
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(forward(cfg, weights, toks)[0][-1].argmax()))
    return toks[len(prompt):]
