"""A plain, slow Munazen: whole sequences in float64, one function per mechanism, straight from the equations.

It shares nothing with the package: it reads the dictionary of `config.json` itself, takes the weights as a
dictionary of tensors by checkpoint name, and keeps no cache: every function sees a whole sequence [n, ...].
`forward(cfg, w, tokens)` returns (logits [n, vocab], the stream summed over its copies after every layer run).
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


def group_rms(x, weight, groups, eps):
    """x [n, c] cut into `groups` equal consecutive parts, each divided by sqrt(mean(part^2) + eps); then * weight."""
    n, c = x.shape
    p = x.view(n, groups, c // groups)
    p = p / torch.sqrt((p * p).mean(-1, keepdim=True) + eps)
    return p.reshape(n, c) * weight


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def rotary_frequencies(dims, base, scaling=None):
    """(frequency of pair i for i < dims/2, the factor on cosine and sine)."""
    i = torch.arange(dims // 2, dtype=F)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def where(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(where(float(scaling["fast"]))), 0)
    hi = min(math.ceil(where(float(scaling["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_pairs(x, angles, magnitude=1.0):
    """x [n, heads, 2m...]: elements (2i, 2i+1), i < m, turned by angles [n, m]; the rest of the head passes."""
    m = angles.shape[1]
    c, s = (torch.cos(angles) * magnitude)[:, None, :], (torch.sin(angles) * magnitude)[:, None, :]
    a, b = x[..., 0:2 * m:2], x[..., 1:2 * m:2]
    out = x.clone()
    out[..., 0:2 * m:2] = a * c - b * s
    out[..., 1:2 * m:2] = b * c + a * s
    return out


def attention_left(h, w, p, m):
    """Softmax attention with biases, rotated q and k, values turned by their position and turned back at the
    query's, one sigmoid gate per head.  h [n, width]; m: the 'left' dictionary of the layer's mixer."""
    n = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(n, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(n, G, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(n, G, dv)
    rot = m["rot"]
    pos = torch.arange(n, dtype=F)
    f, mag = rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
    ang = pos[:, None] * f[None, :]
    q, k = rotate_pairs(q, ang, mag), rotate_pairs(k, ang, mag)
    fv = rot["base"] ** (-2.0 * torch.arange(dv // 2, dtype=F) / dv)
    angv = pos[:, None] * fv[None, :]
    v = rotate_pairs(v, angv)
    gate = torch.sigmoid(h @ w[p + "g"].T)                              # [n, H]
    out = torch.zeros(n, H, dv, dtype=F)
    causal = torch.tril(torch.ones(n, n, dtype=torch.bool))
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * m["scale"]
        s = s.masked_fill(~causal, float("-inf"))
        out[:, head] = torch.softmax(s, dim=-1) @ v[:, g]
    out = rotate_pairs(out, -angv) * gate[:, :, None]
    return out.reshape(n, H * dv) @ w[p + "o"].T + w[p + "o.b"]


def causal_conv(x, weight, bias):
    """x [n, c]; weight [c, taps] whose last column meets the current token; zeros in front of the sequence."""
    n, c = x.shape
    taps = weight.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, c, dtype=F), x], dim=0)
    out = bias[None, :].expand(n, c).clone()
    for j in range(taps):
        out = out + padded[j:j + n] * weight[:, j][None, :]
    return out


def recurrent_right(h, w, p, m):
    """The gated linear recurrence: a branch through gelu, a branch through a convolution and the recurrence."""
    n = h.shape[0]
    width, blocks = m["width"], m["blocks"]
    y = gelu_tanh(h @ w[p + "y"].T + w[p + "y.b"])
    u = causal_conv(h @ w[p + "x"].T + w[p + "x.b"], w[p + "conv"], w[p + "conv.b"])
    ub = u.view(n, blocks, width // blocks)
    r = torch.sigmoid(torch.einsum("nbi,boi->nbo", ub, w[p + "ra"]) + w[p + "ra.b"][None]).reshape(n, width)
    i = torch.sigmoid(torch.einsum("nbi,boi->nbo", ub, w[p + "ri"]) + w[p + "ri.b"][None]).reshape(n, width)
    log_a = -8.0 * r * softplus(w[p + "lam"])[None, :]
    a = torch.exp(log_a)
    drive = torch.sqrt(1.0 - a * a) * i * u
    S = torch.zeros(width, dtype=F)
    states = torch.zeros(n, width, dtype=F)
    for t in range(n):
        S = a[t] * S + drive[t]
        states[t] = S
    return (states * y) @ w[p + "o"].T


def mixer_parallel(h, w, p, m):
    return m["left_scale"] * attention_left(h, w, p + "left.", m["left"]) + \
        m["right_scale"] * recurrent_right(h, w, p + "right.", m["right"])


def mixer_gla(h, w, p, m, eps):
    """Linear attention with a decay per key channel; the state of a head is [dim, vdim]."""
    n = h.shape[0]
    H, d, dv, tau = m["heads"], m["dim"], m["vdim"], float(m["tau"])
    q = (h @ w[p + "q"].T).view(n, H, d) * d ** -0.5
    k = (h @ w[p + "k"].T).view(n, H, d)
    v = (h @ w[p + "v"].T).view(n, H, dv)
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    alpha = torch.sigmoid(z).pow(1.0 / tau).view(n, H, d)
    S = torch.zeros(H, d, dv, dtype=F)
    o = torch.zeros(n, H, dv, dtype=F)
    for t in range(n):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps) * w[p + "norm"]
    g = h @ w[p + "g"].T
    return (o.reshape(n, H * dv) * (g * torch.sigmoid(g))) @ w[p + "o"].T


def poly_norm_mlp(h, w, p, eps):
    z = h @ w[p + "up"].T
    a, b, c, e = w[p + "act"]

    def unit(t):
        return t / torch.sqrt((t * t).mean(-1, keepdim=True) + eps)

    return (a * unit(z) + b * unit(z * z) + c * unit(z ** 3) + e) @ w[p + "down"].T


def layer_runs(cfg):
    """The order in which layers run: the looped span `times` times in a row, then the rest."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    span = list(range(loop["start"], loop["stop"]))
    return list(range(loop["start"])) + span * loop["times"] + list(range(loop["stop"], n))


def forward(cfg, weights, tokens):
    w = {k: (v.to(F) if v.is_floating_point() else v) for k, v in weights.items()}
    eps, groups = cfg["norm"]["eps"], cfg["norm"]["groups"]
    x0 = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    streams = cfg.get("streams")
    xs = [x0.clone() for _ in range(streams or 1)]
    taps = []

    def sublayer(xs, lname, q, fn):
        norm_w = w[f"{lname}.norm{q}"]
        if streams is None:
            return [xs[0] + fn(group_rms(xs[0], norm_w, groups, eps))]
        win, wout, wmix = w[f"{lname}.hc{q}.in"], w[f"{lname}.hc{q}.out"], w[f"{lname}.hc{q}.mix"]
        u = sum(win[s] * xs[s] for s in range(streams))
        y = fn(group_rms(u, norm_w, groups, eps))
        return [sum(wmix[s, t] * xs[s] for s in range(streams)) + wout[t] * y for t in range(streams)]

    for i in layer_runs(cfg):
        lay, lname = cfg["layers"][i], f"l{i}"
        if lay["type"] == "parallel":
            xs = sublayer(xs, lname, 1, lambda h: mixer_parallel(h, w, lname + ".mix.", lay["mixer"]))
        elif lay["type"] == "gla":
            xs = sublayer(xs, lname, 1, lambda h: mixer_gla(h, w, lname + ".mix.", lay["mixer"], eps))
        else:
            raise ValueError(lay["type"])
        if lay.get("mlp") is not None:
            xs = sublayer(xs, lname, 2, lambda h: poly_norm_mlp(h, w, lname + ".mlp.", eps))
        taps.append(sum(xs))
    x = sum(xs)
    logits = group_rms(x, w["final.norm"], groups, eps) @ w["head"].T
    return logits, torch.stack(taps)


def greedy_generate(cfg, weights, prompt, n_new):
    toks = list(prompt)
    for _ in range(n_new):
        logits, _ = forward(cfg, weights, toks)
        toks.append(int(logits[-1].argmax()))
    return toks[len(prompt):]
