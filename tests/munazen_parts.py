"""The Munazen mechanisms one at a time, against the plain functions, for any kernel library: the host tests run
these checks with the tensor-code stand-in on the CPU, the GPU tests with the CUDA kernels in both precisions.

Every check builds one part of the package with weights of its own, feeds requests of unequal length through it three
ways (whole; in portions; a portion and then token by token, all requests in one batch) and compares each with the
plain function on the whole sequence."""

from __future__ import annotations

import types

import numpy as np
import torch

from paged_llm_b200.cache.storage import LayerCache
from paged_llm_b200.engine.context import AttentionPlan, HostBatch
from paged_llm_b200.parts.base import FixedState, PagedKV, materialize
from tests import plain_munazen as plain

F64 = torch.float64


def rand(*shape, seed=0, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * std).to(torch.bfloat16).float()      # values both precisions hold


def tol(dtype, scale=1.0):
    return (2e-5 if dtype == torch.float32 else 1.6e-2) * scale


def make_ctx(ops, device, q_lens, k_lens, plan_keys=(), slots=None):
    S = len(q_lens)
    host = HostBatch(list(q_lens), [k - q for q, k in zip(q_lens, k_lens)], list(slots) if slots is not None else [-1] * S)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a, np.int32)).to(device)      # noqa: E731
    plans = {}
    if hasattr(ops, "plan_attention"):
        for key in plan_keys:
            plan = ops.plan_attention(q_lens, k_lens, *key)
            small, large = plan["small"].reshape(-1, 4), plan["large"].reshape(-1, 4)
            plans[key] = AttentionPlan(dev(small) if len(small) else None, dev(large) if len(large) else None,
                                       dev(plan["splits"]), len(small), len(large), plan["max_splits"],
                                       plan["num_small_tokens"])
    pos = np.concatenate([np.arange(k - q, k) for q, k in zip(q_lens, k_lens)])
    tseq = np.concatenate([np.full(q, s) for s, q in enumerate(q_lens)])
    return types.SimpleNamespace(ops=ops, num_tokens=sum(q_lens), num_seqs=S, host=host, cu_seqlens_q=dev(host.cu),
                                 seq_lens_k=dev(k_lens), positions=dev(pos), token_seq=dev(tseq), max_q_len=max(q_lens),
                                 state_slots=dev(host.state_slots), attention_plans=plans, padded=False)


def _cache_for(req, n_req, lens, ps, dtype, device, seed):
    """A view for one requirement: pages handed out by a random permutation and poisoned, or zeroed state slots."""
    if isinstance(req, tuple):
        parts = [_cache_for(r, n_req, lens, ps, dtype, device, seed + i) for i, r in enumerate(req)]
        tables = [t for _, ts in parts for t in ts]
        views = []
        for view, ts in parts:
            views.append(view)
        return LayerCache("parts", -1, True, parts=tuple(views)), tables
    if isinstance(req, FixedState):
        return LayerCache("fixed_state", -1, True, state=torch.zeros((n_req, *req.shape), device=device)), []
    assert isinstance(req, PagedKV)
    g = torch.Generator().manual_seed(seed)
    n = [-(-L // ps) for L in lens]
    total = sum(n) + 3
    perm = torch.randperm(total, generator=g)
    bt = torch.full((n_req, max(n) + 1), -1, dtype=torch.int32)
    o = 0
    for s in range(n_req):
        bt[s, :n[s]] = perm[o:o + n[s]]
        o += n[s]
    kv = torch.full((total, 2, req.num_kv_heads, ps, req.head_dim), float("nan"), dtype=dtype, device=device)
    return LayerCache("paged_kv", 0, True, kv=kv, window=req.window), [bt]


def run_mixer(ops, device, mixer, hs, dtype, ps=8, ways=("whole", (0.6, 0.4), (0.25, 0.05, 0.7), "decode")):
    """Feeds each request's hidden rows through the mixer in several ways; returns the outputs per way."""
    ops.set_compute_dtype(dtype)
    lens = [h.shape[0] for h in hs]
    results = []
    for w, way in enumerate(ways):
        cache, tables = _cache_for(mixer.cache_requirement(), len(hs), lens, ps, dtype, device, seed=w)
        outs = [[] for _ in hs]
        done = [0] * len(hs)
        while any(d < n for d, n in zip(done, lens)):
            q_lens = []
            for s, n in enumerate(lens):
                if way == "whole":
                    q_lens.append(n - done[s])
                elif way == "decode":
                    q_lens.append(max(1, n // 2) if done[s] == 0 else min(1, n - done[s]))
                elif way[0] == "every":                     # ("every", k): portions of k tokens from the start
                    q_lens.append(min(way[1], n - done[s]))
                else:
                    cut = [max(1, round(f * n)) for f in way]
                    cut[-1] = max(0, n - sum(cut[:-1]))
                    ends = np.cumsum(cut)
                    k = int(np.searchsorted(ends, done[s], side="right"))
                    q_lens.append(min(cut[k], n - done[s]) if k < len(cut) else n - done[s])
            live = [s for s, q in enumerate(q_lens) if q > 0]
            ql = [q_lens[s] for s in live]
            kl = [done[s] + q_lens[s] for s in live]
            keys = [mixer.attention_plan_key()] if getattr(mixer, "attention_plan_key", lambda: None)() is not None else []
            ctx = make_ctx(ops, device, ql, kl, keys, slots=live)
            ctx.block_tables = [t[live].to(device).contiguous() for t in tables]
            h = torch.cat([hs[s][done[s]:done[s] + q_lens[s]] for s in live]).to(dtype).to(device).contiguous()
            out = materialize(mixer.forward(h, ctx, cache), ops).float().cpu()
            o = 0
            for s in live:
                outs[s].append(out[o:o + q_lens[s]])
                o += q_lens[s]
                done[s] += q_lens[s]
        results.append(torch.cat([torch.cat(o) for o in outs]))
    return results


def load(part, weights, dtype, device):
    """Hands a part its tensors by checkpoint name: matrices in the compute dtype, the rest as float32."""
    specs = part.tensor_specs()
    part.load({n: (w.to(dtype) if specs[n].role == "matrix" else w.float()).to(device) for n, w in weights.items()})
    return part


def rotary(head_dim, dims, base, scaling, ops, device, length=4096):
    from paged_llm_b200.parts.rope import RotaryEncoding
    enc = RotaryEncoding({}, head_dim=head_dim, theta=base, rotary_dim=dims, pairing="interleaved",
                         scaling=dict(scaling, type="yarn") if scaling else None)
    enc.prepare(length, device, ops)
    return enc


# ---------------------------------------------------------------- attention with rotated values
def attention_weights(W, m, seed):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    return {"a.q": rand(H * d, W, seed=seed, std=W ** -0.5), "a.q.b": rand(H * d, seed=seed + 1, std=0.2),
            "a.k": rand(G * d, W, seed=seed + 2, std=W ** -0.5), "a.k.b": rand(G * d, seed=seed + 3, std=0.2),
            "a.v": rand(G * dv, W, seed=seed + 4, std=W ** -0.5), "a.v.b": rand(G * dv, seed=seed + 5, std=0.2),
            "a.g": rand(H, W, seed=seed + 6, std=W ** -0.5), "a.o": rand(W, H * dv, seed=seed + 7, std=(H * dv) ** -0.5),
            "a.o.b": rand(W, seed=seed + 8, std=0.2)}


def attention_part(W, m, w, dtype, ops, device):
    from paged_llm_b200.parts.attention import RotatedValueAttention
    rot = m["rot"]
    names = {"q_proj": "a.q", "k_proj": "a.k", "v_proj": "a.v", "g_proj": "a.g", "o_proj": "a.o", "q_proj_bias": "a.q.b",
             "k_proj_bias": "a.k.b", "v_proj_bias": "a.v.b", "o_proj_bias": "a.o.b"}
    part = RotatedValueAttention(names, hidden_size=W, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"],
                                 value_dim=m["vdim"], scale=m["scale"],
                                 position=rotary(m["dim"], rot["dims"], rot["base"], rot.get("scaling"), ops, device),
                                 value_position=rotary(m["vdim"], m["vdim"], rot["base"], None, ops, device))
    return load(part, w, dtype, device)


def check_attention(ops, device, dtype, W, m, lens, seed=0, scale_tol=3.0, weights=None, hs=None, ways=None, ps=8):
    w = weights if weights is not None else attention_weights(W, m, seed)
    part = attention_part(W, m, w, dtype, ops, device)
    hs = hs if hs is not None else [rand(n, W, seed=seed + 20 + i) for i, n in enumerate(lens)]
    want = torch.cat([plain.attention_left(h.double(), {k: v.double() for k, v in w.items()}, "a.", m) for h in hs])
    kw = {"ways": ways} if ways else {}
    for way, got in enumerate(run_mixer(ops, device, part, hs, dtype, ps=ps, **kw)):
        err = (got.double() - want).abs().max()
        assert err <= tol(dtype, scale_tol * max(1.0, float(want.abs().max()))), f"way {way}: {err:.3e}"
    return want


def loud_key_setup(W, m, n, loud, seed=0):
    """Weights and inputs in which token `loud` of n carries a key whose score with every later query stands far above
    the rest, and a value of its own: the key's channel lies behind the rotated part of the head, the queries get it
    from their bias, the key from one input channel that only the loud token has."""
    d, dims = m["dim"], m["rot"]["dims"]
    assert dims < d, "the loud channel must not turn with the position"
    w = attention_weights(W, m, seed)
    ch = d - 1
    for name in ("a.q", "a.k", "a.v"):
        w[name][:, 0] = 0.0                                 # input channel 0 reaches nothing but the loud key and value
    w["a.g"][:, 0] = 0.0
    for head in range(m["heads"]):
        w["a.q.b"][head * d + ch] = 6.0
    for g in range(m["kv_heads"]):
        w["a.k"][g * d + ch, 0] = 1.0
        w["a.v"][g * m["vdim"]:(g + 1) * m["vdim"], 0] = 0.5
    h = rand(n, W, seed=seed + 50, std=0.05)
    h[:, 0] = 0.0
    h[loud, 0] = 8.0 / (m["scale"] * 6.0) * 2.0              # score 16 above the others
    return w, h


# ---------------------------------------------------------------- convolution + gated recurrence
def recurrence_weights(W, m, seed, lam=None):
    c, b = m["width"], m["blocks"]
    bw = c // b
    return {"r.y": rand(c, W, seed=seed, std=W ** -0.5), "r.y.b": rand(c, seed=seed + 1, std=0.2),
            "r.x": rand(c, W, seed=seed + 2, std=W ** -0.5), "r.x.b": rand(c, seed=seed + 3, std=0.2),
            "r.conv": rand(c, m["conv"], seed=seed + 4, std=0.5), "r.conv.b": rand(c, seed=seed + 5, std=0.1),
            "r.ra": rand(b, bw, bw, seed=seed + 6, std=bw ** -0.5), "r.ra.b": rand(b, bw, seed=seed + 7, std=0.3),
            "r.ri": rand(b, bw, bw, seed=seed + 8, std=bw ** -0.5), "r.ri.b": rand(b, bw, seed=seed + 9, std=0.3),
            "r.lam": rand(c, seed=seed + 10) - 3.0 if lam is None else torch.full((c,), float(lam)),
            "r.o": rand(W, c, seed=seed + 11, std=c ** -0.5)}


def recurrence_part(W, m, w, dtype, device):
    from paged_llm_b200.parts.recurrent import GatedLinearRecurrence
    names = {"y_proj": "r.y", "y_bias": "r.y.b", "x_proj": "r.x", "x_bias": "r.x.b", "conv": "r.conv", "conv_bias": "r.conv.b",
             "recurrence_gate": "r.ra", "recurrence_gate_bias": "r.ra.b", "input_gate": "r.ri", "input_gate_bias": "r.ri.b",
             "lam": "r.lam", "o_proj": "r.o"}
    part = GatedLinearRecurrence(names, hidden_size=W, width=m["width"], blocks=m["blocks"], conv_taps=m["conv"])
    return load(part, w, dtype, device)


def check_recurrence(ops, device, dtype, W, m, lens, seed=0, lam=None, hs=None, scale_tol=3.0, ways=None):
    w = recurrence_weights(W, m, seed, lam)
    part = recurrence_part(W, m, w, dtype, device)
    hs = hs if hs is not None else [rand(n, W, seed=seed + 20 + i) for i, n in enumerate(lens)]
    want = torch.cat([plain.recurrent_right(h.double(), {k: v.double() for k, v in w.items()}, "r.", m) for h in hs])
    kw = {"ways": ways} if ways else {}
    for way, got in enumerate(run_mixer(ops, device, part, hs, dtype, **kw)):
        err = (got.double() - want).abs().max()
        assert err <= tol(dtype, scale_tol * max(1.0, float(want.abs().max()))), f"way {way}: {err:.3e}"
    return want


# ---------------------------------------------------------------- gated linear attention
def gla_weights(W, m, seed, rank=6, decay_bias=None):
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    return {"g.q": rand(H * d, W, seed=seed, std=W ** -0.5), "g.k": rand(H * d, W, seed=seed + 1, std=W ** -0.5),
            "g.v": rand(H * dv, W, seed=seed + 2, std=W ** -0.5), "g.g": rand(H * dv, W, seed=seed + 3, std=W ** -0.5),
            "g.o": rand(W, H * dv, seed=seed + 4, std=(H * dv) ** -0.5), "g.norm": 1.0 + rand(dv, seed=seed + 5, std=0.2),
            "g.a1": rand(rank, W, seed=seed + 6, std=W ** -0.5), "g.a2": rand(H * d, rank, seed=seed + 7, std=rank ** -0.5),
            "g.a2.b": 1.0 + rand(H * d, seed=seed + 8) if decay_bias is None else torch.full((H * d,), float(decay_bias))}


def gla_part(W, m, w, eps, dtype, device):
    from paged_llm_b200.parts.linear_attention import GatedLinearAttention
    names = {"q_proj": "g.q", "k_proj": "g.k", "v_proj": "g.v", "g_proj": "g.g", "o_proj": "g.o", "norm": "g.norm",
             "decay_down": "g.a1", "decay_up": "g.a2", "decay_bias": "g.a2.b"}
    part = GatedLinearAttention(names, hidden_size=W, num_heads=m["heads"], head_dim=m["dim"], value_dim=m["vdim"],
                                tau=m["tau"], eps=eps)
    return load(part, w, dtype, device)


def check_gla(ops, device, dtype, W, m, lens, seed=0, eps=1e-5, decay_bias=None, hs=None, scale_tol=3.0, ways=None):
    w = gla_weights(W, m, seed, decay_bias=decay_bias)
    part = gla_part(W, m, w, eps, dtype, device)
    hs = hs if hs is not None else [rand(n, W, seed=seed + 20 + i) for i, n in enumerate(lens)]
    want = torch.cat([plain.mixer_gla(h.double(), {k: v.double() for k, v in w.items()}, "g.", m, eps) for h in hs])
    kw = {"ways": ways} if ways else {}
    for way, got in enumerate(run_mixer(ops, device, part, hs, dtype, **kw)):
        err = (got.double() - want).abs().max()
        assert err <= tol(dtype, scale_tol * max(1.0, float(want.abs().max()))), f"way {way}: {err:.3e}"
    return want


# ---------------------------------------------------------------- norms over several streams, PolyNorm
def check_stream_norm(ops, device, dtype, rows, W, S, G, seed=0):
    """The sublayer boundary: the copies take a branch in, the next input is formed and normed in parts."""
    ops.set_compute_dtype(dtype)
    x0 = rand(rows, S * W, seed=seed, std=2.0)
    br = rand(rows, W, seed=seed + 1)
    mix, outw, inw = rand(S, S, seed=seed + 2, std=0.5), 1.0 + rand(S, seed=seed + 3, std=0.3), rand(S, seed=seed + 4)
    nw = 1.0 + rand(W, seed=seed + 5, std=0.2)
    eps = 1e-5
    xs = x0.double().view(rows, S, W)
    new = torch.einsum("st,rsw->rtw", mix.double(), xs) + outw.double()[None, :, None] * br.double()[:, None, :]
    u = torch.einsum("s,rsw->rw", inw.double(), new)
    want = plain.group_rms(u, nw.double(), G, eps)
    x = x0.clone().to(device)
    d = lambda t: t.to(device)      # noqa: E731
    y = ops.stream_norm(x, S, d(br.to(dtype)), d(mix), d(outw), d(inw), d(nw), G, eps)
    assert y.dtype == dtype
    assert (x.cpu().double().view(rows, S, W) - new).abs().max() <= 1e-5      # the copies are float32 in both precisions
    assert (y.float().cpu().double() - want).abs().max() <= tol(dtype, 2.0 * float(want.abs().max()))
    # without a branch: the plain sum of the copies, normed (what the final norm sees)
    y = ops.stream_norm(x0.clone().to(device), S, None, None, None, None, d(nw), G, eps)
    want = plain.group_rms(xs.sum(1), nw.double(), G, eps)
    assert (y.float().cpu().double() - want).abs().max() <= tol(dtype, 2.0 * float(want.abs().max()))


def check_poly_norm(ops, device, dtype, rows, F, seed=0):
    ops.set_compute_dtype(dtype)
    z = rand(rows, F, seed=seed, std=1.5)
    coef = torch.tensor([0.9, 0.4, -0.2, 0.1])
    zd = z.double()
    unit = lambda t: t / torch.sqrt((t * t).mean(-1, keepdim=True) + 1e-6)      # noqa: E731
    want = 0.9 * unit(zd) + 0.4 * unit(zd * zd) - 0.2 * unit(zd ** 3) + 0.1
    got = ops.poly_norm(z.to(dtype).to(device), coef.to(device), 1e-6)
    assert got.dtype == dtype
    assert (got.float().cpu().double() - want).abs().max() <= tol(dtype, 2.0 * float(want.abs().max()))
