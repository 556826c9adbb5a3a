"""The Munazen decoder on the host: configuration, the model as data, the cache's needs, each mechanism alone and the
engine's host logic (runner, cache manager, state slots, replay, scheduler) with the kernel library replaced by the
tensor-code stand-in, against the plain implementation."""

from __future__ import annotations

import math

import numpy as np
import pytest
import torch

from paged_llm_b200.config.model import ConfigError
from paged_llm_b200.config.munazen import MunazenConfig
from paged_llm_b200.config.registry import parse_model_config
from paged_llm_b200.models.causal_lm import build_model
from paged_llm_b200.parts.base import FixedState, PagedKV, cache_leaves
from tests import munazen_parts as parts
from tests import plain_munazen as plain
from tests import schedules
from tests.helpers import requests_for
from tests.munazen_cases import (CASE_A, CASE_B, CASE_C, CASES, YARN, case_folder, generated_case, left, make_folder,
                                 plain_greedy, plain_logits, rounding_error)
from tests.torch_ops import TorchOps

F32_TOL = 2e-5
F32 = torch.float32


def close(got, want, what, rounding=None):
    """Largest difference within F32_TOL of the largest logit; with `rounding` (per position, the root mean square of what
    float32 alone does to the plain model) a position passes too if its root mean square error is within 10 times that
    (two float32 runs of an ill-conditioned position differ from each other by several times their distance to float64)."""
    assert got.shape == want.shape, what
    assert np.isfinite(got).all(), what
    err = np.abs(got - want)
    bad = err.max(axis=1) > F32_TOL * max(1.0, float(np.abs(want).max()))
    if rounding is not None:
        bad &= np.sqrt((err.astype(np.float64) ** 2).mean(axis=1)) > 10.0 * rounding
    assert not bad.any(), f"{what}: max |diff| {err.max():.3e}, first bad row {int(np.argmax(bad))} ({err[int(np.argmax(bad))].max():.3e})"


def replay(folder, steps, max_tokens, block_size=8, slots=4):
    from paged_llm_b200.engine.replay import TraceReplayer

    rp = TraceReplayer(folder, "float32", max_tokens, device="cpu", ops=TorchOps(), block_size=block_size, max_num_seqs=slots)
    for state in rp.storage._state_tensors():
        state.fill_(float("nan"))                      # a slot that is not zeroed at a request's start shows
    outputs = {}
    for rec in steps:
        out = rp.step(rec)
        if out is not None:
            outputs[rec["step"]] = out
    assert not rp.live
    rp.cm.check_invariants([])
    for g in range(len(rp.cm.pools)):
        assert rp.cm.num_free_in_group(g) == rp.cm.pools[g].num_pages, "pages were lost"
    assert rp.cm.num_free_state_slots == rp.cm.num_state_slots, "state slots were lost"
    return outputs, rp


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: case_folder(tmp_path_factory, name) for name in CASES}


@pytest.fixture(scope="module")
def ops():
    return TorchOps()


# ---------------------------------------------------------------- configuration
def test_configuration_round_trip():
    for hf, _ in CASES.values():
        arch, cfg = parse_model_config(hf)
        assert arch.name == "Munazen"
        assert MunazenConfig.from_hf_dict(cfg.to_hf_dict()) == cfg
        specs = build_model(arch.build_spec(cfg)).tensor_specs()
        assert cfg.num_parameters == sum(int(np.prod(s.draw_shape or s.shape)) for s in specs.values())


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="conv"), "not implemented"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(vdim=15), "even"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(blocks=5), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=18), "dims"),
    (lambda c: c["layers"][1]["mixer"].update(tau=0.0), "tau"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "dense only"),
    (lambda c: c["norm"].update(groups=5), "groups"),
    (lambda c: c["loop"].update(stop=7), "loop"),
    (lambda c: c.update(streams=0), "streams"),
    (lambda c: c.pop("width"), "width"),
])
def test_configuration_refusals(change, message):
    import copy
    hf = copy.deepcopy(CASE_A)
    change(hf)
    with pytest.raises(ConfigError, match=message):
        parse_model_config(hf)


def test_the_model_as_data():
    """Case A: layers 0 and 1 run three times, each run with a cache and state of its own; a parallel mixer needs pages
    for its attention and a slot for its recurrence; the linear-attention layer has no feed-forward."""
    arch, cfg = parse_model_config(CASE_A)
    assert cfg.layer_runs() == [0, 1, 0, 1, 0, 1, 2]
    model = build_model(arch.build_spec(cfg))
    slots = model.cache_slots()
    assert len(slots) == 7 and all(s.shares is None for s in slots)
    a = CASE_A["layers"][0]["mixer"]
    assert slots[0].requirement == (PagedKV(2, 32, None), FixedState((3 * 48,)))          # heads of 16 and 32 -> 32; 3 taps
    assert slots[1].requirement == FixedState((2 * 8 * 16,))
    assert slots[6].requirement == (PagedKV(2, 32, None), FixedState((2 * 40,)))
    assert len([r for s in slots for r in cache_leaves(s.requirement) if isinstance(r, FixedState)]) == 7
    names = set(model.tensor_specs())
    assert {"embed", "head", "final.norm", "l0.hc1.mix", "l0.hc2.out", "l0.mix.left.q.b", "l0.mix.right.ra", "l0.mlp.act",
            "l1.mix.a2.b", "l1.hc1.in"} <= names
    assert not any(n.startswith(("l1.mlp", "l1.norm2", "l1.hc2")) for n in names), "a layer without a feed-forward"
    assert model.has_fixed_state and a["left"]["vdim"] == 32
    # one stream: plain residual sums and no tensors of the hyper-connections
    arch, cfg = parse_model_config(CASE_B)
    assert not any(".hc" in n for n in build_model(arch.build_spec(cfg)).tensor_specs())


def test_rank_of_the_decay_follows_the_checkpoint(tmp_path):
    """The inner size of the decay's two matrices is written nowhere but in their shapes."""
    hf = {"architecture": "Munazen", "vocab": 40, "width": 32, "norm": {"eps": 1e-5, "groups": 1}, "streams": 1,
          "layers": [{"type": "gla", "mixer": {"heads": 2, "dim": 8, "vdim": 8, "tau": 2.0}, "mlp": None}]}
    from tests.munazen_cases import draw_weights
    w = draw_weights(hf, 3)
    g = torch.Generator().manual_seed(1)
    w["l0.mix.a1"] = (torch.randn(5, 32, generator=g) * 0.2).to(torch.bfloat16).float()
    w["l0.mix.a2"] = (torch.randn(16, 5, generator=g) * 0.4).to(torch.bfloat16).float()
    folder = make_folder(tmp_path, hf, 3, weights=w)
    toks = requests_for(40, (19,), seed=1)["r0"]
    steps, max_tokens = schedules.portions({"r0": toks})
    outputs, _ = replay(folder, steps, max_tokens)
    close(schedules.collect(steps, outputs)["r0"], plain_logits(folder, toks), "rank 5")


# ---------------------------------------------------------------- mechanisms by hand
def test_yarn_frequencies_by_hand():
    """dims 8, base 100, original 32, fast 8, slow 1, factor 4: the pair whose wave makes t turns over 32 positions is
    8 ln(32 / (2 pi t)) / (2 ln 100); t = 8 gives -0.39 (floor -1 -> lo 0), t = 1 gives 1.41 (ceil -> hi 2).  Pairs
    0..3 have ramps 0, 1/2, 1, 1."""
    from paged_llm_b200.parts.rope import RotaryEncoding
    enc = RotaryEncoding({}, head_dim=16, theta=100.0, rotary_dim=8, pairing="interleaved", scaling=dict(YARN, type="yarn"))
    f, mag = enc.frequencies()
    base = [100.0 ** (-2 * i / 8) for i in range(4)]
    want = [base[0], base[1] / 4 * 0.5 + base[1] * 0.5, base[2] / 4, base[3] / 4]
    assert np.allclose(f.numpy(), want, rtol=1e-6)
    assert math.isclose(mag, 0.1 * math.log(4.0) + 1.0)
    pf, pmag = plain.rotary_frequencies(8, 100.0, YARN)
    assert np.allclose(pf.numpy(), want, rtol=1e-12) and pmag == mag
    # the ramp's two ends on the same pair: the difference is replaced by 0.001
    sc = {"factor": 2.0, "original": 64, "fast": 1.0, "slow": 1.0}
    lo = math.floor(8 * math.log(64 / (2 * math.pi)) / (2 * math.log(100.0)))
    f2, _ = RotaryEncoding({}, head_dim=8, theta=100.0, rotary_dim=8, pairing="interleaved", scaling=dict(sc, type="yarn")).frequencies()
    p2, _ = plain.rotary_frequencies(8, 100.0, sc)
    assert np.allclose(f2.numpy(), p2.numpy(), rtol=1e-6)
    assert lo == 2 and math.isclose(f2[2].item(), base[2], rel_tol=1e-6) and math.isclose(f2[3].item(), base[3] / 2, rel_tol=1e-6)


def test_rotated_values_see_the_distance_only(ops):
    """One key takes all the weight.  The output at query i is then the value of that key turned by (j - i): moving
    both by the same number of positions changes nothing, moving one of them does."""
    m = left(2, 1, 8, 12, dims=4, base=50.0, scale=1.0)
    W = 16
    outs = {}
    for n, loud in ((40, 10), (47, 17), (40, 11)):
        w, h = parts.loud_key_setup(W, m, n, loud, seed=2)
        for name in ("a.v", "a.g"):
            w[name][:, 1:] = 0.0                          # values and gates are the same at every position
        w["a.v.b"][:] = 0.0
        w["a.o"] = torch.eye(W, 24)                        # the heads' outputs come out as they are
        w["a.o.b"][:] = 0.0
        outs[(n, loud)] = plain.attention_left(h.double(), {k: v.double() for k, v in w.items()}, "a.", m)
        parts.check_attention(ops, "cpu", F32, W, m, None, weights=w, hs=[h], ways=("whole", "decode", ("every", 2)))
    same = (outs[(40, 10)][-1] - outs[(47, 17)][-1]).abs().max()
    moved = (outs[(40, 10)][-1] - outs[(40, 11)][-1]).abs().max()
    assert same < 1e-4 and moved > 1e-2, (same, moved)


def test_recurrence_by_hand(ops):
    """One channel, one tap: with gates r, i and u known, S_1 = sqrt(1 - a_1^2) i_1 u_1 from S = 0 (the first token has
    no special case), S_2 = a_2 S_1 + sqrt(1 - a_2^2) i_2 u_2, a = exp(-8 r softplus(lam))."""
    W, m = 2, {"width": 1, "blocks": 1, "conv": 1}
    w = {"r.y": torch.tensor([[0.0, 1.0]]), "r.y.b": torch.tensor([0.5]), "r.x": torch.tensor([[1.0, 0.0]]),
         "r.x.b": torch.tensor([0.25]), "r.conv": torch.tensor([[2.0]]), "r.conv.b": torch.tensor([-0.5]),
         "r.ra": torch.tensor([[[0.5]]]), "r.ra.b": torch.tensor([[0.125]]), "r.ri": torch.tensor([[[-1.0]]]),
         "r.ri.b": torch.tensor([[0.25]]), "r.lam": torch.tensor([-1.0]), "r.o": torch.tensor([[1.0], [0.0]])}
    h = torch.tensor([[1.0, 0.5], [-0.5, 2.0]])
    sig = lambda z: 1 / (1 + math.exp(-z))      # noqa: E731
    S, want = 0.0, []
    for x0, x1 in h.tolist():
        u = 2.0 * (x0 + 0.25) - 0.5
        a = math.exp(-8.0 * sig(0.5 * u + 0.125) * math.log1p(math.exp(-1.0)))
        S = a * S + math.sqrt(1 - a * a) * sig(-u + 0.25) * u
        z = x1 + 0.5
        want.append(S * 0.5 * z * (1 + math.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3))))
    got = plain.recurrent_right(h.double(), {k: v.double() for k, v in w.items()}, "r.", m)
    assert np.allclose(got[:, 0].numpy(), want, rtol=1e-12)
    part = parts.recurrence_part(W, m, w, F32, "cpu")
    for out in parts.run_mixer(ops, "cpu", part, [h], F32, ways=("whole", "decode")):
        assert np.allclose(out[:, 0].numpy(), want, rtol=1e-5)


def test_linear_attention_by_hand(ops):
    """One head, two key channels, one value channel... the decay multiplies the rows of the state that belong to key
    channels, and the newest key and value are in the state before the query reads it."""
    m, eps = {"heads": 1, "dim": 2, "vdim": 2, "tau": 2.0}, 1e-5
    W = 4
    w = parts.gla_weights(W, m, seed=5, rank=2)
    h = parts.rand(3, W, seed=6)
    hd = h.double()
    q, k, v = (hd @ w[n].double().T for n in ("g.q", "g.k", "g.v"))
    z = (hd @ w["g.a1"].double().T) @ w["g.a2"].double().T + w["g.a2.b"].double()
    alpha = torch.sigmoid(z) ** 0.5
    S = torch.zeros(2, 2, dtype=torch.float64)
    rows = []
    for t in range(3):
        for c in range(2):
            S[c] = alpha[t, c] * S[c] + k[t, c] * v[t]
        o = (S * (q[t] * 2 ** -0.5)[:, None]).sum(0)
        o = o / torch.sqrt((o * o).mean() + eps) * w["g.norm"].double()
        g = hd[t] @ w["g.g"].double().T
        rows.append((o * g * torch.sigmoid(g)) @ w["g.o"].double().T)
    want = torch.stack(rows)
    assert (plain.mixer_gla(hd, {n: t.double() for n, t in w.items()}, "g.", m, eps) - want).abs().max() < 1e-12
    part = parts.gla_part(W, m, w, eps, F32, "cpu")
    for out in parts.run_mixer(ops, "cpu", part, [h], F32, ways=("whole", "decode")):
        assert (out.double() - want).abs().max() < 1e-5


def test_poly_norm_by_hand(ops):
    """Two inner values (3, -4), a..e = 1, 2, 3, 0.5: N(z) = z / sqrt(12.5), N(z^2) = (9, 16) / sqrt(168.5),
    N(z^3) = (27, -64) / sqrt(2412.5)."""
    z = torch.tensor([[3.0, -4.0]])
    got = ops.poly_norm(z, torch.tensor([1.0, 2.0, 3.0, 0.5]), 0.0)
    want = [3 / math.sqrt(12.5) + 2 * 9 / math.sqrt(168.5) + 3 * 27 / math.sqrt(2412.5) + 0.5,
            -4 / math.sqrt(12.5) + 2 * 16 / math.sqrt(168.5) - 3 * 64 / math.sqrt(2412.5) + 0.5]
    assert np.allclose(got.numpy()[0], want, rtol=1e-6)


def test_hyper_connections_by_hand(ops):
    """Two streams of width 1: the mix matrix is indexed [from, to], and every new copy is formed from the old ones."""
    x = torch.tensor([[1.0, 10.0]])
    mix = torch.tensor([[1.0, 2.0], [3.0, 4.0]])
    y = ops.stream_norm(x, 2, torch.tensor([[0.5]]), mix, torch.tensor([2.0, -2.0]), torch.tensor([1.0, 0.5]),
                        torch.tensor([3.0]), 1, 0.0)
    assert x.tolist() == [[1.0 * 1 + 3.0 * 10 + 1.0, 2.0 * 1 + 4.0 * 10 - 1.0]]        # (32, 41)
    assert y.tolist() == [[3.0]]                                                     # u = 32 + 20.5 > 0, normed to 1, times 3


# ---------------------------------------------------------------- each mixer alone, through prompts and decoding
@pytest.mark.parametrize("W,m", [
    (48, left(4, 2, 16, 24, dims=8, base=100.0, scaling=YARN, scale=0.25)),
    (32, left(6, 1, 24, 40, dims=12, base=1e6, scaling=dict(YARN, factor=8.0, original=64))),      # heads that pad the cache
    (40, left(3, 3, 32, 16, base=500.0, scale=0.3)),                                                # values shorter than keys
    (24, left(1, 1, 8, 8, dims=2)),
])
def test_attention_mixer_alone(ops, W, m):
    parts.check_attention(ops, "cpu", F32, W, m, [1, 37, 20, 2])


@pytest.mark.parametrize("W,m", [(48, {"width": 36, "blocks": 3, "conv": 3}), (32, {"width": 20, "blocks": 1, "conv": 1}),
                                 (24, {"width": 64, "blocks": 4, "conv": 6}), (16, {"width": 8, "blocks": 8, "conv": 2})])
def test_recurrence_mixer_alone(ops, W, m):
    parts.check_recurrence(ops, "cpu", F32, W, m, [1, 37, 20, 2], ways=("whole", (0.6, 0.4), "decode", ("every", 2)))


@pytest.mark.parametrize("W,m", [(48, {"heads": 2, "dim": 12, "vdim": 20, "tau": 4.0}), (32, {"heads": 1, "dim": 40, "vdim": 8, "tau": 1.0}),
                                 (24, {"heads": 5, "dim": 4, "vdim": 4, "tau": 16.0})])
def test_linear_attention_mixer_alone(ops, W, m):
    parts.check_gla(ops, "cpu", F32, W, m, [1, 37, 20, 2], ways=("whole", (0.6, 0.4), "decode", ("every", 2)))


@pytest.mark.parametrize("rows,W,S,G", [(9, 48, 3, 2), (1, 32, 1, 1), (5, 40, 5, 4), (4, 24, 2, 3)])
def test_stream_norm_alone(ops, rows, W, S, G):
    parts.check_stream_norm(ops, "cpu", F32, rows, W, S, G)
    parts.check_poly_norm(ops, "cpu", F32, rows, W * 3 + 1)


def test_one_far_key_among_hundreds(ops):
    """Key 3 of 700 takes the weight of every later query, in a prompt, in portions and token by token; without it the
    outputs differ, so a fault in reaching it would show."""
    m = left(4, 2, 16, 24, dims=8, base=100.0, scaling=YARN, scale=0.25)
    W, n = 32, 700
    w, h = parts.loud_key_setup(W, m, n, 3, seed=4)
    want = parts.check_attention(ops, "cpu", F32, W, m, None, weights=w, hs=[h], ways=("whole", (0.9, 0.1), ("every", 64)), ps=16)
    h2 = h.clone()
    h2[3, 0] = 0.0
    quiet = plain.attention_left(h2.double(), {k: v.double() for k, v in w.items()}, "a.", m)
    assert (quiet[-1] - want[-1]).abs().max() > 0.1, "the far key must matter"


def test_long_recurrence_keeps_a_far_token(ops):
    """Decays close to one: the first token still shows after 400 more, in portions and token by token."""
    W, m = 16, {"width": 12, "blocks": 2, "conv": 3}
    h = parts.rand(401, W, seed=9, std=0.3)
    h[0] *= 30.0
    want = parts.check_recurrence(ops, "cpu", F32, W, m, None, lam=-7.0, hs=[h], ways=((0.37, 0.63), "decode"))
    h2 = h.clone()
    h2[0] /= 30.0
    w = parts.recurrence_weights(W, m, 0, -7.0)
    quiet = plain.recurrent_right(h2.double(), {k: v.double() for k, v in w.items()}, "r.", m)
    assert (quiet[-1] - want[-1]).abs().max() > 1e-2, "the far token must matter"


def test_long_linear_attention_keeps_a_far_token(ops):
    W, m = 16, {"heads": 2, "dim": 8, "vdim": 8, "tau": 16.0}
    h = parts.rand(401, W, seed=9, std=0.3)
    h[0] *= 30.0
    want = parts.check_gla(ops, "cpu", F32, W, m, None, decay_bias=6.0, hs=[h], ways=((0.37, 0.63), "decode"))
    h2 = h.clone()
    h2[0] /= 30.0
    w = parts.gla_weights(W, m, 0, decay_bias=6.0)
    quiet = plain.mixer_gla(h2.double(), {k: v.double() for k, v in w.items()}, "g.", m, 1e-5)
    assert (quiet[-1] - want[-1]).abs().max() > 1e-2, "the far token must matter"


# ---------------------------------------------------------------- the engine's host logic against the plain model
LENGTHS = {"A": (1, 30, 77, 49, 2, 60, 90, 35), "B": (5, 41, 120, 13, 80, 55), "C": (3, 70, 33, 65, 18, 41)}


@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("schedule", ["whole", "tail", "portions", "mixed"])
def test_schedule_matches_plain(folders, name, schedule):
    hf = CASES[name][0]
    reqs = requests_for(hf["vocab"], LENGTHS[name], seed=ord(name))
    steps, max_tokens = getattr(schedules, schedule)(reqs)
    outputs, rp = replay(folders[name], steps, max_tokens)
    got = schedules.collect(steps, outputs)
    for rid, toks in reqs.items():
        close(got[rid], plain_logits(folders[name], toks), f"{schedule}/{name}/{rid}", rounding_error(folders[name], toks))
    if schedule == "mixed":
        assert len(reqs) > 4, "state slots must be used again"


def test_layer_by_layer(folders):
    """The stream summed over its copies after every layer run, a looped layer counted each time."""
    from paged_llm_b200.engine.replay import TraceReplayer
    from tests.munazen_cases import read_folder
    toks = requests_for(CASE_A["vocab"], (23,), seed=2)["r0"]
    cfg, w = read_folder(folders["A"])
    with torch.no_grad():
        _, taps = plain.forward(cfg, w, toks)
    rp = TraceReplayer(folders["A"], "float32", 64, device="cpu", ops=TorchOps(), block_size=8, max_num_seqs=2)
    seen = []
    inner = rp.runner.model.blocks
    for entry in rp.runner.model.schedule:
        block = inner[entry.layer]
        if not hasattr(block, "_plain_forward"):
            block._plain_forward = block.forward

            def spy(x, pending, ctx, cache, block=block):
                x, pending = block._plain_forward(x, pending, ctx, cache)
                # the branch still waits for the next norm: carry it out on a copy
                xs = x.clone().view(x.shape[0], block.streams, -1)
                y = parts.materialize(pending.branch, ctx.ops).float()
                new = torch.einsum("st,rsw->rtw", pending.mix, xs) + pending.out[None, :, None] * y[:, None, :]
                seen.append(new.sum(1))
                return x, pending

            block.forward = spy
    rp.step({"step": 0, "entries": [{"id": "a", "tokens": toks, "want": [0]}], "end": ["a"]})
    assert len(seen) == taps.shape[0] == 7
    for i, (got, want) in enumerate(zip(seen, taps)):
        assert (got.double() - want).abs().max() <= 2e-5 * max(1.0, float(want.abs().max())), f"layer run {i}"


def test_one_stream_without_connection_tensors(tmp_path):
    """`streams: 1` over a checkpoint that has no connection tensors is the plain residual sum."""
    from tests.munazen_cases import draw_weights
    base = {k: v for k, v in CASE_B.items()}
    weights = draw_weights(base, 9)
    with_key = make_folder(tmp_path / "one", dict(base, streams=1), 9, weights=weights)
    without = make_folder(tmp_path / "none", base, 9, weights=weights)
    reqs = requests_for(base["vocab"], (7, 33), seed=4)
    steps, max_tokens = schedules.mixed(reqs, live=2, seed=2)
    outputs, _ = replay(with_key, steps, max_tokens)
    got = schedules.collect(steps, outputs)
    for rid, toks in reqs.items():
        close(got[rid], plain_logits(without, toks), f"one stream/{rid}", rounding_error(without, toks))


def test_state_does_not_leak_between_requests(folders):
    """A slot and pages that are used again start clean: the second request equals itself run alone."""
    reqs = requests_for(CASE_B["vocab"], (40, 37), seed=4)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": reqs["r0"], "want": []}], "end": ["x"]},
             {"step": 1, "entries": [{"id": "y", "tokens": reqs["r1"], "want": list(range(37))}], "end": ["y"]}]
    outputs, rp = replay(folders["B"], steps, 64, slots=1)
    close(outputs[1], plain_logits(folders["B"], reqs["r1"]), "a slot used again")


def test_a_request_left_out_of_a_step_goes_on_later(folders):
    """Request a pauses while b runs; its pages and its state wait for it."""
    reqs = requests_for(CASE_C["vocab"], (30, 21), seed=8)
    a, b = reqs["r0"], reqs["r1"]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:11], "want": list(range(11))}], "end": []},
             {"step": 1, "entries": [{"id": "b", "tokens": b[:20], "want": list(range(20))}], "end": []},
             {"step": 2, "entries": [{"id": "b", "tokens": b[20:], "want": [0]}, {"id": "a", "tokens": a[11:13], "want": [0, 1]}], "end": ["b"]},
             {"step": 3, "entries": [{"id": "a", "tokens": a[13:], "want": list(range(17))}], "end": ["a"]}]
    outputs, _ = replay(folders["C"], steps, 128)
    got = schedules.collect(steps, outputs)
    close(got["a"], plain_logits(folders["C"], a), "paused request")
    close(got["b"], plain_logits(folders["C"], b), "the other request")


@pytest.mark.parametrize("seed", range(8))
def test_generated_configurations(tmp_path, seed):
    hf = generated_case(seed)
    folder = make_folder(tmp_path, hf, seed)
    reqs = requests_for(hf["vocab"], (2, 50, 21, 70, 9), seed=seed)
    steps, max_tokens = schedules.mixed(reqs, live=3, seed=seed)
    outputs, _ = replay(folder, steps, max_tokens, block_size=8, slots=3)
    got = schedules.collect(steps, outputs)
    for rid, toks in reqs.items():
        close(got[rid], plain_logits(folder, toks), f"generated {seed}/{rid}", rounding_error(folder, toks))


def test_greedy_generation_through_the_engine(folders):
    from paged_llm_b200 import LLMEngine, SamplingParams
    prompts = list(requests_for(CASE_A["vocab"], (3, 22, 47, 9, 31), seed=60).values())
    eng = LLMEngine(folders["A"], dtype="float32", device="cpu", ops=TorchOps(), block_size=8, num_gpu_blocks=40,
                    max_model_len=96, max_num_batched_tokens=16, max_num_seqs=3)
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12))
    for p, o in zip(prompts, outs):
        assert o.token_ids == plain_greedy(folders["A"], p, 12)
    assert eng.block_manager.num_free_state_slots == 3


def test_generation_with_preemption_restarts_the_state(folders):
    """So few pages that running requests are preempted: a request that comes back starts at position 0 with a
    zeroed state slot and ends with the tokens of an undisturbed run."""
    from paged_llm_b200 import LLMEngine, SamplingParams
    prompts = list(requests_for(CASE_C["vocab"], (30, 26, 21, 12), seed=70).values())
    eng = LLMEngine(folders["C"], dtype="float32", device="cpu", ops=TorchOps(), block_size=8, num_gpu_blocks=11,
                    max_model_len=88, max_num_batched_tokens=24, max_num_seqs=4)
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=16))
    assert sum(o.num_preemptions for o in outs) > 0, "the pool was meant to run out"
    for p, o in zip(prompts, outs):
        assert o.token_ids == plain_greedy(folders["C"], p, 16)
    assert eng.block_manager.num_free_state_slots == 4
