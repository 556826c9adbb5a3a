"""The Pirerax decoder on the host: configuration, the model as data, the cache's needs, each mechanism alone and the
engine's host logic (runner, cache manager, state slots, replay, scheduler) with the kernel library replaced by the
tensor-code stand-in, against the plain implementation."""

from __future__ import annotations

import copy
import math

import numpy as np
import pytest
import torch

from paged_llm_b200.config.model import ConfigError
from paged_llm_b200.config.pirerax import PireraxConfig
from paged_llm_b200.config.registry import parse_model_config
from paged_llm_b200.models.causal_lm import build_model
from paged_llm_b200.parts.base import FixedState, PagedKV
from tests import pirerax_parts as parts
from tests import plain_pirerax as plain
from tests import schedules
from tests.helpers import requests_for
from tests.pirerax_cases import (CASE_A, CASE_B, CASES, attention, case_folder, generated_case, latent, make_folder, moe,
                                 plain_greedy, plain_logits, rounding_error)
from tests.torch_ops import TorchOps

F32_TOL = 2e-5
F32 = torch.float32


def close(got, want, what, rounding=None):
    """Largest difference within F32_TOL of the largest logit; with `rounding` (per position, the root mean square of what
    float32 alone does to the plain model) a position passes too if its root mean square error is within 10 times that."""
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
        assert arch.name == "Pirerax"
        assert PireraxConfig.from_hf_dict(cfg.to_hf_dict()) == cfg
        back = cfg.to_hf_dict()
        back.pop("torch_dtype")
        assert back == hf
        specs = build_model(arch.build_spec(cfg)).tensor_specs()
        assert cfg.num_parameters == sum(int(np.prod(s.draw_shape or s.shape)) for s in specs.values())


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="conv"), "not implemented"),
    (lambda c: c["layers"][0]["mixer"].update(heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"].update(scale=0.0), "scale"),
    (lambda c: c["layers"][0]["mixer"]["q_temp"].update(every=0), "every"),
    (lambda c: c["layers"][0]["mixer"].update(rot={"dims": 8, "base": 10.0}), "rotates nothing"),
    (lambda c: c["layers"][1]["mixer"]["left"].pop("rot"), "rot"),
    (lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=34), "dims"),
    (lambda c: c["layers"][1]["mixer"]["right"].update(heads=3), "multiple"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=10), "dims"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "moe only"),
    (lambda c: c["layers"][0]["mlp"]["expert"].update(limit=0.0), "limit"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "top"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c.pop("width"), "width"),
])
def test_configuration_refusals(change, message):
    hf = copy.deepcopy(CASE_A)
    change(hf)
    with pytest.raises(ConfigError, match=message):
        parse_model_config(hf)


def test_the_model_as_data():
    """Case A: attention caches heads padded to the larger of key and value size; a parallel mixer needs pages for its
    attention and a slot for the delta rule (convolution inputs, then a matrix per head); latent attention caches one
    head of latent + rotated part; the last layer has no feed-forward."""
    arch, cfg = parse_model_config(CASE_A)
    model = build_model(arch.build_spec(cfg))
    slots = model.cache_slots()
    assert [s.requirement for s in slots] == [
        PagedKV(2, 32, None),                                                          # 16 and 24 -> 32
        (PagedKV(4, 32, None), FixedState((2 * (2 * 2 * 8 + 4 * 16) + 4 * 8 * 16,))),  # 3 taps: two rows of 96 inputs, then S
        PagedKV(1, 32, None),                                                          # 24 + 8
        PagedKV(1, 32, None),
    ]
    names = set(model.tensor_specs())
    assert {"embed", "head", "final.norm", "l0.mix.sink", "l0.mix.q.norm", "l1.mix.left.out", "l1.mix.right.A_log",
            "l1.mix.right.q.conv", "l2.mix.dkv.norm", "l2.mix.sink", "l2.mix.g", "l0.mlp.router", "l0.mlp.e5.down"} <= names
    assert "l1.mix.left.sink" not in names, "the attention of a parallel mixer has an ordinary softmax"
    assert not any(n.startswith(("l3.mlp", "l3.norm2")) for n in names), "a layer without a feed-forward"
    assert model.tensor_specs()["l2.mix.g"].shape == (3, 64) and model.tensor_specs()["l0.mix.g"].shape == (4 * 24, 64)
    assert model.has_fixed_state
    # a model without a parallel layer keeps no state of fixed size
    hf = copy.deepcopy(CASE_A)
    del hf["layers"][1]
    arch, cfg = parse_model_config(hf)
    assert not build_model(arch.build_spec(cfg)).has_fixed_state


# ---------------------------------------------------------------- mechanisms by hand
def test_sink_by_hand(ops):
    """One head, keys and queries all zero (scores 0): n visible keys weigh 1 / (n + e^sink) each, so with equal
    values v the output at position i is v (i + 1) / (i + 1 + e^sink); the gate is sigmoid(0) = 1/2."""
    W, m = 4, attention(1, 1, 2, 2, scale=1.0)
    w = parts.attention_weights(W, m, seed=1)
    for name in ("a.q", "a.k", "a.g"):
        w[name][:] = 0.0
    w["a.v"] = torch.tensor([[1.0, 0, 0, 0], [0, 1.0, 0, 0]])
    w["a.o"] = torch.tensor([[1.0, 0], [0, 1.0], [0, 0], [0, 0]])
    w["a.sink"][:] = math.log(3.0)
    h = torch.tensor([[2.0, -4.0, 0.3, 0.1]] * 5)
    want = torch.tensor([[2.0 * (i + 1) / (i + 4) / 2, -4.0 * (i + 1) / (i + 4) / 2, 0, 0] for i in range(5)], dtype=torch.float64)
    got = plain.grouped_attention(h.double(), {k: v.double() for k, v in w.items()}, "a.", m, 1e-5, True)
    assert (got - want).abs().max() < 1e-7            # (the sink is stored in float32)
    part = parts.attention_part(W, m, w, 1e-5, F32, ops, "cpu")
    for out in parts.run_mixer(ops, "cpu", part, [h], F32, ways=("whole", "decode", ("every", 2))):
        assert (out.double() - want).abs().max() < 1e-6


def test_query_temperature_by_hand():
    """coef 0.5, every 4: positions 0..2 give ln(1) = 0 -> factor 1; 3..6 give floor((p+1)/4) = 1 -> 1 + 0.5 ln 2;
    7 gives 2 -> 1 + 0.5 ln 3.  The factor multiplies the query, so it multiplies the scores."""
    W, m = 8, attention(1, 1, 4, 4, scale=0.7, q_temp=(0.5, 4))
    w = parts.attention_weights(W, m, seed=3, sink=False)
    h = parts.rand(8, W, seed=4).double()
    wd = {k: v.double() for k, v in w.items()}
    got = plain.grouped_attention(h, wd, "a.", m, 1e-5, False, m["q_temp"])
    rows = []
    for p in range(8):
        f = 1.0 + 0.5 * math.log((p + 1) // 4 + 1)
        one = plain.grouped_attention(h[:p + 1], wd, "a.", dict(m, scale=0.7 * f), 1e-5, False)
        rows.append(one[-1])
    assert (got - torch.stack(rows)).abs().max() < 1e-12
    assert math.isclose(1.0 + 0.5 * math.log(8 // 4 + 1), 1.0 + 0.5 * math.log(3.0))


def test_router_by_hand(ops):
    """Six experts in three groups of two, two groups stay, two experts are chosen.  Scores (as logits' sigmoids)
    0.9 0.1 | 0.6 0.55 | 0.7 0.2: group sums 1.0, 1.15, 0.9 -> groups 1 and 0 stay; the best two among their experts
    are expert 0 (0.9) and expert 2 (0.6): expert 4 (0.7) belongs to the group that was dropped.  The weights are the
    scores themselves."""
    s = torch.tensor([[0.9, 0.1, 0.6, 0.55, 0.7, 0.2]], dtype=torch.float64)
    z = torch.log(s / (1 - s))
    r = {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 2}}
    idx, wt = plain.router(torch.ones(1, 1, dtype=torch.float64), z.T.clone(), r)
    assert sorted(idx[0].tolist()) == [0, 2] and np.allclose(sorted(wt[0].tolist()), [0.6, 0.9])
    # the same through the part: one input unit, the router's rows are the logits, experts that return their index
    W = 8
    mlp = moe(8, 100.0, 6, 2, (3, 2))
    w = parts.experts_weights(W, mlp, seed=2)
    w["m.router"] = torch.zeros(6, W)
    w["m.router"][:, 0] = z[0].float()
    h = torch.zeros(1, W)
    h[0, 0] = 1.0
    part = parts.experts_part(W, mlp, w, F32, "cpu")
    import types
    got = part.forward(h, types.SimpleNamespace(ops=ops)).double()
    wd = {k: v.double() for k, v in w.items()}
    want = sum(float(torch.sigmoid(w["m.router"][e, 0].double())) * plain.expert(h.double(), wd, f"m.e{e}.", 100.0) for e in (0, 2))
    assert (got - want).abs().max() < 1e-5
    # without groups expert 4 is chosen beside expert 0
    idx, _ = plain.router(torch.ones(1, 1, dtype=torch.float64), z.T.clone(), {"experts": 6, "top": 2})
    assert sorted(idx[0].tolist()) == [0, 4]


def test_clamped_activation_by_hand():
    """limit 1.5: gate 3 -> 1.5, up -2 -> -1.5: 1.5 sigmoid(1.702 * 1.5) (-0.5); gate -4 stays (only its top is cut),
    up 0.25 stays: -4 sigmoid(-6.808) 1.25."""
    w = {"e.gate": torch.tensor([[3.0], [-4.0]], dtype=torch.float64), "e.up": torch.tensor([[-2.0], [0.25]], dtype=torch.float64),
         "e.down": torch.eye(2, dtype=torch.float64)}
    got = plain.expert(torch.ones(1, 1, dtype=torch.float64), w, "e.", 1.5)[0]
    sig = lambda z: 1 / (1 + math.exp(-z))      # noqa: E731
    assert np.allclose(got.tolist(), [1.5 * sig(1.702 * 1.5) * -0.5, -4.0 * sig(-4 * 1.702) * 1.25], rtol=1e-12)


def test_delta_rule_by_hand(ops):
    """One head, one key channel, one value channel, one tap with weight 1: k = silu(x)/|silu(x)| = +-1 and q = k
    (key size 1, so the scale is 1), so S <- g S; S <- S + beta (v - S k) k; o = S q."""
    W, m = 3, {"heads": 1, "kv_heads": 1, "dim": 1, "vdim": 1, "conv": 1}
    w = parts.delta_weights(W, m, seed=0)
    w.update({"d.q": torch.tensor([[1.0, 0, 0]]), "d.k": torch.tensor([[1.0, 0, 0]]), "d.v": torch.tensor([[0, 1.0, 0]]),
              "d.b": torch.tensor([[0, 0, 1.0]]), "d.a": torch.tensor([[0, 0, 0.5]]), "d.q.conv": torch.ones(1, 1),
              "d.k.conv": torch.ones(1, 1), "d.v.conv": torch.ones(1, 1), "d.A_log": torch.tensor([-1.0]),
              "d.dt_bias": torch.tensor([0.25]), "d.norm": torch.ones(1), "d.g": torch.tensor([[0, 0, 1.0]]),
              "d.o": torch.tensor([[1.0], [0], [0]])})
    h = torch.tensor([[2.0, 1.0, 0.5], [-1.0, 3.0, -0.5], [0.5, -2.0, 1.0]])
    sig = lambda z: 1 / (1 + math.exp(-z))      # noqa: E731
    silu = lambda z: z * sig(z)                 # noqa: E731
    S, outs = 0.0, []
    for x, v_in, c in h.tolist():
        k = silu(x) / math.sqrt(silu(x) ** 2 + 1e-6)
        v = silu(v_in)
        g = math.exp(-math.exp(-1.0) * math.log1p(math.exp(0.5 * c + 0.25)))
        S = g * S
        S = S + k * sig(c) * (v - S * k)
        outs.append(S * k)
    got = plain.gated_delta(h.double(), {k: v.double() for k, v in w.items()}, "d.", m, 0.0)
    # the norm over one value leaves the sign; times silu(gate)
    want = [math.copysign(1.0, o) * silu(c) for o, (_, _, c) in zip(outs, h.tolist())]
    assert np.allclose(got[:, 0].numpy(), want, rtol=1e-9)
    eps = 1e-3
    want = [o / math.sqrt(o * o + eps) * silu(c) for o, (_, _, c) in zip(outs, h.tolist())]
    part = parts.delta_part(W, m, w, eps, F32, "cpu")
    for out in parts.run_mixer(ops, "cpu", part, [h], F32, ways=("whole", "decode")):
        assert np.allclose(out[:, 0].numpy(), want, rtol=1e-5)


# ---------------------------------------------------------------- each mixer alone, through prompts and decoding
@pytest.mark.parametrize("W,m,sink", [
    (48, attention(4, 2, 16, 24, q_temp=(0.5, 4)), True),
    (32, attention(6, 1, 8, 40, scale=0.4), True),                                          # heads that pad the cache
    (40, dict(attention(3, 3, 32, 16, scale=0.3), rot={"dims": 8, "base": 100.0}), False),    # rotation, ordinary softmax
    (40, dict(attention(2, 1, 16, 16), rot={"dims": 16, "base": 1e4}, q_temp={"coef": 2.0, "every": 3}), True),
])
def test_attention_alone(ops, W, m, sink):
    parts.check_attention(ops, "cpu", F32, W, m, (1, 2, 21, 37), seed=3, sink=sink)


@pytest.mark.parametrize("W,m", [
    (48, latent(3, 16, 8, 24, 24, base=500.0)),
    (32, latent(1, 8, 2, 8, 8)),
    (64, latent(4, 32, 16, 16, 40, base=1e6, scale=0.2)),
])
def test_latent_attention_alone(ops, W, m):
    parts.check_latent(ops, "cpu", F32, W, m, (1, 2, 19, 33), seed=5)


@pytest.mark.parametrize("W,m", [
    (48, {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 16, "conv": 3}),
    (32, {"heads": 2, "kv_heads": 2, "dim": 24, "vdim": 8, "conv": 1}),
    (40, {"heads": 3, "kv_heads": 1, "dim": 40, "vdim": 20, "conv": 5}),
])
def test_delta_rule_alone(ops, W, m):
    parts.check_delta(ops, "cpu", F32, W, m, (1, 2, 4, 23), seed=7)


def test_parallel_mixer_alone(ops):
    m = {"left": dict(attention(4, 2, 16, 8), rot={"dims": 8, "base": 100.0}),
         "right": {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 12, "conv": 2}}
    parts.check_parallel(ops, "cpu", F32, 32, m, (1, 3, 18), seed=9)


@pytest.mark.parametrize("mlp", [moe(16, 1.0, 6, 2, (3, 2)), moe(24, 0.5, 4, 1, (1, 1)), moe(8, 7.0, 5, 3), moe(16, 1.5, 8, 4, (4, 2))])
def test_experts_alone(ops, mlp):
    parts.check_experts(ops, "cpu", F32, 32, mlp, 24, seed=11)


def test_one_far_key_among_hundreds(ops):
    """Position 5 holds the one key every head answers to; 400 positions later, in a prompt's portion and decoding, it
    still takes nearly all the weight that the sink leaves."""
    W, m = 16, attention(2, 1, 8, 8, scale=1.0)
    w, h = parts.loud_key(W, m, 420, 5, seed=1)
    want = parts.check_attention(ops, "cpu", F32, W, m, None, weights=w, hs=[h], ways=("whole", "decode", (0.5, 0.5)))
    quiet = parts.check_attention(ops, "cpu", F32, W, m, None, weights=w, hs=[torch.cat([h[:5], h[6:]])], ways=("whole",))
    assert (want[-1] - quiet[-1]).abs().max() > 0.05, "the far key does not show"


def test_a_far_token_through_the_delta_state(ops):
    """A decay close to one and keys of 32 channels (a later key wipes little of an earlier one): what the first token
    wrote still shows 300 tokens later."""
    W, m = 16, {"heads": 2, "kv_heads": 1, "dim": 32, "vdim": 8, "conv": 2}
    w = parts.delta_weights(W, m, seed=4, a_log=-9.0)
    w["d.b"] = w["d.b"] * 0.0                     # beta = 1/2 everywhere
    h = parts.rand(300, W, seed=8)
    want = parts.check_delta(ops, "cpu", F32, W, m, None, weights=w, hs=[h], ways=("whole", "decode", ("every", 2)))
    h2 = h.clone()
    h2[0] = -h2[0]
    other = plain.gated_delta(h2.double(), {k: v.double() for k, v in w.items()}, "d.", m, 1e-5)
    assert (want[-1] - other[-1]).abs().max() > 1e-3, "the first token does not show"


# ---------------------------------------------------------------- the engine
@pytest.mark.parametrize("case", sorted(CASES))
@pytest.mark.parametrize("schedule", ["whole", "tail", "portions", "mixed"])
def test_schedules_against_the_plain_model(folders, case, schedule):
    hf, _ = CASES[case]
    reqs = requests_for(hf["vocab"], (1, 2, 23, 41, 70), seed=7)
    steps, max_tokens = getattr(schedules, schedule)(reqs)
    outputs, rp = replay(folders[case], steps, max_tokens)
    got = schedules.collect(steps, outputs)
    for rid, toks in reqs.items():
        close(got[rid], plain_logits(folders[case], toks), f"{case} {schedule} {rid}", rounding_error(folders[case], toks))


def test_the_stream_after_every_layer(folders):
    """The residual stream of the engine after every layer against the plain model's."""
    from paged_llm_b200.engine.replay import TraceReplayer
    from paged_llm_b200.parts.base import materialize
    from tests.pirerax_cases import read_folder
    folder = folders["A"]
    cfg, w = read_folder(folder)
    toks = requests_for(cfg["vocab"], (29,), seed=2)["r0"]
    rp = TraceReplayer(folder, "float32", 64, device="cpu", ops=TorchOps(), block_size=8, max_num_seqs=2)
    seen = []
    for blk in rp.model.blocks:
        def wrap(f):
            def g(x, pending, ctx, cache):
                x, p = f(x, pending, ctx, cache)
                p = materialize(p, ctx.ops)
                seen.append((x + p.float()).clone())
                return x, p
            return g
        blk.forward = wrap(blk.forward)
    rp.step({"step": 0, "entries": [{"id": "a", "tokens": toks, "want": [0]}], "end": ["a"]})
    with torch.no_grad():
        after = plain.forward(cfg, w, toks)[1]
    for i, s in enumerate(seen):
        assert (s.double() - after[i]).abs().max() < 2e-5 * max(1.0, float(after[i].abs().max())), f"layer {i}"


def test_state_does_not_leak_between_requests(folders):
    """Two live requests in two slots, then a third that takes over a freed slot: each matches its plain run."""
    hf, _ = CASES["B"]
    reqs = requests_for(hf["vocab"], (17, 9, 13), seed=3)
    a, b, c = reqs["r0"], reqs["r1"], reqs["r2"]
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:10], "want": list(range(10))}, {"id": "b", "tokens": b[:4], "want": list(range(4))}], "end": []},
        {"step": 1, "entries": [{"id": "b", "tokens": b[4:], "want": list(range(5))}], "end": ["b"]},           # a sits out
        {"step": 2, "entries": [{"id": "a", "tokens": a[10:12], "want": [0, 1]}, {"id": "c", "tokens": c[:2], "want": [0, 1]}], "end": []},
        {"step": 3, "entries": [{"id": "c", "tokens": c[2:], "want": list(range(11))}, {"id": "a", "tokens": a[12:], "want": list(range(5))}],
         "end": ["a", "c"]},
    ]
    outputs, _ = replay(folders["B"], steps, 128, slots=2)
    got = schedules.collect(steps, outputs)
    for rid, toks in (("a", a), ("b", b), ("c", c)):
        close(got[rid], plain_logits(folders["B"], toks), rid)


@pytest.mark.parametrize("seed", range(8))
def test_generated_configurations(tmp_path, seed):
    hf = generated_case(100 + seed)
    folder = make_folder(tmp_path, hf, 200 + seed)
    reqs = requests_for(hf["vocab"], (2, 19, 33), seed=seed)
    steps, max_tokens = schedules.mixed(reqs, live=3, seed=seed)
    outputs, _ = replay(folder, steps, max_tokens, slots=3)
    got = schedules.collect(steps, outputs)
    for rid, toks in reqs.items():
        close(got[rid], plain_logits(folder, toks), f"seed {seed} {rid}", rounding_error(folder, toks))


def _engine(folder, **kw):
    from paged_llm_b200 import LLMEngine
    return LLMEngine(folder, dtype="float32", device="cpu", ops=TorchOps(), block_size=8, max_model_len=96, **kw)


@pytest.mark.parametrize("case", sorted(CASES))
def test_greedy_generation_through_the_engine(folders, case):
    from paged_llm_b200 import SamplingParams
    hf, _ = CASES[case]
    prompts = list(requests_for(hf["vocab"], (3, 11, 26), seed=5).values())
    eng = _engine(folders[case], num_gpu_blocks=40, max_num_seqs=4, max_num_batched_tokens=16)
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=6))
    for p, o in zip(prompts, outs):
        assert o.token_ids == plain_greedy(folders[case], p, 6)


def test_generation_under_preemption(folders):
    """So few pages that requests are preempted and start again, their state slots zeroed anew."""
    from paged_llm_b200 import SamplingParams
    hf, _ = CASES["A"]
    prompts = list(requests_for(hf["vocab"], (14, 15, 13), seed=6).values())
    eng = _engine(folders["A"], num_gpu_blocks=7, max_num_seqs=3, max_num_batched_tokens=32)
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10))
    assert eng.scheduler.num_preemptions > 0 if hasattr(eng.scheduler, "num_preemptions") else True
    for p, o in zip(prompts, outs):
        assert o.token_ids == plain_greedy(folders["A"], p, 10)
