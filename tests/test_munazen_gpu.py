"""The Munazen decoder on the GPU: each new kernel and each mixer alone against the plain functions, then the engine
under every schedule in both precisions against the plain model."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from tests import munazen_parts as parts
from tests import plain_munazen as plain
from tests import schedules
from tests.helpers import requests_for
from tests.munazen_cases import (CASE_A, CASE_B, CASE_C, CASES, YARN, case_folder, generated_case, left, make_folder,
                                 plain_greedy, plain_logits, rounding_error)

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
F32_TOL, BF16_TOL = 2e-5, 4e-2


@pytest.fixture(scope="module")
def ops():
    from paged_llm_b200.kernels.ops import CudaOps
    return CudaOps("cuda")


def close(got, want, dtype, what, rounding=None):
    """float32: the largest difference within F32_TOL of the largest logit, or the position's root mean square error
    within 10 times what float32 alone does to the plain model there.  bfloat16: within BF16_TOL of the largest logit, or
    (`rounding` then measured in bfloat16) a root mean square error within 3 times what bfloat16 alone does there, or
    within what it does at the request's worst position (one run in bfloat16 is one draw of a position's error)."""
    assert got.shape == want.shape, what
    assert np.isfinite(got).all(), what
    err = np.abs(got - want)
    top = max(1.0, float(np.abs(want).max()))
    if dtype == "bfloat16":
        bad = err.max(axis=1) > BF16_TOL * top
        if rounding is not None:
            rms = np.sqrt((err.astype(np.float64) ** 2).mean(axis=1))
            bad &= (rms > 3.0 * rounding) & (rms > rounding.max())
    else:
        bad = err.max(axis=1) > F32_TOL * top
        if rounding is not None:
            bad &= np.sqrt((err.astype(np.float64) ** 2).mean(axis=1)) > 10.0 * rounding
    assert not bad.any(), f"{what}: max |diff| {err.max():.3e}, first bad row {int(np.argmax(bad))} ({err[int(np.argmax(bad))].max():.3e})"


# ---------------------------------------------------------------- kernels and mixers alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,W,S,G", [(9, 48, 3, 2), (1, 32, 1, 1), (5, 40, 5, 4), (4, 24, 2, 3), (300, 1024, 4, 8), (70, 2048, 8, 1),
                                        (7, 30, 3, 2), (3, 6, 2, 3), (11, 66, 4, 1), (2, 1030, 1, 5)])
def test_stream_norm_alone(ops, dtype, rows, W, S, G):
    parts.check_stream_norm(ops, "cuda", dtype, rows, W, S, G)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,F", [(9, 145), (1, 8), (33, 4096), (200, 1000), (3, 11008)])
def test_poly_norm_alone(ops, dtype, rows, F):
    parts.check_poly_norm(ops, "cuda", dtype, rows, F)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("copies", [1, 3])
def test_embedding_copies(ops, dtype, copies):
    g = torch.Generator().manual_seed(1)
    table = torch.randn(50, 36, generator=g).to(dtype)
    ids = torch.tensor([3, 49, 0, 7], dtype=torch.int32)
    out = ops.embedding(table.cuda(), ids.cuda(), 1.0, copies=copies)
    assert out.dtype == torch.float32 and torch.equal(out.cpu(), table[ids.long()].float().repeat(1, copies))


@pytest.mark.parametrize("dtype", DTYPES)
def test_scaled_sum_and_bias(ops, dtype):
    ops.set_compute_dtype(dtype)
    a, b = parts.rand(7, 40, seed=1).to(dtype), parts.rand(7, 40, seed=2).to(dtype)
    ba, bb = parts.rand(40, seed=3), parts.rand(40, seed=4)
    got = ops.scaled_sum(a.cuda(), 1.2, ba.cuda(), b.cuda(), -0.7, None).cpu()
    assert got.dtype == torch.float32
    assert (got.double() - (1.2 * (a.double() + ba.double()) - 0.7 * b.double())).abs().max() <= 1e-5
    got = ops.scaled_sum(a.cuda(), 0.5, None, b.cuda(), 2.0, bb.cuda()).cpu()
    assert (got.double() - (0.5 * a.double() + 2.0 * (b.double() + bb.double()))).abs().max() <= 1e-5
    y = ops.add_bias(a.cuda().clone(), ba.cuda()).float().cpu()
    assert (y.double() - (a.double() + ba.double())).abs().max() <= parts.tol(dtype, 4.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("W,m", [
    (48, left(4, 2, 16, 24, dims=8, base=100.0, scaling=YARN, scale=0.25)),
    (32, left(6, 1, 24, 40, dims=12, base=1e6, scaling=dict(YARN, factor=8.0, original=64))),
    (40, left(3, 3, 32, 16, base=500.0, scale=0.3)),
    (24, left(1, 1, 8, 8, dims=2)),
    (64, left(8, 2, 64, 128, dims=32, base=1e6, scaling=dict(YARN, factor=16.0, original=128, fast=32.0))),
    (64, left(20, 1, 16, 16)),
])
def test_attention_mixer_alone(ops, dtype, W, m):
    parts.check_attention(ops, "cuda", dtype, W, m, [1, 137, 70, 2], ps=16)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("W,m", [(48, {"width": 36, "blocks": 3, "conv": 3}), (32, {"width": 20, "blocks": 1, "conv": 1}),
                                 (24, {"width": 64, "blocks": 4, "conv": 6}), (16, {"width": 8, "blocks": 8, "conv": 2}),
                                 (64, {"width": 1030, "blocks": 2, "conv": 4}), (64, {"width": 264, "blocks": 33, "conv": 8})])
def test_recurrence_mixer_alone(ops, dtype, W, m):
    parts.check_recurrence(ops, "cuda", dtype, W, m, [1, 137, 70, 2], ways=("whole", (0.6, 0.4), "decode", ("every", 2)))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("W,m", [(48, {"heads": 2, "dim": 12, "vdim": 20, "tau": 4.0}), (32, {"heads": 1, "dim": 40, "vdim": 8, "tau": 1.0}),
                                 (24, {"heads": 5, "dim": 4, "vdim": 4, "tau": 16.0}), (64, {"heads": 3, "dim": 128, "vdim": 256, "tau": 16.0}),
                                 (64, {"heads": 2, "dim": 72, "vdim": 48, "tau": 2.0}), (32, {"heads": 4, "dim": 32, "vdim": 48, "tau": 8.0})])
def test_linear_attention_mixer_alone(ops, dtype, W, m):
    parts.check_gla(ops, "cuda", dtype, W, m, [1, 137, 70, 2], ways=("whole", (0.6, 0.4), "decode", ("every", 2)))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("W,m", [(32, {"heads": 2, "dim": 24, "vdim": 40, "tau": 8.0}), (48, {"heads": 3, "dim": 130, "vdim": 16, "tau": 2.0}),
                                 (16, {"heads": 1, "dim": 8, "vdim": 33, "tau": 16.0})])
def test_linear_attention_long_prompts_in_segments(ops, dtype, W, m):
    """Prompts of two segments and more run their segments side by side: lengths at a segment's edge, one token past
    it and one short of it, beside short requests, whole and in portions that start inside a segment."""
    parts.check_gla(ops, "cuda", dtype, W, m, [700, 3, 257, 256, 255, 130, 520],
                    ways=("whole", (0.45, 0.55), (0.1, 0.9), (0.37, 0.0015, 0.6285)))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("W,m", [(32, {"width": 40, "blocks": 2, "conv": 4}), (24, {"width": 33, "blocks": 1, "conv": 2})])
def test_recurrence_long_prompts(ops, dtype, W, m):
    parts.check_recurrence(ops, "cuda", dtype, W, m, [700, 3, 65, 64, 17, 16, 520], ways=("whole", (0.45, 0.55), (0.1, 0.9)))


@pytest.mark.parametrize("dtype", DTYPES)
def test_one_far_key_among_hundreds(ops, dtype):
    """Key 3 of 900 takes the weight of every later query, in a prompt, in portions and token by token."""
    m = left(4, 2, 16, 24, dims=8, base=100.0, scaling=YARN, scale=0.25)
    W, n = 32, 900
    w, h = parts.loud_key_setup(W, m, n, 3, seed=4)
    want = parts.check_attention(ops, "cuda", dtype, W, m, None, weights=w, hs=[h], ways=("whole", (0.9, 0.1), ("every", 64), "decode"), ps=16)
    h2 = h.clone()
    h2[3, 0] = 0.0
    quiet = plain.attention_left(h2.double(), {k: v.double() for k, v in w.items()}, "a.", m)
    assert (quiet[-1] - want[-1]).abs().max() > 0.1, "the far key must matter"


@pytest.mark.parametrize("loud", [0, 15, 16, 17, 63, 64, 500])
def test_one_key_at_page_borders(ops, loud):
    """The loud key sits at the first token, on either side of a page border, and far back."""
    m = left(2, 1, 8, 12, dims=4, base=50.0, scale=1.0)
    w, h = parts.loud_key_setup(16, m, 520, loud, seed=loud)
    parts.check_attention(ops, "cuda", torch.bfloat16, 16, m, None, weights=w, hs=[h], ways=("whole", (0.97, 0.03), "decode"), ps=16)


def test_long_recurrence_keeps_a_far_token(ops):
    """Decays close to one: the first token still shows after 3,000 more, in portions and token by token."""
    W, m = 16, {"width": 12, "blocks": 2, "conv": 3}
    h = parts.rand(3001, W, seed=9, std=0.3)
    h[0] *= 30.0
    want = parts.check_recurrence(ops, "cuda", torch.float32, W, m, None, lam=-9.0, hs=[h], ways=((0.37, 0.63), (0.999, 0.001), "decode"))
    h2 = h.clone()
    h2[0] /= 30.0
    w = parts.recurrence_weights(W, m, 0, -9.0)
    quiet = plain.recurrent_right(h2.double(), {k: v.double() for k, v in w.items()}, "r.", m)
    assert (quiet[-1] - want[-1]).abs().max() > 3e-3, "the far token must matter"


def test_long_linear_attention_keeps_a_far_token(ops):
    W, m = 16, {"heads": 2, "dim": 8, "vdim": 8, "tau": 16.0}
    h = parts.rand(3001, W, seed=9, std=0.3)
    h[0] *= 30.0
    want = parts.check_gla(ops, "cuda", torch.float32, W, m, None, decay_bias=9.0, hs=[h], ways=((0.37, 0.63), (0.999, 0.001), "decode"))
    h2 = h.clone()
    h2[0] /= 30.0
    w = parts.gla_weights(W, m, 0, decay_bias=9.0)
    quiet = plain.mixer_gla(h2.double(), {k: v.double() for k, v in w.items()}, "g.", m, 1e-5)
    assert (quiet[-1] - want[-1]).abs().max() > 3e-3, "the far token must matter"


# ---------------------------------------------------------------- the engine against the plain model
LENGTHS = {"A": (1, 30, 77, 49, 2, 60, 90, 35), "B": (5, 41, 120, 13, 80, 55), "C": (3, 70, 33, 65, 18, 41)}


def rounding_of(folder, toks, dtype):
    return rounding_error(folder, toks, torch.bfloat16 if dtype == "bfloat16" else torch.float32)


def replay(folder, dtype, steps, max_tokens, block_size=16, slots=4, **kw):
    from paged_llm_b200.engine.replay import TraceReplayer

    rp = TraceReplayer(folder, dtype, max_tokens, block_size=block_size, poison=float("nan"), max_num_seqs=slots, **kw)
    for state in rp.storage._state_tensors():
        state.fill_(float("nan"))                     # a slot that is not zeroed at a request's start shows
    outputs = {}
    for rec in steps:
        out = rp.step(rec)
        if out is not None:
            outputs[rec["step"]] = out
    assert not rp.live, "requests left alive at the end of the trace"
    rp.cm.check_invariants([])
    for g in range(len(rp.cm.pools)):
        assert rp.cm.num_free_in_group(g) == rp.cm.pools[g].num_pages, "pages were lost"
    assert rp.cm.num_free_state_slots == rp.cm.num_state_slots
    return outputs, rp


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: case_folder(tmp_path_factory, name) for name in CASES}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("schedule", ["whole", "tail", "portions", "mixed"])
def test_schedule_matches_plain(folders, name, dtype, schedule):
    hf = CASES[name][0]
    reqs = requests_for(hf["vocab"], LENGTHS[name], seed=ord(name))
    steps, max_tokens = getattr(schedules, schedule)(reqs)
    block = 8 if name == "B" else 16
    outputs, rp = replay(folders[name], dtype, steps, max_tokens, block_size=block)
    got = schedules.collect(steps, outputs)
    for rid, toks in reqs.items():
        close(got[rid], plain_logits(folders[name], toks), dtype, f"{schedule}/{name}/{rid}", rounding_of(folders[name], toks, dtype))
    if schedule == "tail":
        assert rp.runner.num_graph_steps > 0, "decode steps replay graphs: every part of the model can be captured"


@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("schedule", ["tail", "portions", "mixed"])
def test_bfloat16_against_the_float32_engine(folders, name, schedule):
    reqs = requests_for(CASES[name][0]["vocab"], LENGTHS[name], seed=ord(name))
    steps, max_tokens = getattr(schedules, schedule)(reqs)
    a, _ = replay(folders[name], "float32", steps, max_tokens)
    b, _ = replay(folders[name], "bfloat16", steps, max_tokens)
    a, b = schedules.collect(steps, a), schedules.collect(steps, b)
    for rid, toks in reqs.items():
        close(b[rid], a[rid], "bfloat16", f"munazen {schedule}/{name}/{rid}", rounding_of(folders[name], toks, "bfloat16"))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_graph_and_eager_decode_agree(folders, dtype):
    reqs = requests_for(CASE_A["vocab"], (66, 90), seed=5)
    steps, max_tokens = schedules.tail(reqs, last=45)
    a, rp_a = replay(folders["A"], dtype, steps, max_tokens)
    b, rp_b = replay(folders["A"], dtype, steps, max_tokens, enforce_eager=True)
    assert rp_a.runner.num_graph_steps > 0 and rp_b.runner.num_graph_steps == 0
    for k in a:
        close(a[k], b[k], dtype, f"graph vs eager step {k}")


def test_long_decoding(folders):
    """Three hundred tokens one by one behind a short prompt, beside a second request that does the same."""
    reqs = requests_for(CASE_B["vocab"], (330, 311), seed=12)
    steps, max_tokens = schedules.mixed(reqs, live=2, seed=3, prompt_fraction=0.08)
    for dtype in ("float32", "bfloat16"):
        outputs, _ = replay(folders["B"], dtype, steps, max_tokens, block_size=8, slots=2)
        got = schedules.collect(steps, outputs)
        for rid, toks in reqs.items():
            close(got[rid], plain_logits(folders["B"], toks), dtype, f"long decoding {dtype}/{rid}", rounding_of(folders["B"], toks, dtype))


@pytest.mark.parametrize("seed", range(10))
def test_generated_configurations(tmp_path, seed):
    hf = generated_case(100 + seed)
    folder = make_folder(tmp_path, hf, seed)
    reqs = requests_for(hf["vocab"], (2, 50, 21, 70, 9, 130), seed=seed)
    steps, max_tokens = schedules.mixed(reqs, live=3, seed=seed)
    for dtype in ("float32", "bfloat16"):
        outputs, _ = replay(folder, dtype, steps, max_tokens, slots=3)
        got = schedules.collect(steps, outputs)
        for rid, toks in reqs.items():
            close(got[rid], plain_logits(folder, toks), dtype, f"generated {seed}/{dtype}/{rid}", rounding_of(folder, toks, dtype))


def test_greedy_generation_through_the_engine(folders):
    from paged_llm_b200 import LLMEngine, SamplingParams
    prompts = list(requests_for(CASE_A["vocab"], (3, 22, 47, 9, 31), seed=60).values())
    eng = LLMEngine(folders["A"], dtype="float32", block_size=16, num_gpu_blocks=24, max_model_len=96,
                    max_num_batched_tokens=16, max_num_seqs=3)
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12))
    for p, o in zip(prompts, outs):
        assert o.token_ids == plain_greedy(folders["A"], p, 12)
    assert eng.block_manager.num_free_state_slots == 3


def test_generation_with_preemption_restarts_the_state(folders):
    from paged_llm_b200 import LLMEngine, SamplingParams
    prompts = list(requests_for(CASE_C["vocab"], (30, 26, 21, 12), seed=70).values())
    eng = LLMEngine(folders["C"], dtype="float32", block_size=8, num_gpu_blocks=11, max_model_len=88,
                    max_num_batched_tokens=24, max_num_seqs=4)
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=16))
    assert sum(o.num_preemptions for o in outs) > 0, "the pool was meant to run out"
    for p, o in zip(prompts, outs):
        assert o.token_ids == plain_greedy(folders["C"], p, 16)
    assert eng.block_manager.num_free_state_slots == 4
