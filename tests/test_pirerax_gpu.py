"""The Pirerax decoder on the GPU: each new kernel and each mixer alone against the plain functions, then the engine
under every schedule in both precisions against the plain model."""

from __future__ import annotations

import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from tests import pirerax_parts as parts
from tests import plain_pirerax as plain
from tests import schedules
from tests.helpers import requests_for
from tests.pirerax_cases import (CASE_A, CASE_B, CASE_C, CASES, attention, case_folder, clear_requests, generated_case, latent,
                                 make_folder, moe, plain_greedy, plain_logits, rounding_error, wide_case)

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


# ---------------------------------------------------------------- kernels alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,W", [(9, 48), (1, 8), (300, 1024), (33, 2050), (5, 30)])
def test_two_normed_branches(ops, dtype, rows, W):
    """sa rms(a) wa + sb rms(b) wb alone, and with the residual sum and the next norm in the same kernel."""
    ops.set_compute_dtype(dtype)
    a, b = parts.rand(rows, W, seed=1).to(dtype), parts.rand(rows, W, seed=2, std=3.0).to(dtype)
    wa, wb, nw = 1.0 + parts.rand(W, seed=3, std=0.2), 1.0 + parts.rand(W, seed=4, std=0.2), 1.0 + parts.rand(W, seed=5, std=0.2)
    x = parts.rand(rows, W, seed=6)
    unit = lambda t, e: t / torch.sqrt((t * t).mean(-1, keepdim=True) + e)      # noqa: E731
    want = 0.5 * unit(a.double(), 1e-5) * wa.double() + 0.25 * unit(b.double(), 1e-5) * wb.double()
    got = ops.normed_pair_sum(a.cuda(), b.cuda(), wa.cuda(), wb.cuda(), 0.5, 0.25, 1e-5).cpu()
    assert got.dtype == torch.float32 and (got.double() - want).abs().max() < 1e-5
    xd = x.cuda().clone()
    y = ops.normed_pair_add_rms_norm(xd, a.cuda(), b.cuda(), wa.cuda(), wb.cuda(), 0.5, 0.25, 1e-5, nw.cuda(), 1e-6).float().cpu()
    assert (xd.cpu().double() - (x.double() + want)).abs().max() < 1e-5, "the stream takes the sum in"
    assert (y.double() - unit(x.double() + want, 1e-6) * nw.double()).abs().max() < parts.tol(dtype, 2.0)


@pytest.mark.parametrize("mlp,W,rows", [(moe(16, 1.0, 6, 2, (3, 2)), 32, 40), (moe(24, 0.5, 4, 1, (1, 1)), 32, 9), (moe(8, 7.0, 5, 3), 40, 33),
                                        (moe(64, 1.5, 8, 4, (4, 2)), 64, 300), (moe(40, 2.0, 64, 6, (8, 3)), 64, 50),
                                        (moe(64, 1.5, 12, 2, (3, 1)), 128, 2100)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_experts_alone(ops, dtype, mlp, W, rows):
    """Sigmoid scores, groups, the clamped activation, in every form of the products (tiles of 16 and 64 pairs, the
    grouped tcgen05 form from 2,048 pairs on, FFMA chains in float32)."""
    parts.check_experts(ops, "cuda", dtype, W, mlp, rows, seed=13, scale_tol=4.0)


def test_router_choice_by_hand(ops):
    """The kernel's choice on the hand-made case of six experts in three groups (see the host test), and without groups."""
    lib = __import__("paged_llm_b200.kernels.ops", fromlist=["load_module"]).load_module("moe")
    from ctypes import c_void_p
    s = torch.tensor([[0.9, 0.1, 0.6, 0.55, 0.7, 0.2], [0.2, 0.3, 0.9, 0.05, 0.5, 0.6]], dtype=torch.float32)
    z = torch.log(s / (1 - s)).cuda().contiguous()
    idx = torch.empty(4, dtype=torch.int32, device="cuda")
    wt = torch.empty(4, dtype=torch.float32, device="cuda")
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.pl_moe_sigmoid_topk(c_void_p(z.data_ptr()), 6, 2, 6, 2, 3, 2, 2, c_void_p(idx.data_ptr()), c_void_p(wt.data_ptr()), stream) == 0
    assert idx.cpu().view(2, 2).tolist() == [[0, 2], [2, 5]]         # row 1: groups 0.5, 0.95, 1.1 -> experts 2..5 may be chosen
    assert lib.pl_moe_sigmoid_topk(c_void_p(z.data_ptr()), 6, 2, 6, 2, 0, 0, 0, c_void_p(idx.data_ptr()), c_void_p(wt.data_ptr()), stream) == 0
    assert idx.cpu().view(2, 2).tolist() == [[0, 4], [2, 5]]
    assert np.allclose(wt.cpu().view(2, 2).numpy(), [[0.9, 0.7], [0.9, 0.6]], rtol=1e-5)


# ---------------------------------------------------------------- mixers alone
LENS = [1, 137, 70, 2]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("W,m,sink", [
    (48, attention(4, 2, 16, 24, q_temp=(0.5, 4)), True),
    (32, attention(6, 1, 8, 40, scale=0.4), True),
    (40, dict(attention(3, 3, 32, 16, scale=0.3), rot={"dims": 8, "base": 100.0}), False),
    (40, dict(attention(2, 1, 16, 16), rot={"dims": 16, "base": 1e4}, q_temp={"coef": 2.0, "every": 3}), True),
    (64, attention(8, 2, 64, 64, q_temp=(0.5, 64)), True),                                   # tcgen05 prefill, head size 64
    (64, dict(attention(4, 1, 128, 128, scale=0.05), rot={"dims": 64, "base": 5e4}), False),  # head size 128
    (64, attention(20, 1, 16, 16), True),
])
def test_attention_alone(ops, dtype, W, m, sink):
    parts.check_attention(ops, "cuda", dtype, W, m, LENS, seed=3, sink=sink, ps=16)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("W,m", [
    (48, latent(3, 16, 8, 24, 24, base=500.0)), (32, latent(1, 8, 2, 8, 8)), (64, latent(4, 32, 16, 16, 40, base=1e6, scale=0.2)),
    (64, latent(8, 64, 32, 64, 96, base=2e4)), (64, latent(2, 48, 64, 32, 192)),
])
def test_latent_attention_alone(ops, dtype, W, m):
    parts.check_latent(ops, "cuda", dtype, W, m, LENS, seed=5, ps=16)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("W,m", [
    (48, {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 16, "conv": 3}), (32, {"heads": 2, "kv_heads": 2, "dim": 24, "vdim": 8, "conv": 1}),
    (40, {"heads": 3, "kv_heads": 1, "dim": 40, "vdim": 20, "conv": 5}), (64, {"heads": 2, "kv_heads": 1, "dim": 128, "vdim": 40, "conv": 4}),
    (64, {"heads": 1, "kv_heads": 1, "dim": 200, "vdim": 17, "conv": 2}), (32, {"heads": 6, "kv_heads": 3, "dim": 64, "vdim": 64, "conv": 4}),
])
def test_delta_rule_alone(ops, dtype, W, m):
    """Every form of the recurrence's kernel (key sizes up to 32, 64, 128, 256; 8, 16 and 32 lanes per column), sizes
    that fill neither lanes nor columns."""
    try:
        for lanes in (0, 16, 32):
            ops.delta_lanes = lanes
            parts.check_delta(ops, "cuda", dtype, W, m, LENS, seed=7, ways=("whole", (0.6, 0.4), "decode", ("every", 2)))
    finally:
        ops.delta_lanes = 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_parallel_mixer_alone(ops, dtype):
    m = {"left": dict(attention(4, 2, 16, 8), rot={"dims": 8, "base": 100.0}), "right": {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 12, "conv": 2}}
    parts.check_parallel(ops, "cuda", dtype, 32, m, [1, 3, 70], seed=9)
    m = {"left": dict(attention(2, 2, 64, 64), rot={"dims": 64, "base": 5e4}), "right": {"heads": 4, "kv_heads": 2, "dim": 32, "vdim": 32, "conv": 4}}
    parts.check_parallel(ops, "cuda", dtype, 128, m, [140, 2, 33], seed=10)


# ---------------------------------------------------------------- weights made so that a fault shows
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m", [attention(2, 1, 8, 8, scale=1.0), attention(4, 2, 64, 64, scale=1.0)])
@pytest.mark.parametrize("loud", [5, 15, 16, 31, 32])
def test_one_far_key_among_hundreds(ops, dtype, m, loud):
    """One key that every head answers to, far back and on both sides of page borders (pages of 16), in a prompt's
    portions (every attention kernel form: the float32 kernel, mma.sync tiles, tcgen05 at head size 64, split decode)."""
    W = 16
    w, h = parts.loud_key(W, m, 900, loud, seed=1)
    want = parts.check_attention(ops, "cuda", dtype, W, m, None, weights=w, hs=[h], ps=16,
                                 ways=("whole", "decode", (0.5, 0.5), (0.02, 0.98)))
    if loud == 5:
        quiet = plain.grouped_attention(torch.cat([h[:5], h[6:]]).double(), {k: v.double() for k, v in w.items()}, "a.", m, 1e-5, True)
        assert (want[-1] - quiet[-1]).abs().max() > 0.05, "the far key does not show"


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_large_sink_takes_the_weight(ops, dtype):
    """sink = 12 against scores near zero: every output shrinks by about n / (n + e^12); leaving the sink out, counting it
    per split or scaling it would show at once."""
    W, m = 16, attention(2, 1, 16, 16, scale=0.25)
    w = parts.attention_weights(W, m, seed=2)
    for name in ("a.q", "a.k"):
        w[name] = w[name] * 0.01
    w["a.sink"][:] = 12.0
    h = parts.rand(700, W, seed=3)
    want = parts.check_attention(ops, "cuda", dtype, W, m, None, weights=w, hs=[h], ps=16, ways=("whole", "decode", (0.3, 0.7)))
    assert want.abs().max() < 0.05


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_far_token_through_the_delta_state(ops, dtype):
    W, m = 16, {"heads": 2, "kv_heads": 1, "dim": 32, "vdim": 8, "conv": 2}
    w = parts.delta_weights(W, m, seed=4, a_log=-9.0)
    w["d.b"] = w["d.b"] * 0.0
    h = parts.rand(300, W, seed=8)
    want = parts.check_delta(ops, "cuda", dtype, W, m, None, weights=w, hs=[h], ways=("whole", "decode", ("every", 2)), scale_tol=4.0)
    h2 = h.clone()
    h2[0] = -h2[0]
    other = plain.gated_delta(h2.double(), {k: v.double() for k, v in w.items()}, "d.", m, 1e-5)
    assert (want[-1] - other[-1]).abs().max() > 1e-3, "the first token does not show"


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


def requests_of(folders, name, dtype, lengths=None, seed=None):
    """float32 takes any request; bfloat16 takes requests on which no router has a close call."""
    hf = CASES[name][0]
    lengths = lengths or LENGTHS[name]
    seed = ord(name) if seed is None else seed
    if dtype == "float32":
        return requests_for(hf["vocab"], lengths, seed=seed)
    return clear_requests(folders[name], hf["vocab"], lengths, seed=seed)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("schedule", ["whole", "tail", "portions", "mixed"])
def test_schedule_matches_plain(folders, name, dtype, schedule):
    reqs = requests_of(folders, name, dtype)
    steps, max_tokens = getattr(schedules, schedule)(reqs)
    block = 8 if name == "B" else 16
    outputs, rp = replay(folders[name], dtype, steps, max_tokens, block_size=block)
    got = schedules.collect(steps, outputs)
    for rid, toks in reqs.items():
        close(got[rid], plain_logits(folders[name], toks), dtype, f"{schedule}/{name}/{rid}", rounding_of(folders[name], toks, dtype))
    if schedule == "tail":
        assert rp.runner.num_graph_steps > 0, "decode steps replay graphs: every part of the model can be captured"


@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("schedule", ["tail", "mixed"])
def test_bfloat16_against_the_float32_engine(folders, name, schedule):
    reqs = requests_of(folders, name, "bfloat16")
    steps, max_tokens = getattr(schedules, schedule)(reqs)
    a, _ = replay(folders[name], "float32", steps, max_tokens)
    b, _ = replay(folders[name], "bfloat16", steps, max_tokens)
    a, b = schedules.collect(steps, a), schedules.collect(steps, b)
    for rid, toks in reqs.items():
        close(b[rid], a[rid], "bfloat16", f"{schedule}/{name}/{rid}", rounding_of(folders[name], toks, "bfloat16"))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_graph_and_eager_decode_agree(folders, dtype):
    reqs = requests_of(folders, "A", dtype, (66, 90), seed=5)
    steps, max_tokens = schedules.tail(reqs, last=45)
    a, rp_a = replay(folders["A"], dtype, steps, max_tokens)
    b, rp_b = replay(folders["A"], dtype, steps, max_tokens, enforce_eager=True)
    assert rp_a.runner.num_graph_steps > 0 and rp_b.runner.num_graph_steps == 0
    for k in a:
        close(a[k], b[k], dtype, f"graph vs eager step {k}")


def test_long_decoding(folders):
    """Three hundred tokens one by one behind a short prompt, beside a second request that does the same; the
    temperature of case C's queries steps every 16 positions on the way."""
    for name in ("B", "C"):
        for dtype in ("float32", "bfloat16"):
            reqs = requests_of(folders, name, dtype, (330, 311), seed=12)
            steps, max_tokens = schedules.mixed(reqs, live=2, seed=3, prompt_fraction=0.08)
            outputs, _ = replay(folders[name], dtype, steps, max_tokens, block_size=8, slots=2)
            got = schedules.collect(steps, outputs)
            for rid, toks in reqs.items():
                close(got[rid], plain_logits(folders[name], toks), dtype, f"long decoding {name}/{dtype}/{rid}",
                      rounding_of(folders[name], toks, dtype))


def test_first_tokens(folders):
    """Requests of one and two tokens, alone and in one batch."""
    for name in ("A", "B", "C"):
        reqs = requests_for(CASES[name][0]["vocab"], (1, 2, 1, 2), seed=3)
        steps = [{"step": 0, "entries": [{"id": k, "tokens": t, "want": list(range(len(t)))} for k, t in reqs.items()], "end": list(reqs)}]
        outputs, _ = replay(folders[name], "float32", steps, 256)
        got = schedules.collect(steps, outputs)
        for rid, toks in reqs.items():
            close(got[rid], plain_logits(folders[name], toks), "float32", f"first tokens {name}/{rid}")


@pytest.mark.parametrize("seed", range(10))
def test_generated_configurations(tmp_path, seed):
    hf = generated_case(100 + seed)
    folder = make_folder(tmp_path, hf, seed)
    for dtype in ("float32", "bfloat16"):
        lengths = (2, 50, 21, 70, 9, 130)
        reqs = requests_for(hf["vocab"], lengths, seed=seed) if dtype == "float32" else clear_requests(folder, hf["vocab"], lengths, seed=seed)
        steps, max_tokens = schedules.mixed(reqs, live=3, seed=seed)
        outputs, _ = replay(folder, dtype, steps, max_tokens, slots=3)
        got = schedules.collect(steps, outputs)
        for rid, toks in reqs.items():
            close(got[rid], plain_logits(folder, toks), dtype, f"generated {seed}/{dtype}/{rid}", rounding_of(folder, toks, dtype))


@pytest.mark.parametrize("seed", [6, 10, 13])
def test_wide_generated_configurations(tmp_path, seed):
    """Drawn configurations at widths of 256 to 512 under a mixed schedule, float32 against the plain model and bfloat16
    against the float32 engine (which is measured against the plain model in the same test)."""
    hf = wide_case(seed)
    folder = make_folder(tmp_path, hf, seed)
    reqs = clear_requests(folder, hf["vocab"], (3, 90, 1, 33, 140), seed=seed)
    steps, max_tokens = schedules.mixed(reqs, live=4, seed=seed)
    a, _ = replay(folder, "float32", steps, max_tokens)
    b, _ = replay(folder, "bfloat16", steps, max_tokens)
    a, b = schedules.collect(steps, a), schedules.collect(steps, b)
    for rid, toks in reqs.items():
        close(a[rid], plain_logits(folder, toks), "float32", f"wide {seed}/float32/{rid}", rounding_of(folder, toks, "float32"))
        close(b[rid], a[rid], "bfloat16", f"wide {seed}/bfloat16/{rid}", rounding_of(folder, toks, "bfloat16"))


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


def test_trace_runner_as_a_program(folders, tmp_path):
    """bin/trace_run on case B: two requests in portions and single tokens, the files it writes against the plain model."""
    import json
    reqs = requests_for(CASE_B["vocab"], (40, 23), seed=9)
    steps, max_tokens = schedules.mixed(reqs, live=2, seed=1)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folders["B"], "--dtype", "float32", "--out",
                        str(out), "--max-tokens", str(max_tokens), "--max-requests", "2"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [ln for ln in p.stdout.splitlines() if ln.startswith("done")] == [f"done {s['step']}" for s in steps]
    vocab = CASE_B["vocab"]
    outputs = {s["step"]: np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, vocab) for s in steps
               if any(e["want"] for e in s["entries"])}
    got = schedules.collect(steps, outputs)
    for rid, toks in reqs.items():
        close(got[rid], plain_logits(folders["B"], toks), "float32", f"trace_run {rid}")
    assert math.isfinite(float(got["r0"].sum()))
