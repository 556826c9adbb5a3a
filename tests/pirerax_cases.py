"""Small Pirerax configurations for the tests, which differ from each other in every size, constant and order of
layers, and helpers to write their folders with random weights and to ask the plain model.

The weights are drawn here so that a fault shows: sinks of the size of the scores, decays between about 0.4 and 0.99
per token, beta away from 0 and 1, convolution taps of weight, norm weights away from 1; the delta rule's queries lean
on their keys (see `draw_weights`).
"""

from __future__ import annotations

import random

import numpy as np
import torch

from paged_llm_b200.config.registry import parse_model_config
from paged_llm_b200.models.causal_lm import build_model
from tests import plain_pirerax
from tests.rokarax_cases import make_folder as _write_folder
from tests.rokarax_cases import read_folder  # noqa: F401  (re-exported)


def attention(heads, kv, dim, vdim, scale=None, q_temp=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": dim ** -0.5 if scale is None else scale}
    if q_temp is not None:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return m


def latent(heads, dim, rot_dim, vdim, kv_rank, base=10000.0, scale=None):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
            "scale": (dim + rot_dim) ** -0.5 if scale is None else scale, "rot": {"dims": rot_dim, "base": base}}


def parallel(lft, dims, base, heads, kv, dim, vdim, conv):
    return {"left": dict(lft, rot={"dims": dims, "base": base}),
            "right": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}}


def moe(ff, limit, experts, top, groups=None):
    router = {"experts": experts, "top": top}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": router}


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


# A: starts with plain attention whose temperature steps every 4 positions; values longer than keys; a parallel layer
# with as many kv heads as query heads, a full rotation, two q/k heads for four value heads of the delta rule, three
# taps; latent attention whose cached head (24 + 8) pads to 32; the last layer has no feed-forward and no temperature.
CASE_A = {
    "architecture": "Pirerax", "vocab": 131, "width": 64, "norm": {"eps": 1e-5},
    "layers": [
        layer("attention", attention(4, 2, 16, 24, q_temp=(0.5, 4)), moe(40, 1.0, 6, 2, (3, 2))),
        layer("parallel", parallel(attention(4, 4, 32, 16, scale=0.2), 32, 100.0, 4, 2, 8, 16, 3), moe(24, 2.5, 6, 3, (2, 1))),
        layer("latent_attention", latent(3, 16, 8, 24, 24, base=500.0), moe(40, 1.0, 6, 2, (3, 2))),
        layer("attention", attention(2, 1, 32, 16, scale=0.3), None),
    ],
}

# B: starts with latent attention; one kv head for six query heads; a convolution of one tap (no history) and one of
# five; one expert per token out of one group; three of five experts without groups; key sizes of the delta rule
# that fill neither the lanes of a column (24, 40) nor the columns of a block (8, 20).
CASE_B = {
    "architecture": "Pirerax", "vocab": 77, "width": 96, "norm": {"eps": 1e-6},
    "layers": [
        layer("latent_attention", latent(2, 32, 16, 16, 40, base=1e6, scale=0.11), moe(16, 7.0, 4, 1, (1, 1))),
        layer("parallel", parallel(attention(6, 1, 16, 32), 8, 1e4, 2, 2, 24, 8, 1), moe(56, 0.75, 5, 3)),
        layer("parallel", parallel(attention(2, 2, 48, 16, scale=0.1), 2, 50.0, 3, 1, 40, 20, 5), None),
    ],
}

# C: starts with a parallel layer; heads of 64 (the tensor-core prefill kernels); eight query heads on two kv heads;
# four of eight experts out of two of four groups; a temperature that steps every 16 positions with a large factor;
# a wide latent (64 + 32 -> 96).
CASE_C = {
    "architecture": "Pirerax", "vocab": 300, "width": 128, "norm": {"eps": 1e-5},
    "layers": [
        layer("parallel", parallel(attention(2, 2, 64, 64), 16, 3000.0, 2, 1, 64, 32, 2), moe(64, 1.5, 8, 4, (4, 2))),
        layer("attention", attention(8, 2, 16, 16, q_temp=(1.5, 16)), moe(32, 3.0, 8, 1, (4, 1))),
        layer("latent_attention", latent(4, 48, 32, 48, 64, base=2e4), moe(64, 1.5, 8, 4, (4, 2))),
    ],
}

CASES = {"A": (CASE_A, 41), "B": (CASE_B, 42), "C": (CASE_C, 43)}


def generated_case(seed: int) -> dict:
    """A configuration drawn from a seed: widths, head counts and sizes, rotations, the delta rule's sizes, the experts,
    their groups and the order of layers all vary, within what the design allows."""
    rng = random.Random(seed)
    width = rng.choice([48, 64, 96, 160])
    layers = []
    for _ in range(rng.randint(2, 4)):
        kind = rng.choice(["attention", "latent_attention", "parallel"])
        if kind == "attention":
            kv, dim = rng.choice([1, 2, 3]), rng.choice([8, 16, 24, 64])
            m = attention(kv * rng.choice([1, 2, 4]), kv, dim, rng.choice([dim, 8, 40]), scale=rng.choice([0.7, 1.0, 1.4]) * dim ** -0.5,
                          q_temp=rng.choice([None, (0.5, 64), (0.25, 3), (2.0, 10)]))
        elif kind == "latent_attention":
            rot = rng.choice([2, 8, 16])
            m = latent(rng.choice([1, 2, 5]), rng.choice([8, 16, 40]), rot, rng.choice([8, 16, 24]), rng.choice([8, 24, 48]),
                       base=rng.choice([100.0, 2e4, 1e6]))
        else:
            kv, dim = rng.choice([1, 2]), rng.choice([16, 32, 64])
            g = rng.choice([1, 2])
            m = parallel(attention(kv * rng.choice([1, 2, 4]), kv, dim, rng.choice([dim, 16, 48])),
                         rng.choice([dim, dim // 2, 2]), rng.choice([100.0, 5e4]),
                         g * rng.choice([1, 2, 3]), g, rng.choice([4, 8, 20, 32, 72]), rng.choice([8, 16, 24, 48]),
                         rng.choice([1, 2, 3, 4, 6]))
        mlp = None
        if rng.random() < 0.8:
            count = rng.choice([1, 2, 3, 4])
            per = rng.choice([1, 2, 3])
            keep = rng.randint(1, count)
            groups = rng.choice([None, (count, keep)])
            allowed = count * per if groups is None else keep * per
            mlp = moe(rng.choice([8, 24, 64]), rng.choice([0.5, 1.5, 7.0]), count * per, rng.randint(1, min(allowed, 4)), groups)
        layers.append(layer(kind, m, mlp))
    return {"architecture": "Pirerax", "vocab": rng.choice([50, 131, 300, 777]), "width": width,
            "norm": {"eps": rng.choice([1e-6, 1e-5])}, "layers": layers}


def wide_case(seed: int) -> dict:
    """A drawn configuration at widths of 256 to 512 with heads of 32 to 128, three to five layers: the sizes at which the
    tensor-core kernels, four-element accesses and the larger builds of the attention kernels run."""
    rng = random.Random(seed)
    layers = []
    for _ in range(rng.randint(3, 5)):
        kind = rng.choice(["attention", "latent_attention", "parallel"])
        if kind == "attention":
            kv, dim = rng.choice([1, 2, 4]), rng.choice([32, 64, 128])
            m = attention(kv * rng.choice([1, 2, 4]), kv, dim, rng.choice([dim, 48, 96]), scale=rng.choice([0.8, 1.0]) * dim ** -0.5,
                          q_temp=rng.choice([None, (0.5, 64), (0.3, 32)]))
        elif kind == "latent_attention":
            m = latent(rng.choice([2, 4, 8]), rng.choice([32, 64, 96]), rng.choice([16, 32, 64]), rng.choice([32, 64, 96]),
                       rng.choice([64, 96, 128, 160]), base=rng.choice([1e4, 2e4, 5e5]))
        else:
            kv, dim, g = rng.choice([1, 2, 4]), rng.choice([32, 64, 128]), rng.choice([1, 2, 4])
            m = parallel(attention(kv * rng.choice([1, 2, 4]), kv, dim, rng.choice([dim, 64, 96])), rng.choice([dim, dim // 2, 16]),
                         rng.choice([1e4, 1e6]), g * rng.choice([1, 2, 4]), g, rng.choice([16, 48, 64, 128]), rng.choice([32, 80, 128]),
                         rng.choice([2, 3, 4]))
        mlp = None
        if rng.random() < 0.9:
            count, per = rng.choice([1, 2, 4]), rng.choice([2, 4])
            keep = rng.randint(1, count)
            groups = rng.choice([None, (count, keep), (count, keep)])
            allowed = count * per if groups is None else keep * per
            mlp = moe(rng.choice([32, 64, 128]), rng.choice([1.0, 1.5, 7.0]), count * per, rng.randint(1, min(allowed, 4)), groups)
        layers.append(layer(kind, m, mlp))
    return {"architecture": "Pirerax", "vocab": rng.choice([320, 1000]), "width": rng.choice([256, 384, 512]),
            "norm": {"eps": rng.choice([1e-6, 1e-5])}, "layers": layers}


def draw_weights(hf_cfg: dict, seed: int) -> dict[str, torch.Tensor]:
    """Every tensor the model expects, in float32 with values that bfloat16 holds exactly."""
    arch, cfg = parse_model_config(hf_cfg)
    specs = build_model(arch.build_spec(cfg)).tensor_specs()
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name in sorted(specs):
        shape = specs[name].draw_shape or specs[name].shape
        r = torch.randn(shape, generator=g)
        if name.endswith(".sink"):
            t = 1.0 + r                                            # of the size of the scores: leaving it out shows
        elif name.endswith(".A_log"):
            t = -3.0 + 3.0 * torch.rand(shape, generator=g)        # exp(A_log) between 0.05 and 1
        elif name.endswith(".dt_bias"):
            t = 0.5 * r
        elif name.endswith(".right.q.conv"):
            t = out[name.replace(".q.conv", ".k.conv")] + 0.15 * r
        elif name.endswith(".conv"):
            t = 0.5 * r
        elif name.endswith(".right.q"):
            # the delta rule's queries lean towards their own keys: the norm behind a nearly empty state keeps only the
            # sign of q . k of the first tokens, which stays away from zero this way also in bfloat16
            t = out[name[:-1] + "k"] + 0.4 * r * (1.2 / np.sqrt(shape[-1]))
        elif "norm" in name or name.endswith(".out"):
            t = 1.0 + 0.2 * r
        elif name == "embed":
            t = 0.5 * r
        elif name.endswith(".router"):
            t = r * (2.0 / np.sqrt(shape[-1]))                     # scores spread over (0, 1)
        else:
            t = r * (1.2 / np.sqrt(shape[-1]))                     # matrices: outputs of the order of their inputs
        out[name] = t.to(torch.bfloat16).float().contiguous()
    return out


def make_folder(path, hf_cfg: dict, seed: int, dtype: str = "bfloat16", weights=None) -> str:
    return _write_folder(path, hf_cfg, seed, dtype, weights if weights is not None else draw_weights(hf_cfg, seed))


def case_folder(tmp_path_factory, name: str) -> str:
    hf, seed = CASES[name]
    return make_folder(tmp_path_factory.mktemp(f"pirerax{name}"), hf, seed)


def plain_logits(folder: str, tokens) -> np.ndarray:
    cfg, w = read_folder(folder)
    with torch.no_grad():
        return plain_pirerax.forward(cfg, w, tokens)[0].to(torch.float32).numpy()


def rounding_error(folder: str, tokens, dtype=torch.float32) -> np.ndarray:
    """Per position, the root mean square over the vocabulary of the difference between the plain model run in `dtype`
    and in float64: what rounding alone does to these weights."""
    cfg, w = read_folder(folder)
    with torch.no_grad():
        exact = plain_pirerax.forward(cfg, w, tokens)[0]
        with plain_pirerax.precision(dtype):
            rounded = plain_pirerax.forward(cfg, w, tokens)[0]
    return (rounded.double() - exact).pow(2).mean(dim=1).sqrt().numpy()


def clear_requests(folder: str, vocab: int, lengths, seed: int = 0, margin: float = 0.02) -> dict[str, list[int]]:
    """Random requests on which no router of the model comes close to a tie (the last kept group and the last chosen
    expert lead the next by `margin` at every token): a bfloat16 engine then chooses the experts the plain model
    chooses, and the two differ by rounding only.  A length for which 60 draws find no such request is shortened."""
    cfg, w = read_folder(folder)
    out = {}
    for i, n in enumerate(lengths):
        while f"r{i}" not in out:
            for attempt in range(60):
                g = torch.Generator().manual_seed(seed * 100003 + i * 401 + attempt)
                toks = torch.randint(0, vocab, (n,), generator=g).tolist()
                margins: list[float] = []
                with torch.no_grad():
                    plain_pirerax.forward(cfg, w, toks, margins)
                if min(margins, default=1.0) >= margin:
                    out[f"r{i}"] = toks
                    break
            else:
                if n <= 2:
                    raise AssertionError("no request without a close call, however short")
                n = max(2, n * 2 // 3)
    return out


def plain_greedy(folder: str, prompt, n: int) -> list[int]:
    cfg, w = read_folder(folder)
    with torch.no_grad():
        return plain_pirerax.greedy_generate(cfg, w, prompt, n)
