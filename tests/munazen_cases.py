"""Small Munazen configurations for the tests, which differ from each other in every size, constant and order of
layers, and helpers to write their folders with random weights and to ask the plain model.

The weights are drawn here so that the vectors that shape the recurrences get values that show a fault: decays close
to one keep far tokens alive, hyper-connection matrices are far from the identity, the activation's four numbers are
all of weight.
"""

from __future__ import annotations

import random

import numpy as np
import torch

from paged_llm_b200.config.registry import parse_model_config
from paged_llm_b200.models.causal_lm import build_model
from tests import plain_munazen
from tests.rokarax_cases import make_folder as _write_folder
from tests.rokarax_cases import read_folder  # noqa: F401  (re-exported)

YARN = {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}


def left(heads, kv, dim, vdim, dims=None, base=10000.0, scaling=None, scale=None):
    rot = {"dims": dim if dims is None else dims, "base": base}
    if scaling is not None:
        rot["scaling"] = scaling
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": dim ** -0.5 if scale is None else scale,
            "rot": rot}


def parallel(lft, width, blocks, conv, left_scale=1.0, right_scale=1.0):
    return {"left": lft, "right": {"width": width, "blocks": blocks, "conv": conv}, "left_scale": left_scale,
            "right_scale": right_scale}


def gla(heads, dim, vdim, tau):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}


def layer(kind, mixer, ff):
    return {"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


# A: two streams, norms in two parts, the first two layers run three times; a partial rotation with YaRN, values
# twice as wide as keys, three blocks of gates, three taps; the linear-attention layer has no feed-forward.
CASE_A = {
    "architecture": "Munazen", "vocab": 131, "width": 64, "norm": {"eps": 1e-5, "groups": 2}, "streams": 2,
    "loop": {"start": 0, "stop": 2, "times": 3},
    "layers": [
        layer("parallel", parallel(left(4, 2, 16, 32, dims=8, scaling=YARN), 48, 3, 3, 0.8, 1.3), 96),
        layer("gla", gla(2, 8, 16, 4.0), None),
        layer("parallel", parallel(left(2, 2, 32, 16, base=500.0, scale=0.3), 40, 1, 2, 1.5, 0.5), 40),
    ],
}

# B: one stream and plain residual sums, norms over the whole row, no loop; starts with linear attention; one kv head
# for six query heads, heads that pad the cache (24 and 40 in 48), a convolution of one tap (no history).
CASE_B = {
    "architecture": "Munazen", "vocab": 77, "width": 96, "norm": {"eps": 1e-6, "groups": 1},
    "layers": [
        layer("gla", gla(3, 16, 32, 16.0), 64),
        layer("parallel", parallel(left(6, 1, 24, 40, dims=12, base=1e6, scaling=dict(YARN, factor=8.0, original=64)), 64, 4, 1), None),
        layer("gla", gla(1, 64, 8, 1.0), 72),
    ],
}

# C: four streams, norms in four parts, all layers run twice; key and value sizes of the linear attention that fill
# neither the lanes of a column nor the columns of a block; as many kv heads as query heads; five taps.
CASE_C = {
    "architecture": "Munazen", "vocab": 300, "width": 128, "norm": {"eps": 1e-5, "groups": 4}, "streams": 4,
    "loop": {"start": 0, "stop": 2, "times": 2},
    "layers": [
        layer("gla", gla(2, 40, 24, 8.0), 100),
        layer("parallel", parallel(left(3, 3, 64, 64, scaling=dict(YARN, factor=2.0)), 96, 2, 5, 1.0, 1.0), 160),
    ],
}

CASES = {"A": (CASE_A, 31), "B": (CASE_B, 32), "C": (CASE_C, 33)}


def generated_case(seed: int) -> dict:
    """A configuration drawn from a seed: widths, head counts and sizes, the rotation, the recurrence's sizes, the
    streams, the norm's parts, the loop and the order of layers all vary, within what the design allows."""
    rng = random.Random(seed)
    width = rng.choice([48, 64, 96, 160, 192])
    layers = []
    for _ in range(rng.randint(2, 4)):
        kind = rng.choice(["parallel", "gla"])
        ff = rng.choice([None, 24, 64, 100])
        if kind == "parallel":
            kv = rng.choice([1, 2, 3])
            dim = rng.choice([8, 16, 24, 48, 64])
            scaling = None
            if rng.random() < 0.6:
                scaling = {"factor": rng.choice([2.0, 4.0, 16.0]), "original": rng.choice([16, 64, 256]),
                           "fast": rng.choice([8.0, 32.0]), "slow": rng.choice([1.0, 2.0])}
            lft = left(kv * rng.choice([1, 2, 4]), kv, dim, rng.choice([dim, 8, 16, 40, 80]),
                       dims=rng.choice([dim, dim, max(2, dim // 2), 2]), base=rng.choice([100.0, 10000.0, 1e6]),
                       scaling=scaling, scale=rng.choice([0.7, 1.0, 1.4]) * dim ** -0.5)
            blocks = rng.choice([1, 2, 3, 4])
            m = parallel(lft, blocks * rng.choice([8, 12, 20, 33]), blocks, rng.choice([1, 2, 3, 4, 6]),
                         rng.choice([0.5, 1.0, 1.2]), rng.choice([0.7, 1.0, 1.1]))
        else:
            m = gla(rng.choice([1, 2, 3, 5]), rng.choice([4, 8, 20, 32, 72]), rng.choice([8, 16, 24, 48]),
                    rng.choice([1.0, 4.0, 16.0]))
        layers.append(layer(kind, m, ff))
    cfg = {"architecture": "Munazen", "vocab": rng.choice([50, 131, 300, 777]), "width": width,
           "norm": {"eps": rng.choice([1e-6, 1e-5]), "groups": rng.choice([g for g in (1, 2, 3, 4, 8) if width % g == 0])},
           "layers": layers}
    streams = rng.choice([None, 1, 2, 3, 5])
    if streams is not None:
        cfg["streams"] = streams
    if rng.random() < 0.7:
        start = rng.randrange(len(layers))
        cfg["loop"] = {"start": start, "stop": rng.randint(start + 1, len(layers)), "times": rng.choice([1, 2, 3])}
    return cfg


def draw_weights(hf_cfg: dict, seed: int) -> dict[str, torch.Tensor]:
    """Every tensor the model expects, in float32 with values that bfloat16 holds exactly."""
    arch, cfg = parse_model_config(hf_cfg)
    specs = build_model(arch.build_spec(cfg)).tensor_specs()
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name in sorted(specs):
        shape = specs[name].draw_shape or specs[name].shape
        r = torch.randn(shape, generator=g)
        if name.endswith(".lam"):
            t = -5.0 + 4.0 * torch.rand(shape, generator=g)        # decays between about 0.5 and 0.99 per token
        elif name.endswith(".a2.b"):
            t = 1.0 + r                                            # sigmoid(z)^(1/tau) close to one for most channels
        elif name.endswith(".b"):
            t = 0.1 * r
        elif name.endswith(".conv"):
            t = 0.5 * r
        elif ".hc" in name and name.endswith(".mix"):
            t = torch.eye(shape[0]) * 0.7 + 0.3 * r
        elif ".hc" in name and name.endswith(".in"):
            t = 0.6 + 0.3 * r
        elif ".hc" in name:
            t = 1.0 + 0.3 * r
        elif name.endswith(".act"):
            t = torch.tensor([1.0, 0.4, 0.2, 0.05]) + 0.05 * r
        elif "norm" in name:
            t = 1.0 + 0.2 * r
        elif name == "embed":
            t = 0.5 * r
        elif name.endswith(".mix.q") and name[:-1] + "k" in out:
            # linear attention: queries that lean towards their own keys, so that q . k of the first tokens, whose sign
            # is all that the norm behind a nearly empty state keeps, stays away from zero also in bfloat16
            t = out[name[:-1] + "k"] + 0.5 * r * (1.2 / np.sqrt(shape[-1]))
        else:
            t = r * (1.2 / np.sqrt(shape[-1]))                     # matrices: outputs of the order of their inputs
        out[name] = t.to(torch.bfloat16).float().contiguous()
    return out


def make_folder(path, hf_cfg: dict, seed: int, dtype: str = "bfloat16", weights=None) -> str:
    return _write_folder(path, hf_cfg, seed, dtype, weights if weights is not None else draw_weights(hf_cfg, seed))


def case_folder(tmp_path_factory, name: str) -> str:
    hf, seed = CASES[name]
    return make_folder(tmp_path_factory.mktemp(f"munazen{name}"), hf, seed)


def plain_logits(folder: str, tokens) -> np.ndarray:
    cfg, w = read_folder(folder)
    with torch.no_grad():
        return plain_munazen.forward(cfg, w, tokens)[0].to(torch.float32).numpy()


def rounding_error(folder: str, tokens, dtype=torch.float32) -> np.ndarray:
    """Per position, the root mean square over the vocabulary of the difference between the plain model run in `dtype`
    and in float64: what rounding alone does to these weights (a norm over a nearly empty state of the linear
    attention, or over a query and key that nearly cancel, magnifies it; in bfloat16 the sign of the first token's
    query-key product, which is all that the norm behind the linear attention keeps of it, can turn)."""
    cfg, w = read_folder(folder)
    with torch.no_grad():
        exact = plain_munazen.forward(cfg, w, tokens)[0]
        with plain_munazen.precision(dtype):
            rounded = plain_munazen.forward(cfg, w, tokens)[0]
    return (rounded.double() - exact).pow(2).mean(dim=1).sqrt().numpy()


def plain_greedy(folder: str, prompt, n: int) -> list[int]:
    cfg, w = read_folder(folder)
    with torch.no_grad():
        return plain_munazen.greedy_generate(cfg, w, prompt, n)
