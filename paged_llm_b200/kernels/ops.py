"""The kernel library as the parts see it: `CudaOps`.

Every method launches hand-written CUDA kernels of `csrc/` (compiled for
sm_100a at first use, called through ctypes on the current stream) on torch
tensors.  There is no CPU fallback: without a CUDA device or without nvcc the
constructor raises.  The only library calls are the bfloat16 matrix products
(cuBLAS through torch), where the reference's engine also calls a library
(`nn.Linear`, pagedllm/model/llama.py:141-144); float32 products use this
package's own CUDA-core kernel so that no reduced-precision mode can slip in.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p

import numpy as np
import torch

from ..csrc import build
from . import plan as planning
from .errors import KernelError

PL_F32, PL_BF16 = 0, 1
_DTYPE_CODE = {torch.float32: PL_F32, torch.bfloat16: PL_BF16}


class LazyNorm:
    """RMSNorm(x) * weight that no kernel has formed yet: the product that comes next
    normalises while it loads.  `part` holds the sums of squares of x that the product
    in front left (per 16 columns and token)."""

    def __init__(self, x: torch.Tensor, part: torch.Tensor, weight: torch.Tensor, eps: float):
        self.x, self.part, self.weight, self.eps = x, part, weight, eps
        self.shape = x.shape
        self.dtype = torch.bfloat16


class AttnParams(ctypes.Structure):
    _fields_ = [
        ("q", c_void_p), ("kv", c_void_p), ("out", c_void_p), ("block_table", c_void_p), ("cu_q", c_void_p),
        ("k_lens", c_void_p), ("work", c_void_p), ("scratch", c_void_p), ("scratch_floats", c_longlong),
        ("q_stride", c_int), ("out_stride", c_int), ("bt_stride", c_int), ("n_work", c_int), ("max_splits", c_int),
        ("nh", c_int), ("nkv", c_int), ("d", c_int), ("ps", c_int), ("window", c_int), ("is_small", c_int),
        ("scale", c_float), ("ps_shift", c_int), ("counters", c_void_p), ("num_pages", c_int), ("cluster", c_int),
        ("softcap", c_float), ("slopes", c_void_p), ("rope_table", c_void_p), ("rope_len", c_int),
        ("pad_seqs", c_int), ("pad_to", c_int), ("chunk", c_int), ("dist_bias", c_void_p), ("dist_len", c_int),
        ("sink", c_void_p),
    ]


ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}       # codes of the gate's activation in the kernels
# the routed experts' kernels also take the clamped form with a limit L:
# g = min(gate, L), u = clamp(up, -L, L), g * sigmoid(1.702 g) * (u + 1)
EXPERT_ACTIVATIONS = dict(ACTIVATIONS, swish_clamped=2)


def attention_plan_key(num_heads: int, num_kv_heads: int, window, head_dim: int, chunk=None) -> tuple:
    """What a step's attention work lists depend on: (query heads per kv head, kv heads, window, head size) and,
    for a chunked mask, the chunk."""
    key = (num_heads // num_kv_heads, num_kv_heads, window, head_dim)
    return key + (chunk,) if chunk else key


_LIBS: dict[str, ctypes.CDLL] = {}


def load_module(name: str) -> ctypes.CDLL:
    """The compiled module `name`, built first if need be."""
    lib = _LIBS.get(name)
    if lib is None:
        path = build.build_module(name)
        lib = ctypes.CDLL(path)
        lib.pl_last_error.restype = ctypes.c_char_p
        _LIBS[name] = lib
    return lib


# Every wait inside a kernel (on an mbarrier of a TMA ring or of tcgen05) is bounded; a wait that
# gives up adds one to a counter of its module, which these exports read.
_TIMEOUT_EXPORTS = ("pl_gemm_skinny_timeouts", "pl_gemm_tc_timeouts", "pl_attention_tc_timeouts")


def _check(lib, rc: int) -> None:
    if rc != 0:
        raise KernelError(lib.pl_last_error().decode())


def head_dim_build(d: int) -> int:
    if d % 16 or d <= 0:
        raise KernelError(f"head_dim={d}: the attention kernels take head sizes in steps of 16")
    for b in build.HEAD_DIM_BUILDS:
        if d <= b:
            return b
    raise KernelError(f"head_dim={d} is larger than the largest attention build ({build.HEAD_DIM_BUILDS[-1]})")


class CudaOps:
    supports_graphs = True
    SMALL_ROWS = 16
    MIN_SPLIT_KEYS = 128
    MAX_CLUSTER = int(os.environ.get("PAGED_LLM_B200_MAX_CLUSTER", "8"))     # blocks of a decode-attention cluster
    MAX_SPLITS = 32

    def __init__(self, device="cuda"):
        self.device = torch.device(device)
        if self.device.type != "cuda" or not torch.cuda.is_available():
            raise KernelError("paged_llm_b200 runs on a CUDA device only (no CPU path); none is available")
        major, minor = torch.cuda.get_device_capability(self.device)
        if major < 10:
            raise KernelError(f"the kernels are built for sm_100a (B200); this device is sm_{major}{minor}")
        self.core = load_module("core")
        self.compute_dtype = torch.bfloat16
        self.num_sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        self._scratch: list[torch.Tensor] = []
        self._pinned_stream = None
        self._attn_lib = None
        self._attn_fn = None
        self.launches = 0                 # kernels of this package launched so far
        self.use_skinny = True            # few-token products on this package's weight-streaming kernel
        # Many tokens: this package's tcgen05 kernel (pairs of blocks on 256 x 256 tiles, fused epilogues) where it is at least
        # as fast as the library product followed by the elementwise kernel.  Measured: the gate/up product
        # with SiLU-mul from 2,048 tokens on (77 us against 87 us, timed alone); the narrower products and fewer
        # tokens are faster through the library.  PAGED_LLM_B200_GEMM_TC lists the kinds ("silu", "add", "plain", "all",
        # "" for none) to run on it from 129 tokens on instead.
        tc_for = os.environ.get("PAGED_LLM_B200_GEMM_TC")
        self.gemm_tc_min_tokens = 2048 if tc_for is None else 129
        tc_for = "silu,moe" if tc_for is None else tc_for
        self.gemm_tc_for = {"silu", "add", "plain", "moe"} if tc_for == "all" else {t for t in tc_for.split(",") if t}
        # (token, expert) pairs of a step from which the routed experts' products take the grouped tcgen05 form
        self.moe_tc_min_pairs = 2048
        self.cluster_attention = os.environ.get("PAGED_LLM_B200_NO_CLUSTER") is None   # decode attention as clusters
        # decode steps of more than 16 tokens: rotary positions and the cache write inside the attention kernel
        self.rope_in_attention = os.environ.get("PAGED_LLM_B200_NO_ROPE_IN_ATTENTION") is None
        # long work-list ranges of decode attention in a ring of three 64-key tiles (head sizes up to 64)
        self.deep_list = os.environ.get("PAGED_LLM_B200_NO_DEEP_LIST") is None
        # lanes that share a column of the delta rule's state (8 unless 16 or 32 is asked for, for measurements)
        self.delta_lanes = int(os.environ.get("PAGED_LLM_B200_DELTA_LANES", "0"))
        self._argmax_ws = None            # (packed winners, arrival counters) of the multi-block argmax
        self._sample_dev = None           # the sampling parameters of a step on the device, and their pinned ring
        self._sample_ring: list = []
        self._sample_keep: list = []
        self._sample_pos = 0
        self._argmax_keep: list = []
        self._attn_counters = None        # arrival counters of the split merge inside the attention kernel
        self._attn_counters_keep: list = []
        self._norm_part = None            # sums of squares that an adding product leaves for the next one
        self._norm_part_keep: list = []
        # the library matrix products must not reduce in bfloat16
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False

    def set_compute_dtype(self, dtype: torch.dtype) -> None:
        if dtype not in _DTYPE_CODE:
            raise KernelError(f"compute dtype {dtype} is not supported (bfloat16 or float32)")
        self.compute_dtype = dtype

    @property
    def _stream(self):
        if self._pinned_stream is not None:
            return self._pinned_stream
        return c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def pin_stream(self) -> None:
        """Looks the current stream up once and launches on it until `unpin_stream` (asking torch for the
        current stream costs more than the rest of a launch; the step function pins it for the length of a
        step and again wherever it changes the stream itself)."""
        self._pinned_stream = c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def unpin_stream(self) -> None:
        self._pinned_stream = None

    @staticmethod
    def _p(t: torch.Tensor | None):
        return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)

    def _code(self, t: torch.Tensor) -> int:
        try:
            return _DTYPE_CODE[t.dtype]
        except KeyError:
            raise KernelError(f"tensor of dtype {t.dtype} where float32 or bfloat16 is expected") from None

    def kernel_timeouts(self) -> int:
        """Bounded waits inside kernels that gave up since the process started, over all loaded
        modules.  Reading the counters waits for the device."""
        total = 0
        for lib in list(_LIBS.values()):
            for name in _TIMEOUT_EXPORTS:
                try:
                    fn = getattr(lib, name)
                except AttributeError:
                    continue
                n = int(fn())
                if n < 0:
                    raise KernelError(f"{name}: the counter could not be read")
                total += n
        return total

    def check_kernels(self) -> None:
        """Raises if a kernel gave up on a wait: what it computed afterwards is not to be trusted."""
        n = self.kernel_timeouts()
        if n:
            raise KernelError(f"{n} bounded wait(s) inside kernels gave up (a TMA copy or a tensor-core product "
                              "never signalled its barrier); results since the last check may be wrong")

    def copy_h2d(self, dst: torch.Tensor, src: torch.Tensor, nbytes: int) -> None:
        """Asynchronous copy of `nbytes` from pinned host memory to the device on the current stream."""
        _check(self.core, self.core.pl_copy_h2d(self._p(dst), self._p(src), c_longlong(nbytes), self._stream))

    def fill_normal(self, out: torch.Tensor, seed: int, key: int, mean: float = 0.0, std: float = 1.0) -> torch.Tensor:
        """out[...] = mean + std * N(0, 1) from the counter-based stream (seed, key): the values depend
        on nothing else.  For random weights drawn on the device."""
        assert out.is_contiguous() and out.is_cuda
        _check(self.core, self.core.pl_fill_normal(self._p(out), self._code(out), c_longlong(out.numel()),
                                                   ctypes.c_ulonglong(seed & (2 ** 64 - 1)),
                                                   ctypes.c_ulonglong(key & (2 ** 64 - 1)), c_float(mean), c_float(std),
                                                   self._stream))
        self.launches += 1
        return out

    # ---- embedding, norms, activation ------------------------------------------
    def embedding(self, table: torch.Tensor, ids: torch.Tensor, scale: float = 1.0, copies: int = 1) -> torch.Tensor:
        """Rows of `table` as the float32 stream, each element times `scale`; with `copies` > 1 every row is laid
        out that many times side by side (a model of several residual streams)."""
        T, (V, H) = ids.numel(), table.shape
        if copies > 1:
            lib = load_module("streams")
            out = torch.empty((T, H * copies), dtype=torch.float32, device=self.device)
            _check(lib, lib.pl_embedding_copies(self._p(table), self._code(table), self._p(ids), self._p(out), T, H, V,
                                                c_float(scale), copies, self._stream))
            self.launches += 1
            return out
        out = torch.empty((T, H), dtype=torch.float32, device=self.device)
        _check(self.core, self.core.pl_embedding(self._p(table), self._code(table), self._p(ids), self._p(out),
                                                 T, H, V, c_float(scale), self._stream))
        self.launches += 1
        return out

    def rms_norm(self, x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
        return self._norm(x, None, w, eps)

    def add_rms_norm(self, x: torch.Tensor, branch: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
        return self._norm(x, branch, w, eps)

    def _norm(self, x, branch, w, eps):
        assert x.dtype == torch.float32 and x.is_contiguous(), "the residual stream is contiguous float32"
        rows, H = x.shape
        y = torch.empty((rows, H), dtype=self.compute_dtype, device=self.device)
        if branch is not None:
            assert branch.shape == x.shape and branch.is_contiguous()
        bcode = self._code(branch) if branch is not None else PL_F32
        _check(self.core, self.core.pl_rmsnorm(self._p(x), self._p(branch), bcode, self._p(w), self._code(w),
                                               self._p(y), self._code(y), rows, H, c_float(eps), self._stream))
        self.launches += 1
        return y

    def dyt(self, x: torch.Tensor | None, branch: torch.Tensor | None, post, pre, out_dtype=None):
        """Dynamic tanh around the residual sum, one kernel: x += post(branch) in place (x the float32 stream),
        then pre(x) in the compute dtype.  `post` and `pre` are (alpha, weight, bias) float32 tensors on the device or
        None: without `post` the branch is added as it is; without `pre` nothing is returned.  With x None the result
        is pre(post(branch)): a norm of a tensor that is not the stream."""
        src = x if x is not None else branch
        rows, H = src.shape
        assert src.is_contiguous() and (x is None or x.dtype == torch.float32)
        if branch is not None:
            assert branch.shape == src.shape and branch.is_contiguous()
        y = torch.empty((rows, H), dtype=out_dtype or self.compute_dtype, device=self.device) if pre is not None else None
        po = post or (None, None, None)
        pr = pre or (None, None, None)
        for t in (*po, *pr):
            assert t is None or (t.dtype == torch.float32 and t.is_contiguous())
        _check(self.core, self.core.pl_dyt(self._p(x), self._p(branch), self._code(branch) if branch is not None else PL_F32,
                                           self._p(po[0]), self._p(po[1]), self._p(po[2]), self._p(pr[0]), self._p(pr[1]),
                                           self._p(pr[2]), self._p(y), self._code(y) if y is not None else PL_F32,
                                           c_longlong(rows), H, self._stream))
        self.launches += 1
        return y

    def silu_mul(self, gate_up: torch.Tensor) -> torch.Tensor:
        return self.act_mul(gate_up, "silu")

    def act_mul(self, gate_up: torch.Tensor, activation: str = "silu") -> torch.Tensor:
        """act(gate) * up for rows [gate | up]; the activation is "silu" or "gelu_tanh", in float32 inside."""
        rows, two_i = gate_up.shape
        assert gate_up.is_contiguous() and two_i % 2 == 0
        out = torch.empty((rows, two_i // 2), dtype=gate_up.dtype, device=self.device)
        _check(self.core, self.core.pl_act_mul(self._p(gate_up), self._p(out), self._code(gate_up), rows, two_i // 2,
                                               ACTIVATIONS[activation], self._stream))
        self.launches += 1
        return out

    def add_rows(self, x: torch.Tensor, branch=None, extra: torch.Tensor | None = None) -> torch.Tensor:
        """x += branch + extra in place, in float32 (x is the residual stream; either addend may be None)."""
        assert x.dtype == torch.float32 and x.is_contiguous()
        if branch is not None:
            assert branch.shape == x.shape and branch.is_contiguous()
        if extra is not None:
            assert extra.shape == x.shape and extra.is_contiguous() and extra.dtype == torch.float32
        if branch is None and extra is None:
            return x
        _check(self.core, self.core.pl_add_rows(self._p(x), self._p(branch), self._code(branch) if branch is not None else PL_F32,
                                                self._p(extra), c_longlong(x.numel()), self._stream))
        self.launches += 1
        return x

    def gather_rows(self, x: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
        n, H = idx.numel(), x.shape[1]
        assert x.is_contiguous()
        out = torch.empty((n, H), dtype=x.dtype, device=self.device)
        _check(self.core, self.core.pl_gather_rows(self._p(x), self._p(idx), self._p(out), self._code(x), n, H,
                                                   x.shape[0], self._stream))
        self.launches += 1
        return out

    # ---- matrix products ---------------------------------------------------------
    def materialize(self, h):
        """A tensor for `h`, which may be a `LazyNorm`."""
        if isinstance(h, LazyNorm):
            return self.rms_norm(h.x, h.weight, h.eps)
        return h

    def _norm_args(self, h):
        """(X pointer, row stride, partial sums, norm weight, its dtype code, eps) for a product."""
        if isinstance(h, LazyNorm):
            return (self._p(h.x), h.x.shape[1], self._p(h.part), self._p(h.weight), self._code(h.weight), c_float(h.eps))
        return (self._p(h), h.shape[1], c_void_p(0), c_void_p(0), 0, c_float(0.0))

    def _skinny_ok(self, h, N: int) -> bool:
        """Few tokens: the weight-streaming kernel of this package instead of the library."""
        M, K = h.shape
        return self.use_skinny and h.dtype == torch.bfloat16 and 1 <= M <= 16 and K >= 32 and K % 32 == 0

    def _gemm_tc_ok(self, h, w: torch.Tensor, kind: str) -> bool:
        M, K = h.shape
        return (kind in self.gemm_tc_for and h.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
                and M >= self.gemm_tc_min_tokens
                and K >= 64 and K % 64 == 0 and w.is_contiguous())

    def _gemm_tc(self, h: torch.Tensor, w: torch.Tensor, out, resid, N: int, epi: int) -> None:
        M, K = h.shape
        assert h.stride(1) == 1 and h.stride(0) % 8 == 0
        lib, fn = self.core, self.core.pl_gemm_tc
        _check(lib, fn(self._p(h), h.stride(0), self._p(w), self._p(out), out.shape[1] if out is not None else 0,
                       self._p(resid), M, N, K, epi, self._stream))
        self.launches += 1

    def linear(self, h, w: torch.Tensor, out_float32: bool = False) -> torch.Tensor:
        """h [M, K] @ w[N, K]^T.  float32: this package's CUDA-core kernel; bfloat16 with few
        tokens: this package's weight-streaming kernel; else the library product with
        float32 accumulation.  `h` may be a `LazyNorm`."""
        M, K = h.shape
        N = w.shape[0]
        assert w.shape[1] == K and w.is_contiguous()
        if self._skinny_ok(h, N) and w.dtype == torch.bfloat16:
            x, ldx, part, nw, nwc, eps = self._norm_args(h)
            out = torch.empty((M, N), dtype=torch.float32 if out_float32 else torch.bfloat16, device=self.device)
            _check(self.core, self.core.pl_gemm_skinny(x, ldx, self._p(w), self._p(out), N, M, N, K,
                                                       1 if out_float32 else 0, part, nw, nwc, eps, self._stream))
            self.launches += 1
            return out
        h = self.materialize(h)
        assert h.is_contiguous()
        if self._gemm_tc_ok(h, w, "plain") and N % 8 == 0:
            out = torch.empty((M, N), dtype=torch.float32 if out_float32 else torch.bfloat16, device=self.device)
            self._gemm_tc(h, w, out, None, N, 1 if out_float32 else 0)
            return out
        if h.dtype == torch.float32:
            assert w.dtype == torch.float32
            out = torch.empty((M, N), dtype=torch.float32, device=self.device)
            _check(self.core, self.core.pl_gemm_f32(self._p(h), self._p(w), self._p(out), M, N, K, K, K, N,
                                                    self._stream))
            self.launches += 1
            return out
        assert h.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
        if out_float32:
            return torch.mm(h, w.t(), out_dtype=torch.float32)
        return torch.nn.functional.linear(h, w)

    def linear_add_rms_norm(self, h, w, x, norm_w, eps):
        """x += h @ w^T (float32 stream, in place), then RMSNorm(x) * norm_w.  With few tokens
        the product's epilogue adds and the result is a `LazyNorm` that the next product
        forms while loading; else the product is followed by the fused sum+norm kernel."""
        M, K = h.shape
        N = w.shape[0]
        if not isinstance(h, LazyNorm) and self._skinny_ok(h, N) and N % 16 == 0 and N % 32 == 0:
            assert x.dtype == torch.float32 and x.is_contiguous() and x.shape == (M, N) and h.is_contiguous()
            if self._norm_part is None or self._norm_part.numel() < N:
                self._norm_part_keep.append(self._norm_part)        # captured graphs hold the old address
                self._norm_part = torch.zeros(max(N, 1 << 16), dtype=torch.float32, device=self.device)
            _check(self.core, self.core.pl_gemm_skinny_add(self._p(h), K, self._p(w), self._p(x), M, N, K,
                                                           self._p(self._norm_part), self._stream))
            self.launches += 1
            return LazyNorm(x, self._norm_part, norm_w, eps)
        if (not isinstance(h, LazyNorm) and self._gemm_tc_ok(h, w, "add") and x.dtype == torch.float32
                and x.is_contiguous() and N % 4 == 0):
            self._gemm_tc(h, w, None, x, N, 3)
            return self.rms_norm(x, norm_w, eps)
        return self.add_rms_norm(x, self.linear(h, w), norm_w, eps)

    def gated_silu_linear(self, h, w_gate_up: torch.Tensor) -> torch.Tensor:
        return self.gated_act_linear(h, w_gate_up, "silu")

    def gated_act_linear(self, h, w_gate_up: torch.Tensor, activation: str = "silu") -> torch.Tensor:
        """act(h Wg^T) * (h Wu^T) for W = [Wg; Wu]: one kernel for few tokens, else the
        product followed by the activation kernel."""
        M, K = h.shape
        I = w_gate_up.shape[0] // 2
        if self._skinny_ok(h, 2 * I):
            x, ldx, part, nw, nwc, eps = self._norm_args(h)
            out = torch.empty((M, I), dtype=torch.bfloat16, device=self.device)
            _check(self.core, self.core.pl_gemm_skinny_silu(x, ldx, self._p(w_gate_up), self._p(out), I, M, I, K,
                                                            part, nw, nwc, eps, ACTIVATIONS[activation], self._stream))
            self.launches += 1
            return out
        h = self.materialize(h)
        if self._gemm_tc_ok(h, w_gate_up, "silu") and h.is_contiguous() and I % 8 == 0:
            out = torch.empty((M, I), dtype=torch.bfloat16, device=self.device)
            if activation == "silu":
                self._gemm_tc(h, w_gate_up, out, None, I, 2)
            else:
                _check(self.core, self.core.pl_gemm_tc_act(self._p(h), h.stride(0), self._p(w_gate_up), self._p(out), I, M, I,
                                                           K, ACTIVATIONS[activation], self._stream))
                self.launches += 1
            return out
        return self.act_mul(self.linear(h, w_gate_up), activation)

    def qkv_rope_write(self, h, w_qkv, nh, nkv, d, position, ctx, kv, block_table, write=True,
                       value_from_key=False) -> torch.Tensor:
        """The fused q/k/v projection with rotary positions applied to q and k and k, v
        written to the cache.  Returns the [T, (nh + 2 nkv) d] buffer whose first nh*d
        columns are the rotated queries.  `value_from_key`: there is no value projection (w_qkv
        stacks q and k only, the buffer is [T, (nh + nkv) d]) and the value written beside a key
        is that key as projected, before its rotation."""
        M, K = h.shape
        N = (nh + (1 if value_from_key else 2) * nkv) * d
        assert w_qkv.shape[0] == N
        fusable = (self._skinny_ok(h, N) and position is not None and position.pairing == "half"
                   and position.rotary_dim == d and M == ctx.num_tokens)
        if not fusable:
            qkv = self.linear(h, w_qkv)
            self.rope_kv_write(qkv, nh, nkv, d, position, ctx, kv, block_table, write=write,
                               value_from_key=value_from_key)
            return qkv
        x, ldx, part, nw, nwc, eps = self._norm_args(h)
        qkv = torch.empty((M, N), dtype=torch.bfloat16, device=self.device)
        assert kv.dtype == torch.bfloat16 and kv.is_contiguous()
        _check(self.core, self.core.pl_gemm_skinny_rope(
            x, ldx, self._p(w_qkv), self._p(qkv), N, M, K, nh, nkv, d, self._p(position.table),
            position.table.shape[0], self._p(ctx.positions), self._p(ctx.token_seq), self._p(block_table),
            block_table.shape[1], self._p(kv), kv.shape[0], kv.shape[3], 1 if write else 0, part, nw, nwc, eps,
            1 if value_from_key else 0, self._stream))
        self.launches += 1
        return qkv

    # ---- mixers that are not plain grouped-query attention ----------------------------
    def heads_linear(self, x: torch.Tensor, col0: int, head_stride: int, w: torch.Tensor,
                     out_float32: bool = False) -> torch.Tensor:
        """A product per head: out[t, h, :] = w[h] @ x[t, col0 + h * head_stride : ... + K] for w [heads, N, K];
        returns [T, heads * N].  float32: this package's CUDA-core product, head by head on strided operands;
        bfloat16: the library's batched product."""
        T, ld = x.shape
        nh, N, K = w.shape
        assert x.is_contiguous() and w.is_contiguous() and col0 + (nh - 1) * head_stride + K <= ld and w.dtype == x.dtype
        if x.dtype == torch.float32:
            out = torch.empty((T, nh * N), dtype=torch.float32, device=self.device)
            for h in range(nh):
                _check(self.core, self.core.pl_gemm_f32(c_void_p(x.data_ptr() + 4 * (col0 + h * head_stride)),
                                                        c_void_p(w.data_ptr() + 4 * h * N * K),
                                                        c_void_p(out.data_ptr() + 4 * h * N), T, N, K, ld, K, nh * N,
                                                        self._stream))
                self.launches += 1
            return out
        xv = torch.as_strided(x, (nh, T, K), (head_stride, ld, 1), x.storage_offset() + col0)
        if out_float32:
            return torch.bmm(xv, w.transpose(1, 2), out_dtype=torch.float32).transpose(0, 1).reshape(T, nh * N)
        return torch.bmm(xv, w.transpose(1, 2)).transpose(0, 1).reshape(T, nh * N)

    def normed_qkv_write(self, proj, nh, nkv, d, dv, D, q_weight, k_weight, eps, ctx, kv, block_table, has_kv=True,
                         write=True, position=None, query_temperature=None) -> torch.Tensor:
        """proj rows [q: nh*d | k: nkv*d | v: nkv*dv | ...]: q and k are each divided by the root mean square
        of the whole projection (all heads at once) and multiplied by their weights; returns the queries as
        [T, nh*D] (heads padded to D with zeros) and writes keys and values, padded the same way, to their page
        slots.  Without `has_kv` the rows hold no k and v (the layer reads another layer's cache).  `position` (a
        prepared rotary encoding): q and k are rotated after their norms.  `query_temperature` (coef, every): the
        query at position p is multiplied by 1 + coef * ln(floor((p + 1) / every) + 1)."""
        T, ld = proj.shape
        assert proj.is_contiguous() and kv.is_contiguous() and kv.dtype == proj.dtype and kv.shape[4] == D
        q = torch.empty((T, nh * D), dtype=proj.dtype, device=self.device)
        _check(self.core, self.core.pl_normed_qkv_write(
            self._p(proj), self._code(proj), T, ld, self._p(q_weight), self._p(k_weight), c_float(eps), self._p(q),
            self._p(kv), self._p(ctx.positions), self._p(ctx.token_seq), self._p(block_table), block_table.shape[1],
            kv.shape[0], kv.shape[3], nh, nkv, d, dv, D, 1 if has_kv else 0, 1 if write else 0, *self._rot_args(position),
            c_float(query_temperature[0] if query_temperature else 0.0), int(query_temperature[1]) if query_temperature else 0,
            self._stream))
        self.launches += 1
        return q

    def head_gate(self, o, nh, D, dv, gate=None) -> torch.Tensor:
        """[T, nh*dv]: the first dv columns of each head of o [T, nh*D], times sigmoid(gate) if a gate
        (a column view [T, nh*dv] of a row-major tensor) is given."""
        T = o.shape[0]
        assert o.is_contiguous() and o.shape[1] == nh * D
        out = torch.empty((T, nh * dv), dtype=o.dtype, device=self.device)
        ldg = 0
        if gate is not None:
            assert gate.dtype == o.dtype and gate.stride(1) == 1 and gate.shape == (T, nh * dv)
            ldg = gate.stride(0)
        _check(self.core, self.core.pl_head_gate(self._p(o), self._code(o), T, D, self._p(gate), ldg, self._p(out), nh, dv,
                                                 self._stream))
        self.launches += 1
        return out

    def latent_kv_write(self, down, q_rank, kv_rank, rot_dim, D, q_weight, c_weight, eps, position, ctx, kv, block_table,
                        write=True, norm_q=True):
        """down rows [query latent: q_rank | key/value latent: kv_rank | rotated key part: rot_dim]: both latents
        are RMS-normed (float32) with their weights; the normed query latent is returned [T, q_rank]; the cache
        (one kv head of size D) gets the key [latent | rotated part | 0] and the value [latent | 0].  Without `norm_q`
        the first q_rank columns are not a latent (the queries themselves, projected straight from the input): they
        are left alone and nothing is returned."""
        T, ld = down.shape
        assert down.is_contiguous() and kv.is_contiguous() and kv.dtype == down.dtype and kv.shape[4] == D and kv.shape[2] == 1
        cq = torch.empty((T, q_rank), dtype=down.dtype, device=self.device) if norm_q else None
        _check(self.core, self.core.pl_latent_kv_write(
            self._p(down), self._code(down), T, ld, self._p(q_weight), self._p(c_weight), c_float(eps), self._p(cq),
            self._p(kv), self._p(ctx.positions), self._p(ctx.token_seq), self._p(block_table), block_table.shape[1],
            kv.shape[0], kv.shape[3], *self._rot_args(position), q_rank, kv_rank, rot_dim, D, 1 if write else 0,
            1 if norm_q else 0, self._stream))
        self.launches += 1
        return cq

    def latent_queries(self, q_abs, q, nh, d, rot_dim, kv_rank, D, position, ctx) -> torch.Tensor:
        """[T, nh*D] with head h = [q_abs[t, h] (kv_rank) | rotated q[t, h, d:d+rot_dim] | 0]; the heads of q are the
        first nh * (d + rot_dim) columns of its rows."""
        T = q.shape[0]
        assert q.is_contiguous() and q_abs.is_contiguous() and q.shape[1] >= nh * (d + rot_dim) and q_abs.shape[1] == nh * kv_rank
        out = torch.empty((T, nh * D), dtype=q.dtype, device=self.device)
        _check(self.core, self.core.pl_latent_q(self._p(q_abs), self._p(q), self._code(q), T, self._p(out),
                                                self._p(ctx.positions), self._p(ctx.token_seq), *self._rot_args(position),
                                                nh, d, rot_dim, kv_rank, D, q.shape[1], self._stream))
        self.launches += 1
        return out

    def ssm_mix(self, zx, inner, groups, state_size, heads, head_dim, conv_w, conv_b, dt_bias, a_log, d_skip, norm_w,
                norm_groups, eps, state, ctx) -> torch.Tensor:
        """The state-space mixer between its two projections.  zx rows [z: inner | x: inner | B: G*N | C: G*N |
        dt: heads] in the compute dtype; `state` [slots, (taps-1)*(inner+2GN) + heads*head_dim*N] float32 holds each
        request's convolution inputs and recurrent state and is updated in place.  Returns the gated, normed
        output [T, inner] in the compute dtype.  Three kernels: convolution + SiLU with dt and the decay;
        the recurrence, token by token in float32; gate and norm in parts."""
        lib = load_module("ssm")
        T, ld = zx.shape
        G, N, H, P = groups, state_size, heads, head_dim
        C = inner + 2 * G * N
        taps = conv_w.shape[1]
        assert zx.is_contiguous() and ld == 2 * inner + 2 * G * N + H and state.dtype == torch.float32 and state.is_contiguous()
        assert state.shape[1] == (taps - 1) * C + H * P * N
        dev = self.device
        xbc = torch.empty((T, C), dtype=torch.float32, device=dev)
        dt = torch.empty((T, H), dtype=torch.float32, device=dev)
        decay = torch.empty((T, H), dtype=torch.float32, device=dev)
        y = torch.empty((T, inner), dtype=torch.float32, device=dev)
        S = ctx.num_seqs
        _check(lib, lib.pl_ssm_conv(self._p(zx), self._code(zx), ld, inner, C, 2 * inner + 2 * G * N, H, self._p(conv_w),
                                    self._p(conv_b), taps, self._p(dt_bias), self._p(a_log), self._p(state),
                                    c_longlong(state.shape[1]), self._p(ctx.cu_seqlens_q), self._p(ctx.state_slots), S, T,
                                    self._p(xbc), self._p(dt), self._p(decay), self._stream))
        _check(lib, lib.pl_ssm_scan(self._p(xbc), C, inner, G, N, H, P, self._p(dt), self._p(decay), self._p(d_skip),
                                    self._p(state), c_longlong(state.shape[1]), c_longlong((taps - 1) * C),
                                    self._p(ctx.cu_seqlens_q), self._p(ctx.state_slots), S, T, self._p(y), self._stream))
        out = torch.empty((T, inner), dtype=zx.dtype, device=dev)
        _check(lib, lib.pl_gated_group_norm(self._p(y), self._p(zx), self._code(zx), ld, self._p(norm_w), c_float(eps),
                                            self._p(out), T, inner, norm_groups, self._p(ctx.token_seq), self._stream))
        self.launches += 3
        return out

    # ---- several residual streams, norms in parts, PolyNorm ---------------------------
    def stream_norm(self, x, streams, branch, mix, out, w_in, norm_w, groups, eps, branch2=None, scales=None, biases=None):
        """One kernel at a sublayer boundary of a model with `streams` copies of the residual stream
        (x: [rows, streams * W] float32, updated in place): the copies take `branch` [rows, W] in
        (x_t <- sum_s mix[s, t] x_s + out[t] * branch with `mix` [S, S] and `out` [S]; without `mix` every copy gets
        + branch), the next input u = sum_s w_in[s] x_s (w_in None: the plain sum) is formed and normed in `groups`
        equal consecutive parts, each divided by its own root mean square, times `norm_w`.  With `branch2` the branch
        is scales[0] * (branch + biases[0]) + scales[1] * (branch2 + biases[1]) (biases float32 [W] or None)."""
        lib = load_module("streams")
        rows, SW = x.shape
        W = SW // streams
        assert x.dtype == torch.float32 and x.is_contiguous() and W * streams == SW
        for t in (mix, out, w_in):
            assert t is None or (t.dtype == torch.float32 and t.is_contiguous())
        if branch is not None:
            assert branch.shape == (rows, W) and branch.is_contiguous()
        if branch2 is not None:
            assert branch2.shape == (rows, W) and branch2.is_contiguous() and branch2.dtype == branch.dtype
        sa, sb = scales if scales is not None else (1.0, 1.0)
        ba, bb = biases if biases is not None else (None, None)
        y = torch.empty((rows, W), dtype=self.compute_dtype, device=self.device)
        _check(lib, lib.pl_stream_norm(self._p(x), self._p(branch), self._p(branch2),
                                       self._code(branch) if branch is not None else PL_F32, self._p(ba), self._p(bb),
                                       c_float(sa), c_float(sb), self._p(mix), self._p(out), self._p(w_in), self._p(norm_w),
                                       self._code(norm_w), self._p(y), self._code(y), c_longlong(rows), streams, W, groups,
                                       c_float(eps), self._stream))
        self.launches += 1
        return y

    def poly_norm(self, z: torch.Tensor, coef: torch.Tensor, eps: float) -> torch.Tensor:
        """coef[0] N(z) + coef[1] N(z^2) + coef[2] N(z^3) + coef[3] row by row, N(v) = v / sqrt(mean(v^2) + eps)."""
        lib = load_module("streams")
        rows, F = z.shape
        assert z.is_contiguous() and coef.dtype == torch.float32 and coef.numel() == 4
        out = torch.empty_like(z)
        _check(lib, lib.pl_poly_norm(self._p(z), self._code(z), self._p(coef), c_float(eps), self._p(out), c_longlong(rows), F,
                                     self._stream))
        self.launches += 1
        return out

    def add_bias(self, y: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
        """y[r, :] += bias in place (bias float32)."""
        lib = load_module("streams")
        rows, W = y.shape
        assert y.is_contiguous() and bias.dtype == torch.float32 and bias.numel() == W
        _check(lib, lib.pl_add_bias(self._p(y), self._code(y), self._p(bias), c_longlong(rows), W, self._stream))
        self.launches += 1
        return y

    def scaled_sum(self, a, scale_a, bias_a, b, scale_b, bias_b) -> torch.Tensor:
        """scale_a * (a + bias_a) + scale_b * (b + bias_b) as float32 (either bias may be None)."""
        lib = load_module("streams")
        rows, W = a.shape
        assert a.is_contiguous() and b.is_contiguous() and a.shape == b.shape and a.dtype == b.dtype
        out = torch.empty((rows, W), dtype=torch.float32, device=self.device)
        _check(lib, lib.pl_scaled_sum(self._p(a), self._p(b), self._code(a), self._p(bias_a), self._p(bias_b), c_float(scale_a),
                                      c_float(scale_b), self._p(out), c_longlong(rows), W, self._stream))
        self.launches += 1
        return out

    # ---- attention whose values are rotated too ---------------------------------------
    @staticmethod
    def _rot_args(position):
        if position is None:
            return c_void_p(0), 0, 0, 0
        t = position.table
        return c_void_p(t.data_ptr()), t.shape[0], position.rotary_dim, 1 if position.pairing == "interleaved" else 0

    def rotated_qkv_write(self, proj, bias, nh, nkv, d, dv, D, position, value_position, ctx, kv, block_table,
                          write=True) -> torch.Tensor:
        """proj rows [q: nh*d | k: nkv*d | v: nkv*dv | ...] (+ `bias`, float32, the same layout): q and k are rotated
        by the token's position with `position`, v with `value_position`; returns the queries [T, nh*D] (heads padded
        to D with zeros) and writes keys and values, padded the same way, to their page slots."""
        T, ld = proj.shape
        assert proj.is_contiguous() and kv.is_contiguous() and kv.dtype == proj.dtype and kv.shape[4] == D
        assert bias is None or (bias.dtype == torch.float32 and bias.numel() == nh * d + nkv * (d + dv))
        q = torch.empty((T, nh * D), dtype=proj.dtype, device=self.device)
        _check(self.core, self.core.pl_rotated_qkv_write(
            self._p(proj), self._code(proj), T, ld, self._p(bias), self._p(q), self._p(kv), self._p(ctx.positions),
            self._p(ctx.token_seq), self._p(block_table), block_table.shape[1], kv.shape[0], kv.shape[3],
            *self._rot_args(position), *self._rot_args(value_position), nh, nkv, d, dv, D, 1 if write else 0, self._stream))
        self.launches += 1
        return q

    def head_unrotate_gate(self, o, nh, D, dv, value_position, ctx, gate=None) -> torch.Tensor:
        """[T, nh*dv]: the first dv columns of each head of o [T, nh*D], turned back by the query's position with
        `value_position`, times sigmoid(gate[t, h]) if a gate (a column view [T, nh] of a row-major tensor) is given."""
        T = o.shape[0]
        assert o.is_contiguous() and o.shape[1] == nh * D
        out = torch.empty((T, nh * dv), dtype=o.dtype, device=self.device)
        ldg = 0
        if gate is not None:
            assert gate.dtype == o.dtype and gate.stride(1) == 1 and gate.shape == (T, nh)
            ldg = gate.stride(0)
        _check(self.core, self.core.pl_head_unrotate_gate(self._p(o), self._code(o), T, D, self._p(gate), ldg,
                                                          self._p(ctx.positions), self._p(ctx.token_seq),
                                                          *self._rot_args(value_position), self._p(out), nh, dv,
                                                          self._stream))
        self.launches += 1
        return out

    # ---- mixers with a state of fixed size: convolution + gated recurrence, gated linear attention --------------
    def causal_conv(self, yx, col0, C, b_in, conv_w, conv_b, state, ctx, activation=None, low=True):
        """u = conv(yx[:, col0:col0+C] + b_in[col0:col0+C]) + conv_b per channel, causal, `taps` wide; the request's
        last taps-1 inputs are the first (taps-1)*C floats of its state slot and are replaced by the new ones.
        Either bias may be None; `activation` "silu" is applied to the result.
        Returns (u float32 [T, C], u in the compute dtype, or None without `low`)."""
        lib = load_module("recurrent")
        T, ld = yx.shape
        taps = conv_w.shape[1]
        assert yx.is_contiguous() and state.dtype == torch.float32 and state.is_contiguous() and state.dim() == 2
        assert conv_w.dtype == torch.float32 and conv_w.shape == (C, taps) and conv_w.is_contiguous()
        u = torch.empty((T, C), dtype=torch.float32, device=self.device)
        if activation not in (None, "silu"):
            raise KernelError(f"causal_conv: activation {activation!r} (silu or none)")
        if not low:
            low = None
        else:
            low = u if yx.dtype == torch.float32 else torch.empty((T, C), dtype=yx.dtype, device=self.device)
        _check(lib, lib.pl_causal_conv(self._p(yx), self._code(yx), ld, col0, C, self._p(b_in), self._p(conv_w),
                                       self._p(conv_b), taps, self._p(state), c_longlong(state.shape[1]),
                                       self._p(ctx.cu_seqlens_q), self._p(ctx.state_slots), ctx.num_seqs, max(T, 1),
                                       self._p(u), self._p(low) if low is not None and low is not u else c_void_p(0),
                                       1 if activation == "silu" else 0, self._stream))
        self.launches += 1
        return u, low

    def delta_rule_scan(self, u, proj, gate_col0, decay_rate, decay_bias, H, G, d, dv, unit_eps, q_scale, state_off, state,
                        ctx) -> torch.Tensor:
        """The gated delta rule's recurrence.  u float32 [T, q: G*d | k: G*d | v: H*dv] (convolved and activated; q and k
        are made unit vectors in place, q also times `q_scale`); proj columns [gate_col0, +2H) hold [b: H | a: H]:
        beta = sigmoid(b), g = exp(decay_rate * softplus(a + decay_bias)).  Per value head (q/k head h // (H // G)):
        S <- g S; w = beta (v - S^T k); S <- S + k w^T; o = S^T q.  S lives `state_off` floats into the request's
        state slot as [H][dv][d] float32 and is updated in place.  Returns o float32 [T, H*dv]."""
        lib = load_module("recurrent")
        T, C = u.shape
        assert u.dtype == torch.float32 and u.is_contiguous() and proj.is_contiguous() and C == 2 * G * d + H * dv
        assert state.dtype == torch.float32 and state.is_contiguous() and state.shape[1] >= state_off + H * dv * d
        assert decay_rate.dtype == torch.float32 and decay_bias.dtype == torch.float32 and decay_rate.numel() == H
        o = torch.empty((T, H * dv), dtype=torch.float32, device=self.device)
        bg = torch.empty((T, 2 * H + G), dtype=torch.float32, device=self.device)
        _check(lib, lib.pl_delta_rule(self._p(u), C, self._p(proj), self._code(proj), proj.shape[1], gate_col0,
                                      self._p(decay_rate), self._p(decay_bias), H, G, d, dv, c_float(unit_eps), c_float(q_scale),
                                      self._p(bg), self._p(state), c_longlong(state.shape[1]), c_longlong(state_off),
                                      self._p(ctx.cu_seqlens_q), self._p(ctx.state_slots), ctx.num_seqs, c_longlong(T),
                                      self._p(o), self.delta_lanes, self._stream))
        self.launches += 2
        return o

    # ---- two branches that are normed before they meet ---------------------------------
    def normed_pair_sum(self, a, b, wa, wb, sa, sb, eps) -> torch.Tensor:
        """sa * rms_norm(a) * wa + sb * rms_norm(b) * wb as float32 (norms over the row, eps inside the root)."""
        rows, W = a.shape
        assert a.is_contiguous() and b.is_contiguous() and a.shape == b.shape and a.dtype == b.dtype
        assert wa.dtype == torch.float32 and wb.dtype == torch.float32 and wa.numel() == W and wb.numel() == W
        out = torch.empty((rows, W), dtype=torch.float32, device=self.device)
        _check(self.core, self.core.pl_normed_pair(self._p(a), self._p(b), self._code(a), self._p(wa), self._p(wb), c_float(sa),
                                                   c_float(sb), c_float(eps), c_void_p(0), self._p(out), c_void_p(0), 0,
                                                   c_float(0.0), c_void_p(0), 0, c_longlong(rows), W, self._stream))
        self.launches += 1
        return out

    def normed_pair_add_rms_norm(self, x, a, b, wa, wb, sa, sb, pair_eps, norm_w, eps) -> torch.Tensor:
        """x += sa * rms_norm(a) * wa + sb * rms_norm(b) * wb (float32 stream, in place), then RMSNorm(x) * norm_w in the
        compute dtype: one kernel."""
        rows, W = x.shape
        assert x.dtype == torch.float32 and x.is_contiguous() and a.shape == x.shape and b.shape == x.shape
        assert a.is_contiguous() and b.is_contiguous() and a.dtype == b.dtype
        assert wa.dtype == torch.float32 and wb.dtype == torch.float32 and wa.numel() == W and wb.numel() == W
        y = torch.empty((rows, W), dtype=self.compute_dtype, device=self.device)
        _check(self.core, self.core.pl_normed_pair(self._p(a), self._p(b), self._code(a), self._p(wa), self._p(wb), c_float(sa),
                                                   c_float(sb), c_float(pair_eps), self._p(x), c_void_p(0), self._p(norm_w),
                                                   self._code(norm_w), c_float(eps), self._p(y), self._code(y),
                                                   c_longlong(rows), W, self._stream))
        self.launches += 1
        return y

    def gated_recurrence(self, gates, b_gates, u, yx, b_in, rate, blocks, taps, state, ctx) -> torch.Tensor:
        """S_t = a S_(t-1) + sqrt(1 - a^2) sigmoid(g_i) u_t with a = exp(rate * sigmoid(g_r)); returns
        S_t * gelu_tanh(yx[:, :C] + b_in[:C]) in the compute dtype.  gates: float32 [T, blocks * 2 * bw], per block
        [recurrence gate | input gate], overwritten when a request brings more than a few tokens (the decays and drives
        of all tokens are then formed in place by a kernel of their own, and the scan only multiplies and adds); S lives
        behind the convolution's inputs in the state slot."""
        lib = load_module("recurrent")
        T, C = u.shape
        ld = yx.shape[1]
        assert gates.dtype == torch.float32 and gates.is_contiguous() and gates.shape == (T, 2 * C)
        assert u.dtype == torch.float32 and u.is_contiguous() and yx.is_contiguous() and state.shape[1] == taps * C
        out = torch.empty((T, C), dtype=yx.dtype, device=self.device)
        _check(lib, lib.pl_gated_recurrence(self._p(gates), self._p(b_gates), self._p(u), self._p(yx), self._code(yx), ld,
                                            self._p(b_in), self._p(rate), C, blocks, self._p(state),
                                            c_longlong(state.shape[1]), c_longlong((taps - 1) * C),
                                            self._p(ctx.cu_seqlens_q), self._p(ctx.state_slots), ctx.num_seqs,
                                            max(int(ctx.max_q_len), 1), c_longlong(T),
                                            self._p(out), self._stream))
        self.launches += 1 if int(ctx.max_q_len) <= 16 else 2
        return out

    def linear_attention_scan(self, proj, z, z_bias, H, d, dv, tau, q_scale, state, ctx) -> torch.Tensor:
        """Gated linear attention's recurrence.  proj rows [q: H*d | k: H*d | v: H*dv | ...]; z float32 [T, H*d] the
        decay's pre-activation (bias `z_bias`): alpha = sigmoid(z)^(1/tau); S_t = diag(alpha_t) S_(t-1) + k_t v_t^T,
        o_t = S_t^T (q_t * q_scale).  state: [slots, H*dv*d] float32, updated in place.  Returns o float32 [T, H*dv].
        z is overwritten by the decays when a request brings a long prompt."""
        lib = load_module("recurrent")
        T, ld = proj.shape
        assert proj.is_contiguous() and z.dtype == torch.float32 and z.is_contiguous() and z.shape == (T, H * d)
        assert state.dtype == torch.float32 and state.is_contiguous() and state.shape[1] == H * dv * d
        o = torch.empty((T, H * dv), dtype=torch.float32, device=self.device)
        # a long prompt is cut into segments that run side by side: each leaves its end state and the product of its decays
        seg, longest = lib.pl_gla_segment(), max(int(ctx.max_q_len), 1)
        cut = longest >= 2 * seg
        seg_state = seg_decay = None
        if cut:
            seg_state = torch.empty((2, -(-T // seg), H * dv * d), dtype=torch.float32, device=self.device)
            seg_state, seg_decay = seg_state[0], seg_state[1]
        _check(lib, lib.pl_gla_scan(self._p(proj), self._code(proj), ld, self._p(z), self._p(z_bias), H, d, dv, c_float(tau),
                                    c_float(q_scale), self._p(state), c_longlong(state.shape[1]), self._p(ctx.cu_seqlens_q),
                                    self._p(ctx.state_slots), ctx.num_seqs, longest, c_longlong(T), self._p(seg_state),
                                    self._p(seg_decay), self._p(o), self._stream))
        self.launches += 3 if cut else 1
        return o

    def head_norm_gate(self, o, proj, g_col0, H, dv, norm_w, eps) -> torch.Tensor:
        """Each head of o (float32 [T, H*dv]) divided by its root mean square over dv, times `norm_w` [dv], times
        silu(proj[:, g_col0 : g_col0 + H*dv]); in the compute dtype."""
        lib = load_module("recurrent")
        T = o.shape[0]
        assert o.is_contiguous() and proj.is_contiguous() and norm_w.dtype == torch.float32 and norm_w.numel() == dv
        out = torch.empty((T, H * dv), dtype=proj.dtype, device=self.device)
        gate = c_void_p(proj.data_ptr() + g_col0 * proj.element_size())
        _check(lib, lib.pl_head_norm_gate(self._p(o), gate, self._code(proj), proj.shape[1], self._p(norm_w), c_float(eps),
                                          self._p(out), c_longlong(T), H, dv, self._stream))
        self.launches += 1
        return out

    # ---- routed experts ----------------------------------------------------------
    def routed_experts(self, h, w_router, w_gate_up, w_down, top_k: int, activation: str = "silu", shared=None,
                       shared_activation: str = "silu", activation_limit: float = 0.0, scoring: str = "softmax_top",
                       groups=None) -> torch.Tensor:
        """The feed-forward of routed experts for the step's tokens: float32 [T, D].

        w_router [E (+1) or more, D]: the router's rows and, with a shared expert, the row of its gate (further rows
        are ignored); w_gate_up
        [E, 2F, D] (gate rows over up rows) and w_down [E, D, F]; `shared` = (gate over up [2Fs, D], down
        [D, Fs]) or None.  Router logits, top-k, the softmax over the chosen logits and the final weighted
        sum are float32.  Kernels: the router's product and choice; (token, choice) pairs sorted by expert on the device; the
        experts' two products over tiles of that list (bfloat16: mma.sync tiles of 64 pairs, or of 16 when
        experts get few pairs as in decoding, or, with many pairs per expert, the grouped form of the tcgen05
        product over rows gathered in sorted order; float32 and odd sizes: FFMA chains in k order); the sum.
        Nothing is read back, so the step can be captured.  `scoring` "sigmoid": the scores sigmoid(z) choose and are the
        weights as they are; `groups` (count, keep, best): only experts of the `keep` groups (of `count` equal groups
        of neighbours) with the largest sum of their `best` largest scores can be chosen.  `activation`
        "swish_clamped" takes `activation_limit`."""
        h = self.materialize(h)
        assert h.is_contiguous() and w_gate_up.is_contiguous() and w_down.is_contiguous() and w_router.is_contiguous()
        T, D = h.shape
        E, F2, _ = w_gate_up.shape
        F = F2 // 2
        assert w_down.shape == (E, D, F) and w_router.shape[0] >= E + (1 if shared is not None else 0) and w_router.shape[1] == D
        assert w_gate_up.dtype == h.dtype and w_down.dtype == h.dtype and w_router.dtype == h.dtype
        lib = load_module("moe")
        dev, code = self.device, self._code(h)
        pairs = T * top_k
        top_idx = torch.empty(pairs, dtype=torch.int32, device=dev)
        top_w = torch.empty(pairs, dtype=torch.float32, device=dev)
        gate = torch.empty(T, dtype=torch.float32, device=dev) if shared is not None else None
        z = self.linear(h, w_router, out_float32=True)          # float32 logits (and the shared expert's gate)
        if scoring == "sigmoid":
            if shared is not None:
                raise KernelError("routed_experts: a shared expert's gate rides with the softmax scoring only")
            count, keep, best = groups if groups is not None else (0, 0, 0)
            _check(lib, lib.pl_moe_sigmoid_topk(self._p(z), z.shape[1], T, E, top_k, count, keep, best, self._p(top_idx),
                                                self._p(top_w), self._stream))
        else:
            _check(lib, lib.pl_moe_topk(self._p(z), z.shape[1], T, E, top_k, 1 if shared is not None else 0,
                                        self._p(top_idx), self._p(top_w), self._p(gate), self._stream))
        tensor_cores = h.dtype == torch.bfloat16 and D % 8 == 0 and F % 8 == 0
        # Many pairs per expert (prompt portions): the experts' products run on the tcgen05 kernel of the dense
        # layers in its grouped form, over rows gathered in the order of the sorted list (tiles of 256 pairs).
        grouped_tc = (tensor_cores and "moe" in self.gemm_tc_for and D % 64 == 0 and F % 64 == 0
                      and pairs >= max(self.moe_tc_min_pairs, 96 * E))
        BM = 256 if grouped_tc else (64 if tensor_cores and pairs >= 32 * E else 16)
        max_tiles = pairs // BM + min(pairs, E)
        cap = max_tiles * BM
        sorted_pairs = torch.empty(cap, dtype=torch.int32, device=dev)
        tile_expert = torch.empty(max_tiles, dtype=torch.int32, device=dev)
        n_tiles = torch.empty(1, dtype=torch.int32, device=dev)
        place = torch.empty(pairs, dtype=torch.int32, device=dev) if grouped_tc else None
        _check(lib, lib.pl_moe_align(self._p(top_idx), pairs, E, BM, cap, self._p(sorted_pairs),
                                     self._p(tile_expert), self._p(n_tiles), self._p(place), self._stream))
        act, lim = EXPERT_ACTIVATIONS[activation], c_float(activation_limit)
        if grouped_tc:
            xs = torch.empty((cap, D), dtype=h.dtype, device=dev)
            _check(lib, lib.pl_moe_gather(self._p(h), D, top_k, self._p(sorted_pairs), self._p(n_tiles), BM, cap, pairs, D,
                                          self._p(xs), self._stream))
            inter = torch.empty((cap, F), dtype=h.dtype, device=dev)
            _check(self.core, self.core.pl_gemm_tc_grouped(self._p(xs), D, self._p(w_gate_up), self._p(inter), F, cap, F, D,
                                                           2, act, lim, E, self._p(n_tiles), self._p(tile_expert), self._stream))
            # (each expert's output is rounded to bfloat16, as a dense layer's branch is; the weighted sum is float32)
            pair_out = torch.empty((cap, D), dtype=torch.bfloat16, device=dev)
            _check(self.core, self.core.pl_gemm_tc_grouped(self._p(inter), F, self._p(w_down), self._p(pair_out), D, cap, D, F,
                                                           0, act, lim, E, self._p(n_tiles), self._p(tile_expert), self._stream))
            self.launches += 5
        else:
            inter = torch.empty((pairs, F), dtype=h.dtype, device=dev)
            _check(lib, lib.pl_moe_gemm(self._p(h), D, top_k, self._p(w_gate_up), self._p(inter), F, self._p(sorted_pairs),
                                        self._p(tile_expert), self._p(n_tiles), c_void_p(0), pairs, F, D, 1, act, lim, code, BM,
                                        max_tiles, 1 if tensor_cores else 0, self._stream))
            pair_out = torch.empty((pairs, D), dtype=torch.float32, device=dev)
            _check(lib, lib.pl_moe_gemm(self._p(inter), F, 1, self._p(w_down), self._p(pair_out), D, self._p(sorted_pairs),
                                        self._p(tile_expert), self._p(n_tiles), self._p(top_w), pairs, D, F, 0, act, lim, code, BM,
                                        max_tiles, 1 if tensor_cores else 0, self._stream))
            self.launches += 4
        s = None
        if shared is not None:
            s = self.linear(self.gated_act_linear(h, shared[0], shared_activation), shared[1])
        y = torch.empty((T, D), dtype=torch.float32, device=dev)
        _check(lib, lib.pl_moe_combine(self._p(pair_out), self._code(pair_out), top_k, self._p(place),
                                       self._p(top_w) if grouped_tc else c_void_p(0),
                                       self._p(s), self._code(s) if s is not None else PL_F32,
                                       self._p(gate), self._p(y), T, D, self._stream))
        self.launches += 1
        return y

    # ---- positions ---------------------------------------------------------------
    def rope_table(self, inv_freq: torch.Tensor, max_positions: int, magnitude: float = 1.0) -> torch.Tensor:
        """[positions, pairs, 2] float32: (cos, sin) of position * inv_freq, both times `magnitude`."""
        inv_freq = inv_freq.to(device=self.device, dtype=torch.float32).contiguous()
        half = inv_freq.numel()
        table = torch.empty((max_positions, half, 2), dtype=torch.float32, device=self.device)
        _check(self.core, self.core.pl_rope_table(self._p(inv_freq), self._p(table), max_positions, half,
                                                  c_float(magnitude), self._stream))
        self.launches += 1
        return table

    def rope_kv_write(self, qkv, nh, nkv, d, position, ctx, kv, block_table, write=True, value_from_key=False):
        T = ctx.num_tokens
        assert qkv.is_contiguous() and qkv.shape[0] == T
        if position is not None:
            table, table_len, rd = position.table, position.table.shape[0], position.rotary_dim
            inter = 1 if position.pairing == "interleaved" else 0
        else:
            table, table_len, rd, inter = None, 0, 0, 0
        num_pages, ps = kv.shape[0], kv.shape[3]
        assert kv.dtype == qkv.dtype and kv.is_contiguous()
        _check(self.core, self.core.pl_rope_kv_write(
            self._p(qkv), self._code(qkv), T, qkv.shape[1], self._p(table), table_len, rd, inter,
            self._p(ctx.positions), self._p(ctx.token_seq), self._p(block_table), block_table.shape[1],
            self._p(kv), num_pages, nh, nkv, d, ps, 1 if write else 0, 1 if value_from_key else 0, self._stream))
        self.launches += 1

    # ---- attention ---------------------------------------------------------------
    def _large_rows(self, head_dim: int) -> int:
        """Query rows of a prefill tile: what the kernel that will run was built with."""
        if self.compute_dtype != torch.bfloat16:
            return 16
        b = head_dim_build(head_dim)
        lib = load_module(f"attn_bf16_d{b}")
        return int(getattr(lib, f"pl_attention_bf16_rows_d{b}")(0))

    CLUSTER_KEYS = 600      # keys a block of a decode-attention cluster may have to walk before more splits pay

    def long_context_class(self, num_requests: int, num_kv_heads: int, max_context: int) -> bool:
        """True if a decode step of this shape is planned as a long-context step (see
        plan.is_long_context).  A step replayed from a graph must stay in the class it was
        captured in, so the runner keeps a graph per class."""
        return planning.is_long_context(num_requests, num_kv_heads, self.num_sms, self.MAX_SPLITS,
                                        self.MAX_CLUSTER if self.cluster_attention else 0, self.CLUSTER_KEYS, max_context)

    def plan_attention(self, q_lens, k_lens, group_size, num_kv_heads, window, head_dim, chunk=None, pad_requests=None,
                       fixed_capacity=False, pad_tokens=None) -> dict:
        return planning.plan_attention(
            q_lens, k_lens, group_size, num_kv_heads, window, chunk=chunk, small_rows=self.SMALL_ROWS,
            large_rows=self._large_rows(head_dim), min_split_keys=self.MIN_SPLIT_KEYS, num_sms=self.num_sms,
            max_splits=self.MAX_SPLITS, pad_requests=pad_requests, fixed_capacity=fixed_capacity,
            cluster_max=self.MAX_CLUSTER if self.cluster_attention else 0, long_keys=self.CLUSTER_KEYS,
            pad_tokens=pad_tokens)

    def _scratch_for(self, floats: int) -> torch.Tensor:
        """Scratch for split partials.  Grown by allocating anew and keeping the
        old buffers, since captured graphs hold their addresses."""
        if not self._scratch or self._scratch[-1].numel() < floats:
            self._scratch.append(torch.empty(max(floats, 1 << 20), dtype=torch.float32, device=self.device))
        return self._scratch[-1]

    def _attention_bf16(self, d: int):
        b = head_dim_build(d)
        lib = load_module(f"attn_bf16_d{b}")
        return lib, getattr(lib, f"pl_attention_bf16_d{b}")

    def _runs_as_clusters(self, plan, ctx, nh: int, nkv: int, bf16: bool) -> bool:
        """Whether this step's attention takes the cluster form of the decode kernel: every request
        is a small item (a decode step), in bfloat16, with contexts short enough."""
        return bool(bf16 and self.cluster_attention and plan.n_small and not plan.n_large
                    and max(ctx.host.q_lens) * (nh // nkv) <= self.SMALL_ROWS and not plan.long_context)

    def qkv_attention(self, h, w_qkv, nh, nkv, d, position, ctx, kv, block_table, scale, window, write=True,
                      softcap=None, slopes=None, chunk=None, value_from_key=False) -> torch.Tensor:
        """The mixer's whole front: fused q/k/v projection, rotary positions on q and k, k and v written
        to the cache, attention over the pages.  Returns [T, nh * d].  It is `qkv_rope_write` followed by
        `paged_attention`, but for a decode step of more than 16 tokens (the projection is a library
        product then, without an epilogue) rotation and cache write happen inside the attention
        kernel instead of in a kernel of their own."""
        M = h.shape[0]
        plan = ctx.attention_plans.get(attention_plan_key(nh, nkv, window, d, chunk))
        inside = (plan is not None and write and softcap is None and slopes is None and position is not None
                  and not value_from_key
                  and position.pairing == "half" and position.rotary_dim == d and M == ctx.num_tokens
                  and not self._skinny_ok(h, (nh + 2 * nkv) * d) and self.compute_dtype == torch.bfloat16
                  and kv.dtype == torch.bfloat16 and self._runs_as_clusters(plan, ctx, nh, nkv, True)
                  and self.rope_in_attention)
        if inside:
            qkv = self.linear(h, w_qkv)
            return self.paged_attention(qkv, nh, nkv, d, kv, block_table, ctx, scale, window, rope=position, chunk=chunk)
        qkv = self.qkv_rope_write(h, w_qkv, nh, nkv, d, position, ctx, kv, block_table, write=write,
                                  value_from_key=value_from_key)
        return self.paged_attention(qkv, nh, nkv, d, kv, block_table, ctx, scale, window, softcap=softcap, slopes=slopes,
                                    chunk=chunk)

    def paged_attention(self, qkv, nh, nkv, d, kv, block_table, ctx, scale, window, softcap=None, slopes=None,
                        rope=None, chunk=None, dist_bias=None, sink=None):
        """Attention of the step's tokens over the paged cache.  `softcap` (scores become
        softcap * tanh(score / softcap)) and `slopes` (a float32 tensor [nh]: head h adds
        slopes[h] * (key position - query position) to its scores) modify the scores; both off
        by default; `dist_bias` (float32 [nh, L]) adds dist_bias[h, min(query position - key position, L - 1)];
        `chunk` c lets a query at position p see the keys from p - p % c on only.  `rope` (a prepared rotary encoding; only where the step runs as clusters, see
        `qkv_attention`): qkv is the unrotated projection, and the kernel rotates q and the step's own
        keys and writes those keys and values to the cache itself.  `sink` (float32 [nh]): the softmax's denominator
        of head h also holds exp(sink[h]), a term without key or value that counts once however the keys are split."""
        T = ctx.num_tokens
        plan = ctx.attention_plans[attention_plan_key(nh, nkv, window, d, chunk)]
        out = torch.empty((T, nh * d), dtype=qkv.dtype, device=self.device)
        p = AttnParams()
        real = sum(ctx.host.q_lens)
        if T > real or getattr(ctx, "padded", False):
            # Rows that pad the step to the size of its graph.  The split-context kernels zero them themselves
            # (a fill kernel between two kernels of a layer would keep them from overlapping: 0.97 against 0.92 ms
            # per step at 12 requests); a step with large items too is not padded in practice and gets the fill.
            if plan.n_large:
                out.zero_()
            else:
                p.pad_seqs, p.pad_to = ctx.num_seqs, T
        p.q, p.kv, p.out = qkv.data_ptr(), kv.data_ptr(), out.data_ptr()
        p.block_table, p.cu_q, p.k_lens = block_table.data_ptr(), ctx.cu_seqlens_q.data_ptr(), ctx.seq_lens_k.data_ptr()
        p.q_stride, p.out_stride, p.bt_stride = qkv.shape[1], nh * d, block_table.shape[1]
        p.nh, p.nkv, p.d, p.ps, p.num_pages = nh, nkv, d, kv.shape[3], kv.shape[0]
        p.window, p.scale, p.max_splits = int(window or 0), float(scale), plan.max_splits
        p.softcap = float(softcap or 0.0)
        p.chunk = int(chunk or 0)
        if slopes is not None:
            assert slopes.dtype == torch.float32 and slopes.numel() == nh and slopes.is_contiguous() and slopes.is_cuda
            p.slopes = slopes.data_ptr()
        if dist_bias is not None:
            assert (dist_bias.dtype == torch.float32 and dist_bias.dim() == 2 and dist_bias.shape[0] == nh
                    and dist_bias.is_contiguous() and dist_bias.is_cuda)
            p.dist_bias, p.dist_len = dist_bias.data_ptr(), dist_bias.shape[1]
        if sink is not None:
            assert sink.dtype == torch.float32 and sink.numel() == nh and sink.is_contiguous() and sink.is_cuda
            p.sink = sink.data_ptr()
        ps = kv.shape[3]
        p.ps_shift = ps.bit_length() - 1 if ps & (ps - 1) == 0 else -1
        p.counters = 0
        bf16 = qkv.dtype == torch.bfloat16
        if bf16:
            lib, fn = self._attention_bf16(d)
        else:
            lib, fn = self.core, self.core.pl_attention_f32
        p.cluster = 0
        if rope is not None:
            if not self._runs_as_clusters(plan, ctx, nh, nkv, bf16) or softcap or slopes is not None or dist_bias is not None:
                raise KernelError("rotary positions inside the attention kernel: only for decode steps that run as "
                                  "clusters, without score modifiers")
            assert qkv.shape[1] == (nh + 2 * nkv) * d and rope.table.is_contiguous() and rope.rotary_dim == d
            p.rope_table, p.rope_len = rope.table.data_ptr(), rope.table.shape[0]
        if self._runs_as_clusters(plan, ctx, nh, nkv, bf16):
            # every request is a small item: the splits of a (request, kv head) are the blocks of
            # a thread-block cluster that merge through distributed shared memory
            p.work, p.n_work, p.is_small, p.cluster = 0, ctx.num_seqs, 1, min(plan.max_splits, self.MAX_CLUSTER)
            p.scratch, p.scratch_floats = 0, 0
            _check(lib, fn(ctypes.byref(p), self._stream))
            self.launches += 1
            return out
        if plan.n_small:
            floats = max(plan.small_tokens, 1) * nh * plan.max_splits * (d + 2)
            scratch = self._scratch_for(floats)
            p.scratch, p.scratch_floats = scratch.data_ptr(), scratch.numel()
            # long ranges and blocks in plenty (two per SM or more): the ring of three 64-key tiles; with fewer
            # blocks eight warps per block do better (one request x 16,384 keys: 1.00 against 1.10 ms per step)
            deep = plan.long_context and self.deep_list and plan.n_small * nkv >= 2 * self.num_sms
            p.work, p.n_work, p.is_small = plan.small.data_ptr(), plan.n_small, 2 if deep else 1
            fused_merge = bf16 and plan.max_splits > 1
            if fused_merge:
                need = ctx.num_seqs * nkv
                if self._attn_counters is None or self._attn_counters.numel() < need:
                    self._attn_counters_keep.append(self._attn_counters)    # captured graphs hold the old address
                    self._attn_counters = torch.zeros(max(need, 4096), dtype=torch.int32, device=self.device)
                p.counters = self._attn_counters.data_ptr()
            _check(lib, fn(ctypes.byref(p), self._stream))
            self.launches += 1
            p.counters = 0
            if plan.max_splits > 1 and not fused_merge:
                _check(self.core, self.core.pl_attention_combine(ctypes.byref(p), self._code(out), self._stream))
                self.launches += 1
        if plan.n_large:
            p.scratch, p.scratch_floats = 0, 0
            p.work, p.n_work, p.is_small = plan.large.data_ptr(), plan.n_large, 0
            p.max_splits = 1
            _check(lib, fn(ctypes.byref(p), self._stream))
            self.launches += 1
        return out

    # ---- cache -------------------------------------------------------------------
    def copy_pages(self, pool: torch.Tensor, pairs) -> None:
        layers, pages = pool.shape[0], pool.shape[1]
        page_bytes = pool[0, 0].numel() * pool.element_size()
        for src, dst in pairs:
            _check(self.core, self.core.pl_copy_page(self._p(pool), layers, c_longlong(pages), c_longlong(page_bytes),
                                                     int(src), int(dst), self._stream))
            self.launches += 1

    # ---- sampling ----------------------------------------------------------------
    def argmax(self, logits: torch.Tensor) -> torch.Tensor:
        rows, V = logits.shape
        assert logits.dtype == torch.float32 and logits.stride(1) == 1
        out = torch.empty(rows, dtype=torch.int32, device=self.device)
        if self._argmax_ws is None or self._argmax_ws[0].numel() < rows:
            self._argmax_keep.append(self._argmax_ws)               # captured graphs hold the old addresses
            self._argmax_ws = (torch.zeros(max(rows, 1024), dtype=torch.int64, device=self.device),
                               torch.zeros(max(rows, 1024), dtype=torch.int32, device=self.device))
        cells, counters = self._argmax_ws
        _check(self.core, self.core.pl_argmax(self._p(logits), self._p(out), rows, V, c_longlong(logits.stride(0)),
                                              self._p(cells), self._p(counters), self._stream))
        self.launches += 1
        return out

    def sample(self, logits, temps, top_k, top_p, seeds, counters) -> torch.Tensor:
        rows, V = logits.shape
        assert logits.dtype == torch.float32 and logits.stride(1) == 1
        dev = self.device
        # The five per-row arrays go up as one copy from pinned memory that does not wait for the step in front
        # of it (five copies from pageable memory each waited for the device: 1.01 against 0.81 ms per step at
        # batch 8).  Layout in 8-byte words: seeds [rows], counters [rows], then temps, top_p, top_k as 4-byte
        # values.
        words = 2 * rows + (3 * rows + 1) // 2
        if self._sample_dev is None or self._sample_dev.numel() < words:
            self._sample_keep.append(self._sample_dev)              # a kernel in flight may still read the old one
            self._sample_dev = torch.empty(max(2 * words, 1024), dtype=torch.int64, device=dev)
            self._sample_ring = [[torch.empty(max(2 * words, 1024), dtype=torch.int64, pin_memory=True), None]
                                 for _ in range(4)]
        slot = self._sample_ring[self._sample_pos % len(self._sample_ring)]
        self._sample_pos += 1
        if slot[1] is not None:
            slot[1].synchronize()                                   # its last copy has left the buffer
        host = slot[0].numpy()
        host[:rows] = np.ascontiguousarray(seeds, np.uint64).view(np.int64)
        host[rows:2 * rows] = np.ascontiguousarray(counters, np.uint64).view(np.int64)
        tail = host[2 * rows:words].view(np.float32)
        tail[:rows] = temps
        tail[rows:2 * rows] = top_p
        tail[2 * rows:3 * rows].view(np.int32)[:] = top_k
        self.copy_h2d(self._sample_dev, slot[0], words * 8)
        slot[1] = torch.cuda.Event()
        slot[1].record()
        s, c = self._sample_dev[:rows], self._sample_dev[rows:2 * rows]
        tail_dev = self._sample_dev[2 * rows:words].view(torch.float32)
        t, pp, k = tail_dev[:rows], tail_dev[rows:2 * rows], tail_dev[2 * rows:3 * rows].view(torch.int32)
        out = torch.empty(rows, dtype=torch.int32, device=dev)
        _check(self.core, self.core.pl_sample(self._p(logits), self._p(out), rows, V, c_longlong(logits.stride(0)),
                                              self._p(t), self._p(k), self._p(pp), self._p(s), self._p(c),
                                              self._stream))
        self.launches += 1
        return out
