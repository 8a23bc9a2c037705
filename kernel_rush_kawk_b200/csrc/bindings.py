"""Python bindings of the CUDA kernels (ctypes over the compiled libraries).

``Kernels`` is the one object through which the engine computes. Every method
launches this package's own kernels on torch's current CUDA stream; the only
library routine on the path is the dense matrix product of many rows in
bfloat16 (cuBLASLt, called by csrc/lt_gemm.cu with the algorithm picked by
measurement; ``torch.matmul`` for layouts that it does not take), which is
where the reference calls the library too (engine/model.py:295,299,301,303 of
willzeng274/kernel-rush-kawk).
There is no fallback: without a CUDA device and the compiled libraries,
construction raises.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_uint, c_void_p

import torch

from .build import build_library

F32, BF16 = 0, 1
_P = c_void_p


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise TypeError(f"kernels take float32 or bfloat16 tensors, got {dtype}")


class KernelError(RuntimeError):
    pass


_SIGNATURES = {
    "krk_rmsnorm": [_P, _P, _P, _P, _P, c_int, c_int, c_int, c_float, c_int, _P],
    "krk_gather_rows": [_P, _P, _P, c_int, c_int, c_int, _P, c_int, _P],
    "krk_swiglu": [_P, _P, c_int, c_int, c_int, _P],
    "krk_qk_norm_rope_write": [_P, _P, _P, c_int, _P, _P, _P, _P, _P, _P, c_int, _P, _P, c_int, c_int, c_int, c_int,
                               c_int, c_float, c_int, _P, c_int, _P],
    "krk_gemm_nt": [_P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, _P],
    "krk_select_tokens": [_P, _P, c_int, c_int, c_float, c_uint, _P, c_uint, _P, _P, _P, _P, _P],
    "krk_gemm_tcgen05": [_P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, _P, _P],
    "krk_selftest_wait_runs_out": [_P, c_int, _P],
    "krk_skinny_linear": [_P, _P, _P, _P, _P, _P, c_int, _P, c_int, c_int, c_int, c_float, c_int, c_int, _P],
    "krk_lt_gemm_bf16": [_P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, _P, _P],
    "krk_lt_gemm_report": [_P, _P],
}
_MIX_SIGNATURES = {
    "krk_embed_scaled": [_P, _P, _P, c_int, c_int, c_int, c_float, _P, c_int, _P, c_int],
    "krk_rmsnorm_wide": [_P, _P, _P, _P, _P, c_float, c_int, c_int, c_float, _P, c_float, _P, _P, c_int, _P],
    "krk_gated_act": [_P, _P, c_int, c_int, c_int, c_int, c_int, c_int, _P, c_float, c_float],
    "krk_hyper_rmsnorm": [_P, _P, _P, _P, _P, _P, _P, c_float, c_int, c_int, c_int, c_float, c_int, _P],
    "krk_bias_row_norm": [_P, c_int, c_int, c_int, c_int, c_int, _P, _P, c_float, c_int, c_int, _P],
    "krk_rotate_norm_write": [_P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, _P, c_int, c_int, c_float, _P, _P,
                              _P, _P, c_int, _P, _P, c_int, c_int, _P, c_int, c_float, c_int, _P],
    "krk_sink_attention": [_P, c_int, c_int, c_float, _P, c_int, c_int, c_int, c_int, c_int, c_int, _P, _P, _P, _P, _P,
                           c_int, _P, _P, c_int, c_float, c_int, c_int, c_int, _P, c_int, c_int, c_int, c_int, _P],
    "krk_sink_attention_single": [_P, c_int, c_int, c_float, _P, c_int, c_int, c_int, c_int, c_int, c_int, _P, _P, _P, _P,
                                  c_int, _P, _P, c_int, c_float, c_int, c_int, _P, c_int, c_int, c_int, _P, c_int, c_int, c_float,
                                  c_int, c_int, _P, c_int, c_int, c_int, c_int, _P],
    "krk_latent_norm_write": [_P, c_int, c_int, c_int, _P, c_float, _P, _P, _P, _P, c_int, c_int, _P, c_int, _P, c_int, _P],
    "krk_head_linear": [_P, c_int, c_int, c_float, _P, c_int, _P, c_int, c_int, c_int, c_int, c_int, _P],
    "krk_embed_bigram": [_P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_longlong, c_longlong, _P, _P, _P, _P, _P, c_int, _P],
    "krk_bias_norm_rotate_write": [_P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, _P, _P, c_float, _P, c_int,
                                   c_int, _P, _P, _P, _P, c_int, _P, _P, c_int, c_int, c_int, _P],
    "krk_mixed_attention": [_P, c_int, c_int, c_float, _P, c_int, c_int, c_int, c_int, c_int, c_int, _P, _P, _P, _P, _P, _P,
                            c_int, _P, _P, c_int, c_float, c_int, _P, c_int, c_int, c_int, c_int, _P],
    "krk_mixed_attention_single": [_P, c_int, c_int, c_float, _P, c_int, c_int, c_int, c_int, c_int, c_int, _P, _P, _P, _P,
                                   _P, c_int, _P, _P, c_int, c_float, c_int, c_int, _P, _P, c_int, c_int, c_int, c_int, _P],
    "krk_mixed_attention_merge": [_P, c_int, c_int, c_float, _P, c_int, c_int, c_int, c_int, _P, c_int, c_int, c_int, c_int, _P],
    "krk_norm_sum": [_P, _P, _P, _P, _P, c_int, _P, c_int, c_int, c_float, c_float, c_int, _P],
    "krk_act_rows": [_P, _P, c_int, c_int, c_int, c_int, c_float, c_float, c_int, _P],
}
_MOE_SIGNATURES = {
    "krk_moe_route": [_P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, _P, c_int],
    "krk_moe_route_groups": [_P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_float, _P],
    "krk_moe_gate_up_pairs": [_P, _P, c_int, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, _P],
    "krk_moe_down_pairs": [_P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, _P],
    "krk_moe_sort": [_P, _P, _P, c_int, c_int, c_int, _P],
    "krk_moe_gather": [_P, _P, c_int, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, _P],
    "krk_moe_combine": [_P, _P, _P, _P, _P, _P, _P, c_int, _P, c_int, c_int, c_int, c_int, _P],
}
_SCAN_SIGNATURES = {
    "krk_token_shift": [_P, _P, c_int, _P, _P, c_int, c_int, c_int, _P, _P, _P, c_int, _P, c_int],
    "krk_linear_recurrence": [c_int, _P, c_int, _P, c_int, _P, c_int, _P, c_int, _P, c_int, _P, c_int, _P, _P, _P, _P, _P,
                              _P, _P, c_int, c_int, _P, _P, c_int, c_int, c_float, c_float, c_float, c_int, c_int, c_int,
                              c_int, _P, _P, _P, c_int, _P, _P, c_int, _P],
    "krk_causal_conv_silu": [_P, _P, c_int, _P, _P, _P, c_int, c_int, c_int, c_int, _P, _P, _P, _P, c_int, _P],
    "krk_ssd_scan": [_P, _P, c_int, _P, c_int, _P, c_int, _P, c_int, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int,
                     c_int, _P, _P, _P, c_int, _P, _P, c_int, _P],
    "krk_gated_group_norm": [_P, c_int, c_int, c_float, _P, _P, c_int, _P, c_int, c_int, c_int, c_float, c_int, _P],
}
_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "sigmoid": 2, "swish_clamped": 3, "xielu": 4}
_ATTN_SIGNATURES = {
    "krk_attention_simple": [_P, _P, c_int, c_int, c_int, _P, _P, _P, _P, c_int, _P, _P, c_int, c_float, c_int, c_int, _P],
    "krk_attention_head_dim": [],
    "krk_attention_prefill": [_P, _P, c_int, c_int, c_int, _P, _P, _P, _P, _P, c_int, _P, _P, c_int, c_int, c_float,
                              c_int, _P],
    "krk_sink_window_prefill": [_P, c_int, c_float, _P, c_int, c_int, c_int, _P, _P, _P, _P, _P, _P, c_int, _P, _P, c_int,
                                c_int, c_float, c_int, c_int, c_int, _P, c_int, c_int, _P],
    "krk_mixed_prefill": [_P, c_int, c_float, _P, c_int, c_int, c_int, _P, _P, _P, _P, _P, _P, _P, c_int, _P, _P, c_int,
                          c_int, c_float, c_int, _P, c_int, c_int, _P, c_int, _P],
    "krk_attention_decode": [_P, _P, c_int, c_int, c_int, _P, _P, _P, c_int, _P, _P, c_int, c_float, c_int, c_int, _P,
                             _P],
    "krk_attention_prefill_tcgen05": [_P, _P, c_int, c_int, c_int, _P, _P, _P, _P, _P, c_int, _P, _P, c_int, c_int, c_int,
                                      c_int, c_float, c_int, _P, _P],
    "krk_attention_decode_fused": [_P, _P, c_int, c_int, c_int, _P, _P, c_int, _P, _P, c_float, _P, _P, _P, c_int, _P,
                                   _P, c_int, c_float, c_int, c_int, c_int, _P, _P],
    "krk_attention_decode_fused_tma": [_P, _P, c_int, c_int, c_int, _P, _P, c_int, _P, _P, c_float, _P, _P, _P, c_int, _P,
                                       _P, c_int, c_int, c_float, c_int, c_int, c_int, _P, _P],
}


def _load(path, signatures) -> ctypes.CDLL:
    lib = ctypes.CDLL(str(path))
    for name, args in signatures.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            continue
        fn.argtypes = args
        fn.restype = c_int
    return lib


def _ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


class Kernels:
    """All kernels, for one device. ``head_dims``: the head sizes whose attention
    libraries are needed (compiled at first use)."""

    SKINNY_MAX_ROWS = 16  # rows up to which the fused skinny kernels serve a bfloat16 product
    # Every block of a skinny product redoes the norm of all rows in its prologue. That is
    # cheaper than a separate norm kernel for one or two rows and dearer beyond.
    FUSED_NORM_MAX_ROWS = 2

    def __init__(self, head_dims=(), device="cuda:0"):
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device: this library computes with its CUDA kernels only")
        self.device = torch.device(device)
        self.core = _load(build_library("core"), _SIGNATURES)
        self._mix = self._scan = self._moe = None
        self.attn: dict[int, ctypes.CDLL] = {}
        for d in head_dims:
            self._attn_lib(int(d))
        self.error = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.has_skinny = hasattr(self.core, "krk_skinny_linear")
        self._partials: dict = {}
        self._select_scratch = None
        self.use_tcgen05_attention = True
        self.use_tma_decode_attention = True
        # Key-split counts that take the TMA-fed single-token attention. It splits keys over a cluster like the
        # cp.async kernel, bit for bit; measured on the 4B shape it wins with one block or two per item (16 sequences
        # at 8,000 tokens of context: 4.95 against 5.53 ms a step) and loses with more (one sequence at 32,000
        # tokens: 4.08 against 3.14 ms), where a block's own pace, not the bytes in flight, is the bound.
        self.tma_decode_splits = {1, 2}
        self.use_tuned_library_gemm = hasattr(self.core, "krk_lt_gemm_bf16")
        # steps of many tokens: prepare / scan / finish kernels instead of the fused one. Bit-equal to it and, on one
        # prompt, no faster (the scan itself bounds both), so it is off; it needs rows * channels * 28 bytes of scratch
        self.split_recurrence = False
        # single-token steps: rotation, value norm and cache write inside the attention kernel (one launch fewer a
        # layer). Right, and slower (8 sequences of the 1.5k-wide preset: 0.608 against 0.563 ms a step; one sequence
        # 0.510 against 0.497): every block of an item repeats the prologue on its critical path, where the kernel of
        # its own runs under the product before it. Off.
        self.fuse_single_token_attention = os.environ.get("KRK_FUSE_SINGLE_ATTENTION") is not None
        self.launches = 0

    def _attn_lib(self, head_dim: int) -> ctypes.CDLL:
        lib = self.attn.get(head_dim)
        if lib is None:
            if head_dim % 2 or head_dim > 256:
                raise KernelError(f"attention kernels take an even head size up to 256, got {head_dim}")
            lib = self.attn[head_dim] = _load(build_library("attn", head_dim), _ATTN_SIGNATURES)
            assert lib.krk_attention_head_dim() == head_dim
        return lib

    # -- plumbing -------------------------------------------------------------
    def _stream(self):
        return torch.cuda.current_stream(self.device).cuda_stream

    def _ok(self, code: int, what: str) -> None:
        self.launches += 1
        if code != 0:
            detail = {-2: "a size is outside what the kernel takes", -3: "the grid would be too large",
                      -4: "unsupported dtype combination"}.get(code, f"CUDA error {code}")
            raise KernelError(f"{what}: {detail}")

    def check(self) -> None:
        """Read the kernels' error word; if a kernel flagged bad input (a token id or position out of
        range: the row was zeroed or skipped) or gave up on a bounded wait since the last look, clear
        the word and raise. The results of the step that raised it are not to be used. The generation
        loop reads the word with every step's tokens, the step function at the end of every
        multi-token step."""
        flag = int(self.error.item())
        if flag:
            self.error.zero_()
            raise KernelError(self.describe(flag))

    @staticmethod
    def describe(flag: int) -> str:
        known = {1: "a token id outside the embedding table reached the device",
                 2: "a position outside the rotary table reached the device",
                 3: "a tensor-core GEMM gave up waiting for a free shared-memory stage",
                 4: "a tensor-core GEMM gave up waiting for a TMA load",
                 5: "a tensor-core GEMM gave up waiting for its accumulator",
                 21: "the wait of the self-test kernel ran out (as it is meant to)"}
        if flag in known:
            return known[flag]
        if 6 <= flag <= 14:
            return f"the tensor-core attention kernel gave up on a barrier wait (code {flag})"
        return f"error flag {flag}"

    def selftest_wait_runs_out(self, limit_us: int = 1000) -> None:
        """Launch a kernel whose only wait, on a barrier nobody arrives at, runs out after ``limit_us``
        and sets the error word; ``check`` then raises. For the tests of the error path."""
        self._ok(self.core.krk_selftest_wait_runs_out(self.error.data_ptr(), int(limit_us), self._stream()), "self-test wait")

    def empty_like(self, x):
        return torch.empty_like(x)

    @staticmethod
    def _resolve(x):
        return x if isinstance(x, torch.Tensor) else x.tensor()

    # -- rows -------------------------------------------------------------------
    def embed(self, table, tokens, n_rows):
        out = torch.empty((n_rows, table.shape[1]), dtype=table.dtype, device=table.device)
        self._ok(self.core.krk_gather_rows(out.data_ptr(), table.data_ptr(), tokens.data_ptr(), n_rows, table.shape[1],
                                           table.shape[0], self.error.data_ptr(), _code(table.dtype), self._stream()),
                 "embedding gather")
        return out

    def gather_rows(self, x, idx):
        n = idx.shape[0]
        out = torch.empty((n, x.shape[1]), dtype=x.dtype, device=x.device)
        self._ok(self.core.krk_gather_rows(out.data_ptr(), x.data_ptr(), idx.data_ptr(), n, x.shape[1], x.shape[0],
                                           self.error.data_ptr(), _code(x.dtype), self._stream()), "row gather")
        return out

    def rmsnorm(self, x, gain, eps):
        out = torch.empty_like(x)
        self._ok(self.core.krk_rmsnorm(out.data_ptr(), None, x.data_ptr(), None, gain.data_ptr(),
                                       int(gain.dtype == torch.float32), x.shape[0], x.shape[1], eps, _code(x.dtype),
                                       self._stream()), "rmsnorm")
        return out

    def add_rmsnorm(self, x, branch, gain, eps, x_new):
        out = torch.empty_like(x)
        self._ok(self.core.krk_rmsnorm(out.data_ptr(), x_new.data_ptr(), x.data_ptr(), branch.data_ptr(),
                                       gain.data_ptr(), int(gain.dtype == torch.float32), x.shape[0], x.shape[1], eps,
                                       _code(x.dtype), self._stream()), "add + rmsnorm")
        return out

    def swiglu(self, gu, intermediate):
        out = torch.empty((gu.shape[0], intermediate), dtype=gu.dtype, device=gu.device)
        self._ok(self.core.krk_swiglu(out.data_ptr(), gu.data_ptr(), gu.shape[0], intermediate, _code(gu.dtype),
                                      self._stream()), "swiglu")
        return out

    # -- matrix products ----------------------------------------------------------
    def _gemm_nt(self, x, w, out_dtype):
        M, K = x.shape
        N = w.shape[0]
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
        self._ok(self.core.krk_gemm_nt(out.data_ptr(), x.data_ptr(), w.data_ptr(), M, N, K, x.stride(0), w.stride(0), N,
                                       _code(x.dtype), _code(out_dtype), self._stream()), "gemm")
        return out

    def gemm_tcgen05(self, x, w, swiglu_rows=0, variant=0, out_float32=False):
        """y = x W^T (bfloat16 inputs) on the tcgen05 tensor cores; with ``swiglu_rows`` = I,
        W is [2I, K] and y is the activated [M, I] product; ``out_float32`` keeps the
        accumulator's precision (output-head logits)."""
        M, K = x.shape
        N = swiglu_rows if swiglu_rows else w.shape[0]
        out = torch.empty((M, N), dtype=torch.float32 if out_float32 else torch.bfloat16, device=x.device)
        self._ok(self.core.krk_gemm_tcgen05(out.data_ptr(), x.data_ptr(), w.data_ptr(), M, N, K, x.stride(0), w.stride(0),
                                            N, int(swiglu_rows > 0), variant, int(out_float32), self.error.data_ptr(),
                                            self._stream()),
                 "tcgen05 gemm")
        return out

    def _skinny(self, x, w, out_dtype, swiglu_rows=0, gate_act=1, act_limit=0.0):
        """x: a tensor or a Normed not yet computed (then the add and the norm run in
        the kernel's prologue)."""
        lazy = not isinstance(x, torch.Tensor)
        src = x.x if lazy else x
        M, K = src.shape
        N = swiglu_rows if swiglu_rows else w.shape[0]
        out = torch.empty((M, N), dtype=out_dtype, device=src.device)
        branch = x.branch if lazy else None
        gain = x.gain if lazy else None
        x_new = x.x_new if lazy and x.branch is not None else None
        self._ok(self.core.krk_skinny_linear(
            out.data_ptr(), src.data_ptr(), w.data_ptr(), _ptr(branch), _ptr(gain), _ptr(x_new),
            int(gain is not None and gain.dtype == torch.float32), None, M, N, K, float(x.eps) if lazy else float(act_limit),
            int(gate_act if swiglu_rows > 0 else 0), _code(out_dtype), self._stream()), "skinny product")
        if lazy:
            x.mark_fused()
        return out

    def _use_skinny(self, x, w) -> bool:
        rows = x.shape[0]
        return (self.has_skinny and w.dtype == torch.bfloat16 and 0 < rows <= self.SKINNY_MAX_ROWS
                and w.shape[1] % 32 == 0 and w.is_contiguous())

    @staticmethod
    def _fits_prologue(x) -> bool:
        """Whether the normalised rows fit the fused kernel's shared memory."""
        rows, k = x.shape
        if rows > Kernels.FUSED_NORM_MAX_ROWS:
            return False
        tiles = 1 if rows <= 8 else 2
        return 65536 + rows * (k + 64) * 2 + 8 * 2 * tiles * 512 <= 216 * 1024

    def _skinny_input(self, x):
        """A Normed goes to the kernel as it is if its norm is still to be done and fits
        the prologue; otherwise its rows are computed first."""
        if isinstance(x, torch.Tensor):
            return x
        if x.done or not self._fits_prologue(x):
            return x.tensor()
        return x

    def linear(self, x, w, out_float32=False):
        """y = x W^T; W is [out, in]. x may be a Normed (see parts/norm.py)."""
        out_dtype = torch.float32 if out_float32 else w.dtype
        if self._use_skinny(x, w):
            return self._skinny(self._skinny_input(x), w, out_dtype)
        x = self._resolve(x)
        if x.shape[0] == 0:
            return torch.empty((0, w.shape[0]), dtype=out_dtype, device=x.device)
        if w.dtype == torch.float32:
            return self._gemm_nt(x, w, out_dtype)
        if out_float32:  # many rows of float32 logits: the tcgen05 GEMM keeps the accumulator's precision
            if (x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
                    and w.data_ptr() % 16 == 0 and hasattr(self.core, "krk_gemm_tcgen05")):
                return self.gemm_tcgen05(x, w, out_float32=True)
            return self._gemm_nt(x, w, out_dtype)
        if (self.use_tuned_library_gemm and x.stride(1) == 1 and w.stride(1) == 1 and x.stride(0) % 8 == 0
                and w.stride(0) % 8 == 0 and w.shape[0] % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0):
            return self._library_gemm(x, w)
        return torch.matmul(x, w.t())

    def _library_gemm(self, x, w):
        """The library's product with the algorithm picked by measurement (csrc/lt_gemm.cu)."""
        M, K = x.shape
        N = w.shape[0]
        out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
        rc = self.core.krk_lt_gemm_bf16(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, x.stride(0), w.stride(0), N, 1,
                                        None, self._stream())
        if rc:
            raise KernelError(f"the library product of {M} x {N} x {K} failed with code {rc}")
        return out

    def library_gemm_report(self):
        """(shape classes with a measured choice, how many of them kept the heuristic's first proposal)."""
        a, b = c_int(0), c_int(0)
        self.core.krk_lt_gemm_report(ctypes.byref(a), ctypes.byref(b))
        return a.value, b.value

    def gate_up_swiglu(self, h, w_gate_up, intermediate):
        if self._use_skinny(h, w_gate_up):
            return self._skinny(self._skinny_input(h), w_gate_up, w_gate_up.dtype, swiglu_rows=intermediate)
        return self.swiglu(self.linear(h, w_gate_up), intermediate)

    # -- attention ------------------------------------------------------------------
    def qk_norm_rope_write(self, qkv, heads, kv_in_row, head_dim, q_gain, k_gain, eps, cos, sin, batch, cache):
        gain = q_gain if q_gain is not None else k_gain
        n_pos = cos.shape[0] if cos is not None else 0x7fffffff
        rot = self._rotated_width(cos, head_dim)
        self._ok(self.core.krk_qk_norm_rope_write(
            qkv.data_ptr(), _ptr(q_gain), _ptr(k_gain), int(gain is not None and gain.dtype == torch.float32),
            _ptr(cos), _ptr(sin), batch.row_seq.data_ptr(), batch.row_pos.data_ptr(), batch.seq_slot.data_ptr(),
            cache.table.data_ptr(), cache.width, cache.k.data_ptr() if kv_in_row else None,
            cache.v.data_ptr() if kv_in_row else None, qkv.shape[0], heads, kv_in_row, head_dim, rot, eps, n_pos,
            self.error.data_ptr(), _code(qkv.dtype), self._stream()), "q/k norm + rope + cache write")

    @staticmethod
    def _rotated_width(cos, head_dim: int) -> int:
        """The width of the head that the tables rotate: all of it, or its first 2 * columns elements."""
        if cos is None:
            return head_dim
        rot = 2 * cos.shape[1]
        if rot > head_dim or not cos.is_contiguous():
            raise KernelError(f"rotary tables of {cos.shape[1]} columns do not fit a head of {head_dim} (at most half of it, contiguous)")
        return rot

    def rope_attention(self, qkv, heads, kv_in_row, head_dim, q_gain, k_gain, eps, cos, sin, batch, cache, scale,
                       window):
        """Per-head q/k norm, rotation, cache write and attention. A single-token step in
        bfloat16 runs them as one kernel; everything else as two."""
        lib = self._attn_lib(head_dim)
        if (batch.is_decode and qkv.dtype == torch.bfloat16 and head_dim % 16 == 0 and kv_in_row > 0
                and hasattr(lib, "krk_attention_decode_fused") and qkv.shape[0] > 0
                and self._rotated_width(cos, head_dim) == head_dim):  # the fused kernel rotates the whole head
            n = batch.n_seqs
            out = torch.empty((n, heads * head_dim), dtype=qkv.dtype, device=qkv.device)
            row_tiles = -(-(heads // cache.kv_heads) // 16)
            # key splits (blocks per cluster) by the number of (sequence, kv head, row tile) items alone,
            # never by lengths, so a captured step stays valid; measured best on B200 at 1, 2 to 4, 8, 16 and 32 or
            # 64 sequences of the 4B shape: 16, 8, 4, 2 and 1 (one block per item runs a deeper page pipeline). One
            # sequence has eight items: sixteen splits are 128 blocks where eight are 64, and what bounds the
            # kernel is the bytes its blocks have in flight (one step of the 4B shape at 32,000 tokens of context:
            # 4.41 -> 3.14 ms, at 8,000: 2.51 -> 2.17, at 1,000: 1.93 -> 1.91; at two sequences sixteen gain nothing)
            items = n * cache.kv_heads * row_tiles
            splits = 16 if items <= 9 else 8 if items <= 37 else 4 if items <= 74 else 2 if items <= 192 else 1
            gain = q_gain if q_gain is not None else k_gain
            n_pos = cos.shape[0] if cos is not None else 0x7fffffff
            if (splits in self.tma_decode_splits and self.use_tma_decode_attention and head_dim % 64 == 0
                    and cache.width <= 1024 and hasattr(lib, "krk_attention_decode_fused_tma")):
                # many sequences: one block or two per (sequence, kv head), pages by TMA into a ring of half page-pairs
                rc = lib.krk_attention_decode_fused_tma(
                    out.data_ptr(), qkv.data_ptr(), qkv.stride(0), heads, cache.kv_heads, _ptr(q_gain), _ptr(k_gain),
                    int(gain is not None and gain.dtype == torch.float32), _ptr(cos), _ptr(sin), eps,
                    batch.seq_slot.data_ptr(), batch.seq_start.data_ptr(), cache.table.data_ptr(), cache.width,
                    cache.k.data_ptr(), cache.v.data_ptr(), cache.k.shape[0], n, scale, int(window or 0), splits, n_pos,
                    self.error.data_ptr(), self._stream())
                if rc != -2:  # -2: the shapes do not fit this kernel's shared memory; the kernel below takes them
                    self._ok(rc, "fused decode attention (TMA)")
                    return out
            self._ok(lib.krk_attention_decode_fused(
                out.data_ptr(), qkv.data_ptr(), qkv.stride(0), heads, cache.kv_heads, _ptr(q_gain), _ptr(k_gain),
                int(gain is not None and gain.dtype == torch.float32), _ptr(cos), _ptr(sin), eps,
                batch.seq_slot.data_ptr(), batch.seq_start.data_ptr(), cache.table.data_ptr(), cache.width,
                cache.k.data_ptr(), cache.v.data_ptr(), n, scale, int(window or 0), splits, n_pos,
                self.error.data_ptr(), self._stream()), "fused decode attention")
            return out
        self.qk_norm_rope_write(qkv, heads, kv_in_row, head_dim, q_gain, k_gain, eps, cos, sin, batch, cache)
        return self.attention(qkv, heads, kv_in_row, head_dim, batch, cache, scale, window)

    def attention(self, qkv, heads, kv_in_row, head_dim, batch, cache, scale, window):
        lib = self._attn_lib(head_dim)
        rows = qkv.shape[0]
        out = torch.empty((rows, heads * head_dim), dtype=qkv.dtype, device=qkv.device)
        if rows == 0:
            return out
        stride = qkv.stride(0)
        win = int(window or 0)
        fast = qkv.dtype == torch.bfloat16 and head_dim % 16 == 0
        if fast and batch.is_decode and hasattr(lib, "krk_attention_decode"):
            splits, parts = self._decode_partials(batch.n_seqs, heads, cache.kv_heads, head_dim)
            self._ok(lib.krk_attention_decode(
                out.data_ptr(), qkv.data_ptr(), stride, heads, cache.kv_heads, batch.seq_slot.data_ptr(),
                batch.seq_start.data_ptr(), cache.table.data_ptr(), cache.width, cache.k.data_ptr(),
                cache.v.data_ptr(), batch.n_seqs, scale, win, splits, parts.data_ptr(), self._stream()),
                "decode attention")
        elif (fast and self.use_tcgen05_attention and head_dim in (64, 128) and hasattr(lib, "krk_attention_prefill_tcgen05")
              and batch.max_q_len * (heads // cache.kv_heads) >= 128 and stride % 8 == 0):
            # long steps: the tcgen05 kernel (128-row tiles of (token, group member) pairs)
            self._ok(lib.krk_attention_prefill_tcgen05(
                out.data_ptr(), qkv.data_ptr(), stride, heads, cache.kv_heads, batch.seq_slot.data_ptr(),
                batch.seq_start.data_ptr(), batch.seq_qlen.data_ptr(), batch.cu_q.data_ptr(), cache.table.data_ptr(),
                cache.width, cache.k.data_ptr(), cache.v.data_ptr(), cache.k.shape[0], batch.n_seqs, batch.max_q_len,
                rows, scale, win, self.error.data_ptr(), self._stream()), "tcgen05 prefill attention")
        elif fast and hasattr(lib, "krk_attention_prefill"):
            self._ok(lib.krk_attention_prefill(
                out.data_ptr(), qkv.data_ptr(), stride, heads, cache.kv_heads, batch.seq_slot.data_ptr(),
                batch.seq_start.data_ptr(), batch.seq_qlen.data_ptr(), batch.cu_q.data_ptr(), cache.table.data_ptr(),
                cache.width, cache.k.data_ptr(), cache.v.data_ptr(), batch.n_seqs, batch.max_q_len, scale, win,
                self._stream()), "prefill attention")
        else:
            self._ok(lib.krk_attention_simple(
                out.data_ptr(), qkv.data_ptr(), stride, heads, cache.kv_heads, batch.row_seq.data_ptr(),
                batch.row_pos.data_ptr(), batch.seq_slot.data_ptr(), cache.table.data_ptr(), cache.width,
                cache.k.data_ptr(), cache.v.data_ptr(), rows, scale, win, _code(qkv.dtype), self._stream()),
                "attention")
        return out

    def _decode_partials(self, n_seqs: int, heads: int, kv_heads: int, head_dim: int):
        """Number of key splits for a decode step and the float32 scratch its partial
        results go through. The split count depends on the batch size only, never on
        lengths, so a captured step stays valid as sequences grow."""
        row_tiles = -(-(heads // kv_heads) // 16)
        splits = max(1, min(32, -(-296 // (n_seqs * kv_heads * row_tiles))))
        key = (n_seqs, heads, head_dim, splits)
        buf = self._partials.get(key)
        if buf is None:
            buf = self._partials[key] = torch.empty(n_seqs * heads * splits * (head_dim + 2), dtype=torch.float32,
                                                    device=self.device)
        return splits, buf

    # -- 32-bit residual stream, windowed attention with a sink, recurrent state -------------------
    @property
    def mix(self) -> ctypes.CDLL:
        """The library of these kernels, compiled and loaded when a model first asks for one of them."""
        if self._mix is None:
            self._mix = _load(build_library("mix"), _MIX_SIGNATURES)
        return self._mix

    @property
    def scan(self) -> ctypes.CDLL:
        """The library of the recurrent-state kernels, compiled and loaded at their first call."""
        if self._scan is None:
            self._scan = _load(build_library("scan"), _SCAN_SIGNATURES)
        return self._scan

    @property
    def moe(self) -> ctypes.CDLL:
        """The library of the routed-experts kernels, compiled and loaded at their first call."""
        if self._moe is None:
            self._moe = _load(build_library("moe"), _MOE_SIGNATURES)
        return self._moe

    @staticmethod
    def _rows_view(t):
        """(pointer, row stride) of a 2-D view whose rows are contiguous."""
        if t.dim() != 2 or t.stride(1) != 1:
            raise KernelError("a kernel input must be a 2-D tensor (or column slice) with contiguous rows")
        return t.data_ptr(), t.stride(0)

    def embed_scaled(self, table, tokens, n_rows, scale, copies=1):
        """float32 rows table[token] * scale, each written ``copies`` times side by side."""
        out = torch.empty((n_rows, copies * table.shape[1]), dtype=torch.float32, device=table.device)
        self._ok(self.mix.krk_embed_scaled(out.data_ptr(), table.data_ptr(), tokens.data_ptr(), n_rows, table.shape[1],
                                           table.shape[0], float(scale), self.error.data_ptr(), _code(table.dtype),
                                           self._stream(), int(copies)), "scaled embedding gather")
        return out

    def hyper_rmsnorm(self, x, branch, fold, read, gain, offset, eps, x_new, out_dtype):
        """Rows of S float32 streams side by side. With a pending ``branch``, the streams are rewritten into ``x_new``
        through ``fold`` (M [S, S] indexed [from, to], then b [S]): x_t = sum_s M[s, t] x_s + b_t * branch. Returns
        norm(sum_s read[s] x_s) * (offset + gain) in ``out_dtype``."""
        S = read.shape[0]
        rows, C = x.shape[0], x.shape[1] // S
        if x.dtype != torch.float32 or not x.is_contiguous() or gain.dtype != torch.float32 or gain.shape[0] != C:
            raise KernelError("the hyper-connection norm reads contiguous float32 streams and a float32 gain")
        if branch is not None and (branch.dtype != out_dtype or not branch.is_contiguous() or branch.shape != (rows, C)
                                   or fold is None or fold.numel() != S * S + S):
            raise KernelError("the pending output must have the path's dtype and one stream's shape, with its M and b")
        out = torch.empty((rows, C), dtype=out_dtype, device=x.device)
        self._ok(self.mix.krk_hyper_rmsnorm(out.data_ptr(), x_new.data_ptr() if branch is not None else None, x.data_ptr(),
                                            _ptr(branch), _ptr(fold) if branch is not None else None, read.data_ptr(),
                                            gain.data_ptr(), float(offset), rows, S, C, float(eps), _code(out_dtype),
                                            self._stream()), "hyper-connection rmsnorm")
        return out

    def bias_row_norm(self, proj, cols, bias, gain, eps):
        """In place on a stacked q | k | v product: ``cols`` = (q0, k0, v0, end) column bounds; float32 ``bias`` over
        q0..end is added (None: none), and with ``gain`` (float32 over q0..v0) the q columns and the k columns are each
        divided by their root mean square and multiplied by it."""
        ptr, stride = self._rows_view(proj)
        q0, k0, v0, end = (int(c) for c in cols)
        if (bias is not None and bias.numel() != end - q0) or (gain is not None and gain.numel() != v0 - q0):
            raise KernelError("bias and gain must cover the columns they are applied to")
        self._ok(self.mix.krk_bias_row_norm(ptr, stride, q0, k0, v0, end, _ptr(bias), _ptr(gain), float(eps), proj.shape[0],
                                            _code(proj.dtype), self._stream()), "projection biases + row norms")

    def rmsnorm_wide(self, x, branch, gain, offset, eps, x_new, out_dtype, branch2=None, scale=1.0, gain2=None):
        """Rows of a float32 stream, normalised into ``out_dtype``; with a branch, ``x_new`` = x + scale * (branch +
        branch2) (float32). With a second gain, two results of the one pass: (rows, rows2)."""
        if x.dtype != torch.float32 or gain.dtype != torch.float32 or not x.is_contiguous():
            raise KernelError("the wide norm reads a contiguous float32 stream and a float32 gain")
        for b in (branch, branch2):
            if b is not None and (b.dtype != out_dtype or not b.is_contiguous() or b.shape != x.shape):
                raise KernelError("the wide norm's branch must have the path's dtype and the stream's shape")
        if gain2 is not None and (gain2.dtype != torch.float32 or gain2.shape != gain.shape):
            raise KernelError("the wide norm's second gain must be float32 and of the first one's size")
        out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
        out2 = torch.empty(x.shape, dtype=out_dtype, device=x.device) if gain2 is not None else None
        self._ok(self.mix.krk_rmsnorm_wide(out.data_ptr(), x_new.data_ptr() if branch is not None else None, x.data_ptr(),
                                           _ptr(branch), gain.data_ptr(), float(offset), x.shape[0], x.shape[1], float(eps),
                                           _ptr(branch2), float(scale), _ptr(gain2), _ptr(out2), _code(out_dtype),
                                           self._stream()), "wide rmsnorm")
        return out if gain2 is None else (out, out2)

    def gated_act(self, gu, intermediate, activation, row_gate_col=None, act_params=None):
        """act(gu[:, :I]) * gu[:, I:2I], times sigmoid(gu[:, row_gate_col]) per row if that column is given.
        "swish_clamped" takes ``act_params`` = (limit, slope)."""
        ptr, stride = self._rows_view(gu)
        out = torch.empty((gu.shape[0], intermediate), dtype=gu.dtype, device=gu.device)
        limit, slope = act_params if act_params is not None else (0.0, 1.0)
        if activation == "swish_clamped" and act_params is None:
            raise KernelError("the clamped activation needs its limit and slope")
        self._ok(self.mix.krk_gated_act(out.data_ptr(), ptr, stride, gu.shape[0], intermediate, _ACTIVATIONS[activation],
                                        -1 if row_gate_col is None else int(row_gate_col), _code(gu.dtype),
                                        self._stream(), float(limit), float(slope)), "gated activation")
        return out

    def latent_norm_write(self, proj, c_col, rank, gain, eps, batch, cache, keep_rows=False):
        """The rows' ``rank`` columns from ``c_col`` on, RMS-normed with a float32 gain, into the cache (one head);
        with ``keep_rows`` the normalised rows are returned as well, [rows, rank]."""
        ptr, stride = self._rows_view(proj)
        if cache.k.dtype != proj.dtype or cache.head_dim != rank or cache.kv_heads != 1 or gain.dtype != torch.float32:
            raise KernelError("the cache does not fit the latent rows it is to receive")
        kept = torch.empty((proj.shape[0], rank), dtype=proj.dtype, device=proj.device) if keep_rows else None
        self._ok(self.mix.krk_latent_norm_write(ptr, stride, int(c_col), int(rank), gain.data_ptr(), float(eps),
                                                batch.row_seq.data_ptr(), batch.row_pos.data_ptr(),
                                                batch.seq_slot.data_ptr(), cache.table.data_ptr(), cache.width,
                                                int(getattr(cache, "keep_pages", 0)), cache.k.data_ptr(), proj.shape[0],
                                                _ptr(kept), _code(proj.dtype), self._stream()), "latent norm + cache write")
        return kept

    def head_linear(self, x, w, out=None, out_col=0, out_scale=1.0):
        """out[r, h, :] = out_scale * W_h x[r, h, :]; W [heads, N, K] contiguous, x [rows, heads * K] (rows may be strided)."""
        heads, N, K = w.shape
        ptr, stride = self._rows_view(x)
        if x.shape[1] != heads * K or w.dtype != x.dtype or not w.is_contiguous():
            raise KernelError("the per-head product reads [rows, heads * K] rows and a contiguous [heads, N, K] weight of one dtype")
        if out is None:
            out = torch.empty((x.shape[0], heads * N), dtype=x.dtype, device=x.device)
        optr, ostride = self._rows_view(out)
        rows = x.shape[0]
        if rows > self.SKINNY_MAX_ROWS and x.dtype == torch.bfloat16:
            # many rows in bfloat16: the library's batched product, one batch entry per head
            y = torch.bmm(x.view(rows, heads, K).transpose(0, 1), w.transpose(1, 2))  # [heads, rows, N]
            dst = out[:, out_col:out_col + heads * N].view(rows, heads, N)
            if out_scale == 1.0:
                dst.copy_(y.transpose(0, 1))
            else:
                torch.mul(y.transpose(0, 1), out_scale, out=dst)
            return out
        self._ok(self.mix.krk_head_linear(optr, ostride, int(out_col), float(out_scale), ptr, stride, w.data_ptr(), heads, N,
                                          K, x.shape[0], _code(x.dtype), self._stream()), "per-head product")
        return out

    # -- routed experts ------------------------------------------------------------------------
    MOE_PAIR_ROWS = 16  # rows up to which every (row, expert) pair reads its expert's weights by itself

    def moe_route(self, x, w, b, top, gate_row=False, over_all=False, sigmoid_groups=None):
        """(experts int32 [rows, top], weights float32 [rows, top], row gate float32 [rows] or None): the ``top`` largest
        of x W^T + b in 32-bit (ties: the lower index) and the softmax over them, or with ``over_all`` their shares of
        the softmax over all experts. With ``gate_row`` the last row of W is no expert but a gate's weights: sigmoid
        of its product is the row gate. ``sigmoid_groups`` = (correction, groups, keep, scale): sigmoid scores, the choice
        by score + correction among the experts of the ``keep`` best of ``groups`` groups of neighbours, the weights
        the chosen scores over their sum, times ``scale``."""
        E = w.shape[0] - int(gate_row)
        rows, K = x.shape
        experts = torch.empty((rows, top), dtype=torch.int32, device=x.device)
        weights = torch.empty((rows, top), dtype=torch.float32, device=x.device)
        row_gate = torch.empty(rows, dtype=torch.float32, device=x.device) if gate_row else None
        logits = self.linear(x, w, out_float32=True)
        if sigmoid_groups is not None:
            correction, groups, keep, scale = sigmoid_groups
            if correction.dtype != torch.float32 or correction.numel() != E:
                raise KernelError("the routing correction is one float32 number per expert")
            self._ok(self.moe.krk_moe_route_groups(experts.data_ptr(), weights.data_ptr(), _ptr(row_gate), logits.data_ptr(),
                                                   correction.data_ptr(), rows, E, int(gate_row), int(top), int(groups),
                                                   int(keep), float(scale), self._stream()), "expert routing within groups")
            return experts, weights, row_gate
        self._ok(self.moe.krk_moe_route(experts.data_ptr(), weights.data_ptr(), _ptr(row_gate), logits.data_ptr(), _ptr(b),
                                        rows, E, int(gate_row), int(top), self._stream(), int(over_all)), "expert routing")
        return experts, weights, row_gate

    def moe_experts(self, x, w_gate_up, w_down, experts, weights, intermediate, activation, add=None, add_gate=None,
                    batch=None):
        """add * add_gate + sum_j weights[r, j] * expert_{experts[r, j]}(x[r]); w_gate_up [E, 2F, K], w_down [E, C, F];
        ``add_gate``: one float32 number per row (None: 1)."""
        rows, top = experts.shape
        E, C, F = w_down.shape
        K = x.shape[1]
        ptr, stride = self._rows_view(x)
        out = torch.empty((rows, C), dtype=x.dtype, device=x.device)
        act = _ACTIVATIONS[activation]
        single = batch is not None and batch.is_decode  # such a step may be replayed from a graph: nothing comes to the host
        if single or rows * top <= max(self.MOE_PAIR_ROWS * top, 2 * E):
            pairs = torch.empty((rows * top, F), dtype=x.dtype, device=x.device)
            self._ok(self.moe.krk_moe_gate_up_pairs(pairs.data_ptr(), ptr, stride, w_gate_up.data_ptr(), experts.data_ptr(),
                                                    rows, top, F, K, act, _code(x.dtype), self._stream()), "experts' gate/up")
            self._ok(self.moe.krk_moe_down_pairs(out.data_ptr(), _ptr(add), _ptr(add_gate), pairs.data_ptr(), w_down.data_ptr(),
                                                 experts.data_ptr(), weights.data_ptr(), rows, top, C, F, _code(x.dtype),
                                                 self._stream()), "experts' down")
            return out
        # many rows: ordered by expert on the device; the experts' row counts come to the host (a step of many
        # tokens is never replayed from a graph)
        offsets = torch.empty(E + 1, dtype=torch.int32, device=x.device)
        place = torch.empty(rows * top, dtype=torch.int32, device=x.device)
        self._ok(self.moe.krk_moe_sort(offsets.data_ptr(), place.data_ptr(), experts.data_ptr(), rows, top, E,
                                       self._stream()), "expert ordering")
        bounds = offsets.tolist()
        most = max(bounds[e + 1] - bounds[e] for e in range(E))
        cap = -(-most // 16) * 16
        batched = x.dtype == torch.bfloat16 and E * cap <= 4 * rows * top
        if not batched:
            cap = 0
        n_rows = E * cap if batched else rows * top
        xg = torch.empty((n_rows, K), dtype=x.dtype, device=x.device)
        self._ok(self.moe.krk_moe_gather(xg.data_ptr(), ptr, stride, place.data_ptr(), experts.data_ptr(), offsets.data_ptr(),
                                         cap, rows, top, K, _code(x.dtype), self._stream()), "expert gather")
        if batched:
            # bfloat16: every expert's rows start at a multiple of cap (the most rows any expert got), and the
            # library's batched product takes all experts at once; the rows beyond an expert's own are never read back
            gu = torch.bmm(xg.view(E, cap, K), w_gate_up.transpose(1, 2))
            h = self.gated_act(gu.view(E * cap, 2 * F), F, activation)
            yg = torch.bmm(h.view(E, cap, F), w_down.transpose(1, 2)).view(E * cap, C)
        else:
            yg = torch.empty((n_rows, C), dtype=x.dtype, device=x.device)
            for e in range(E):
                a, b = bounds[e], bounds[e + 1]
                if b > a:
                    h = self.gate_up_act(xg[a:b], w_gate_up[e], F, activation)
                    yg[a:b] = self.linear(h, w_down[e])
        self._ok(self.moe.krk_moe_combine(out.data_ptr(), _ptr(add), _ptr(add_gate), yg.data_ptr(), place.data_ptr(), experts.data_ptr(),
                                          offsets.data_ptr(), cap, weights.data_ptr(), rows, top, C, _code(x.dtype),
                                          self._stream()), "experts' sum")
        return out

    def gate_up_act(self, h, w_gate_up, intermediate, activation, act_params=None):
        """act(gate h) * (up h) with W = cat(gate, up); silu on few bfloat16 rows runs in the product's epilogue."""
        if act_params is not None:
            if activation == "swish_clamped" and act_params[1] == 1.702 and self._use_skinny(h, w_gate_up):
                # few rows: in the product's epilogue (its clamped swish has the slope 1.702 built in)
                return self._skinny(self._resolve(h), w_gate_up, w_gate_up.dtype, swiglu_rows=intermediate, gate_act=3,
                                    act_limit=act_params[0])
            return self.gated_act(self.linear(h, w_gate_up), intermediate, activation, act_params=act_params)
        if activation == "silu" and self._use_skinny(h, w_gate_up):
            return self.gate_up_swiglu(h, w_gate_up, intermediate)
        if activation == "gelu_tanh" and self._use_skinny(h, w_gate_up):  # few rows: in the product's epilogue
            return self._skinny(self._resolve(h), w_gate_up, w_gate_up.dtype, swiglu_rows=intermediate, gate_act=2)
        return self.gated_act(self.linear(h, w_gate_up), intermediate, activation)

    def rotate_norm_write(self, proj, q_col, k_col, v_col, heads, kv_heads, dim, vdim, inv_freq, rot_dims, value_eps,
                          batch, cache, value_mix=None):
        """Rotate q in place, rotate k into the cache, write v (divided by its root mean square if
        ``value_eps`` is a number) into the cache; columns are offsets into ``proj``'s rows. ``value_mix``
        (v_first rows, lambda): (1 - lambda) v + lambda v_first is what is written."""
        ptr, stride = self._rows_view(proj)
        if cache.k.dtype != proj.dtype or cache.head_dim != dim or cache.v_dim != vdim or cache.kv_heads != kv_heads:
            raise KernelError("the cache does not fit the heads it is to receive")
        mix_ptr, mix_stride, lam = None, 0, 0.0
        if value_mix is not None:
            if value_eps is not None or value_mix[0].dtype != proj.dtype or value_mix[0].shape != (proj.shape[0], kv_heads * vdim):
                raise KernelError("blended values come without a value norm, in the path's dtype, one row per row of the step")
            (mix_ptr, mix_stride), lam = self._rows_view(value_mix[0]), float(value_mix[1])
        self._ok(self.mix.krk_rotate_norm_write(
            ptr, stride, q_col, k_col, v_col, heads, kv_heads, dim, vdim, inv_freq.data_ptr(), rot_dims,
            int(value_eps is not None), float(value_eps or 0.0), batch.row_seq.data_ptr(), batch.row_pos.data_ptr(),
            batch.seq_slot.data_ptr(), cache.table.data_ptr(), cache.width, cache.k.data_ptr(), cache.v.data_ptr(),
            proj.shape[0], int(getattr(cache, "keep_pages", 0)), mix_ptr, mix_stride, lam, _code(proj.dtype),
            self._stream()), "rotation + value norm + cache write")

    def sink_attention_step(self, proj, q_col, k_col, v_col, heads, kv_heads, dim, vdim, inv_freq, rot_dims, value_eps, sink,
                            scale, window, batch, cache, out, out_col, out_scale) -> bool:
        """Rotation, value norm, cache write and attention of a single-token step as one launch (plus the merge of
        the blocks' shares). False if the step or the sizes are not of that kind: nothing was done then."""
        if not self.fuse_single_token_attention:
            return False
        if not (batch.is_decode and proj.shape[0] == batch.n_seqs) or heads // kv_heads > 8 or vdim > 128:
            return False
        return self.sink_attention(proj, q_col, heads, dim, vdim, sink, scale, window, batch, cache, out, out_col, out_scale,
                                   fuse=(k_col, v_col, inv_freq, rot_dims, value_eps))

    def sink_attention(self, proj, q_col, heads, dim, vdim, sink, scale, window, batch, cache, out, out_col, out_scale,
                       fuse=None, keep_first=0, gate=None, gate_rows=None):
        """``keep_first``: a windowed query also sees the sequence's first keys. ``gate`` (column, "head" or "element"):
        the result is multiplied by the sigmoid of those columns of ``gate_rows`` (default: of ``proj``)."""
        ptr, stride = self._rows_view(proj)
        optr, ostride = self._rows_view(out)
        keep_first = int(keep_first) if window else 0
        keep_pages = int(getattr(cache, "keep_pages", 0))
        g_ptr, g_stride, g_col, g_mode = None, 0, 0, 0
        if gate is not None:
            g_rows = proj if gate_rows is None else gate_rows
            if g_rows.dtype != proj.dtype or g_rows.shape[0] != proj.shape[0]:
                raise KernelError("the gate's rows have the queries' dtype and number")
            (g_ptr, g_stride), g_col, g_mode = self._rows_view(g_rows), int(gate[0]), {"head": 1, "element": 2}[gate[1]]
        extras = (keep_first, keep_pages, g_ptr, g_stride, g_col, g_mode)
        if batch.is_decode and proj.shape[0] == batch.n_seqs:
            # one token per sequence: a block per (sequence, kv head), its warps splitting the window's keys. The
            # choice depends on the step's shape alone, so a sequence's results do not depend on its batch
            # blocks per (sequence, kv head) by the number of such items alone, never by lengths, so that a
            # captured step stays valid: enough to give every SM a block while items are few
            items = batch.n_seqs * cache.kv_heads
            splits = 8 if items <= 18 else 4 if items <= 37 else 2 if items <= 74 else 1
            key = ("sink", batch.n_seqs, heads, vdim, splits)
            scratch = self._partials.get(key)
            if scratch is None and splits > 1:
                scratch = self._partials[key] = torch.empty(batch.n_seqs * heads * splits * (vdim + 2),
                                                            dtype=torch.float32, device=self.device)
            rc = self.mix.krk_sink_attention_single(
                optr, ostride, out_col, float(out_scale), ptr, stride, q_col, heads, cache.kv_heads, dim, vdim,
                _ptr(sink), batch.seq_slot.data_ptr(), batch.seq_start.data_ptr(), cache.table.data_ptr(), cache.width,
                cache.k.data_ptr(), cache.v.data_ptr(), batch.n_seqs, float(scale), int(window or 0), splits,
                _ptr(scratch), *((1, fuse[0], fuse[1], fuse[2].data_ptr(), fuse[3], int(fuse[4] is not None),
                                  float(fuse[4] or 0.0)) if fuse else (0, 0, 0, None, 0, 0, 0.0)),
                *extras, _code(proj.dtype), self._stream())
            if rc != -2:  # -2: heads too large for it; the general kernel takes them
                self._ok(rc, "single-token windowed attention with a sink")
                return True
            if fuse:
                return False
        elif fuse:
            return False
        if (proj.dtype == torch.bfloat16 and dim == vdim and dim % 16 == 0 and dim <= 256 and dim in self.attn
                and not batch.is_decode and hasattr(self.attn[dim], "krk_sink_window_prefill")):
            # many tokens per sequence in bfloat16: the tensor-core walk over whole pages (compiled per head size)
            esz = proj.element_size()
            rc = self.attn[dim].krk_sink_window_prefill(
                optr + out_col * esz, ostride, float(out_scale), ptr + q_col * esz, stride, heads, cache.kv_heads,
                _ptr(sink), batch.seq_slot.data_ptr(), batch.seq_start.data_ptr(), batch.seq_qlen.data_ptr(),
                batch.cu_q.data_ptr(), cache.table.data_ptr(), cache.width, cache.k.data_ptr(), cache.v.data_ptr(),
                batch.n_seqs, batch.max_q_len, float(scale), int(window or 0), keep_first, keep_pages,
                None if g_ptr is None else g_ptr + g_col * esz, g_stride, g_mode, self._stream())
            if rc != -2:  # -2: odd strides or offsets; the general kernel takes them
                self._ok(rc, "tensor-core windowed attention with a sink")
                return
        self._ok(self.mix.krk_sink_attention(
            optr, ostride, out_col, float(out_scale), ptr, stride, q_col, heads, cache.kv_heads, dim, vdim, _ptr(sink),
            batch.row_seq.data_ptr(), batch.row_pos.data_ptr(), batch.seq_slot.data_ptr(), cache.table.data_ptr(),
            cache.width, cache.k.data_ptr(), cache.v.data_ptr(), proj.shape[0], float(scale), int(window or 0),
            *extras, _code(proj.dtype), self._stream()), "windowed attention with a sink")

    # -- pair-hash embedding, per-head norms with pair rotation, mixed head scores over blocks of keys ------------
    def embed_bigram(self, table, pairs, state, buckets, mul_prev, mul_cur, batch):
        """float32 rows table[id] + pairs[(id_prev * mul_prev + id * mul_cur) % buckets] (row ``buckets`` at position 0);
        ``state`` int32 [slots, 1] holds every sequence's last token and is brought up to date."""
        if state.dtype != torch.int32 or not state.is_contiguous() or pairs.dtype != table.dtype or pairs.shape[0] != buckets + 1:
            raise KernelError("the pair embedding keeps one int32 per slot and a second table of buckets + 1 rows")
        rows = batch.n_rows
        out = torch.empty((rows, table.shape[1]), dtype=torch.float32, device=table.device)
        self._ok(self.mix.krk_embed_bigram(out.data_ptr(), table.data_ptr(), pairs.data_ptr(), batch.tokens.data_ptr(),
                                           state.data_ptr(), rows, table.shape[1], table.shape[0], int(buckets), int(mul_prev),
                                           int(mul_cur), batch.row_seq.data_ptr(), batch.row_pos.data_ptr(),
                                           batch.cu_q.data_ptr(), batch.seq_slot.data_ptr(), self.error.data_ptr(),
                                           _code(table.dtype), self._stream()), "pair-hash embedding")
        return out

    def bias_norm_rotate_write(self, proj, q_col, k_col, v_col, heads, kv_heads, dim, vdim, bias, qk_gain, eps, inv_freq,
                               rot_dims, pairs, batch, cache):
        """On a stacked q | k | v product: float32 ``bias`` over all three (None: none); with ``qk_gain`` (float32, the q
        weight then the k weight, ``dim`` each) every q and k head is divided by its root mean square and multiplied by
        it; the first ``rot_dims`` elements are rotated (``pairs``: 2i with 2i + 1, else i with i + rot_dims/2); q in
        place, k and v into their pages."""
        ptr, stride = self._rows_view(proj)
        if cache.k.dtype != proj.dtype or cache.head_dim != dim or cache.v_dim != vdim or cache.kv_heads != kv_heads:
            raise KernelError("the cache does not fit the heads it is to receive")
        n = (heads + kv_heads) * dim + kv_heads * vdim
        if (bias is not None and (bias.numel() != n or bias.dtype != torch.float32)) or (
                qk_gain is not None and (qk_gain.numel() != 2 * dim or qk_gain.dtype != torch.float32)):
            raise KernelError("float32 biases cover q, k and v; the float32 gains are one head's q weight and k weight")
        self._ok(self.mix.krk_bias_norm_rotate_write(
            ptr, stride, q_col, k_col, v_col, heads, kv_heads, dim, vdim, _ptr(bias), _ptr(qk_gain), float(eps),
            inv_freq.data_ptr(), int(rot_dims), int(bool(pairs)), batch.row_seq.data_ptr(), batch.row_pos.data_ptr(),
            batch.seq_slot.data_ptr(), cache.table.data_ptr(), cache.width, cache.k.data_ptr(), cache.v.data_ptr(),
            proj.shape[0], int(getattr(cache, "keep_pages", 0)), _code(proj.dtype), self._stream()),
            "biases + head norms + rotation + cache write")

    # bytes up to which a prompt step's tiles leave shares to be merged (measured: 51 MB of shares at 12 heads gain
    # 12 % of the attention's time, 136 MB at 32 heads lose 30 %)
    MIXED_PREFILL_SCRATCH = 64 << 20
    MIXED_SPLITS_MAX = 32  # blocks that share one sequence's keys in a single-token step

    def mixed_attention(self, proj, q_col, heads, dim, vdim, sink, talk, scale, chunk, batch, cache, out, out_col, out_scale,
                        gate=None):
        """Attention over the keys of the query's own block of ``chunk`` positions (None: all earlier keys), the heads'
        scores mixed by ``talk`` [heads, heads] before the softmax (None: not mixed), ``sink`` as in ``sink_attention``,
        ``gate`` (column, "head"). Up to 32 heads, value heads up to 256."""
        ptr, stride = self._rows_view(proj)
        optr, ostride = self._rows_view(out)
        g_col, g_mode = (int(gate[0]), 1) if gate is not None else (0, 0)
        if gate is not None and gate[1] != "head":
            raise KernelError("this attention takes a gate per head only")
        if getattr(cache, "keep_pages", 0) or cache.window:
            raise KernelError("this attention reads a cache that keeps every key")
        if talk is not None and (talk.dtype != torch.float32 or talk.shape != (heads, heads) or not talk.is_contiguous()):
            raise KernelError("the heads' mixing matrix is float32 [heads, heads]")
        chunk = int(chunk or 0)
        if batch.is_decode and proj.shape[0] == batch.n_seqs:
            # by the step's shape alone, never by lengths, so that a captured step stays valid
            most = -(-chunk // 32) if chunk else self.MIXED_SPLITS_MAX
            splits = max(1, min(self.MIXED_SPLITS_MAX, most, 148 // batch.n_seqs))
            key = ("mixed", batch.n_seqs, heads, vdim, splits)
            scratch = self._partials.get(key)
            if scratch is None:
                scratch = self._partials[key] = torch.empty(batch.n_seqs * heads * splits * (vdim + 2), dtype=torch.float32,
                                                            device=self.device)
            self._ok(self.mix.krk_mixed_attention_single(
                optr, ostride, out_col, float(out_scale), ptr, stride, q_col, heads, cache.kv_heads, dim, vdim, _ptr(sink),
                _ptr(talk), batch.seq_slot.data_ptr(), batch.seq_start.data_ptr(), cache.table.data_ptr(), cache.width,
                cache.k.data_ptr(), cache.v.data_ptr(), batch.n_seqs, float(scale), chunk, splits, scratch.data_ptr(),
                ptr, stride, g_col, g_mode, _code(proj.dtype), self._stream()), "single-token attention with mixed scores")
            self.launches += 1
            return
        if (proj.dtype == torch.bfloat16 and dim == vdim and dim in self.attn and hasattr(self.attn[dim], "krk_mixed_prefill")):
            # many tokens per sequence in bfloat16: scores and P.V on the tensor cores (compiled per head size)
            esz = proj.element_size()
            # Few tiles of unequal length (one prompt of a few thousand tokens: a tile sees 1 to chunk / 64 pages) leave
            # SMs idle while the longest runs: then every tile's pages are dealt out over 2 or 4 blocks and a merge
            # kernel adds their shares. By the step's shape; a step of many tokens is never replayed from a graph.
            rows = proj.shape[0]
            tiles = -(-batch.max_q_len // 16) * batch.n_seqs
            pages = -(-min(chunk or batch.max_kv_len, batch.max_kv_len) // 64)
            splits = 1 if tiles >= 592 or pages < 4 else (2 if tiles >= 296 else 4)
            splits = min(splits, pages)
            part = None
            while splits > 1 and rows * heads * splits * (dim + 2) * 4 > self.MIXED_PREFILL_SCRATCH:
                splits //= 2  # the shares are written and read once: beyond this size that costs more than it gains
            if splits > 1:
                need = rows * heads * splits * (dim + 2)
                part = self._partials.get("mixed_prefill")
                if part is None or part.numel() < need:
                    part = self._partials["mixed_prefill"] = torch.empty(need, dtype=torch.float32, device=self.device)
            rc = self.attn[dim].krk_mixed_prefill(
                optr + out_col * esz, ostride, float(out_scale), ptr + q_col * esz, stride, heads, cache.kv_heads, _ptr(sink),
                _ptr(talk), batch.seq_slot.data_ptr(), batch.seq_start.data_ptr(), batch.seq_qlen.data_ptr(),
                batch.cu_q.data_ptr(), cache.table.data_ptr(), cache.width, cache.k.data_ptr(), cache.v.data_ptr(),
                batch.n_seqs, batch.max_q_len, float(scale), chunk, ptr + g_col * esz, stride, g_mode, self._stream(),
                splits, _ptr(part))
            if rc != -2:  # -2: a shape it does not take; the general kernel does
                self._ok(rc, "tensor-core attention with mixed scores")
                if splits > 1:
                    self._ok(self.mix.krk_mixed_attention_merge(optr, ostride, out_col, float(out_scale), part.data_ptr(), heads,
                                                               vdim, splits, rows, ptr, stride, g_col, g_mode,
                                                               _code(proj.dtype), self._stream()),
                             "merge of a prompt's key splits")
                return
        self._ok(self.mix.krk_mixed_attention(
            optr, ostride, out_col, float(out_scale), ptr, stride, q_col, heads, cache.kv_heads, dim, vdim, _ptr(sink),
            _ptr(talk), batch.row_seq.data_ptr(), batch.row_pos.data_ptr(), batch.seq_slot.data_ptr(),
            cache.table.data_ptr(), cache.width, cache.k.data_ptr(), cache.v.data_ptr(), proj.shape[0], float(scale), chunk,
            ptr, stride, g_col, g_mode, _code(proj.dtype), self._stream()), "attention with mixed scores")

    def norm_sum(self, outs, gains, eps, scale):
        """scale * sum_b rmsnorm(outs[b]) * gains[b]: up to four [rows, C] inputs of the path's dtype, float32 gains [n, C]."""
        first = outs[0]
        n = len(outs)
        if any(o.shape != first.shape or o.dtype != first.dtype or not o.is_contiguous() for o in outs) or (
                gains.dtype != torch.float32 or gains.shape != (n, first.shape[1]) or not gains.is_contiguous()):
            raise KernelError("the summed norms read contiguous rows of one shape and dtype and float32 gains [n, C]")
        out = torch.empty_like(first)
        ptrs = [o.data_ptr() for o in outs] + [None] * (4 - n)
        self._ok(self.mix.krk_norm_sum(out.data_ptr(), *ptrs, n, gains.data_ptr(), first.shape[0], first.shape[1], float(eps),
                                       float(scale), _code(first.dtype), self._stream()), "norms of several outputs, summed")
        return out

    def act_rows(self, z, activation, params=(0.0, 0.0)):
        """An activation without a gate over [rows, I]; "xielu" takes (softplus(p), 1/2 + softplus(q))."""
        ptr, stride = self._rows_view(z)
        out = torch.empty(z.shape, dtype=z.dtype, device=z.device)
        self._ok(self.mix.krk_act_rows(out.data_ptr(), ptr, stride, z.shape[0], z.shape[1], _ACTIVATIONS[activation],
                                       float(params[0]), float(params[1]), _code(z.dtype), self._stream()), "activation")
        return out

    def token_shift(self, h, last_state, mu, batch, store=False):
        """[mixes, rows, hidden]: h + (h_prev - h) * mu, the row before a step's first coming from ``last_state``;
        with ``store`` every sequence's last row of the step then takes its place there."""
        if last_state.dtype != torch.float32 or not last_state.is_contiguous() or mu.dtype != torch.float32:
            raise KernelError("the token shift keeps a contiguous float32 row per slot and reads float32 blend weights")
        ptr, stride = self._rows_view(h)
        rows, C = h.shape
        out = torch.empty((mu.shape[0], rows, C), dtype=h.dtype, device=h.device)
        self._ok(self.scan.krk_token_shift(out.data_ptr(), ptr, stride, last_state.data_ptr(), mu.data_ptr(), mu.shape[0],
                                          C, rows, batch.row_seq.data_ptr(), batch.cu_q.data_ptr(),
                                          batch.seq_slot.data_ptr(), _code(h.dtype), self._stream(), int(store)), "token shift")
        return out

    def linear_recurrence(self, kind, r, k, v, gate, lora, w2, w0, heads, dim, norm_w, eps, state, batch, out, out_col,
                          out_scale, rate=None, rate_bias=None, decay_scale=1.0, bonus=None, last_rows=None):
        """The scan of a matrix-state mixer over a step's rows ("wkv" or "delta"); see csrc/recurrent.cu."""
        views = [self._rows_view(t) for t in (r, k, v, gate)]
        rate_v = self._rows_view(rate) if rate is not None else (None, 0)
        lora_v = self._rows_view(lora)
        optr, ostride = self._rows_view(out)
        last_ptr, last_stride, C, last_state = None, 0, 0, None
        if last_rows is not None:
            (last_ptr, last_stride), C, last_state = self._rows_view(last_rows[0]), last_rows[0].shape[1], last_rows[1]
        if state.dtype != torch.float32 or not state.is_contiguous() or not w2.is_contiguous() or w2.dtype != r.dtype:
            raise KernelError("the recurrence keeps a contiguous float32 state and reads W2 in the path's dtype")
        rows = r.shape[0]
        prep = o_raw = None
        if not batch.is_decode and dim % 4 == 0 and self.split_recurrence:
            # steps of many tokens: decays and gates over all rows at once, the scan between them (float32 scratch)
            prep = torch.empty(rows * heads * 6 * dim, dtype=torch.float32, device=r.device)
            o_raw = torch.empty(rows * heads * dim, dtype=torch.float32, device=r.device)
        rc = self.scan.krk_linear_recurrence(
            {"wkv": 0, "delta": 1}[kind], views[0][0], views[0][1], views[1][0], views[1][1], views[2][0], views[2][1],
            views[3][0], views[3][1], rate_v[0], rate_v[1], lora_v[0], lora_v[1], w2.data_ptr(), w0.data_ptr(),
            _ptr(rate_bias), _ptr(bonus), norm_w.data_ptr(), state.data_ptr(), last_ptr, last_stride, C,
            _ptr(last_state), optr, ostride, out_col, float(out_scale), float(eps), float(decay_scale), heads, dim,
            lora.shape[1], batch.n_seqs, batch.cu_q.data_ptr(), batch.seq_qlen.data_ptr(), batch.seq_slot.data_ptr(),
            rows, _ptr(prep), _ptr(o_raw), _code(r.dtype), self._stream())
        self._ok(rc, f"{kind} recurrence (heads of up to 256 channels)")

    # -- state-space mixer ------------------------------------------------------------------
    SSD_CHUNK = 128  # tokens per chunk where one sequence's step is long enough to be scanned in chunks

    def causal_conv_silu(self, x, w, b, tail, batch):
        """silu(b + short causal convolution over each sequence's rows); ``tail`` [slots, taps - 1, channels] holds
        every sequence's last inputs and is brought up to date. x may be a column slice; w [taps, channels] float32."""
        ptr, stride = self._rows_view(x)
        rows, ch = x.shape
        taps = w.shape[0]
        if w.shape[1] != ch or not w.is_contiguous():
            raise KernelError("the convolution's weights come tap-major, [taps, channels], contiguous")
        if tail.dtype != x.dtype or not tail.is_contiguous() or tail.shape[1:] != (max(taps - 1, 1), ch):
            raise KernelError("the convolution's stored inputs have the path's dtype and [taps - 1, channels] per slot")
        out = torch.empty((rows, ch), dtype=x.dtype, device=x.device)
        self._ok(self.scan.krk_causal_conv_silu(out.data_ptr(), ptr, stride, w.data_ptr(), b.data_ptr(), tail.data_ptr(),
                                               taps, ch, rows, batch.n_seqs, batch.row_seq.data_ptr(),
                                               batch.cu_q.data_ptr(), batch.seq_qlen.data_ptr(), batch.seq_slot.data_ptr(),
                                               _code(x.dtype), self._stream()), "causal convolution + silu")
        self.launches += int(taps > 1)
        return out

    def ssd_scan(self, x, B, C, dt, dt_bias, a_log, skip, heads, P, N, groups, state, batch):
        """The scan of a state-space mixer over a step's rows (csrc/ssd.cu): float32 y [rows, heads * P]; ``state``
        [slots, heads, N, P] float32 is read and left as the sequences' new state."""
        views = [self._rows_view(t) for t in (x, B, C, dt)]
        rows = x.shape[0]
        if state.dtype != torch.float32 or not state.is_contiguous() or state.shape[1:] != (heads, N, P):
            raise KernelError("the scan keeps a contiguous float32 state [slots, heads, N, P]")
        y = torch.empty((rows, heads * P), dtype=torch.float32, device=x.device)
        chunk, cs, cd = 0, None, None
        if not batch.is_decode and batch.max_q_len >= 2 * self.SSD_CHUNK:
            chunk = self.SSD_CHUNK
            n_chunks = -(-batch.max_q_len // chunk)
            cs = torch.empty((batch.n_seqs * n_chunks * heads, N * P), dtype=torch.float32, device=x.device)
            cd = torch.empty(batch.n_seqs * n_chunks * heads, dtype=torch.float32, device=x.device)
            self.launches += 2
        self._ok(self.scan.krk_ssd_scan(y.data_ptr(), views[0][0], views[0][1], views[1][0], views[1][1], views[2][0],
                                        views[2][1], views[3][0], views[3][1], dt_bias.data_ptr(), a_log.data_ptr(),
                                        skip.data_ptr(), state.data_ptr(), heads, P, N, groups, batch.n_seqs,
                                        batch.max_q_len, batch.cu_q.data_ptr(), batch.seq_qlen.data_ptr(),
                                        batch.seq_slot.data_ptr(), chunk, _ptr(cs), _ptr(cd), _code(x.dtype),
                                        self._stream()), "state-space scan (a head's state must fit a block's registers)")
        return y

    def gated_group_norm(self, y, gate_rows, weight, parts, eps, out, out_col, out_scale):
        """out[:, out_col:...] = group_norm(y * silu(gate_rows)) * weight * out_scale; y float32, ``parts`` equal parts
        each divided by its own root mean square."""
        zptr, zstride = self._rows_view(gate_rows)
        optr, ostride = self._rows_view(out)
        rows, inner = y.shape
        if y.dtype != torch.float32 or not y.is_contiguous() or gate_rows.dtype != out.dtype:
            raise KernelError("the gated norm reads float32 rows and a gate of the path's dtype")
        self._ok(self.scan.krk_gated_group_norm(optr, ostride, int(out_col), float(out_scale), y.data_ptr(), zptr, zstride,
                                               weight.data_ptr(), rows, inner, int(parts), float(eps), _code(out.dtype),
                                               self._stream()), "gated group norm")

    # -- token selection ------------------------------------------------------------
    def select_tokens(self, logits, temperature, seed, requests, step, feed=None, out=None):
        """One token per row. ``feed``: the batch description of a single-token step; the
        kernel then also writes the chosen tokens into it and moves its positions on by
        one, so that the next step can run without the host."""
        n, vocab = logits.shape
        tokens = out if out is not None else torch.empty(n, dtype=torch.int32, device=logits.device)
        logits = logits.contiguous()
        f = (None, None, None) if feed is None else (feed.tokens.data_ptr(), feed.row_pos.data_ptr(),
                                                     feed.seq_start.data_ptr())
        if self._select_scratch is None or self._select_scratch.numel() < n:
            self._select_scratch = torch.zeros(max(n, 256), dtype=torch.int64, device=self.device)
        self._ok(self.core.krk_select_tokens(tokens.data_ptr(), logits.data_ptr(), n, vocab, temperature,
                                             seed & 0xFFFFFFFF, requests.data_ptr(), step & 0xFFFFFFFF, *f,
                                             self._select_scratch.data_ptr(), self._stream()), "token selection")
        return tokens


_cached: dict = {}


def load_kernels(head_dims=(), device="cuda:0") -> Kernels:
    """The process-wide Kernels object of a device, with the given head sizes loaded."""
    key = str(torch.device(device))
    k = _cached.get(key)
    if k is None:
        k = _cached[key] = Kernels(head_dims, device)
    for d in head_dims:
        k._attn_lib(int(d))
    return k
