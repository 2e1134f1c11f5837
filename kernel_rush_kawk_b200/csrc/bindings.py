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
from ctypes import c_float, c_int, c_uint, c_void_p

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
_ATTN_SIGNATURES = {
    "krk_attention_simple": [_P, _P, c_int, c_int, c_int, _P, _P, _P, _P, c_int, _P, _P, c_int, c_float, c_int, c_int, _P],
    "krk_attention_head_dim": [],
    "krk_attention_prefill": [_P, _P, c_int, c_int, c_int, _P, _P, _P, _P, _P, c_int, _P, _P, c_int, c_int, c_float,
                              c_int, _P],
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

    def _skinny(self, x, w, out_dtype, swiglu_rows=0):
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
            int(gain is not None and gain.dtype == torch.float32), None, M, N, K, float(x.eps) if lazy else 0.0,
            int(swiglu_rows > 0), _code(out_dtype), self._stream()), "skinny product")
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
