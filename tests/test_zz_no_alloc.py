"""The allocation-free decode attention entry point, called through its exported C
symbol, against the regular entry point.

Some callers of these kernels cannot allocate device memory (a fixed memory budget,
an allocator that must not be re-entered, a plug-in that only gets its buffers);
``krk_attention_decode_noalloc`` keeps its split-partials scratch in a fixed array
inside the library for them. It must give what ``krk_attention_decode`` gives with a
caller's scratch buffer, on two calls in a row (the array keeps the first call's
contents), and must refuse a request that does not fit its array.

This file sorts last so that a run that stops at the first failure has run every
other test before it.
"""

import ctypes
import math
import random
from ctypes import c_char_p, c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

PAGE = 64
P = c_void_p


def load(head_dim):
    from kernel_rush_kawk_b200.csrc.build import build_library

    lib = ctypes.CDLL(str(build_library("attn", head_dim)))
    lib.krk_attention_decode.argtypes = [P, P, c_int, c_int, c_int, P, P, P, c_int, P, P, c_int, c_float, c_int, c_int, P, P]
    lib.krk_attention_decode.restype = c_int
    lib.krk_attention_decode_noalloc.argtypes = [P, P, c_int, c_int, c_int, P, P, P, c_int, P, P, c_int, c_float, c_int,
                                                 c_int, P]
    lib.krk_attention_decode_noalloc.restype = c_int
    lib.krk_attention_decode_noalloc_strerror.argtypes = [c_int]
    lib.krk_attention_decode_noalloc_strerror.restype = c_char_p
    return lib


def case(seed, n_seqs, heads, kv_heads, D, lengths):
    g = torch.Generator(device="cuda").manual_seed(seed)
    n_pages, width = 48, 8
    rnd = lambda *shape: torch.randn(shape, generator=g, device="cuda").to(torch.bfloat16)
    k, v = rnd(n_pages, kv_heads, PAGE, D), rnd(n_pages, kv_heads, PAGE, D)
    order = list(range(n_pages))
    random.Random(seed).shuffle(order)
    table = torch.tensor(order[:n_seqs * width], dtype=torch.int32, device="cuda").view(n_seqs, width)
    qkv = rnd(n_seqs, (heads + 2 * kv_heads) * D)
    slots = torch.arange(n_seqs, dtype=torch.int32, device="cuda")
    starts = torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device="cuda")
    return dict(k=k, v=v, table=table, width=width, qkv=qkv, slots=slots, starts=starts)


@pytest.mark.parametrize("shape", [(4, 8, 2, 64, [70, 300, 5, 129]), (2, 32, 8, 128, [500, 64])])
def test_noalloc_matches_the_regular_entry_point_twice_in_a_row(shape):
    n_seqs, heads, kv_heads, D, lengths = shape
    lib = load(D)
    stream = torch.cuda.current_stream().cuda_stream
    scale = 1.0 / math.sqrt(D)
    for call, (seed, splits) in enumerate(((1, 5), (2, 3))):  # the second call finds the first one's leftovers
        c = case(seed, n_seqs, heads, kv_heads, D, lengths)
        want = torch.empty((n_seqs, heads * D), dtype=torch.bfloat16, device="cuda")
        got = torch.full_like(want, float("nan"))
        scratch = torch.empty(n_seqs * heads * splits * (D + 2), dtype=torch.float32, device="cuda")
        args = (c["qkv"].data_ptr(), c["qkv"].stride(0), heads, kv_heads, c["slots"].data_ptr(), c["starts"].data_ptr(),
                c["table"].data_ptr(), c["width"], c["k"].data_ptr(), c["v"].data_ptr(), n_seqs, scale, 0, splits)
        assert lib.krk_attention_decode(want.data_ptr(), *args, scratch.data_ptr(), stream) == 0
        rc = lib.krk_attention_decode_noalloc(got.data_ptr(), *args, stream)
        assert rc == 0, lib.krk_attention_decode_noalloc_strerror(rc).decode()
        torch.cuda.synchronize()
        scale_ref = want.float().abs().max().item()
        err = (got.float() - want.float()).abs().max().item()
        assert torch.isfinite(got.float()).all() and err <= 0.02 * scale_ref + 1e-3, (call, err)


def test_noalloc_refuses_what_does_not_fit():
    D, heads, kv_heads, n_seqs = 128, 32, 8, 64
    lib = load(D)
    # 64 sequences x 32 heads x 32 splits x 130 floats = 34 MB: beyond the 4 MiB array; refused before any launch
    dummy = torch.zeros(16, dtype=torch.int32, device="cuda")
    rc = lib.krk_attention_decode_noalloc(dummy.data_ptr(), dummy.data_ptr(), 6144, heads, kv_heads, dummy.data_ptr(),
                                          dummy.data_ptr(), dummy.data_ptr(), 8, dummy.data_ptr(), dummy.data_ptr(),
                                          n_seqs, 0.1, 0, 32, torch.cuda.current_stream().cuda_stream)
    assert rc == -5
    assert b"4 MiB" in lib.krk_attention_decode_noalloc_strerror(rc)
    torch.cuda.synchronize()
