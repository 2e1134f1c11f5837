"""The allocation-free decode attention entry point, called through its exported C
symbol, against the regular entry point and against the plain attention of the tests.

Some callers of these kernels cannot allocate device memory (a fixed memory budget,
an allocator that must not be re-entered, a plug-in that only gets its buffers);
``krk_attention_decode_noalloc`` keeps its split-partials scratch in a fixed array
inside the library for them. It must give what ``krk_attention_decode`` gives with a
caller's scratch buffer, bit for bit (it is the same arithmetic in the same order),
on two calls in a row (the array keeps the first call's contents); both must agree
with the plain attention within the kernels' tolerance; and a request that does not
fit the array, or whose head counts make no sense, must be refused before any launch.

This file sorts last so that a run that stops at the first failure has run every
other test before it.
"""

import ctypes
import math
import random
from ctypes import c_char_p, c_float, c_int, c_void_p
from types import SimpleNamespace

import pytest
import torch

from helpers import assert_close
from torch_ops import TorchOps

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
    qkv[:, :heads * D] *= 3.0  # sharp scores: one wrong key or a lost split shows
    slots = torch.arange(n_seqs, dtype=torch.int32, device="cuda")
    starts = torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device="cuda")
    return dict(k=k, v=v, table=table, width=width, qkv=qkv, slots=slots, starts=starts)


def plain_attention(c, heads, kv_heads, D, lengths, scale, window):
    batch = SimpleNamespace(slots=list(range(len(lengths))), starts=[n - 1 for n in lengths], q_lens=[1] * len(lengths))
    cache = SimpleNamespace(k=c["k"], v=c["v"], table=c["table"], width=c["width"], kv_heads=kv_heads)
    return TorchOps(torch.bfloat16).attention(c["qkv"], heads, kv_heads, D, batch, cache, scale, window or None)


# (sequences, q heads, kv heads, head size, lengths, window, split counts of the two calls); the last case has
# more splits than its sequences have pages, so some splits are empty
CASES = [
    (4, 8, 2, 64, [70, 300, 5, 129], 0, (5, 3)),
    (2, 32, 8, 128, [500, 64], 0, (3, 5)),
    (3, 8, 2, 64, [200, 90, 331], 100, (4, 2)),
    (2, 4, 4, 64, [60, 130], 0, (7, 6)),
]


@pytest.mark.parametrize("shape", CASES)
def test_noalloc_matches_the_regular_entry_point_twice_in_a_row(shape):
    n_seqs, heads, kv_heads, D, lengths, window, split_counts = shape
    lib = load(D)
    stream = torch.cuda.current_stream().cuda_stream
    scale = 1.0 / math.sqrt(D)
    for call, splits in enumerate(split_counts):  # the second call finds the first one's leftovers in the array
        c = case(call + 1, n_seqs, heads, kv_heads, D, lengths)
        want = torch.empty((n_seqs, heads * D), dtype=torch.bfloat16, device="cuda")
        got = torch.full_like(want, float("nan"))
        scratch = torch.empty(n_seqs * heads * splits * (D + 2), dtype=torch.float32, device="cuda")
        args = (c["qkv"].data_ptr(), c["qkv"].stride(0), heads, kv_heads, c["slots"].data_ptr(), c["starts"].data_ptr(),
                c["table"].data_ptr(), c["width"], c["k"].data_ptr(), c["v"].data_ptr(), n_seqs, scale, window, splits)
        assert lib.krk_attention_decode(want.data_ptr(), *args, scratch.data_ptr(), stream) == 0
        rc = lib.krk_attention_decode_noalloc(got.data_ptr(), *args, stream)
        assert rc == 0, lib.krk_attention_decode_noalloc_strerror(rc).decode()
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"call {call}: the two entry points run the same kernels and must agree bit for bit"
        ref = plain_attention(c, heads, kv_heads, D, lengths, scale, window)
        assert_close(got, ref, "bfloat16", f"call {call} against the plain attention", kernel=True)


def test_noalloc_refuses_what_does_not_fit_and_what_makes_no_sense():
    D, heads, kv_heads, n_seqs = 128, 32, 8, 64
    lib = load(D)
    dummy = torch.zeros(16, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream

    def call(HQ, HKV, q_stride, n, splits):
        return lib.krk_attention_decode_noalloc(dummy.data_ptr(), dummy.data_ptr(), q_stride, HQ, HKV, dummy.data_ptr(),
                                                dummy.data_ptr(), dummy.data_ptr(), 8, dummy.data_ptr(), dummy.data_ptr(),
                                                n, 0.1, 0, splits, stream)

    # 64 sequences x 32 heads x 32 splits x 130 floats = 34 MB: beyond the 4 MiB array; refused before any launch
    rc = call(heads, kv_heads, 6144, n_seqs, 32)
    assert rc == -5
    assert b"4 MiB" in lib.krk_attention_decode_noalloc_strerror(rc)
    # head counts and strides are checked before anything is divided or launched
    for HQ, HKV, stride in ((32, 0, 6144), (0, 8, 6144), (30, 8, 6144), (32, 8, 100)):
        rc = call(HQ, HKV, stride, 2, 2)
        assert rc == -7, (HQ, HKV, stride, rc)
        assert b"multiple" in lib.krk_attention_decode_noalloc_strerror(rc)
    torch.cuda.synchronize()
