"""Each CUDA kernel alone against its plain torch reference (tests/torch_ops.py), at
sizes other than the tiny models': widths that are no power of two, head sizes in
steps of 16, odd group counts. Inputs are made so that a fault shows: one far key
whose score stands out, a window's edge, pages scattered over the pool."""

import math
import random
from types import SimpleNamespace

import pytest
import torch

from helpers import assert_close
from torch_ops import PAGE, TorchOps

pytestmark = pytest.mark.gpu

DTYPES = (torch.float32, torch.bfloat16)
NAME = {torch.float32: "float32", torch.bfloat16: "bfloat16"}


@pytest.fixture(scope="module")
def ops():
    from kernel_rush_kawk_b200.csrc import load_kernels

    return load_kernels(())


def rand(shape, dtype, seed, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, generator=g, device="cuda", dtype=torch.float32) * scale).to(dtype)


def close(got, ref, dtype, what):
    assert_close(got, ref, NAME[dtype], what, kernel=True)


# -- rows -------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [48, 250, 2560, 5123])
def test_rmsnorm_and_add_rmsnorm(ops, dtype, hidden):
    ref = TorchOps(dtype)
    x, b = rand((7, hidden), dtype, 1, 3.0), rand((7, hidden), dtype, 2)
    gain = (1 + 0.1 * rand((hidden,), torch.float32, 3)).to(dtype)
    close(ops.rmsnorm(x, gain, 1e-5), ref.rmsnorm(x, gain, 1e-5), dtype, "rmsnorm")
    xn, xr = torch.empty_like(x), torch.empty_like(x)
    close(ops.add_rmsnorm(x, b, gain, 1e-6, xn), ref.add_rmsnorm(x, b, gain, 1e-6, xr), dtype, "add+rmsnorm")
    assert torch.equal(xn, xr), "the new residual stream is defined to the bit"
    if dtype == torch.bfloat16:  # a gain kept in 32-bit on the bfloat16 path
        close(ops.rmsnorm(x, gain.float(), 1e-5), ref.rmsnorm(x, gain.float(), 1e-5), dtype, "rmsnorm, float32 gain")


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_row_gather(ops, dtype):
    table = rand((301, 80), dtype, 4)
    ids = torch.tensor([0, 300, 17, 17, 5], dtype=torch.int32, device="cuda")
    assert torch.equal(ops.embed(table, ids, 5), table[ids.long()])
    assert torch.equal(ops.gather_rows(table, ids[:2]), table[ids[:2].long()])
    odd = rand((10, 37), dtype, 5)
    assert torch.equal(ops.gather_rows(odd, ids[:1]), odd[:1])
    ops.check()


def test_a_token_outside_the_table_is_flagged(ops):
    from kernel_rush_kawk_b200.csrc import KernelError

    table = rand((16, 32), torch.float32, 6)
    out = ops.embed(table, torch.tensor([3, 16], dtype=torch.int32, device="cuda"), 2)
    assert torch.equal(out[1], torch.zeros_like(out[1]))
    with pytest.raises(KernelError):
        ops.check()
    ops.check()  # the flag is cleared


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu(ops, dtype):
    gu = rand((9, 2 * 333), dtype, 7, 2.0)
    ref = TorchOps(dtype)
    g, u = gu[:, :333].float(), gu[:, 333:].float()
    want = (ref.rt(g / (1 + torch.exp(-g))) * u).to(dtype)
    close(ops.swiglu(gu, 333), want, dtype, "swiglu")


# -- matrix products ----------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("mnk", [(1, 70, 96), (5, 301, 80), (64, 192, 64), (130, 257, 333), (16, 2560, 4096)])
def test_linear(ops, dtype, mnk):
    m, n, k = mnk
    x, w = rand((m, k), dtype, 8), rand((n, k), dtype, 9, 0.05)
    ref = TorchOps(dtype)
    close(ops.linear(x, w), ref.linear(x, w), dtype, f"linear {mnk}")
    close(ops.linear(x, w, out_float32=True), ref.linear(x, w, out_float32=True), dtype, f"linear {mnk}, float32 out")


@pytest.mark.parametrize("mnk", [(1, 2560, 9728), (8, 2560, 4096), (16, 2560, 9728), (13, 1000, 2080), (3, 48, 2048),
                                 (9, 2000, 4128)])
def test_few_row_products_that_split_k_over_a_cluster(ops, mnk):
    """Few output features and a long K: the bfloat16 product splits K over the four blocks of a cluster and adds
    the parts in the first block's shared memory. Sizes off the grid (features no multiple of 16, chunks that do
    not divide by four), both output types, and the same bits on every run."""
    m, n, k = mnk
    dtype = torch.bfloat16
    x, w = rand((m, k), dtype, 84), rand((n, k), dtype, 85, 0.05)
    ref = TorchOps(dtype)
    got = ops.linear(x, w)
    close(got, ref.linear(x, w), dtype, f"linear {mnk}")
    close(ops.linear(x, w, out_float32=True), ref.linear(x, w, out_float32=True), dtype, f"linear {mnk}, float32 out")
    for _ in range(3):
        assert torch.equal(ops.linear(x, w), got), "the sum over the cluster's parts must not depend on timing"


def test_library_gemm_with_measured_algorithm(ops):
    """Products of more than 16 rows in bfloat16 go to the library with the algorithm picked by timing its
    proposals: the first call of a shape class measures, later calls (other row counts of the class, a view
    with a wider row stride, a stream capture) reuse the choice, and all of them give the plain product."""
    dtype = torch.bfloat16
    ref = TorchOps(dtype)
    assert ops.use_tuned_library_gemm
    before, _ = ops.library_gemm_report()
    w = rand((1096, 520), dtype, 91, 0.05)
    # 300, 400 and 512 are one class, measured at 300; 4,500 and 6,000 are one, measured on the first 4,096 rows
    for m in (17, 64, 300, 400, 512, 700, 4500, 6000):
        x = rand((m, 520), dtype, 92 + m)
        close(ops.linear(x, w), ref.linear(x, w), dtype, f"library product, {m} rows")
    after, _ = ops.library_gemm_report()
    assert after - before == 5, "classes: 17, 64, 512 (300, 400, 512), 768 (700), 8192 (4500, 6000)"
    wide = rand((300, 1040), dtype, 93)
    x = wide[:, :520]  # rows 1,040 apart
    close(ops.linear(x, w), ref.linear(x.contiguous(), w), dtype, "library product of a strided view")
    ops.use_tuned_library_gemm = False
    try:
        other = ops.linear(x, w)
    finally:
        ops.use_tuned_library_gemm = True
    close(ops.linear(x, w), other, dtype, "measured choice against the heuristic's")
    # a class first met under capture runs the heuristic's first proposal and stays unmeasured
    x = rand((33, 520), dtype, 94)
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            y = ops.linear(x, w)
        graph.replay()
    torch.cuda.current_stream().wait_stream(stream)
    torch.cuda.synchronize()
    close(y, ref.linear(x, w), dtype, "library product in a captured graph")
    assert ops.library_gemm_report()[0] == after + 1, "the strided view's class was measured, the captured one was not"


@pytest.mark.parametrize("mnk", [(128, 128, 64), (128, 128, 512), (256, 384, 2560), (130, 200, 72), (77, 3000, 1000),
                                 (2048, 2560, 4096)])
def test_tcgen05_gemm(ops, mnk):
    m, n, k = mnk
    dtype = torch.bfloat16
    x, w = rand((m, k), dtype, 80), rand((n, k), dtype, 81, 0.05)
    ref = TorchOps(dtype)
    close(ops.gemm_tcgen05(x, w), ref.linear(x, w), dtype, f"tcgen05 gemm {mnk}")
    close(ops.gemm_tcgen05(x, w, out_float32=True), ref.linear(x, w, out_float32=True), dtype, f"tcgen05 gemm {mnk}, float32 out")
    ops.check()


def test_tcgen05_logits_tiles_of_every_width(ops):
    """Float32 logits take 256-, 224- or 192-wide tiles, whichever fills its rounds of blocks best: a vocabulary of
    151,936 at up to 128 rows takes 224, 3,000 columns take 192, 148 x 256 columns take 256."""
    dtype = torch.bfloat16
    ref = TorchOps(dtype)
    for m, n, k in ((64, 151936, 64), (20, 3000, 96), (33, 148 * 256, 64)):
        x, w = rand((m, k), dtype, 86), rand((n, k), dtype, 87, 0.05)
        close(ops.gemm_tcgen05(x, w, out_float32=True), ref.linear(x, w, out_float32=True), dtype, f"logits {m} x {n} x {k}")
    ops.check()


@pytest.mark.parametrize("mik", [(128, 128, 128), (300, 272, 160), (2048, 9728, 2560)])
def test_tcgen05_gemm_with_swiglu_epilogue(ops, mik):
    m, inter, k = mik
    dtype = torch.bfloat16
    x, w = rand((m, k), dtype, 82), rand((2 * inter, k), dtype, 83, 0.05)
    ref = TorchOps(dtype)
    close(ops.gemm_tcgen05(x, w, swiglu_rows=inter), ref.gate_up_swiglu(x, w, inter), dtype, f"tcgen05 gate/up {mik}")
    ops.check()


@pytest.mark.parametrize("rows", [1, 3, 8, 13, 16])
@pytest.mark.parametrize("nk", [(96, 64), (160, 2560), (301, 96), (2560, 9728)])
def test_fused_norm_linear_bfloat16(ops, rows, nk):
    """The decode-time product with the residual add and the norm in its prologue."""
    from kernel_rush_kawk_b200.parts.norm import Normed

    n, k = nk
    dtype = torch.bfloat16
    ref = TorchOps(dtype)
    x, b = rand((rows, k), dtype, 10, 2.0), rand((rows, k), dtype, 11)
    gain = (1 + 0.1 * rand((k,), torch.float32, 12)).to(dtype)
    w = rand((n, k), dtype, 13, 0.05)
    for branch in (b, None):
        xn, xr = torch.empty_like(x), torch.empty_like(x)
        lazy = Normed(ops, x, branch, gain, 1e-6, xn if branch is not None else x)
        got = ops.linear(lazy, w)
        h = ref.add_rmsnorm(x, branch, gain, 1e-6, xr) if branch is not None else ref.rmsnorm(x, gain, 1e-6)
        close(got, ref.linear(h, w), dtype, f"norm+linear rows {rows} {nk}")
        if branch is not None:
            assert torch.equal(xn, xr)
    lazy = Normed(ops, x, b, gain, 1e-6, torch.empty_like(x))
    got = ops.linear(lazy, w, out_float32=True)
    close(got, ref.linear(ref.add_rmsnorm(x, b, gain, 1e-6, torch.empty_like(x)), w, out_float32=True), dtype, "float32 out")


@pytest.mark.parametrize("rows", [1, 8, 11])
def test_fused_gate_up_swiglu_bfloat16(ops, rows):
    from kernel_rush_kawk_b200.parts.norm import Normed

    dtype, k, inter = torch.bfloat16, 160, 272
    ref = TorchOps(dtype)
    x, b = rand((rows, k), dtype, 14, 2.0), rand((rows, k), dtype, 15)
    gain = (1 + 0.1 * rand((k,), torch.float32, 16)).to(dtype)
    w = rand((2 * inter, k), dtype, 17, 0.08)
    lazy = Normed(ops, x, b, gain, 1e-6, torch.empty_like(x))
    got = ops.gate_up_swiglu(lazy, w, inter)
    h = ref.add_rmsnorm(x, b, gain, 1e-6, torch.empty_like(x))
    close(got, ref.gate_up_swiglu(h, w, inter), dtype, "norm + gate/up + swiglu")
    close(ops.gate_up_swiglu(h, w, inter), ref.gate_up_swiglu(h, w, inter), dtype, "gate/up + swiglu")


# -- attention -----------------------------------------------------------------------
def make_cache(n_pages, kv_heads, head_dim, n_slots, width, dtype, seed):
    """A cache view whose pages are handed out in a shuffled order, filled with noise so
    that reading a page one does not own shows."""
    from kernel_rush_kawk_b200.cache import KVView

    k = rand((n_pages, kv_heads, PAGE, head_dim), dtype, seed, 1.0)
    v = rand((n_pages, kv_heads, PAGE, head_dim), dtype, seed + 1, 1.0)
    order = list(range(n_pages))
    random.Random(seed).shuffle(order)
    table = torch.tensor(order[:n_slots * width], dtype=torch.int32, device="cuda").view(n_slots, width)
    return KVView(k, v, table, width, None, kv_heads, head_dim)


def make_batch(slots, starts, q_lens):
    rows = sum(q_lens)
    dev = "cuda"
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    row_seq = [s for s, n in enumerate(q_lens) for _ in range(n)]
    row_pos = [st + t for st, n in zip(starts, q_lens) for t in range(n)]
    return SimpleNamespace(n_rows=rows, n_seqs=len(slots), row_seq=i32(row_seq), row_pos=i32(row_pos),
                           seq_slot=i32(slots), seq_start=i32(starts), seq_qlen=i32(q_lens), cu_q=i32(cu),
                           slots=slots, starts=starts, q_lens=q_lens, max_q_len=max(q_lens),
                           max_kv_len=max(s + n for s, n in zip(starts, q_lens)), is_decode=max(q_lens) == 1)


ATTN_SHAPES = [  # heads, kv_heads, head_dim
    (4, 2, 16), (6, 2, 32), (5, 1, 48), (8, 8, 64), (14, 2, 80), (32, 8, 128),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", ATTN_SHAPES)
@pytest.mark.parametrize("window", [None, 40])
def test_rope_write_then_attention_prefill_and_decode(ops, dtype, shape, window):
    heads, kv_heads, D = shape
    ref = TorchOps(dtype)
    width, n_slots = 6, 4
    cache = make_cache(40, kv_heads, D, n_slots, width, dtype, 20)
    cache.window = window
    ref_cache = SimpleNamespace(**vars(cache))
    ref_cache.k, ref_cache.v = cache.k.clone(), cache.v.clone()
    theta = 10000.0
    inv = 1.0 / (theta ** (torch.arange(0, D, 2, device="cuda").float() / D))
    ang = torch.arange(width * PAGE, device="cuda").float()[:, None] * inv[None, :]
    cos, sin = ang.cos().to(dtype), ang.sin().to(dtype)
    qg = (1.5 + 0.1 * rand((D,), torch.float32, 21)).to(dtype)
    kg = (1.5 + 0.1 * rand((D,), torch.float32, 22)).to(dtype)
    scale = 1.0 / math.sqrt(D)
    width_row = (heads + 2 * kv_heads) * D
    # step 1: three sequences start with unequal prompts; step 2: they go on by pieces
    # of unequal length (one of them a single token); step 3: one token each
    steps = [([2, 0, 3], [0, 0, 0], [70, 5, 129]), ([2, 0, 3], [70, 5, 129], [33, 1, 64]),
             ([3, 2, 0], [193, 103, 6], [1, 1, 1])]
    for s, (slots, starts, q_lens) in enumerate(steps):
        batch = make_batch(slots, starts, q_lens)
        qkv = rand((batch.n_rows, width_row), dtype, 30 + s, 1.0)
        # make one far key stand out for the last query of the longest sequence: its key
        # and that query point the same way, strongly
        qkv_ref = qkv.clone()
        ops.qk_norm_rope_write(qkv, heads, kv_heads, D, qg, kg, 1e-6, cos, sin, batch, cache)
        ref.qk_norm_rope_write(qkv_ref, heads, kv_heads, D, qg, kg, 1e-6, cos, sin, batch, ref_cache)
        close(qkv[:, :heads * D], qkv_ref[:, :heads * D], dtype, f"rotated queries, step {s}")
        close(cache.k, ref_cache.k, dtype, f"key pages, step {s}")
        assert torch.equal(cache.v, ref_cache.v), "values are copied raw"
        ref_cache.k.copy_(cache.k)  # same keys on both sides from here on
        qkv_ref[:, :heads * D] = qkv[:, :heads * D]
        got = ops.attention(qkv, heads, kv_heads, D, batch, cache, scale, window)
        want = ref.attention(qkv_ref, heads, kv_heads, D, batch, ref_cache, scale, window)
        close(got, want, dtype, f"attention, step {s}, shape {shape}, window {window}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(3, 1, 16), (6, 2, 32), (8, 8, 64), (32, 8, 128), (7, 1, 128), (2, 1, 256), (5, 1, 48)])
def test_rope_write_many_rows(ops, dtype, shape):
    """Steps with hundreds of rows take the block-per-row kernel (bfloat16, head sizes 16..256 in powers of
    two); every row's position, page and head must come out as with few rows."""
    heads, kv_heads, D = shape
    ref = TorchOps(dtype)
    width, n_slots = 8, 4
    cache = make_cache(40, kv_heads, D, n_slots, width, dtype, 23)
    ref_cache = SimpleNamespace(**vars(cache))
    ref_cache.k, ref_cache.v = cache.k.clone(), cache.v.clone()
    inv = 1.0 / (1e6 ** (torch.arange(0, D, 2, device="cuda").float() / D))
    ang = torch.arange(width * PAGE, device="cuda").float()[:, None] * inv[None, :]
    cos, sin = ang.cos().to(dtype), ang.sin().to(dtype)
    qg = (1.5 + 0.1 * rand((D,), torch.float32, 24)).to(dtype)
    kg = (0.7 + 0.1 * rand((D,), torch.float32, 25)).to(dtype)
    batch = make_batch([1, 3, 0], [37, 0, 130], [200, 90, 41])
    qkv = rand((batch.n_rows, (heads + 2 * kv_heads) * D), dtype, 26, 1.0)
    qkv_ref = qkv.clone()
    ops.qk_norm_rope_write(qkv, heads, kv_heads, D, qg, kg, 1e-5, cos, sin, batch, cache)
    ref.qk_norm_rope_write(qkv_ref, heads, kv_heads, D, qg, kg, 1e-5, cos, sin, batch, ref_cache)
    close(qkv[:, :heads * D], qkv_ref[:, :heads * D], dtype, "rotated queries")
    close(cache.k, ref_cache.k, dtype, "key pages")
    assert torch.equal(cache.v, ref_cache.v), "values are copied raw"
    assert torch.equal(qkv[:, heads * D:], qkv_ref[:, heads * D:]), "the step's own k and v columns stay as they were"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(3, 1, 16, 8), (6, 2, 48, 20), (8, 2, 128, 64), (5, 1, 80, 2)])
@pytest.mark.parametrize("gains", [True, False])
def test_rope_write_rotates_part_of_the_head(ops, dtype, shape, gains):
    """Tables narrower than half the head: the first rot elements are rotated in pairs (i, i + rot/2), the
    others only normalised (over the whole head); few rows and many; then a single-token step, which must
    not take the kernel that rotates whole heads."""
    heads, kv_heads, D, rot = shape
    ref = TorchOps(dtype)
    width, n_slots = 8, 4
    cache = make_cache(40, kv_heads, D, n_slots, width, dtype, 41)
    ref_cache = SimpleNamespace(**vars(cache))
    ref_cache.k, ref_cache.v = cache.k.clone(), cache.v.clone()
    inv = 1.0 / (1e4 ** (torch.arange(0, rot, 2, device="cuda").float() / rot))
    ang = torch.arange(width * PAGE, device="cuda").float()[:, None] * inv[None, :]
    cos, sin = ang.cos().to(dtype).contiguous(), ang.sin().to(dtype).contiguous()
    qg = (1.5 + 0.1 * rand((D,), torch.float32, 42)).to(dtype) if gains else None
    kg = (0.7 + 0.1 * rand((D,), torch.float32, 43)).to(dtype) if gains else None
    scale = 1.0 / math.sqrt(D)
    for s, (slots, starts, q_lens) in enumerate([([1, 3, 0], [0, 0, 0], [300, 7, 41]), ([3, 1], [7, 300], [5, 1]),
                                                 ([0, 1, 3], [41, 301, 12], [1, 1, 1])]):
        batch = make_batch(slots, starts, q_lens)
        qkv = rand((batch.n_rows, (heads + 2 * kv_heads) * D), dtype, 44 + s, 1.0)
        qkv_ref = qkv.clone()
        if s < 2:
            ops.qk_norm_rope_write(qkv, heads, kv_heads, D, qg, kg, 1e-5, cos, sin, batch, cache)
            ref.qk_norm_rope_write(qkv_ref, heads, kv_heads, D, qg, kg, 1e-5, cos, sin, batch, ref_cache)
            close(qkv[:, :heads * D], qkv_ref[:, :heads * D], dtype, f"rotated queries, step {s}")
            if not gains:
                got_q = qkv[:, :heads * D].view(-1, heads, D)
                assert torch.equal(got_q[..., rot:], qkv_ref[:, :heads * D].view(-1, heads, D)[..., rot:]), "beyond rot: untouched"
        else:
            got = ops.rope_attention(qkv, heads, kv_heads, D, qg, kg, 1e-5, cos, sin, batch, cache, scale, None)
            want = ref.rope_attention(qkv_ref, heads, kv_heads, D, qg, kg, 1e-5, cos, sin, batch, ref_cache, scale, None)
            close(got, want, dtype, "single-token step with a partial rotation")
        close(cache.k, ref_cache.k, dtype, f"key pages, step {s}")
        assert torch.equal(cache.v, ref_cache.v), "values are copied raw"
        ref_cache.k.copy_(cache.k)


@pytest.mark.parametrize("rows", [3, 300])
def test_a_position_outside_the_rotary_table_is_flagged(ops, rows):
    """A row whose position lies beyond the tables is reported through the error word and stores
    nothing; the other rows are done as usual (both row kernels: few rows and many)."""
    from kernel_rush_kawk_b200.csrc import KernelError

    dtype, heads, kv_heads, D = torch.bfloat16, 4, 2, 32
    width = 8
    cache = make_cache(16, kv_heads, D, 1, width, dtype, 31)
    before_k = cache.k.clone()
    n_pos = rows + 5
    inv = 1.0 / (1e4 ** (torch.arange(0, D, 2, device="cuda").float() / D))
    ang = torch.arange(n_pos, device="cuda").float()[:, None] * inv[None, :]
    cos, sin = ang.cos().to(dtype), ang.sin().to(dtype)
    batch = make_batch([0], [0], [rows])
    batch.row_pos[1] = n_pos + 7  # one bad row
    qkv = rand((rows, (heads + 2 * kv_heads) * D), dtype, 32)
    raw = qkv.clone()
    ops.qk_norm_rope_write(qkv, heads, kv_heads, D, None, None, 1e-6, cos, sin, batch, cache)
    with pytest.raises(KernelError):
        ops.check()
    assert torch.equal(qkv[1], raw[1]), "the bad row is left as it was"
    page, off = int(cache.table[0, 0]), 1
    assert torch.equal(cache.k[page, :, off], before_k[page, :, off]), "and its key is not stored"
    assert not torch.equal(qkv[2, :heads * D], raw[2, :heads * D]), "the rows around it are rotated"
    ops.check()


@pytest.mark.parametrize("shape", ATTN_SHAPES + [(40, 2, 64)])
@pytest.mark.parametrize("window", [None, 70])
@pytest.mark.parametrize("n_seqs", [1, 3, 40, 100])
def test_fused_decode_attention_against_the_two_kernel_path(ops, shape, window, n_seqs):
    """Single-token steps in bfloat16: norm + rotation + cache write + attention + merge in
    one launch, against the plain reference of each stage; 1, 3 and 40 sequences give
    cluster sizes 8, 4 or 2, and 1; with one block per (sequence, kv head, row tile), head
    sizes 64 and 128 take the TMA-fed kernel (at 100 sequences also the shape with two row tiles)."""
    heads, kv_heads, D = shape
    dtype = torch.bfloat16
    ref = TorchOps(dtype)
    width = 6
    cache = make_cache(n_seqs * width + 3, kv_heads, D, n_seqs, width, dtype, 70)
    cache.window = window
    ref_cache = SimpleNamespace(**vars(cache))
    ref_cache.k, ref_cache.v = cache.k.clone(), cache.v.clone()
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, device="cuda").float() / D))
    ang = torch.arange(width * PAGE, device="cuda").float()[:, None] * inv[None, :]
    cos, sin = ang.cos().to(dtype), ang.sin().to(dtype)
    qg = (1.5 + 0.1 * rand((D,), torch.float32, 71)).to(dtype)
    kg = (1.5 + 0.1 * rand((D,), torch.float32, 72)).to(dtype)
    rnd = random.Random(5)
    starts = [rnd.choice([0, 1, 63, 64, 127, 200, 383]) for _ in range(n_seqs)]
    slots = list(range(n_seqs))
    rnd.shuffle(slots)
    batch = make_batch(slots, starts, [1] * n_seqs)
    qkv = rand((n_seqs, (heads + 2 * kv_heads) * D), dtype, 73)
    qkv_ref = qkv.clone()
    scale = 1.0 / math.sqrt(D)
    got = ops.rope_attention(qkv, heads, kv_heads, D, qg, kg, 1e-6, cos, sin, batch, cache, scale, window)
    want = ref.rope_attention(qkv_ref, heads, kv_heads, D, qg, kg, 1e-6, cos, sin, batch, ref_cache, scale, window)
    close(cache.k, ref_cache.k, dtype, "key pages after the fused step")
    assert torch.equal(cache.v, ref_cache.v)
    close(got, want, dtype, f"fused decode attention {shape} window {window} seqs {n_seqs}")


@pytest.mark.parametrize("shape", [(8, 8, 64), (32, 8, 128), (40, 2, 64), (4, 4, 256)])
@pytest.mark.parametrize("window", [None, 150])
def test_tma_fed_decode_attention_equals_the_cp_async_kernel(ops, shape, window):
    """Many sequences, long ones among them (18 pages through a ring of 6 or 12 units, so every unit is
    reused), a page table that wraps under the window: the TMA-fed kernel and the cp.async kernel walk
    the keys in the same order and must agree to the bit, cache pages included."""
    heads, kv_heads, D = shape
    dtype = torch.bfloat16
    n_seqs, width = 120, 18
    rnd = random.Random(9)
    starts = [rnd.choice([0, 5, 63, 64, 65, 500, 1000, 1151]) for _ in range(n_seqs)]
    slots = list(range(n_seqs))
    rnd.shuffle(slots)
    batch = make_batch(slots, starts, [1] * n_seqs)
    qg = (1.5 + 0.1 * rand((D,), torch.float32, 81)).to(dtype)
    kg = (1.5 + 0.1 * rand((D,), torch.float32, 82)).to(dtype)
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, device="cuda").float() / D))
    ang = torch.arange(width * PAGE, device="cuda").float()[:, None] * inv[None, :]
    cos, sin = ang.cos().to(dtype), ang.sin().to(dtype)
    scale = 1.0 / math.sqrt(D)
    results = []
    for use_tma in (True, False):
        cache = make_cache(n_seqs * width + 3, kv_heads, D, n_seqs, width, dtype, 80)
        cache.window = window
        qkv = rand((n_seqs, (heads + 2 * kv_heads) * D), dtype, 83)
        ops.use_tma_decode_attention = use_tma
        try:
            out = ops.rope_attention(qkv, heads, kv_heads, D, qg, kg, 1e-6, cos, sin, batch, cache, scale, window)
        finally:
            ops.use_tma_decode_attention = True
        results.append((out, cache.k, cache.v))
    ops.check()
    for a, b, what in zip(results[0], results[1], ("output", "key pages", "value pages")):
        assert torch.equal(a, b), f"{what} differ between the TMA-fed and the cp.async kernel"


@pytest.mark.parametrize("shape", [(8, 8, 64), (32, 8, 128), (40, 2, 64)])
@pytest.mark.parametrize("n_seqs", [1, 3, 9])
@pytest.mark.parametrize("window", [None, 150])
def test_tma_fed_decode_attention_with_key_splits(ops, shape, n_seqs, window):
    """Few sequences: the keys of a (sequence, kv head) are split over a cluster of 16, 8 or 4 blocks, each with
    a TMA ring of its own, and meet in the first block's shared memory. Sequences of one key, of fewer pages
    than splits and of 40 pages; the same splits in the cp.async kernel give the same bits."""
    heads, kv_heads, D = shape
    dtype = torch.bfloat16
    ref = TorchOps(dtype)
    width = 40
    rnd = random.Random(19 + n_seqs)
    starts = [rnd.choice([0, 63, 64, 200, 1000, 2559]) for _ in range(n_seqs)]
    starts[0] = 2559
    slots = list(range(n_seqs))
    rnd.shuffle(slots)
    batch = make_batch(slots, starts, [1] * n_seqs)
    qg = (1.5 + 0.1 * rand((D,), torch.float32, 81)).to(dtype)
    kg = (1.5 + 0.1 * rand((D,), torch.float32, 82)).to(dtype)
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, device="cuda").float() / D))
    ang = torch.arange(width * PAGE, device="cuda").float()[:, None] * inv[None, :]
    cos, sin = ang.cos().to(dtype), ang.sin().to(dtype)
    scale = 1.0 / math.sqrt(D)
    results = []
    before = ops.tma_decode_splits
    for splits_by_tma in ({1, 2, 4, 8, 16}, set()):
        cache = make_cache(n_seqs * width + 3, kv_heads, D, n_seqs, width, dtype, 80)
        cache.window = window
        qkv = rand((n_seqs, (heads + 2 * kv_heads) * D), dtype, 83)
        ops.tma_decode_splits = splits_by_tma
        try:
            out = ops.rope_attention(qkv, heads, kv_heads, D, qg, kg, 1e-6, cos, sin, batch, cache, scale, window)
        finally:
            ops.tma_decode_splits = before
        results.append((out, cache.k, cache.v))
    ops.check()
    for a, b, what in zip(results[0], results[1], ("output", "key pages", "value pages")):
        assert torch.equal(a, b), f"{what} differ between the TMA-fed and the cp.async kernel"
    ref_cache = make_cache(n_seqs * width + 3, kv_heads, D, n_seqs, width, dtype, 80)
    ref_cache.window = window
    want = ref.rope_attention(rand((n_seqs, (heads + 2 * kv_heads) * D), dtype, 83), heads, kv_heads, D, qg, kg, 1e-6, cos, sin,
                              batch, ref_cache, scale, window)
    close(results[0][0], want, dtype, f"TMA-fed decode attention with key splits {shape} seqs {n_seqs} window {window}")


@pytest.mark.parametrize("shape", [(8, 8, 64), (32, 8, 128)])
def test_tma_fed_decode_attention_round_a_wrapped_ring_of_pages(ops, shape):
    """A window of 150 keys in a ring of 6 pages, sequences thousands of tokens long: the positions' pages
    are table entries modulo the ring, and the kernel's own ring of units turns several times per block.
    Against the plain attention over the same pages."""
    heads, kv_heads, D = shape
    dtype = torch.bfloat16
    ref = TorchOps(dtype)
    n_seqs, width, window = 110, 6, 150
    rnd = random.Random(11)
    starts = [rnd.choice([149, 150, 383, 384, 1000, 2047, 4999]) for _ in range(n_seqs)]
    slots = list(range(n_seqs))
    rnd.shuffle(slots)
    batch = make_batch(slots, starts, [1] * n_seqs)
    cache = make_cache(n_seqs * width + 3, kv_heads, D, n_seqs, width, dtype, 90)
    cache.window = window
    ref_cache = SimpleNamespace(**vars(cache))
    ref_cache.k, ref_cache.v = cache.k.clone(), cache.v.clone()
    qkv = rand((n_seqs, (heads + 2 * kv_heads) * D), dtype, 91)
    qkv_ref = qkv.clone()
    scale = 1.0 / math.sqrt(D)
    got = ops.rope_attention(qkv, heads, kv_heads, D, None, None, 1e-6, None, None, batch, cache, scale, window)
    want = ref.rope_attention(qkv_ref, heads, kv_heads, D, None, None, 1e-6, None, None, batch, ref_cache, scale, window)
    ops.check()
    assert torch.equal(cache.k, ref_cache.k) and torch.equal(cache.v, ref_cache.v)
    close(got, want, dtype, f"TMA-fed decode attention round a wrapped ring {shape}")


@pytest.mark.parametrize("shape", [(8, 2, 64), (32, 8, 128), (6, 2, 128), (5, 1, 64)])
@pytest.mark.parametrize("window", [None, 100])
def test_tcgen05_prefill_attention(ops, shape, window):
    """Long steps in bfloat16 at head sizes 64 and 128 take the tcgen05 kernel: prompts of
    unequal lengths from position 0, then pieces that continue them, against the plain
    reference; with the mma.sync kernel of the same library as a second opinion."""
    heads, kv_heads, D = shape
    dtype = torch.bfloat16
    ref = TorchOps(dtype)
    width, n_slots = 10, 3
    cache = make_cache(34, kv_heads, D, n_slots, width, dtype, 90)
    cache.window = window
    scale = 1.0 / math.sqrt(D)
    row_w = (heads + 2 * kv_heads) * D
    steps = [([1, 2, 0], [0, 0, 0], [300, 129, 64]), ([2, 1], [129, 300], [200, 131])]
    for s, (slots, starts, q_lens) in enumerate(steps):
        batch = make_batch(slots, starts, q_lens)
        qkv = rand((batch.n_rows, row_w), dtype, 91 + s, 1.0)
        # the step's own keys and values go into the cache first, as in the engine
        ops.qk_norm_rope_write(qkv, heads, kv_heads, D, None, None, 1e-6, None, None, batch, cache)
        assert ops.use_tcgen05_attention
        got = ops.attention(qkv, heads, kv_heads, D, batch, cache, scale, window)
        ops.check()
        want = ref.attention(qkv, heads, kv_heads, D, batch, cache, scale, window)
        close(got, want, dtype, f"tcgen05 attention step {s} {shape} window {window}")
        ops.use_tcgen05_attention = False
        try:
            other = ops.attention(qkv, heads, kv_heads, D, batch, cache, scale, window)
        finally:
            ops.use_tcgen05_attention = True
        close(got, other, dtype, "tcgen05 against mma.sync")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("q_len", [1, 37])
def test_one_far_key_among_hundreds_decides(ops, dtype, q_len):
    """Key 3 of 700 is made to match the last query; its value is a marker. The output
    must be the marker, which a kernel that skipped or misplaced the key would miss."""
    heads, kv_heads, D = 4, 2, 64
    width = 12
    cache = make_cache(30, kv_heads, D, 2, width, dtype, 40)
    cache.k.mul_(0.05)
    total = 700
    slot, start = 1, total - q_len
    batch = make_batch([slot], [start], [q_len])
    qkv = rand((q_len, (heads + 2 * kv_heads) * D), dtype, 41, 0.05)
    direction = torch.zeros(D, device="cuda")
    direction[5] = 8.0
    page = int(cache.table[slot, 0])
    cache.k[page, :, 3] = direction.to(dtype)
    cache.v[page, :, 3] = 7.0
    qkv.view(q_len, heads + 2 * kv_heads, D)[-1, :heads] = (direction * 4).to(dtype)
    got = ops.attention(qkv, heads, kv_heads, D, batch, cache, 1.0 / math.sqrt(D), None)
    want = TorchOps(dtype).attention(qkv, heads, kv_heads, D, batch, cache, 1.0 / math.sqrt(D), None)
    close(got, want, dtype, "far key")
    assert (got[-1].float() - 7.0).abs().max().item() < 0.1


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_windows_edge(ops, dtype):
    """With a window of 50 the key 50 places back is out and the key 49 back is in: a
    marker on either side tells."""
    heads, kv_heads, D, window = 2, 1, 32, 50
    cache = make_cache(8, kv_heads, D, 1, 8, dtype, 50)
    cache.k.mul_(0.02)
    cache.window = window
    pos = 300
    batch = make_batch([0], [pos], [1])
    direction = torch.zeros(D, device="cuda")
    direction[0] = 10.0
    for back, marker in ((50, -5.0), (49, 3.0)):
        p = pos - back
        page = int(cache.table[0, p // PAGE])
        cache.k[page, 0, p % PAGE] = direction.to(dtype)
        cache.v[page, 0, p % PAGE] = marker
    qkv = rand((1, (heads + 2 * kv_heads) * D), dtype, 51, 0.02)
    qkv.view(1, heads + 2 * kv_heads, D)[0, :heads] = (direction * 3).to(dtype)
    got = ops.attention(qkv, heads, kv_heads, D, batch, cache, 1.0 / math.sqrt(D), window)
    assert (got.float() - 3.0).abs().max().item() < 0.1


# -- token selection --------------------------------------------------------------------
def test_greedy_takes_the_lowest_index_on_ties(ops):
    logits = rand((5, 1001), torch.float32, 60)
    logits[2, 17] = logits[2, 900] = 50.0
    req = torch.arange(5, dtype=torch.int32, device="cuda")
    got = ops.select_tokens(logits, 0.0, 0, req, 0)
    assert got.tolist() == logits.argmax(dim=-1).tolist() and got[2].item() == 17


def test_temperature_draws_match_the_plain_sampler(ops):
    import plain_qwen3 as plain

    logits = rand((6, 777), torch.float32, 61, 2.0)
    req = torch.tensor([5, 0, 9, 1, 2, 3], dtype=torch.int32, device="cuda")
    got = ops.select_tokens(logits, 0.7, 99, req, 4).tolist()
    want = [plain.sample_temperature(logits[r].cpu(), 0.7, 99, int(req[r]), 4) for r in range(6)]
    assert got == want
    # draws follow softmax(logits / T): chi-square-free sanity on a 3-way distribution
    small = torch.tensor([[2.0, 1.0, 0.0]], device="cuda").repeat(1, 1)
    counts = [0, 0, 0]
    one = torch.zeros(1, dtype=torch.int32, device="cuda")
    for step in range(3000):
        counts[ops.select_tokens(small, 1.0, 7, one, step).item()] += 1
    probs = torch.softmax(small[0], -1).tolist()
    for c, p in zip(counts, probs):
        assert abs(c / 3000 - p) < 0.03
