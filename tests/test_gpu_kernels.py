"""Each kernel alone against a plain float32 reference of the same operation, at sizes the engine's
tiny models do not use (GPU)."""
import math

import pytest
import torch

from tests.plain import qwen3_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    from jllm_serve_b200.csrc import ops as o
    o.require_device()
    return o


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator().manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed_rows(ops, dtype):
    table = rnd(517, 72, dtype=dtype)
    ids = torch.tensor([0, 516, 3, 3, 100], dtype=torch.int32, device=DEV)
    out = torch.empty(5, 72, device=DEV)
    ops.embed_rows(ids, table, out)
    assert torch.equal(out, table.float()[ids.long()])


@pytest.mark.parametrize("dim", [72, 1000, 4096, 5120])
@pytest.mark.parametrize("gain_dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm(ops, dim, gain_dtype):
    x, gain = rnd(7, dim, scale=3.0), (1 + 0.1 * rnd(dim)).to(gain_dtype)
    want = P.rmsnorm(x.cpu(), gain.float().cpu(), 1e-5)
    out = torch.empty(7, dim, device=DEV)
    ops.rmsnorm(x, gain, 1e-5, out)
    assert torch.allclose(out.cpu(), want, rtol=2e-6, atol=1e-6)
    out16 = torch.empty(7, dim, dtype=torch.bfloat16, device=DEV)
    ops.rmsnorm(x, gain, 1e-5, out16)
    assert torch.allclose(out16.float().cpu(), want, rtol=2 ** -8, atol=1e-6)
    idx = torch.tensor([6, 0, 6], dtype=torch.int32, device=DEV)          # gathered rows (the head's input)
    sel = torch.empty(3, dim, device=DEV)
    ops.rmsnorm(x, gain, 1e-5, sel, row_index=idx)
    assert torch.equal(sel, out[idx.long()])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu(ops, dtype):
    gu = rnd(5, 2 * 200, dtype=dtype, scale=2.0)
    out = torch.empty(5, 200, dtype=dtype, device=DEV)
    ops.swiglu(gu, out)
    g, u = gu.float().cpu()[:, :200], gu.float().cpu()[:, 200:]
    want = P.silu(g) * u
    tol = 1e-6 if dtype == torch.float32 else 2 ** -8
    assert torch.allclose(out.float().cpu(), want, rtol=tol, atol=1e-6)


def gemm_want(a, w, bias=None, base=None):
    y = a.double().cpu() @ w.double().cpu().t()
    if bias is not None:
        y = y + bias.double().cpu()
    if base is not None:
        y = y + base.double().cpu()
    return y.float()


@pytest.mark.parametrize("M,N,K", [(1, 7, 5), (3, 130, 72), (65, 64, 129), (200, 517, 96)])
def test_gemm_plain_float32(ops, M, N, K):
    a, w, bias = rnd(M, K), rnd(N, K, seed=1), rnd(N, seed=2)
    out = torch.empty(M, N, device=DEV)
    ops.gemm_plain(a, w, out, bias)
    assert torch.allclose(out.cpu(), gemm_want(a, w, bias), rtol=1e-5, atol=1e-5)
    base = rnd(M, N, seed=3)
    acc = base.clone()
    ops.gemm_plain(a, w, acc, None, accumulate=True)
    assert torch.allclose(acc.cpu(), gemm_want(a, w, None, base), rtol=1e-5, atol=1e-5)
    # a row's result does not depend on the rows beside it: bit for bit
    one = torch.empty(1, N, device=DEV)
    ops.gemm_plain(a[M // 2:M // 2 + 1], w, one, bias)
    assert torch.equal(one[0], out[M // 2])


def test_gemm_plain_strided_and_bfloat16(ops):
    big = rnd(9, 300, dtype=torch.bfloat16)
    a, w = big[:, 100:172], rnd(50, 72, dtype=torch.bfloat16, seed=4)      # a view with a row stride of 300
    out = torch.zeros(9, 80, dtype=torch.bfloat16, device=DEV)
    ops.gemm_plain(a, w, out[:, :50])
    assert torch.allclose(out[:, :50].float().cpu(), gemm_want(a, w), rtol=2 ** -7, atol=1e-3)
    assert float(out[:, 50:].abs().max()) == 0


@pytest.mark.parametrize("M", [1, 5, 8, 9, 16, 31, 33, 64])
@pytest.mark.parametrize("N,K", [(40, 64), (517, 72), (6144, 4096), (4736, 1000)])
def test_gemm_small_m(ops, M, N, K):
    a, w = rnd(M, K, dtype=torch.bfloat16), rnd(N, K, dtype=torch.bfloat16, seed=1, scale=0.05)
    bias = rnd(N, dtype=torch.bfloat16, seed=2)
    want = gemm_want(a, w, bias)
    out = torch.empty(M, N, device=DEV)
    ops.gemm_small_m(a, w, out, bias)
    tol = 1e-4 * math.sqrt(K)
    assert torch.allclose(out.cpu(), want, rtol=1e-4, atol=tol * 0.05)
    base = rnd(M, N, seed=3)
    acc = base.clone()
    ops.gemm_small_m(a, w, acc, None, accumulate=True)
    assert torch.allclose(acc.cpu(), gemm_want(a, w, None, base), rtol=1e-4, atol=tol * 0.05)
    out16 = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    ops.gemm_small_m(a, w, out16)
    assert torch.allclose(out16.float().cpu(), gemm_want(a, w), rtol=2 ** -7, atol=2e-3)


@pytest.mark.parametrize("M", [1, 5, 8, 16, 17, 33, 64, 100, 128, 129, 200, 256])
@pytest.mark.parametrize("N,K", [(40, 64), (517, 72), (6144, 4096), (4096, 12288), (4736, 1000), (128, 8)])
def test_gemm_stream(ops, M, N, K):
    """The weight-stream product over a packed weight: whole tiles and tiles whose k blocks fall to several blocks,
    bias, the residual add, bfloat16 output, few blocks (every block walks many tiles), and the same bits twice."""
    a, w = rnd(M, K, dtype=torch.bfloat16), rnd(N, K, dtype=torch.bfloat16, seed=1, scale=0.05)
    packed = ops.pack_weight(w)
    assert torch.equal(packed.unpack(), w)
    bias = rnd(N, dtype=torch.bfloat16, seed=2)
    want = gemm_want(a, w, bias)
    out = torch.full((M, N), float("nan"), device=DEV)
    ops.gemm_stream(a, packed, out, bias)
    assert ops.gemm_tcgen05_error() == 0
    tol = 1e-4 * math.sqrt(K) * 0.05
    assert torch.allclose(out.cpu(), want, rtol=1e-4, atol=tol), float((out.cpu() - want).abs().max())
    base = rnd(M, N, seed=3)
    for blocks in (0, 3, 7):
        acc, again = base.clone(), base.clone()
        ops.gemm_stream(a, packed, acc, bias, accumulate=True, max_blocks=blocks)
        ops.gemm_stream(a, packed, again, bias, accumulate=True, max_blocks=blocks)
        assert torch.allclose(acc.cpu(), gemm_want(a, w, bias, base), rtol=1e-4, atol=tol), blocks
        assert torch.equal(acc, again), "the parts of a tile are added in k order: two runs give the same bits"
    out16 = torch.zeros(M, N + 8, dtype=torch.bfloat16, device=DEV)
    ops.gemm_stream(a, packed, out16[:, :N])
    assert torch.allclose(out16[:, :N].float().cpu(), gemm_want(a, w), rtol=2 ** -7, atol=2e-3)
    assert float(out16[:, N:].abs().max()) == 0 and ops.gemm_tcgen05_error() == 0


@pytest.mark.parametrize("M", [1, 8, 20, 64, 128, 250])
@pytest.mark.parametrize("hidden,K", [(8, 8), (200, 72), (12288, 4096), (1000, 136)])
def test_gemm_stream_with_swiglu_epilogue(ops, M, hidden, K):
    a = rnd(M, K, dtype=torch.bfloat16)
    gate, up = rnd(hidden, K, dtype=torch.bfloat16, seed=1, scale=0.05), rnd(hidden, K, dtype=torch.bfloat16, seed=2, scale=0.05)
    w = torch.stack([gate.view(hidden // 8, 8, K), up.view(hidden // 8, 8, K)], dim=1).reshape(2 * hidden, K).contiguous()
    want = P.silu(gemm_want(a, gate)) * gemm_want(a, up)
    for blocks in (0, 5):
        out = torch.full((M, hidden), float("nan"), dtype=torch.bfloat16, device=DEV)
        ops.gemm_stream(a, ops.pack_weight(w), out, swiglu=True, max_blocks=blocks)
        assert ops.gemm_tcgen05_error() == 0
        assert torch.allclose(out.float().cpu(), want, rtol=2 ** -7, atol=1e-3), float((out.float().cpu() - want).abs().max())


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (1, 8, 8), (100, 517, 72), (300, 1000, 200), (2048, 6144, 4096),
                                   (257, 4096, 12288), (64, 300, 4096), (129, 257, 136)])
def test_gemm_tcgen05(ops, M, N, K):
    a, w = rnd(M, K, dtype=torch.bfloat16), rnd(N, K, dtype=torch.bfloat16, seed=1, scale=0.05)
    bias = rnd(N, dtype=torch.bfloat16, seed=2)
    want = gemm_want(a, w, bias)
    out = torch.full((M, N), float("nan"), device=DEV)
    ops.gemm_tcgen05(a, w, out, bias)
    assert ops.gemm_tcgen05_error() == 0
    tol = 1e-4 * math.sqrt(K) * 0.05
    assert torch.allclose(out.cpu(), want, rtol=1e-4, atol=tol), float((out.cpu() - want).abs().max())
    base = rnd(M, N, seed=3)
    acc = base.clone()
    ops.gemm_tcgen05(a, w, acc, None, accumulate=True, max_blocks=3)    # few blocks: every block walks many tiles
    assert torch.allclose(acc.cpu(), gemm_want(a, w, None, base), rtol=1e-4, atol=tol)
    out16 = torch.zeros(M, N + 8, dtype=torch.bfloat16, device=DEV)
    ops.gemm_tcgen05(a, w, out16[:, :N])
    assert torch.allclose(out16[:, :N].float().cpu(), gemm_want(a, w), rtol=2 ** -7, atol=2e-3)
    assert float(out16[:, N:].abs().max()) == 0 and ops.gemm_tcgen05_error() == 0
    # streamed (equal runs of (tile, k block) pairs per block, also with few blocks): the parts of a tile are added
    # in k order by whichever block comes last, so two runs give the same bits
    for blocks in (0, 5):
        one, two = base.clone(), base.clone()
        ops.gemm_tcgen05(a, w, one, None, accumulate=True, stream_mode=1, max_blocks=blocks)
        ops.gemm_tcgen05(a, w, two, None, accumulate=True, stream_mode=1, max_blocks=blocks)
        assert torch.allclose(one.cpu(), gemm_want(a, w, None, base), rtol=1e-4, atol=tol) and torch.equal(one, two)
    ops.gemm_tcgen05(a, w, out16[:, :N], stream_mode=1)
    assert torch.allclose(out16[:, :N].float().cpu(), gemm_want(a, w), rtol=2 ** -7, atol=2e-3)
    assert ops.gemm_tcgen05_error() == 0


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (1, 8, 8), (100, 517, 72), (300, 1000, 200), (2048, 6144, 4096),
                                   (257, 4096, 12288), (700, 384, 136), (129, 257, 1032)])
def test_gemm_pair(ops, M, N, K):
    """Two SMs to a 256 x 256 tile (tcgen05 cta_group::2): the product with a bias, the residual add with few pairs (each
    walks many tiles and both accumulators), bfloat16 into a view with columns beside it, the SwiGLU epilogue; rows and
    columns that end inside a tile, inside a block's half of it, and a tile whose second half of W does not exist."""
    if ops.resident_pairs() < 1:
        pytest.skip("the device runs no pair of blocks of this kernel")
    a, w = rnd(M, K, dtype=torch.bfloat16), rnd(N, K, dtype=torch.bfloat16, seed=1, scale=0.05)
    bias = rnd(N, dtype=torch.bfloat16, seed=2)
    tol = 1e-4 * math.sqrt(K) * 0.05
    out = torch.full((M, N), float("nan"), device=DEV)
    ops.gemm_pair(a, w, out, bias)
    assert ops.gemm_tcgen05_error() == 0
    assert torch.allclose(out.cpu(), gemm_want(a, w, bias), rtol=1e-4, atol=tol), float((out.cpu() - gemm_want(a, w, bias)).abs().max())
    base = rnd(M, N, seed=3)
    for pairs in (3, 0):
        acc = base.clone()
        ops.gemm_pair(a, w, acc, None, accumulate=True, max_pairs=pairs, stream_mode=2)
        assert torch.allclose(acc.cpu(), gemm_want(a, w, None, base), rtol=1e-4, atol=tol)
    # streamed: the tiles of the last round are cut up over the pairs, whose parts are added in k order (the same bits twice)
    for pairs in (3, 5, 0):
        one, two = base.clone(), base.clone()
        ops.gemm_pair(a, w, one, None, accumulate=True, max_pairs=pairs, stream_mode=1)
        ops.gemm_pair(a, w, two, None, accumulate=True, max_pairs=pairs, stream_mode=1)
        assert torch.allclose(one.cpu(), gemm_want(a, w, None, base), rtol=1e-4, atol=tol) and torch.equal(one, two)
    out16 = torch.zeros(M, N + 8, dtype=torch.bfloat16, device=DEV)
    for mode in (2, 1):
        out16[:, :N].fill_(float("nan"))
        ops.gemm_pair(a, w, out16[:, :N], stream_mode=mode, max_pairs=7 if mode == 1 else 0)
        assert torch.allclose(out16[:, :N].float().cpu(), gemm_want(a, w), rtol=2 ** -7, atol=2e-3)
        assert float(out16[:, N:].abs().max()) == 0
    # the same bits as the one-SM kernel: the same products summed in the same order, k block by k block
    single, again = torch.empty(M, N, device=DEV), torch.empty(M, N, device=DEV)
    ops.gemm_tcgen05(a, w, single, bias)
    ops.gemm_pair(a, w, again, bias, stream_mode=2)
    assert torch.equal(single, again)
    if N % 16 == 0:
        hidden = N // 2
        g = gemm_want(a, w.view(hidden // 8, 2, 8, K)[:, 0].reshape(hidden, K))
        u = gemm_want(a, w.view(hidden // 8, 2, 8, K)[:, 1].reshape(hidden, K))
        h = torch.full((M, hidden), float("nan"), dtype=torch.bfloat16, device=DEV)
        ops.gemm_pair(a, w, h, swiglu=True)
        assert torch.allclose(h.float().cpu(), P.silu(g) * u, rtol=2 ** -7, atol=1e-3)
    assert ops.gemm_tcgen05_error() == 0


def test_gemm_pair_random_shapes(ops):
    """Random shapes of the paired product (rows, columns and k that end anywhere inside tiles, few pairs or all): the
    one-SM product's bits and the plain float32 product's values; with the last round's tiles cut up over the pairs
    (their parts are added in another grouping) the values, and the same bits when run again."""
    import random
    if ops.resident_pairs() < 1:
        pytest.skip("the device runs no pair of blocks of this kernel")
    rng = random.Random(11)
    for trial in range(14):
        M = rng.choice([rng.randint(1, 300), rng.randint(300, 1500)])
        N = rng.choice([rng.randint(1, 600), 8 * rng.randint(1, 400)])
        K = 8 * rng.randint(1, 160)
        a, w = rnd(M, K, dtype=torch.bfloat16, seed=trial), rnd(N, K, dtype=torch.bfloat16, seed=100 + trial, scale=0.05)
        bias = rnd(N, dtype=torch.bfloat16, seed=200 + trial)
        ld = N + rng.choice([0, 4, 5])
        base = rnd(M, ld, seed=300 + trial)
        got, ref = base.clone(), base.clone()
        pairs, mode = rng.choice([0, 1, 3, 9]), rng.choice([1, 2])
        ops.gemm_pair(a, w, got[:, :N], bias, accumulate=True, max_pairs=pairs, stream_mode=mode)
        ops.gemm_tcgen05(a, w, ref[:, :N], bias, accumulate=True)
        what = f"trial {trial}: M={M} N={N} K={K} ld={ld} pairs={pairs} mode={mode}"
        assert ops.gemm_tcgen05_error() == 0, what
        if mode == 2:
            assert torch.equal(got, ref), what
        else:
            again = base.clone()
            ops.gemm_pair(a, w, again[:, :N], bias, accumulate=True, max_pairs=pairs, stream_mode=mode)
            assert torch.equal(got, again) and torch.equal(got[:, N:], base[:, N:]), what
        tol = 1e-4 * math.sqrt(K) * 0.05
        assert torch.allclose(got[:, :N].cpu(), gemm_want(a, w, bias, base[:, :N]), rtol=1e-4, atol=tol), what


@pytest.mark.parametrize("M,N,K", [(512, 4096, 12288), (300, 6144, 4096), (256, 1000, 520)])
def test_gemm_pair_streamed_with_fewer_tiles_than_pairs(ops, M, N, K):
    """Fewer 256 x 256 tiles than the device runs pairs: streamed, every tile's k blocks are cut up over ALL pairs (a
    tile then has two to four parts, one of which finishes it): the plain product's values, and the same bits twice."""
    if ops.resident_pairs() < 1:
        pytest.skip("the device runs no pair of blocks of this kernel")
    assert -(-M // 256) * -(-N // 256) < ops.resident_pairs()
    a, w = rnd(M, K, dtype=torch.bfloat16), rnd(N, K, dtype=torch.bfloat16, seed=1, scale=0.05)
    bias, base = rnd(N, dtype=torch.bfloat16, seed=2), rnd(M, N, seed=3)
    want = gemm_want(a, w, bias, base)
    tol = 1e-4 * math.sqrt(K) * 0.05
    got, again = base.clone(), base.clone()
    ops.gemm_pair(a, w, got, bias, accumulate=True, stream_mode=1)
    ops.gemm_pair(a, w, again, bias, accumulate=True, stream_mode=1)
    assert ops.gemm_tcgen05_error() == 0
    assert torch.allclose(got.cpu(), want, rtol=1e-4, atol=tol), float((got.cpu() - want).abs().max())
    assert torch.equal(got, again)
    out16 = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.gemm_pair(a, w, out16, stream_mode=1)
    assert torch.allclose(out16.float().cpu(), gemm_want(a, w), rtol=2 ** -7, atol=2e-3) and ops.gemm_tcgen05_error() == 0


@pytest.mark.parametrize("kernel", ["tiles", "pair"])
@pytest.mark.parametrize("M,N,K", [(300, 1000, 200), (2048, 4096, 512), (129, 260, 136), (31, 36, 64), (513, 7936, 72)])
def test_gemm_float32_output_by_bulk_copies(ops, M, N, K, kernel):
    """A float32 output whose rows allow a tensor map leaves the tcgen05 products by tiled bulk copies of 32 x 32 blocks
    (the residual add as a reduce where the data lies): the same bits as the epilogue warps' own loads and stores, for
    the product with a bias and for the add, into a view that starts 16 bytes into wider rows; what lies beside the
    view, and beyond M and N inside the last blocks, is left alone."""
    if kernel == "pair" and ops.resident_pairs() < 1:
        pytest.skip("the device runs no pair of blocks of this kernel")
    go = ops.gemm_pair if kernel == "pair" else ops.gemm_tcgen05
    a, w = rnd(M, K, dtype=torch.bfloat16), rnd(N, K, dtype=torch.bfloat16, seed=1, scale=0.05)
    bias = rnd(N, dtype=torch.bfloat16, seed=2)
    tol = 1e-4 * math.sqrt(K) * 0.05
    base = rnd(M + 3, N + 12, seed=3)
    results = {}
    for plain in (False, True):
        ops.gemm_plain_stores(plain)
        try:
            wide = base.clone()
            view = wide[:M, 4:4 + N]
            go(a, w, view, bias)
            fresh = view.clone()
            go(a, w, view, None, accumulate=True)
            results[plain] = (fresh, view.clone(), wide)
        finally:
            ops.gemm_plain_stores(False)
    fresh, added, wide = results[False]
    assert ops.gemm_tcgen05_error() == 0
    assert torch.allclose(fresh.cpu(), gemm_want(a, w, bias), rtol=1e-4, atol=tol)
    assert torch.allclose(added.cpu(), gemm_want(a, w, None, fresh), rtol=1e-4, atol=tol)
    assert torch.equal(fresh, results[True][0]) and torch.equal(added, results[True][1])
    untouched = torch.ones_like(base, dtype=torch.bool)
    untouched[:M, 4:4 + N] = False
    assert torch.equal(wide[untouched], base[untouched])


@pytest.mark.parametrize("width", [32, 64, 128, 192, 256])
@pytest.mark.parametrize("M,N,K", [(64, 4096, 4096), (33, 517, 72), (200, 1000, 1032), (128, 24576, 512)])
def test_gemm_tcgen05_tile_widths(ops, M, N, K, width):
    """Every width of the output tile, chosen by hand: the product, the residual add, the streamed product and
    the SwiGLU epilogue give what the default width gives."""
    a, w = rnd(M, K, dtype=torch.bfloat16), rnd(N, K, dtype=torch.bfloat16, seed=1, scale=0.05)
    bias = rnd(N, dtype=torch.bfloat16, seed=2)
    tol = 1e-4 * math.sqrt(K) * 0.05
    out = torch.full((M, N), float("nan"), device=DEV)
    ops.gemm_tcgen05(a, w, out, bias, tile_width=width)
    assert torch.allclose(out.cpu(), gemm_want(a, w, bias), rtol=1e-4, atol=tol)
    base = rnd(M, N, seed=3)
    acc, split = base.clone(), base.clone()
    ops.gemm_tcgen05(a, w, acc, None, accumulate=True, tile_width=width, max_blocks=5)
    ops.gemm_tcgen05(a, w, split, None, accumulate=True, tile_width=width, stream_mode=1)
    want = gemm_want(a, w, None, base)
    assert torch.allclose(acc.cpu(), want, rtol=1e-4, atol=tol) and torch.allclose(split.cpu(), want, rtol=1e-4, atol=tol)
    if N % 16 == 0:
        hidden = N // 2
        g = gemm_want(a, w.view(hidden // 8, 2, 8, K)[:, 0].reshape(hidden, K))
        u = gemm_want(a, w.view(hidden // 8, 2, 8, K)[:, 1].reshape(hidden, K))
        h = torch.full((M, hidden), float("nan"), dtype=torch.bfloat16, device=DEV)
        ops.gemm_tcgen05(a, w, h, swiglu=True, tile_width=width)
        assert torch.allclose(h.float().cpu(), P.silu(g) * u, rtol=2 ** -7, atol=1e-3)
    assert ops.gemm_tcgen05_error() == 0


@pytest.mark.parametrize("M", [1, 8, 20, 33, 200])
@pytest.mark.parametrize("hidden,K", [(8, 8), (200, 72), (12288, 4096), (1000, 136)])
def test_gemm_with_swiglu_epilogue(ops, M, hidden, K):
    """gate and up rows interleaved in blocks of 8: the product's epilogue gives silu(gate) * up directly."""
    a = rnd(M, K, dtype=torch.bfloat16)
    gate, up = rnd(hidden, K, dtype=torch.bfloat16, seed=1, scale=0.05), rnd(hidden, K, dtype=torch.bfloat16, seed=2, scale=0.05)
    w = torch.stack([gate.view(hidden // 8, 8, K), up.view(hidden // 8, 8, K)], dim=1).reshape(2 * hidden, K).contiguous()
    g, u = gemm_want(a, gate), gemm_want(a, up)
    want = P.silu(g) * u
    out = torch.full((M, hidden), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.gemm_bf16(a, w, out, swiglu=True)
    assert ops.gemm_tcgen05_error() == 0
    assert torch.allclose(out.float().cpu(), want, rtol=2 ** -7, atol=1e-3), float((out.float().cpu() - want).abs().max())
    out32 = torch.full((M, hidden), float("nan"), device=DEV)
    ops.gemm_tcgen05(a, w, out32, swiglu=True)
    # float32 sums of K bfloat16 products differ from float64 by about 1e-4 sqrt(K) 0.05, times |up| of a few
    assert torch.allclose(out32.cpu(), want, rtol=1e-3, atol=1e-4 * math.sqrt(K) * 0.05 * 4 + 1e-5)


def test_gemm_small_m_refuses_what_it_cannot_do(ops):
    a, w = rnd(3, 12, dtype=torch.bfloat16), rnd(8, 12, dtype=torch.bfloat16)
    with pytest.raises(ops.KernelError, match="K % 8"):
        ops.gemm_small_m(a, w, torch.empty(3, 8, device=DEV))
    assert not ops.gemm_bf16_fits(a, w, None)


# ---- q/k norm + RoPE + cache write, and attention over a shuffled, poisoned pool --------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,Hkv,hd,rot,norm", [(6, 2, 48, 24, True), (4, 4, 16, 16, False), (8, 1, 128, 128, True),
                                                (2, 2, 80, 0, True), (3, 1, 64, 64, True), (5, 5, 256, 256, False),
                                                (4, 2, 128, 64, True)])
def test_qk_norm_rope_store(ops, dtype, H, Hkv, hd, rot, norm):
    R, page, pages, eps = 11, 4, 9, 1e-5
    width = (H + 2 * Hkv) * hd
    qkv = rnd(R, width, dtype=dtype)
    qg, kg = (1 + 0.1 * rnd(hd)).to(dtype), (1 + 0.1 * rnd(hd, seed=1)).to(dtype)
    positions = torch.tensor([5, 6, 7, 0, 1, 2, 3, 30, 31, 32, 33], dtype=torch.int32)
    slots = torch.randperm(pages * page)[:R].to(torch.int32)
    cos, sin = P.rope_table(range(40), rot, 50000.0) if rot else (None, None)
    kc = torch.full((pages, Hkv, page, hd), float("nan"), dtype=dtype, device=DEV)
    vc = torch.full_like(kc, float("nan"))
    x = qkv.float().cpu().reshape(R, H + 2 * Hkv, hd)
    q, k, v = x[:, :H], x[:, H:H + Hkv], x[:, H + Hkv:]
    if norm:
        q, k = P.rmsnorm(q, qg.float().cpu(), eps), P.rmsnorm(k, kg.float().cpu(), eps)
    if rot:
        q, k = P.apply_rope(q, cos[positions.long()], sin[positions.long()]), \
            P.apply_rope(k, cos[positions.long()], sin[positions.long()])
    work = qkv.clone()
    ops.qk_norm_rope_store(work, qg if norm else None, kg if norm else None, eps,
                           cos.to(DEV) if rot else None, sin.to(DEV) if rot else None, rot, positions.to(DEV),
                           slots.to(DEV), kc, vc, H, Hkv, hd, page)
    tol = dict(rtol=1e-5, atol=1e-6) if dtype == torch.float32 else dict(rtol=2 ** -7, atol=1e-3)
    got = work.float().cpu().reshape(R, H + 2 * Hkv, hd)
    assert torch.allclose(got[:, :H], q, **tol)
    assert torch.equal(got[:, H:], x[:, H:])                       # keys and values in the buffer are left alone
    for r in range(R):
        pg, off = int(slots[r]) // page, int(slots[r]) % page
        assert torch.allclose(kc[pg, :, off].float().cpu(), k[r], **tol)
        assert torch.allclose(vc[pg, :, off].float().cpu(), v[r].to(dtype).float(), **tol)
    written = torch.zeros(pages * page, dtype=torch.bool)
    written[slots.long()] = True
    rest = kc.float().cpu().permute(0, 2, 1, 3).reshape(pages * page, -1)[~written]
    assert torch.isnan(rest).all()                                   # nothing else was touched


def rows_close(got, want, what="", share=2 ** -7, floor=2e-4):
    """Every row within `share` of ITS OWN largest |value| (plus a floor for rounding of values near zero): an absolute
    tolerance sized for the largest row would let a damaged row of small values through. Returns the worst ratio."""
    got, want = got.float().cpu(), want.float().cpu()
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    tol = share * want.abs().amax(dim=-1, keepdim=True) + floor
    ratio = ((got - want).abs() / tol).amax(dim=-1)
    worst = int(ratio.argmax())
    assert float(ratio[worst]) <= 1.0, (f"{what}: row {worst} differs by {float((got[worst] - want[worst]).abs().max()):.3e}, "
                                        f"its largest |value| is {float(want[worst].abs().max()):.3e}")
    return float(ratio[worst])


MODES = ("random", "far", "planted")


def attention_case(ops, dtype, H, Hkv, hd, page, lens, window, scale, make_far_key=False, q_lens=None, planted=False):
    """Several requests of `lens` cached positions each; the last `q_len` positions of each are the step's rows.
    `make_far_key` (True or "far"): one early key that the last query matches strongly. `planted` (or the mode
    "planted"): one key in every 64-key tile that EVERY query matches strongly, with a value that tells which tile
    it came from, so every row's result is large and a tile that is dropped, doubled or misplaced changes it."""
    planted = planted or make_far_key == "planted"
    make_far_key = make_far_key is True or make_far_key == "far"
    torch.manual_seed(H * 1000 + hd + page)
    nseq = len(lens)
    q_lens = q_lens or [min(l, 1 + 3 * i) for i, l in enumerate(lens)]
    pages_needed = sum(-(-l // page) for l in lens)
    pool = pages_needed + 5
    perm = torch.randperm(pool).tolist()
    kc = torch.full((pool, Hkv, page, hd), float("nan"), dtype=dtype, device=DEV)
    vc = torch.full_like(kc, float("nan"))
    max_blocks = max(-(-l // page) for l in lens) + 2
    tables = torch.full((nseq, max_blocks), -1, dtype=torch.int32)
    rows_q, row_seg, row_pos, wants = [], [], [], []
    for s, L in enumerate(lens):
        k, v, q = torch.randn(L, Hkv, hd), torch.randn(L, Hkv, hd), torch.randn(L, H, hd)
        if make_far_key:
            # one early key that the last query matches strongly: a fault that drops or misplaces far keys shows
            far = 1 if L > 3 else 0
            k[far, :, :] = 0
            k[far, :, 0] = 6.0 / scale / max(1.0, hd ** 0.5)
            q[L - 1, :, :] *= 0.05
            q[L - 1, :, 0] = hd ** 0.5
            v[far] = 7.0
        if planted:
            marks = torch.arange(17 if L > 17 else 0, L, 64)
            k[:, :, 1] = 0                     # only the planted keys answer to the queries' large component
            k[marks] = 0
            k[marks, :, 1] = 1.0
            v[marks] = (10.0 * (1 + torch.arange(len(marks), dtype=torch.float32)))[:, None, None] * (1 + 0.1 * torch.randn(len(marks), Hkv, hd))
            q *= 0.3
            q[:, :, 1] = 8.0 / scale
        k, v, q = k.to(dtype).float(), v.to(dtype).float(), q.to(dtype).float()
        for b in range(-(-L // page)):
            pg = perm.pop()
            tables[s, b] = pg
            n = min(page, L - b * page)
            kc[pg, :, :n] = k[b * page:b * page + n].transpose(0, 1).to(dtype).to(DEV)
            vc[pg, :, :n] = v[b * page:b * page + n].transpose(0, 1).to(dtype).to(DEV)
        want = P.causal_gqa_attention(q, k, v, scale, window).reshape(L, H * hd)
        for p in range(L - q_lens[s], L):
            rows_q.append(q[p].reshape(-1))
            row_seg.append(s)
            row_pos.append(p)
            wants.append(want[p])
    qd = torch.stack(rows_q).to(dtype).to(DEV)
    out = torch.empty_like(qd)
    return qd, kc, vc, out, torch.tensor(row_seg, dtype=torch.int32, device=DEV), \
        torch.tensor(row_pos, dtype=torch.int32, device=DEV), tables.to(DEV), torch.stack(wants), q_lens


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,Hkv,hd,page,window", [(6, 2, 48, 16, 0), (4, 4, 16, 4, 0), (8, 1, 128, 16, 0),
                                                   (6, 3, 80, 8, 21), (4, 2, 256, 16, 0), (2, 1, 32, 1, 7)])
def test_attention_plain(ops, dtype, H, Hkv, hd, page, window):
    lens, scale = [1, 17, 64, 131, 300], 1.0 / math.sqrt(hd)
    for far in MODES:
        q, kc, vc, out, rseg, rpos, tables, want, _ = attention_case(ops, dtype, H, Hkv, hd, page, lens, window, scale,
                                                                      far)
        ops.attention_plain(q, q.stride(0), kc, vc, out, rseg, rpos, tables, q.shape[0], H, Hkv, hd, page, window, scale)
        if dtype == torch.float32:
            rows_close(out, want, f"plain {far}", share=1e-5, floor=1e-6)
        else:
            rows_close(out, want, f"plain {far}")


def check_attention_prefill(ops, H, Hkv, hd, page, window, lens, q_lens, kernel):
    scale = 1.0 / math.sqrt(hd)
    for far in MODES:
        q, kc, vc, out, rseg, rpos, tables, want, q_lens = attention_case(ops, torch.bfloat16, H, Hkv, hd, page, lens,
                                                                          window, scale, far, q_lens)
        out.fill_(float("nan"))
        starts = [sum(q_lens[:i]) for i in range(len(lens))]
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
        ops.attention_prefill(q, kc, vc, out, i32(starts), i32(q_lens), i32(lens), tables, q.shape[0], H, Hkv, hd, page,
                              window, scale, kernel=kernel)
        assert ops.attention_prefill_tc_error() == 0
        rows_close(out, want, f"prefill {kernel} {far}")


@pytest.mark.parametrize("kernel", ["mma", "tc", "pair"])
@pytest.mark.parametrize("H,Hkv,hd,page,window", [(6, 2, 64, 16, 0), (4, 4, 128, 4, 0), (32, 8, 128, 16, 0),
                                                   (6, 3, 64, 8, 21), (4, 1, 256, 16, 0), (2, 1, 64, 1, 7),
                                                   (8, 2, 128, 16, 100)])
def test_attention_prefill(ops, H, Hkv, hd, page, window, kernel):
    """Portions of prompts (and single rows) of several requests in one launch, starting anywhere in a page."""
    if kernel != "mma" and hd != 128:
        pytest.skip("the tcgen05 kernels are built for head size 128")
    check_attention_prefill(ops, H, Hkv, hd, page, window, [1, 17, 64, 131, 300, 1000, 77], [1, 17, 30, 131, 200, 65, 1],
                            kernel)


@pytest.mark.parametrize("kernel", ["tc", "pair"])
@pytest.mark.parametrize("H,Hkv,page,window", [(2, 1, 1, 0), (3, 3, 2, 0), (4, 2, 32, 0), (2, 2, 64, 300), (6, 1, 128, 0),
                                               (4, 2, 16, 128), (2, 1, 8, 129), (2, 2, 16, 1)])
def test_attention_prefill_tcgen05_tiles(ops, H, Hkv, page, window, kernel):
    """The tcgen05 kernel over several query tiles and many key tiles: portions that start and end anywhere
    relative to the 128-key tiles, every page size, windows at, below and above a tile."""
    check_attention_prefill(ops, H, Hkv, 128, page, window, [128, 129, 700, 1500, 256, 383],
                            [128, 2, 513, 300, 129, 255], kernel)


@pytest.mark.parametrize("splits", [1, 3, 8])
@pytest.mark.parametrize("H,Hkv,hd,page,window", [(6, 2, 48, 16, 0), (4, 4, 16, 4, 0), (32, 8, 128, 16, 0),
                                                   (6, 3, 80, 8, 21), (16, 1, 256, 16, 0), (2, 1, 32, 1, 7),
                                                   (8, 2, 64, 16, 100)])
def test_attention_decode(ops, H, Hkv, hd, page, window, splits):
    """One query per request: rows of the decode kernel against the plain attention, also split over blocks."""
    lens, scale = [1, 17, 64, 131, 300, 1000], 1.0 / math.sqrt(hd)
    for far in MODES:
        q, kc, vc, out, rseg, rpos, tables, want, q_lens = attention_case(ops, torch.bfloat16, H, Hkv, hd, page, lens,
                                                                          window, scale, far)
        # keep the last row of every request only: one query position per row
        last = torch.tensor([sum(q_lens[:i + 1]) - 1 for i in range(len(lens))], device=DEV)
        q1, rseg1, rpos1, want1 = q[last].contiguous(), rseg[last].contiguous(), rpos[last].contiguous(), want[last.cpu()]
        out1 = torch.full_like(q1, float("nan"))
        scratch = torch.full((ops.attention_decode_scratch_floats(len(lens), H, hd, splits) + 1,), float("nan"),
                             device=DEV)
        ops.attention_decode(q1, kc, vc, out1, rseg1, rpos1, tables, len(lens), H, Hkv, hd, page, window, scale, splits,
                             scratch)
        rows_close(out1, want1, f"decode splits {splits} {far}")
        # the partials added up by the last block of every pair (head sizes 64, 128, 256) or by a kernel of their own:
        # the same bits; and again, with the counters that the first launch must have left at zero
        again, apart = torch.full_like(q1, float("nan")), torch.full_like(q1, float("nan"))
        ops.attention_decode(q1, kc, vc, again, rseg1, rpos1, tables, len(lens), H, Hkv, hd, page, window, scale, splits,
                             scratch)
        ops.attention_decode_separate_combine(True)
        try:
            ops.attention_decode(q1, kc, vc, apart, rseg1, rpos1, tables, len(lens), H, Hkv, hd, page, window, scale,
                                 splits, scratch)
        finally:
            ops.attention_decode_separate_combine(False)
        assert torch.equal(out1, again) and torch.equal(out1, apart)


@pytest.mark.parametrize("how,n", [("split", 1), ("split", 3), ("split", 8), ("split", 20), ("flat", 5), ("flat", 40)])
@pytest.mark.parametrize("H,Hkv,hd,page,window,norm", [(32, 8, 128, 16, 0, True), (16, 1, 256, 16, 0, False),
                                                        (8, 2, 64, 8, 100, True), (6, 3, 64, 1, 0, True),
                                                        (4, 4, 128, 4, 70, False)])
def test_attention_decode_fresh(ops, H, Hkv, hd, page, window, norm, how, n):
    """The decode attention that norms and rotates its own rows and writes their keys and values: the same bits, in
    its output and in the cache, as the row-wise kernel followed by the decode attention; positions at the start, the
    end and the middle of pages and of 64-key tiles; what the cache held at the newest position does not matter."""
    import random
    rng = random.Random(H * 100 + hd + n)
    lens = [1, 17, 64, 65, 131, 300, 1000, 128, 2]
    R, eps, scale = len(lens), 1e-6, 1.0 / math.sqrt(hd)
    pages_of = [-(-L // page) for L in lens]
    pool = sum(pages_of) + 7
    order = list(range(pool))
    rng.shuffle(order)
    tables = torch.full((R, max(pages_of) + 1), -1, dtype=torch.int32)
    at = 0
    for r, npg in enumerate(pages_of):
        tables[r, :npg] = torch.tensor(order[at:at + npg], dtype=torch.int32)
        at += npg
    kc = (rnd(pool, Hkv, page, hd, seed=5) * 0.5).to(torch.bfloat16)
    vc = rnd(pool, Hkv, page, hd, seed=6).to(torch.bfloat16)
    positions = torch.tensor([L - 1 for L in lens], dtype=torch.int32)
    slots = torch.tensor([int(tables[r, (L - 1) // page]) * page + (L - 1) % page for r, L in enumerate(lens)], dtype=torch.int32)
    for r in range(R):          # nothing may be read of what the cache holds at the newest position
        kc[int(slots[r]) // page, :, int(slots[r]) % page] = float("nan")
        vc[int(slots[r]) // page, :, int(slots[r]) % page] = float("nan")
    qkv = rnd(R, (H + 2 * Hkv) * hd, dtype=torch.bfloat16, seed=7)
    qg, kg = (1 + 0.1 * rnd(hd, seed=8)).to(torch.bfloat16), (1 + 0.1 * rnd(hd, seed=9)).to(torch.bfloat16)
    cos, sin = P.rope_table(range(max(lens) + 1), hd, 50000.0)
    cos, sin = cos.to(DEV), sin.to(DEV)
    seg, pos, tab = torch.arange(R, dtype=torch.int32, device=DEV), positions.to(DEV), tables.to(DEV)
    if how == "flat":
        n = min(n, 62 * Hkv)
        scratch = torch.full((ops.attention_decode_flat_scratch_floats(R, H, Hkv, hd, n),), float("nan"), device=DEV)
    else:
        scratch = torch.full((ops.attention_decode_scratch_floats(R, H, hd, n) + 1,), float("nan"), device=DEV)
    # apart: the row-wise kernel, then the attention
    work, kc_a, vc_a = qkv.clone(), kc.clone(), vc.clone()
    ops.qk_norm_rope_store(work, qg if norm else None, kg if norm else None, eps, cos, sin, hd, pos, slots.to(DEV), kc_a, vc_a,
                           H, Hkv, hd, page)
    out_a = torch.full((R, H * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    if how == "flat":
        ops.attention_decode_flat(work, kc_a, vc_a, out_a, seg, pos, tab, R, H, Hkv, hd, page, window, scale, n, scratch)
    else:
        ops.attention_decode(work, kc_a, vc_a, out_a, seg, pos, tab, R, H, Hkv, hd, page, window, scale, n, scratch)
    # in one
    kc_b, vc_b = kc.clone(), vc.clone()
    out_b = torch.full((R, H * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops._call("jllm_attention_decode_fresh", qkv.data_ptr(), qkv.stride(0), qg.data_ptr() if norm else None,
              kg.data_ptr() if norm else None, ops._DT[qg.dtype], int(norm), eps, cos.data_ptr(), sin.data_ptr(),
              kc_b.data_ptr(), vc_b.data_ptr(), out_b.data_ptr(), out_b.stride(0), seg.data_ptr(), pos.data_ptr(),
              tab.data_ptr(), tab.stride(0), R, H, Hkv, hd, page, window, scale, int(how == "flat"), n, scratch.data_ptr(),
              ops._stream())
    assert torch.isfinite(out_a.float()).all()
    assert torch.equal(out_a, out_b)
    assert torch.equal(kc_a.view(torch.int16), kc_b.view(torch.int16)) and torch.equal(vc_a.view(torch.int16), vc_b.view(torch.int16))
    assert torch.equal(work[:, H * hd:], qkv[:, H * hd:])


def test_attention_decode_fresh_random_shapes(ops):
    """Random rows, lengths, splits and page sizes: the attention that finishes its own rows against the row-wise kernel
    followed by the attention (bits of the output and of the cache)."""
    import random
    rng = random.Random(23)
    for trial in range(14):
        H, Hkv, hd = rng.choice([(8, 2, 128), (4, 4, 64), (16, 2, 128), (4, 1, 256)])
        page = rng.choice([1, 4, 16, 32])
        lens = [rng.choice([1, 2, 63, 64, 65, 128, rng.randint(1, 700)]) for _ in range(rng.randint(1, 9))]
        R, eps, scale = len(lens), 1e-6, 1.0 / math.sqrt(hd)
        norm, splits = rng.random() < 0.7, rng.choice([1, 2, 5, 8, 13])
        if trial >= 10:                 # the last trials: thousands of keys, many splits
            page, splits = rng.choice([16, 64]), rng.choice([4, 13, 32])
            lens = [rng.randint(3000, 40000) for _ in range(rng.randint(1, 5))] + [rng.randint(1, 100)]
            R = len(lens)
        pages_of = [-(-L // page) for L in lens]
        pool = sum(pages_of) + 3
        order = list(range(pool))
        rng.shuffle(order)
        tables = torch.full((R, max(pages_of) + 1), -1, dtype=torch.int32)
        at = 0
        for r, npg in enumerate(pages_of):
            tables[r, :npg] = torch.tensor(order[at:at + npg], dtype=torch.int32)
            at += npg
        kc = (rnd(pool, Hkv, page, hd, seed=trial) * 0.5).to(torch.bfloat16)
        vc = rnd(pool, Hkv, page, hd, seed=50 + trial).to(torch.bfloat16)
        positions = torch.tensor([L - 1 for L in lens], dtype=torch.int32)
        slots = torch.tensor([int(tables[r, (L - 1) // page]) * page + (L - 1) % page for r, L in enumerate(lens)],
                             dtype=torch.int32)
        qkv = rnd(R, (H + 2 * Hkv) * hd, dtype=torch.bfloat16, seed=70 + trial)
        qg, kg = (1 + 0.1 * rnd(hd, seed=8)).to(torch.bfloat16), (1 + 0.1 * rnd(hd, seed=9)).to(torch.bfloat16)
        cos, sin = P.rope_table(range(max(lens) + 1), hd, 10000.0)
        cos, sin = cos.to(DEV), sin.to(DEV)
        seg, pos, tab = torch.arange(R, dtype=torch.int32, device=DEV), positions.to(DEV), tables.to(DEV)
        scratch = torch.full((ops.attention_decode_scratch_floats(R, H, hd, splits) + 1,), float("nan"), device=DEV)
        work, kc_a, vc_a = qkv.clone(), kc.clone(), vc.clone()
        ops.qk_norm_rope_store(work, qg if norm else None, kg if norm else None, eps, cos, sin, hd, pos, slots.to(DEV), kc_a,
                               vc_a, H, Hkv, hd, page)
        out_a = torch.full((R, H * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
        ops.attention_decode(work, kc_a, vc_a, out_a, seg, pos, tab, R, H, Hkv, hd, page, 0, scale, splits, scratch)
        kc_b, vc_b = kc.clone(), vc.clone()
        out_b = torch.full((R, H * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
        ops._call("jllm_attention_decode_fresh", qkv.data_ptr(), qkv.stride(0), qg.data_ptr() if norm else None,
                  kg.data_ptr() if norm else None, ops._DT[qg.dtype], int(norm), eps, cos.data_ptr(), sin.data_ptr(),
                  kc_b.data_ptr(), vc_b.data_ptr(), out_b.data_ptr(), out_b.stride(0), seg.data_ptr(), pos.data_ptr(),
                  tab.data_ptr(), tab.stride(0), R, H, Hkv, hd, page, 0, scale, 0, splits, scratch.data_ptr(), ops._stream())
        what = f"trial {trial}: heads {H}/{Hkv} of {hd}, page {page}, lens {lens}, {splits} splits, norm {norm}"
        assert torch.isfinite(out_a.float()).all(), what
        assert torch.equal(out_a, out_b), what
        assert torch.equal(kc_a.view(torch.int16), kc_b.view(torch.int16)), what
        assert torch.equal(vc_a.view(torch.int16), vc_b.view(torch.int16)), what


@pytest.mark.parametrize("blocks", [1, 7, 40, 296])
@pytest.mark.parametrize("H,Hkv,hd,page,window", [(32, 8, 128, 16, 0), (16, 1, 256, 16, 0), (8, 2, 64, 16, 100),
                                                   (6, 3, 64, 8, 21), (4, 4, 128, 4, 0)])
def test_attention_decode_dealt_out_evenly(ops, H, Hkv, hd, page, window, blocks):
    """The key tiles of all (row, kv head) pairs in equal runs over `blocks` blocks: runs that end inside a pair,
    pairs that spread over many blocks, blocks with nothing to do."""
    lens, scale = [1, 17, 64, 131, 300, 1000, 65, 2], 1.0 / math.sqrt(hd)
    blocks = min(blocks, 62 * Hkv)
    for far in MODES:
        q, kc, vc, out, rseg, rpos, tables, want, q_lens = attention_case(ops, torch.bfloat16, H, Hkv, hd, page, lens,
                                                                          window, scale, far)
        last = torch.tensor([sum(q_lens[:i + 1]) - 1 for i in range(len(lens))], device=DEV)
        q1, rseg1, rpos1, want1 = q[last].contiguous(), rseg[last].contiguous(), rpos[last].contiguous(), want[last.cpu()]
        out1 = torch.full_like(q1, float("nan"))
        scratch = torch.full((ops.attention_decode_flat_scratch_floats(len(lens), H, Hkv, hd, blocks),), float("nan"),
                             device=DEV)
        ops.attention_decode_flat(q1, kc, vc, out1, rseg1, rpos1, tables, len(lens), H, Hkv, hd, page, window, scale,
                                  blocks, scratch)
        rows_close(out1, want1, f"decode dealt out over {blocks} blocks {far}")
        again, apart = torch.full_like(q1, float("nan")), torch.full_like(q1, float("nan"))
        ops.attention_decode_flat(q1, kc, vc, again, rseg1, rpos1, tables, len(lens), H, Hkv, hd, page, window, scale,
                                  blocks, scratch)
        ops.attention_decode_separate_combine(True)
        try:
            ops.attention_decode_flat(q1, kc, vc, apart, rseg1, rpos1, tables, len(lens), H, Hkv, hd, page, window, scale,
                                      blocks, scratch)
        finally:
            ops.attention_decode_separate_combine(False)
        assert torch.equal(out1, again) and torch.equal(out1, apart)


def test_attention_decode_dealt_out_evenly_random_shapes(ops):
    """Random numbers of rows, lengths and blocks: the evenly dealt kernel against one block per (row, kv head)."""
    import random
    rng = random.Random(7)
    H, Hkv, hd, page, scale = 8, 2, 128, 16, 1.0 / math.sqrt(128)
    for trial in range(12):
        lens = [rng.choice([1, 2, 63, 64, 65, rng.randint(1, 900)]) for _ in range(rng.randint(1, 12))]
        blocks = rng.randint(1, 62 * Hkv)
        q, kc, vc, out, rseg, rpos, tables, want, q_lens = attention_case(ops, torch.bfloat16, H, Hkv, hd, page, lens, 0,
                                                                          scale, False, [1] * len(lens))
        a, b = torch.full_like(q, float("nan")), torch.full_like(q, float("nan"))
        scratch = torch.full((ops.attention_decode_flat_scratch_floats(len(lens), H, Hkv, hd, blocks),), float("nan"),
                             device=DEV)
        ops.attention_decode_flat(q, kc, vc, a, rseg, rpos, tables, len(lens), H, Hkv, hd, page, 0, scale, blocks, scratch)
        ops.attention_decode(q, kc, vc, b, rseg, rpos, tables, len(lens), H, Hkv, hd, page, 0, scale)
        rows_close(a, want, f"trial {trial}: dealt out, lens {lens}, {blocks} blocks")
        rows_close(b, want, f"trial {trial}: one block per pair, lens {lens}")


# ---- choosing tokens -----------------------------------------------------------------------------------------

def test_argmax_lowest_index_among_equals(ops):
    logits = rnd(4, 151936)
    logits[1, 70000] = logits[1, 150000] = 50.0
    logits[2, 0] = 60.0
    logits[3, 151935] = 60.0
    out = torch.empty(4, dtype=torch.int32, device=DEV)
    ops.argmax(logits, out)
    assert out.tolist() == [P.argmax_lowest(logits[0].cpu()), 70000, 0, 151935]
    ops.argmax(logits, out, vocab=151000)                    # padding rows of the head are never chosen
    assert out.tolist()[3] == P.argmax_lowest(logits[3, :151000].cpu())
    # rows dealt out over several blocks and rows with one block each, widths that end inside a group of four columns,
    # equal maxima in different blocks' stretches, a view with wider rows, a row of NaNs; twice (the counters are left at zero)
    for rows, vocab, ld in ((1, 151936, 151936), (3, 50001, 50004), (40, 32003, 32004), (200, 9001, 9004), (2, 777, 780),
                            (5, 40000, 40001)):
        wide = rnd(rows, ld, seed=rows)
        wide[0, 5] = wide[0, vocab - 1] = 70.0
        if rows > 2:
            wide[1, vocab - 2] = wide[1, vocab // 2] = 70.0
            wide[2, :] = float("nan")
        view = wide[:, :vocab]
        want = [P.argmax_lowest(view[r].cpu()) if not torch.isnan(view[r]).all() else 0 for r in range(rows)]
        got = torch.full((rows,), -1, dtype=torch.int32, device=DEV)
        for _ in range(2):
            got.fill_(-1)
            ops.argmax(view, got)
            assert got.tolist() == want, (rows, vocab, ld)


@pytest.mark.parametrize("T,k,p,mp", [(0.8, 0, 1.0, 0.0), (1.0, 20, 0.95, 0.0), (0.6, 0, 0.9, 0.0), (1.3, 0, 1.0, 0.05),
                                      (0.7, 5, 1.0, 0.3), (1.0, 2000, 0.5, 0.0), (0.9, 3, 0.5, 0.9)])
def test_sample_follows_the_plain_walk(ops, T, k, p, mp):
    V, rows = 1000, 24
    logits = rnd(rows, V, scale=2.5, seed=int(T * 10) + k)
    logits[:, 17] = logits[:, 400]                              # equal logits: the lower index comes first
    g = torch.Generator().manual_seed(5)
    u = torch.rand(rows, generator=g, dtype=torch.float64)
    u[0], u[1] = 0.0, 0.999999
    f = lambda v, dt: torch.full((rows,), v, dtype=dt, device=DEV)
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    ops.sample(logits, f(T, torch.float32), f(k, torch.int32), f(p, torch.float32), f(mp, torch.float32), u.to(DEV), out)
    for r in range(rows):
        idx, w = P.sampling_weights(logits[r].cpu(), T, k, p, mp)
        assert out[r].item() == P.draw(idx, w, float(u[r])), (r, float(u[r]))


def test_sample_rows_have_their_own_parameters(ops):
    logits = rnd(3, 517, scale=3.0)
    out = torch.empty(3, dtype=torch.int32, device=DEV)
    t = torch.tensor([0.0, 1.0, 1.0], device=DEV)
    k = torch.tensor([0, 1, 4], dtype=torch.int32, device=DEV)
    ops.sample(logits, t, k, torch.ones(3, device=DEV), torch.zeros(3, device=DEV),
               torch.tensor([0.3, 0.3, 0.99999], dtype=torch.float64, device=DEV), out)
    top4 = torch.topk(logits[2], 4).indices.tolist()
    assert out[0].item() == int(logits[0].argmax()) and out[1].item() == int(logits[1].argmax())
    assert out[2].item() == top4[3]
