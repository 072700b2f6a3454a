"""The kernels that the layer-norm, chunked-attention and latent-attention parts add, each alone against its plain
PyTorch version (tests/ref_ops.py), in 32-bit and in bfloat16: the layer norm with the residual addition; the
prepared q/k/v (norm per head, over the whole projection or none, rotation, heads wider in the cache than in the
projection, the page write); every attention kernel with chunks (the first and last position of a chunk, chunks of
one position, longer than a context, no multiple of a tile); the latent rows' preparation and latent attention over
pages (spans beside single tokens, contexts across many pages); gates, the bounded gated activation, capped logits
and the stretched rotation table; sizes that are no power of two and no multiple of a warp."""
import pytest
import torch

import ref_ops
from test_gpu_kernels import fill_pages, make_step
from zig_ai_b200.cache.manager import CacheView

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
STRETCH = (4.0, 32.0, 8.0, 1.0)


def ops():
    from zig_ai_b200.kernels import ops as o
    o.require(extra=("layernorm", "qkv_prepare", "latent_attention"))
    return o


def tol(dtype):
    return dict(atol=3e-5, rtol=3e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("N,H,eps", [(5, 96, 1e-6), (3, 1000, 1e-5), (17, 4104, 1e-3), (1, 66, 1e-5), (70, 1024, 1e-5),
                                     (65, 2048, 1e-5), (64, 1540, 1e-3), (300, 4096, 1e-5), (513, 1001, 1e-6), (9, 4, 1e-5)])
def test_add_layernorm(dtype, N, H, eps):
    o = ops()
    g = torch.Generator().manual_seed(2)
    h = (torch.randn(N, H, generator=g) * 3 + 1.5).cuda()          # a mean far from zero: the variance is about the mean
    delta = torch.randn(N, H, generator=g).to(dtype).cuda()
    w = (1 + 0.1 * torch.randn(H, generator=g)).cuda()
    b = (0.3 * torch.randn(H, generator=g)).cuda()
    h1, h2 = h.clone(), h.clone()
    a = o.add_layernorm(h1, delta, w, b, eps, dtype)
    want = ref_ops.add_layernorm(h2, delta, w, b, eps, dtype)
    assert torch.equal(h1, h2)                                     # the 32-bit residual sum is exact
    assert torch.allclose(a.float(), want.float(), **tol(dtype))
    a = o.add_layernorm(h1, None, w, b, eps, dtype)
    assert torch.allclose(a.float(), ref_ops.add_layernorm(h2, None, w, b, eps, dtype).float(), **tol(dtype))
    assert torch.equal(h1, h2)


@pytest.mark.parametrize("scaling", [None, STRETCH, (16.0, 24.0, 4.0, 0.5)])
def test_rotation_table_plain_and_stretched(scaling):
    o = ops()
    step = make_step(o, torch.float32, [0, 700, 31], [9, 1, 40], 16, 128, 3)
    for dims, theta in ((8, 10000.0), (32, 250000.0), (6, 300.0)):
        a = o.rope_table(step, dims, theta, torch.device("cuda"), scaling)
        b = ref_ops.rope_table(step, dims, theta, torch.device("cuda"), scaling)
        assert a.shape == (50, dims // 2, 2) and torch.allclose(a.cpu(), b.cpu(), atol=2e-7, rtol=0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,D,Dv,rot,scope", [(4, 2, 16, 16, 8, 2), (3, 1, 32, 8, 32, 2), (6, 3, 24, 40, 0, 2), (2, 2, 128, 128, 64, 2),
                                                (5, 5, 10, 6, 4, 1), (8, 2, 64, 64, 64, 0), (8, 1, 128, 64, 32, 2)])
def test_qkv_prepare(dtype, H, G, D, Dv, rot, scope):
    """q, k and v from a wider stacked projection (a gate's columns behind them): the norm in its three scopes, the
    rotation, heads padded to the cache's size, and the rows written at the right page and offset."""
    o = ops()
    g = torch.Generator().manual_seed(5)
    Dp, ps, num_pages = max(D, Dv), 8, 64
    ctx, q_lens = [0, 7, 30, 3], [9, 1, 20, 1]
    step = make_step(o, dtype, ctx, q_lens, ps, num_pages, 6)
    N = sum(q_lens)
    y = torch.randn(N, (H + G) * D + G * Dv + H, generator=g).to(dtype).cuda()
    q_w = (1 + 0.2 * torch.randn(H * D if scope == 2 else D, generator=g)).cuda() if scope else None
    k_w = (1 + 0.2 * torch.randn(G * D if scope == 2 else D, generator=g)).cuda() if scope else None
    table = o.rope_table(step, rot, 10000.0, y.device, STRETCH) if rot else None
    pages_a = torch.full((num_pages, 2, G, ps, Dp), 7.0, dtype=dtype, device="cuda")
    pages_b = pages_a.clone()
    va, vb = CacheView(0, pages_a, step.block_tables[0], ps), CacheView(0, pages_b, step.block_tables[0], ps)
    a = o.qkv_prepare(y, q_w, k_w, 1e-5, scope, table, rot, step, va, H, G, D, Dv, Dp, True)
    b = ref_ops.qkv_prepare(y, q_w, k_w, 1e-5, scope, table, rot, step, vb, H, G, D, Dv, Dp, True)
    assert torch.allclose(a.float(), b.float(), **tol(dtype))
    assert torch.allclose(pages_a.float(), pages_b.float(), **tol(dtype))
    keep = pages_a.clone()
    o.qkv_prepare(y * 2, q_w, k_w, 1e-5, scope, table, rot, step, va, H, G, D, Dv, Dp, False)      # write off: the pages stay
    assert torch.equal(pages_a, keep)
    assert o.read_status() == 0


CHUNK_SHAPES = [(4, 2, 16, 8, 11), (3, 1, 32, 8, 1), (6, 3, 48, 4, 7), (8, 2, 80, 32, 64), (16, 8, 64, 16, 96),
                (2, 2, 128, 16, 112), (8, 1, 128, 64, 100), (5, 5, 112, 16, 5000), (2, 1, 200, 16, 33)]


@pytest.mark.parametrize("dtype,impl", [(torch.float32, None), (torch.bfloat16, None), (torch.bfloat16, "general")])
@pytest.mark.parametrize("Hq,Hkv,D,ps,chunk", CHUNK_SHAPES)
def test_chunked_attention_mixed_spans(dtype, impl, Hq, Hkv, D, ps, chunk):
    """Spans that start at 0, inside a page and far into a request, of 1 to 150 rows, with chunks that end inside
    spans, at their first row and at their last; what a chunk must not see holds values that would drown the rest."""
    o = ops()
    g = torch.Generator().manual_seed(8)
    ctx, q_lens = [0, ps - 1, 2 * ps, 301, 5, 63], [150, 2, 1, 1, 37, 66]
    num_pages = 256
    step = make_step(o, dtype, ctx, q_lens, ps, num_pages, 9)
    pages = fill_pages(step, ctx, q_lens, ps, Hkv, D, dtype, num_pages, g)
    q = torch.randn(sum(q_lens), Hq * D, generator=g).to(dtype).cuda()
    view = CacheView(0, pages, step.block_tables[0], ps)
    a = o.paged_attention(q, step, view, Hq, Hkv, D, D ** -0.5, None, impl=impl, chunk=chunk)
    b = ref_ops.paged_attention(q, step, view, Hq, Hkv, D, D ** -0.5, None, chunk=chunk)
    assert torch.allclose(a.float(), b.float(), **tol(dtype))
    if chunk < 150:
        plain = ref_ops.paged_attention(q, step, view, Hq, Hkv, D, D ** -0.5, None)
        assert not torch.allclose(b.float(), plain.float(), **tol(dtype))          # the chunks do change the result


@pytest.mark.parametrize("impl", ["tcgen05", "mma"])
@pytest.mark.parametrize("Hq,Hkv,ps,chunk", [(16, 8, 16, 64), (4, 1, 64, 96), (2, 2, 8, 100), (6, 3, 128, 1), (3, 1, 32, 300)])
def test_chunked_span_attention_head_size_64(impl, Hq, Hkv, ps, chunk):
    o = ops()
    dtype, D = torch.bfloat16, 64
    g = torch.Generator().manual_seed(28)
    ctx, q_lens = [0, ps - 1, 1100, 301, 5, 127, 640], [400, 2, 130, 1, 37, 129, 128]
    num_pages = (sum(c + n for c, n in zip(ctx, q_lens)) // ps) + 16
    step = make_step(o, dtype, ctx, q_lens, ps, num_pages, 29)
    pages = fill_pages(step, ctx, q_lens, ps, Hkv, D, dtype, num_pages, g)
    q = torch.randn(sum(q_lens), Hq * D, generator=g).to(dtype).cuda()
    view = CacheView(0, pages, step.block_tables[0], ps)
    a = o.paged_attention(q, step, view, Hq, Hkv, D, D ** -0.5, None, impl=impl, chunk=chunk)
    b = ref_ops.paged_attention(q, step, view, Hq, Hkv, D, D ** -0.5, None, chunk=chunk)
    assert torch.allclose(a.float(), b.float(), **tol(dtype))
    assert o.tc_status() == 0


@pytest.mark.parametrize("Hq,Hkv,D,ps,chunk", CHUNK_SHAPES)
def test_chunked_attention_single_tokens(Hq, Hkv, D, ps, chunk):
    """Every span one token: queries at the first and the last position of a chunk and of a block of keys."""
    o = ops()
    for dtype in DTYPES:
        g = torch.Generator().manual_seed(18)
        ctx = [0, 1, 254, 255, 256, 700, 63, 1029] + [chunk - 1, chunk, 3 * chunk - 1, 3 * chunk][:4 if chunk < 300 else 0]
        q_lens = [1] * len(ctx)
        num_pages = 2048
        step = make_step(o, dtype, ctx, q_lens, ps, num_pages, 19)
        pages = fill_pages(step, ctx, q_lens, ps, Hkv, D, dtype, num_pages, g)
        q = torch.randn(len(ctx), Hq * D, generator=g).to(dtype).cuda()
        view = CacheView(0, pages, step.block_tables[0], ps)
        a = o.paged_attention(q, step, view, Hq, Hkv, D, D ** -0.5, None, chunk=chunk)
        b = ref_ops.paged_attention(q, step, view, Hq, Hkv, D, D ** -0.5, None, chunk=chunk)
        assert torch.allclose(a.float(), b.float(), **tol(dtype)), dtype


def latent_pages(step, ctx, q_lens, ps, W, dtype, num_pages, g):
    """Random rows at every position the step's requests hold; a large finite value everywhere else."""
    pages = torch.full((num_pages, ps, W), 60.0, dtype=dtype, device="cuda")
    bt = step.block_tables[0].cpu().long()
    for s, (c, n) in enumerate(zip(ctx, q_lens)):
        p = torch.arange(c + n)
        pages[bt[s, p // ps].cuda(), (p % ps).cuda(), :] = torch.randn(c + n, W, generator=g).to(dtype).cuda()
    return pages


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,D,Dr,R", [(4, 48, 32, 160), (3, 12, 8, 24), (5, 4, 16, 40), (2, 20, 6, 17), (16, 64, 64, 256), (9, 8, 2, 300)])
def test_latent_prepare(dtype, H, D, Dr, R):
    o = ops()
    g = torch.Generator().manual_seed(7)
    ps, num_pages = 8, 64
    ctx, q_lens = [0, 7, 30, 3], [9, 1, 20, 1]
    step = make_step(o, dtype, ctx, q_lens, ps, num_pages, 6)
    N = sum(q_lens)
    y = torch.randn(N, H * (D + Dr) + 5 + R + Dr, generator=g).to(dtype).cuda()
    q, dkv = y[:, :H * (D + Dr)].view(N, H, D + Dr), y[:, H * (D + Dr) + 5:]
    w = (1 + 0.2 * torch.randn(R, generator=g)).cuda()
    table = o.rope_table(step, Dr, 10000.0, y.device, STRETCH)
    pages_a = torch.full((num_pages, ps, R + Dr), 7.0, dtype=dtype, device="cuda")
    pages_b = pages_a.clone()
    va, vb = CacheView(0, pages_a, step.block_tables[0], ps), CacheView(0, pages_b, step.block_tables[0], ps)
    a = o.latent_prepare(q, dkv, w, 1e-5, table, step, va, H, D, Dr, R)
    b = ref_ops.latent_prepare(q, dkv, w, 1e-5, table, step, vb, H, D, Dr, R)
    assert torch.allclose(a.float(), b.float(), **tol(dtype)) and torch.allclose(pages_a.float(), pages_b.float(), **tol(dtype))
    keep = pages_a.clone()
    a2 = o.latent_prepare(q, None, None, 1e-5, table, step, va, H, D, Dr, R)         # a layer that borrows its rows writes none
    assert torch.equal(a, a2) and torch.equal(pages_a, keep)
    assert o.read_status() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,R,Dr,ps", [(4, 160, 32, 64), (7, 128, 16, 32), (3, 24, 8, 8), (5, 40, 16, 16), (2, 17, 6, 8), (16, 256, 64, 32), (9, 300, 2, 16),
                                       (1, 512, 64, 16)])
def test_latent_attention_spans_and_single_tokens(dtype, H, R, Dr, ps):
    o = ops()
    g = torch.Generator().manual_seed(11)
    for ctx, q_lens in (([0, ps - 1, 2 * ps, 301, 5, 63], [150, 2, 1, 1, 37, 66]), ([0, 1, 254, 255, 256, 700, 63, 1029], [1] * 8)):
        num_pages = sum(-(-(c + n) // ps) for c, n in zip(ctx, q_lens)) + 8
        step = make_step(o, dtype, ctx, q_lens, ps, num_pages, 12)
        pages = latent_pages(step, ctx, q_lens, ps, R + Dr, dtype, num_pages, g)
        N = sum(q_lens)
        q_lat = torch.randn(N, H, R, generator=g).to(dtype).cuda()
        q_rot = torch.randn(N, H, Dr, generator=g).to(dtype).cuda()
        view = CacheView(0, pages, step.block_tables[0], ps)
        scale = (R + Dr) ** -0.5
        b = ref_ops.latent_attention(q_lat, q_rot, step, view, H, R, Dr, scale)
        # (bfloat16 with sizes the tensor-core kernels take: the one the step's size picks, both by name, the general one)
        for impl in (None, "general") + (("mma_rows", "mma_ranges") if dtype == torch.bfloat16 and R % 32 == 0 and Dr % 16 == 0 else ()):
            a = o.latent_attention(q_lat, q_rot, step, view, H, R, Dr, scale, impl=impl)
            assert torch.allclose(a.float(), b.float(), **tol(dtype)), (q_lens, impl)
        step.max_kv_len = 5000                      # more ranges of keys than any request needs (a captured graph's bound)
        a2 = o.latent_attention(q_lat, q_rot, step, view, H, R, Dr, scale)
        assert torch.allclose(a2.float(), b.float(), **tol(dtype)), q_lens
    assert o.read_status() == 0


@pytest.mark.parametrize("H,R,Dr,ps", [(16, 256, 32, 64), (20, 128, 64, 16), (128, 512, 64, 64), (4, 160, 16, 32)])
def test_latent_attention_on_tensor_cores_many_rows(H, R, Dr, ps):
    """Enough rows that no key ranges are made, spans of several hundred rows over long contexts, more than 16 heads,
    ranks of one, two and four blocks of 128 columns and of a block and a quarter."""
    o = ops()
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(21)
    ctx, q_lens = [0, 700, 33], [400 if H < 100 else 40, 130 if H < 100 else 9, 1]
    num_pages = sum(-(-(c + n) // ps) for c, n in zip(ctx, q_lens)) + 8
    step = make_step(o, dtype, ctx, q_lens, ps, num_pages, 22)
    pages = latent_pages(step, ctx, q_lens, ps, R + Dr, dtype, num_pages, g)
    N = sum(q_lens)
    q_lat = torch.randn(N, H, R, generator=g).to(dtype).cuda()
    q_rot = torch.randn(N, H, Dr, generator=g).to(dtype).cuda()
    view = CacheView(0, pages, step.block_tables[0], ps)
    scale = (R + Dr) ** -0.5
    b = ref_ops.latent_attention(q_lat, q_rot, step, view, H, R, Dr, scale)
    for impl in ("mma_rows", "mma_ranges"):
        a = o.latent_attention(q_lat, q_rot, step, view, H, R, Dr, scale, impl=impl)
        assert torch.allclose(a.float(), b.float(), **tol(dtype)), impl
    assert o.read_status() == 0


@pytest.mark.parametrize("M", [1, 5, 8, 16, 40])
@pytest.mark.parametrize("K,F,limit", [(256, 384, 1.0), (1024, 3072, 7.0), (192, 100, 0.5)])
def test_product_with_the_bounded_gated_activation(M, K, F, limit):
    """Few rows: the activation is the product kernel's epilogue; more rows: a kernel of its own behind the product."""
    o = ops()
    g = torch.Generator().manual_seed(23)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(2 * F, K, generator=g) * K ** -0.5 * 2).to(torch.bfloat16).cuda()
    a = o.linear_clamped_glu(x, w, F, limit, 1.702)
    b = ref_ops.linear_clamped_glu(x, w, F, limit, 1.702)
    assert a.shape == (M, F) and torch.allclose(a.float(), b.float(), atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_latent_attention_finds_one_far_row(dtype):
    """One cached row far back, in the first page, carries a score that stands out: its latent is the result."""
    o = ops()
    g = torch.Generator().manual_seed(13)
    H, R, Dr, ps = 4, 64, 16, 16
    for far, ctx, n in ((0, 900, 1), (15, 900, 1), (16, 640, 130), (3, 0, 300)):
        step = make_step(o, dtype, [ctx], [n], ps, 128, 14)
        pages = latent_pages(step, [ctx], [n], ps, R + Dr, dtype, 128, g) * 0.1
        q_lat = (torch.randn(n, H, R, generator=g) * 0.1).to(dtype).cuda()
        q_rot = torch.randn(n, H, Dr, generator=g).to(dtype).cuda()
        page = int(step.block_tables[0][0, far // ps])
        pages[page, far % ps, R:] = 8.0
        q_rot[-1] = 8.0                                     # the last row's rotated part lines up with that row's
        view = CacheView(0, pages, step.block_tables[0], ps)
        a = o.latent_attention(q_lat, q_rot, step, view, H, R, Dr, 1.0)
        want = pages[page, far % ps, :R].float()
        assert torch.allclose(a[-1].float(), want.expand(H, R), atol=2e-2), (far, ctx, n)


@pytest.mark.parametrize("dtype", DTYPES)
def test_gates_activation_and_capped_logits(dtype):
    o = ops()
    g = torch.Generator().manual_seed(15)
    for N, H, Dh in ((7, 6, 128), (33, 3, 20), (1, 5, 7)):
        x = torch.randn(N, H * Dh, generator=g).to(dtype).cuda()
        wide = torch.randn(N, H * Dh + H + 3, generator=g).to(dtype).cuda()
        for per_head, gate in ((True, wide[:, 3:3 + H]), (False, wide[:, 3:3 + H * Dh])):
            a, b = o.sigmoid_gate(x, gate, H, Dh, per_head), ref_ops.sigmoid_gate(x, gate, H, Dh, per_head)
            assert torch.allclose(a.float(), b.float(), **tol(dtype))
    for N, F, limit in ((9, 384, 1.0), (40, 100, 0.5), (3, 7, 2.0)):
        gu = (torch.randn(N, 2 * F, generator=g) * 2).to(dtype).cuda()
        a, b = o.clamped_glu(gu, F, limit, 1.702), ref_ops.clamped_glu(gu, F, limit, 1.702)
        assert torch.allclose(a.float(), b.float(), **tol(dtype))
        assert float(a.float().max()) <= limit * (limit + 1) + 1e-2
    logits = (torch.randn(5, 577, generator=g) * 40).cuda()
    for scale, cap in ((0.5, 15.0), (1.0, None), (2.0, 30.0)):
        want = ref_ops.scale_softcap(logits, scale, cap)
        got = o.scale_softcap(logits.clone(), scale, cap)
        assert torch.allclose(got, want, atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("dtype", DTYPES)
def test_products_with_a_bias_and_per_head(dtype):
    o = ops()
    g = torch.Generator().manual_seed(17)
    for N in (1, 9, 200):
        x = torch.randn(N, 66, generator=g).to(dtype).cuda()
        w = (torch.randn(150, 66, generator=g) * 0.1).to(dtype).cuda()
        b = torch.randn(150, generator=g).to(dtype).cuda()
        assert torch.allclose(o.linear(x, w, bias=b).float(), ref_ops.linear(x, w, bias=b).float(), **tol(dtype))
        wide = torch.randn(N, 5 * (12 + 6) + 4, generator=g).to(dtype).cuda()
        q = wide[:, :5 * 18].view(N, 5, 18)[:, :, :12]                       # the unrotated parts of five heads
        wh = (torch.randn(5, 24, 12, generator=g) * 0.3).to(dtype).cuda()
        a, b2 = o.head_linear(q, wh), ref_ops.head_linear(q, wh)
        assert a.shape == (N, 5, 24) and a.is_contiguous() and torch.allclose(a.float(), b2.float(), **tol(dtype))


@pytest.mark.parametrize("M", [1, 3, 8, 13, 16])
@pytest.mark.parametrize("K,O", [(256, 512), (1024, 1536), (2048, 320), (192, 96)])
def test_layer_norm_inside_the_few_rows_product(M, K, O):
    """The layer norm (with the residual addition) as the product kernel's prologue against the norm's own kernel and
    the product behind it: bfloat16 and 32-bit results, gathered rows, and the bounded gated activation as the epilogue;
    the residual stream after the addition is the same either way."""
    from zig_ai_b200.parts.base import LazyNorm, Residual
    o = ops()
    g = torch.Generator().manual_seed(31)
    dt = torch.bfloat16
    h = (torch.randn(M, K, generator=g) * 2 + 0.7).cuda()
    delta = torch.randn(M, K, generator=g).to(dt).cuda()
    gamma = (1 + 0.2 * torch.randn(K, generator=g)).cuda()
    beta = (0.5 * torch.randn(K, generator=g)).cuda()
    w = (torch.randn(O, K, generator=g) * K ** -0.5).to(dt).cuda()
    h_ref = h.clone()
    x_ref = ref_ops.add_layernorm(h_ref, delta, gamma, beta, 1e-5, dt)
    for out_dtype in (dt, torch.float32):
        res = Residual(h.clone())
        got = o.linear(LazyNorm(res, delta, gamma, 1e-5, dt, beta=beta), w, out_dtype=out_dtype)
        want = ref_ops.linear(x_ref, w, out_dtype)
        assert torch.allclose(got.float(), want.float(), atol=3e-2, rtol=3e-2), out_dtype
        assert torch.allclose(res.data, h_ref, atol=1e-6, rtol=0)
    rows = torch.tensor([M - 1, 0], dtype=torch.int32).cuda()
    res = Residual(h.clone())
    got = o.linear(LazyNorm(res, delta, gamma, 1e-5, dt, rows=rows, beta=beta), w, out_dtype=torch.float32)
    assert torch.allclose(got, ref_ops.linear(x_ref[rows.long()], w, torch.float32), atol=3e-2, rtol=3e-2)
    if O % 2 == 0:
        res = Residual(h.clone())
        got = o.linear_clamped_glu(LazyNorm(res, delta, gamma, 1e-5, dt, beta=beta), w, O // 2, 0.8, 1.702)
        want = ref_ops.linear_clamped_glu(x_ref, w, O // 2, 0.8, 1.702)
        assert got.shape == (M, O // 2) and torch.allclose(got.float(), want.float(), atol=3e-2, rtol=3e-2)
