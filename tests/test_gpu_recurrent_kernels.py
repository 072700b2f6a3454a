"""The kernels of the recurrent mixers (causal convolution, selective scan, minimal gated recurrence, gated
delta rule) and the small kernels that go with them, each alone against its plain PyTorch version
(tests/ref_ops.py), in 32-bit and in bfloat16: spans of several lengths beside single tokens, a second
step that continues from the state the first one left, a step of single tokens only, empty spans, sizes
that are no power of two and no multiple of a warp."""
import pytest
import torch

import ref_ops
from test_gpu_kernels import make_step

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
# the last two are long enough for the passes over chunks of rows (chunks that end inside and at a request's end,
# a request shorter than a chunk, one of exactly two chunks)
STEPS = ([1, 3, 4, 11, 1], [5, 1, 1, 2, 9], [1, 1, 1, 1, 1], [2, 37, 1, 1, 6], [200, 1, 63, 128, 70], [64, 65, 300, 2, 1])
MANY_SINGLES = [1] * 20           # more single tokens than the one-kernel paths for few requests take


def ops():
    from zig_ai_b200.kernels import ops as o
    o.require(extra=("causal_conv", "selective_scan", "min_gru", "gated_delta"))
    return o


def tol(dtype):
    return dict(atol=3e-5, rtol=3e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("C,L,bias,act", [(96, 4, True, True), (64, 3, False, True), (200, 2, True, False), (48, 1, False, True),
                                          (130, 7, True, True)])
def test_causal_conv_spans_and_state(dtype, C, L, bias, act):
    o = ops()
    g = torch.Generator().manual_seed(4)
    w = (torch.randn(C, L, generator=g) * 0.3).cuda()
    b = (torch.randn(C, generator=g) * 0.3).cuda() if bias else None
    state_a = torch.randn(6, max(L - 1, 1), C, generator=g).cuda()
    state_b = state_a.clone()
    for q_lens in STEPS:
        step = make_step(o, dtype, [3] * 5, q_lens, 8, 256, 5)
        wide = torch.randn(sum(q_lens), C + 24, generator=g).to(dtype).cuda()
        x = wide[:, 8:8 + C]                                   # a column slice of a wider matrix
        ya = o.causal_conv(x, w, b, state_a, step, act, True)
        yb = ref_ops.causal_conv(x, w, b, state_b, step, act, True)
        assert torch.allclose(ya.float(), yb.float(), **tol(dtype)), q_lens
        assert torch.allclose(state_a, state_b, atol=1e-6, rtol=1e-6), q_lens
    keep = state_a.clone()
    step = make_step(o, dtype, [3] * 5, [2, 4, 1, 1, 3], 8, 64, 5)
    x = torch.randn(11, C, generator=g).to(dtype).cuda()
    o.causal_conv(x, w, b, state_a, step, act, False)          # write_state off: the history stays
    assert torch.equal(state_a, keep)
    assert torch.equal(state_a[0], state_b[0])                 # the null slot was never touched


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("I,S,R", [(96, 20, 12), (70, 3, 5), (33, 16, 1), (40, 40, 7), (20, 100, 9), (12, 200, 3)])
def test_selective_scan(dtype, I, S, R):
    o = ops()
    g = torch.Generator().manual_seed(6)
    w_dt = (torch.randn(I, R, generator=g) * 0.5).to(dtype).cuda()
    b_dt = (torch.randn(I, generator=g) * 0.5).cuda()
    a_log = (torch.randn(I, S, generator=g) * 0.5).cuda()
    d = torch.randn(I, generator=g).cuda()
    state_a = torch.randn(6, I, S, generator=g).cuda()
    state_b = state_a.clone()
    for q_lens in STEPS:
        step = make_step(o, dtype, [3] * 5, q_lens, 8, 256, 5)
        N = sum(q_lens)
        x = torch.randn(N, I, generator=g).to(dtype).cuda()
        proj = torch.randn(N, R + 2 * S + 3, generator=g).to(dtype).cuda()
        z = torch.randn(N, 2 * I, generator=g).to(dtype).cuda()[:, I:]
        ya = o.selective_scan(x, proj, z, w_dt, b_dt, a_log, d, state_a, step, R, True)
        yb = ref_ops.selective_scan(x, proj, z, w_dt, b_dt, a_log, d, state_b, step, R, True)
        assert torch.allclose(ya.float(), yb.float(), **tol(dtype)), q_lens
        assert torch.allclose(state_a, state_b, atol=1e-4, rtol=1e-4), q_lens
    assert torch.equal(state_a[0], state_b[0])


@pytest.mark.parametrize("dtype", DTYPES)
def test_selective_scan_single_tokens_aligned_rows(dtype):
    """A step of single tokens sums the step size's product itself, 16 bytes a load where the rows allow it."""
    o = ops()
    g = torch.Generator().manual_seed(13)
    I, S, R = 72, 16, 32
    w_dt = (torch.randn(I, R, generator=g) * 0.5).to(dtype).cuda()
    b_dt, a_log, d = (torch.randn(I, generator=g) * 0.5).cuda(), (torch.randn(I, S, generator=g) * 0.5).cuda(), torch.randn(I, generator=g).cuda()
    state_a = torch.randn(6, I, S, generator=g).cuda()
    state_b = state_a.clone()
    for _ in range(3):
        step = make_step(o, dtype, [3] * 5, [1] * 5, 8, 64, 5)
        x = torch.randn(5, I, generator=g).to(dtype).cuda()
        proj = torch.randn(5, R + 2 * S, generator=g).to(dtype).cuda()
        z = torch.randn(5, I, generator=g).to(dtype).cuda()
        ya = o.selective_scan(x, proj, z, w_dt, b_dt, a_log, d, state_a, step, R, True)
        yb = ref_ops.selective_scan(x, proj, z, w_dt, b_dt, a_log, d, state_b, step, R, True)
        assert torch.allclose(ya.float(), yb.float(), **tol(dtype))
        assert torch.allclose(state_a, state_b, atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("W", [200, 70, 1, 130])
def test_min_gru(dtype, W):
    o = ops()
    g = torch.Generator().manual_seed(7)
    bz, bx = torch.randn(W, generator=g).cuda(), torch.randn(W, generator=g).cuda()
    state_a = torch.randn(6, W, generator=g).cuda()
    state_b = state_a.clone()
    for q_lens in STEPS:
        step = make_step(o, dtype, [3] * 5, q_lens, 8, 256, 5)
        zxg = (torch.randn(sum(q_lens), 3 * W, generator=g) * 2).to(dtype).cuda()
        ya = o.min_gru(zxg, bz, bx, state_a, step, True)
        yb = ref_ops.min_gru(zxg, bz, bx, state_b, step, True)
        assert torch.allclose(ya.float(), yb.float(), **tol(dtype)), q_lens
        assert torch.allclose(state_a, state_b, atol=1e-5, rtol=1e-5), q_lens
    assert torch.equal(state_a[0], state_b[0])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,D,V", [(6, 2, 32, 40), (2, 2, 16, 24), (3, 1, 40, 33), (4, 2, 64, 128), (2, 1, 128, 48),
                                     (1, 1, 200, 20), (2, 1, 8, 70)])
def test_gated_delta(dtype, H, G, D, V):
    o = ops()
    g = torch.Generator().manual_seed(8)
    a_log, dt_bias = torch.randn(H, generator=g).cuda() * 0.5, torch.randn(H, generator=g).cuda() * 0.5
    norm_w = (1 + 0.1 * torch.randn(V, generator=g)).cuda()
    state_a = (torch.randn(22, H, D, V, generator=g) * 0.3).cuda()
    state_b = state_a.clone()
    cols = 2 * G * D + H * V
    for q_lens in STEPS + (MANY_SINGLES,):
        step = make_step(o, dtype, [3] * len(q_lens), q_lens, 8, 256, 5)
        N = sum(q_lens)
        qkv = torch.randn(N, cols, generator=g).to(dtype).cuda()
        rest = torch.randn(N, H * V + 2 * H, generator=g).to(dtype).cuda()
        gate, b, a = rest[:, :H * V], rest[:, H * V:H * V + H], rest[:, H * V + H:]
        ya = o.gated_delta(qkv, b, a, gate, a_log, dt_bias, norm_w, 1e-5, state_a, step, H, G, D, V, True)
        yb = ref_ops.gated_delta(qkv, b, a, gate, a_log, dt_bias, norm_w, 1e-5, state_b, step, H, G, D, V, True)
        assert torch.allclose(ya.float(), yb.float(), **tol(dtype)), q_lens
        assert torch.allclose(state_a, state_b, atol=1e-4, rtol=1e-4), q_lens
    assert torch.equal(state_a[0], state_b[0])


@pytest.mark.parametrize("dtype", DTYPES)
def test_empty_spans_change_nothing(dtype):
    """A step may hold spans without tokens (a captured step shape is filled up with them)."""
    o = ops()
    g = torch.Generator().manual_seed(9)
    step = make_step(o, dtype, [3, 0, 5], [4, 0, 2], 8, 64, 5)
    W = 40
    state = torch.randn(6, W, generator=g).cuda()
    before = state.clone()
    zxg = torch.randn(6, 3 * W, generator=g).to(dtype).cuda()
    o.min_gru(zxg, None, None, state, step, True)
    assert torch.equal(state[2], before[2]) and not torch.equal(state[1], before[1])
    conv_state = torch.randn(6, 3, W, generator=g).cuda()
    before = conv_state.clone()
    o.causal_conv(zxg[:, :W], torch.randn(W, 4, generator=g).cuda(), None, conv_state, step, True, True)
    assert torch.equal(conv_state[2], before[2]) and not torch.equal(conv_state[3], before[3])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind", ["gelu", "gelu_tanh", "silu", "relu"])
@pytest.mark.parametrize("shape", [(3, 192), (7, 1001)])
def test_activation_and_weighted_sum(dtype, kind, shape):
    o = ops()
    g = torch.Generator().manual_seed(10)
    x = (torch.randn(*shape, generator=g) * 3).to(dtype).cuda()
    y = (torch.randn(*shape, generator=g) * 3).to(dtype).cuda()
    assert torch.allclose(o.activation(x, kind).float(), ref_ops.activation(x, kind).float(), **tol(dtype))
    assert torch.allclose(o.weighted_sum(x, y, 0.8, -1.3).float(), ref_ops.weighted_sum(x, y, 0.8, -1.3).float(), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("N,H", [(5, 96), (3, 1000), (40, 2050)])
def test_norm_of_the_pending_term(dtype, N, H):
    o = ops()
    g = torch.Generator().manual_seed(11)
    h = (torch.randn(N, H, generator=g) * 3).cuda()
    delta = (torch.randn(N, H, generator=g) * 5).to(dtype).cuda()
    w, wd = (1 + 0.1 * torch.randn(H, generator=g)).cuda(), (1 + 0.1 * torch.randn(H, generator=g)).cuda()
    h1, h2 = h.clone(), h.clone()
    a = o.add_rmsnorm(h1, delta, w, 1e-6, dtype, wd, 1e-5)
    b = ref_ops.add_rmsnorm(h2, delta, w, 1e-6, dtype, wd, 1e-5)
    assert torch.allclose(h1, h2, atol=1e-5, rtol=1e-5)
    assert torch.allclose(a.float(), b.float(), **tol(dtype))
    rows = torch.tensor([N - 1, 0, N // 2], dtype=torch.int32).cuda()
    assert torch.allclose(o.gather_add(h, delta, rows, wd, 1e-5), ref_ops.gather_add(h, delta, rows, wd, 1e-5), atol=1e-5, rtol=1e-5)
    table = torch.randn(50, H, generator=g).to(dtype).cuda()
    ids = torch.randint(0, 50, (N,), generator=g, dtype=torch.int32).cuda()
    assert torch.allclose(o.embed(ids, table, 7.25), ref_ops.embed(ids, table, 7.25), atol=0, rtol=1e-6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,D,Dv", [(4, 2, 16, 16), (3, 1, 32, 48), (2, 2, 40, 24), (6, 2, 64, 64)])
@pytest.mark.parametrize("normed", [True, False])
def test_value_norm_and_padding(dtype, H, G, D, Dv, normed):
    o = ops()
    g = torch.Generator().manual_seed(12)
    qkv = torch.randn(9, H * D + G * D + G * Dv, generator=g).to(dtype).cuda()
    want = ref_ops.value_norm_pad(qkv.clone(), H, G, D, Dv, 1e-5, normed)
    got = o.value_norm_pad(qkv, H, G, D, Dv, 1e-5, normed)
    assert got.shape == want.shape
    assert torch.allclose(got.float(), want.float(), **tol(dtype))
