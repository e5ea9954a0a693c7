"""Parity of the sm_100a quantized linear against the CPU oracle (B200 only).

int32 accumulators: bit-exact.  int8 outputs: bit-exact against the oracle's
statement of the same epilogue and within 1 LSB of the reference's fake-quant
golden.  fp16 / fp32 outputs: rtol 1e-2, atol 1e-3.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-2, 1e-3


@pytest.fixture(scope="module")
def ops():
    assert torch.cuda.is_available()
    from bladedisc_b200 import ops as o
    yield o
    assert o.kernel_status() == 0, "a kernel's bounded wait ran out"


def _rand_i8(rng, shape):
    return rng.integers(-127, 128, shape, dtype=np.int8)


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _check_requant(run, want, exact_ok=True):
    """`run(exact_division)` returns the int8 result.  The exact form equals the divide-based oracle bit for
    bit (`exact_ok=False`: an activation computed by libdevice instead of libm allows one level); the default
    reciprocal form may differ by one level, and only at rounding ties, so on a tiny share of the values."""
    got = run(True)
    d = np.abs(got.astype(np.int32) - want.astype(np.int32))
    assert d.max() <= (0 if exact_ok else 1), f"exact division: {np.count_nonzero(d)} mismatches, max {d.max()}"
    fast = run(False)
    d = np.abs(fast.astype(np.int32) - want.astype(np.int32))
    assert d.max() <= 1 and (d > 0).mean() < 1e-3, f"reciprocal form: flip rate {(d > 0).mean():.2e}, max {d.max()}"


# (M, K, N): every path, ragged edges, K not a multiple of the 128-byte tile,
# N not a multiple of the vector width, one row, one tile exactly.
ACC_SHAPES = [
    (1, 768, 768), (7, 768, 3072), (64, 3072, 768), (33, 144, 80), (16, 128, 128), (64, 4096, 512),
    (128, 256, 256), (129, 256, 384), (333, 768, 768), (200, 144, 72), (256, 128, 136), (1024, 768, 3072),
    (1024, 3072, 768), (130, 2064, 264),
]


@pytest.mark.parametrize("M,K,N", ACC_SHAPES)
def test_accumulators_bit_exact(ops, M, K, N):
    from oracle import c
    rng = np.random.default_rng(M * 131 + K * 7 + N)
    a, w = _rand_i8(rng, (M, K)), _rand_i8(rng, (N, K))
    want = c.qgemm_acc(a, w)
    got = ops.qgemm(_dev(a), _dev(w), out_dtype=torch.int32).cpu().numpy()
    assert got.shape == want.shape
    assert (got == want).all(), f"path {ops.qgemm_path(M, N, K)}: {np.count_nonzero(got != want)} mismatches"


@pytest.mark.parametrize("path,M", [("tiled", 96), ("tiled", 1), ("small_m", 128), ("small_m", 100),
                                    ("simt", 70), ("small_m", 5), ("skinny", 1), ("skinny", 70),
                                    ("skinny", 128), ("skinny", 300)])
def test_forced_paths_agree(ops, path, M):
    from oracle import c
    rng = np.random.default_rng(11)
    a, w = _rand_i8(rng, (M, 640)), _rand_i8(rng, (392, 640))
    got = ops.qgemm(_dev(a), _dev(w), out_dtype=torch.int32, path=path).cpu().numpy()
    assert (got == c.qgemm_acc(a, w)).all()


@pytest.mark.parametrize("M,K,N", [(256, 128, 256), (1, 128, 16), (300, 640, 392), (512, 2064, 520), (1000, 768, 72),
                                   (2048, 1024, 1024), (777, 144, 264)])
@pytest.mark.parametrize("out_dtype", [torch.int32, torch.int8, torch.float16, torch.float32])
def test_cta_pair_path(ops, M, K, N, out_dtype):
    """The 2-CTA (256 x 256 tile, TMA-store epilogue) kernel, forced on shapes that
    exercise ragged rows / columns / K tails and both store routes (N = 72 with
    int8 output is not 16-byte aligned per row, so it leaves by direct stores)."""
    from oracle import c
    rng = np.random.default_rng(M + K + N)
    a, w = _rand_i8(rng, (M, K)), _rand_i8(rng, (N, K))
    acc = c.qgemm_acc(a, w)
    if out_dtype == torch.int32:
        got = ops.qgemm(_dev(a), _dev(w), out_dtype=torch.int32, path="pair").cpu().numpy()
        assert (got == acc).all()
        return
    sw = (rng.random(N) * 9e-3 + 1e-3).astype(np.float32)
    bias = (rng.standard_normal(N) * 0.5).astype(np.float32)
    s_x, s_out = np.float32(0.02), np.float32(0.05)
    kw = dict(x_scale=_dev(np.array([s_x])), w_scale=_dev(sw), bias=_dev(bias), path="pair")
    if out_dtype == torch.int8:
        _, want = c.qgemm_epilogue(acc, x_scale=s_x, w_scale=sw, out_scale=s_out, bias=bias, div_out=True)
        # canary rows around the result: a store that runs past the tensor edge would touch them
        buf = torch.full((M + 2, N), 99, dtype=torch.int8, device="cuda")

        def run(exact):
            ops.qgemm(_dev(a), _dev(w), out_scale=_dev(np.array([s_out])), out=buf[1:M + 1], exact_division=exact, **kw)
            return buf[1:M + 1].cpu().numpy()
        _check_requant(run, want)
        assert (buf[0] == 99).all() and (buf[M + 1] == 99).all()
    else:
        want, _ = c.qgemm_epilogue(acc, x_scale=s_x, w_scale=sw, bias=bias)
        got = ops.qgemm(_dev(a), _dev(w), out_dtype=out_dtype, **kw).float().cpu().numpy()
        if out_dtype == torch.float32:
            assert (got == want).all()
        else:
            ok = np.abs(want) < 60000
            assert np.allclose(got[ok], want[ok], rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("M,K,N", [(1, 256, 520), (3, 4096, 1000), (9, 768, 768), (16, 128, 16), (33, 144, 80), (64, 4096, 520), (100, 640, 392),
                                   (128, 2064, 264), (129, 256, 384), (300, 640, 1000), (333, 768, 3072),
                                   (48, 3072, 72), (600, 1024, 777),
                                   # one row tile, K >= 4096, few channels: K cut over a cluster of 4, 4 (K tail:
                                   # 33 blocks, the last rank short), 3 and 2 blocks
                                   (128, 8192, 1024), (16, 4112, 1000), (40, 6272, 5120), (33, 8192, 8200),
                                   # more channels than 148 blocks of 128 hold: blocks of 160, 224 and 256 channels
                                   (16, 256, 22016), (64, 128, 32000), (33, 144, 37880),
                                   # three row tiles of 240-channel blocks
                                   (333, 256, 11008),
                                   # K split with 2, 2 (K tail), 3 and 4 row tiles
                                   (256, 8192, 1024), (200, 4224, 2048), (384, 6272, 2000), (512, 4096, 1024)])
@pytest.mark.parametrize("out_dtype", [torch.int32, torch.int8, torch.float16, torch.float32])
def test_skinny_path(ops, M, K, N, out_dtype):
    """The few-row kernel (fine channel blocks over the full K, one box per
    operand and stage when K is a multiple of 128, per-block boxes otherwise),
    forced on ragged rows / columns / K tails, several row tiles, both
    store routes (N = 72 or 777 with int8 output leaves by scalar stores), and
    with K split over a thread-block cluster (partial tiles added through
    distributed shared memory)."""
    from oracle import c
    rng = np.random.default_rng(M * 3 + K + N)
    a, w = _rand_i8(rng, (M, K)), _rand_i8(rng, (N, K))
    acc = c.qgemm_acc(a, w)
    if out_dtype == torch.int32:
        got = ops.qgemm(_dev(a), _dev(w), out_dtype=torch.int32, path="skinny").cpu().numpy()
        assert (got == acc).all()
        return
    sw = (rng.random(N) * 9e-3 + 1e-3).astype(np.float32)
    bias = (rng.standard_normal(N) * 0.5).astype(np.float32)
    sx = (rng.random(M) * 0.03 + 0.01).astype(np.float32)  # per-row (dynamic) activation scales
    s_out = np.float32(0.05)
    kw = dict(x_scale=_dev(sx), w_scale=_dev(sw), bias=_dev(bias), path="skinny")
    if out_dtype == torch.int8:
        _, want = c.qgemm_epilogue(acc, x_scale=sx, w_scale=sw, out_scale=s_out, bias=bias, div_out=True)
        buf = torch.full((M + 2, N), 99, dtype=torch.int8, device="cuda")

        def run(exact):
            ops.qgemm(_dev(a), _dev(w), out_scale=_dev(np.array([s_out])), out=buf[1:M + 1], exact_division=exact, **kw)
            return buf[1:M + 1].cpu().numpy()
        _check_requant(run, want)
        assert (buf[0] == 99).all() and (buf[M + 1] == 99).all()
    else:
        want, _ = c.qgemm_epilogue(acc, x_scale=sx, w_scale=sw, bias=bias)
        got = ops.qgemm(_dev(a), _dev(w), out_dtype=out_dtype, **kw).float().cpu().numpy()
        if out_dtype == torch.float32:
            assert (got == want).all()
        else:
            ok = np.abs(want) < 60000
            assert np.allclose(got[ok], want[ok], rtol=RTOL, atol=ATOL)


def test_auto_path_by_rows(ops):
    assert ops.qgemm_path(1, 4096, 4096) == "gemv"
    assert ops.qgemm_path(8, 4096, 4096) == "gemv"
    assert ops.qgemm_path(4, 4096, 11008) == "gemv"
    assert ops.qgemm_path(5, 4096, 11008) == "skinny"
    assert ops.qgemm_path(7, 11008, 4096) == "skinny"
    assert ops.qgemm_path(64, 4096, 4096) == "skinny"
    assert ops.qgemm_path(128, 768, 3072) == "skinny"
    assert ops.qgemm_path(333, 4096, 4096) == "skinny"
    assert ops.qgemm_path(1024, 4096, 4096) in ("tiled", "pair")
    assert ops.qgemm_path(16384, 4096, 4096) == "pair"


@pytest.mark.parametrize("M", [1, 2, 3, 4, 5, 8])
@pytest.mark.parametrize("K,N", [(768, 768), (4096, 1000), (16, 5), (2064, 77), (16384, 130)])
def test_gemv_path(ops, M, K, N):
    """M <= 8 takes the dp4a matrix-vector kernel: exact sums, same epilogue, odd N and K tails."""
    from oracle import c
    assert ops.qgemm_path(M, N, K) == "gemv"
    rng = np.random.default_rng(M * 1000 + K + N)
    a, w = _rand_i8(rng, (M, K)), _rand_i8(rng, (N, K))
    acc = c.qgemm_acc(a, w)
    assert (ops.qgemm(_dev(a), _dev(w), out_dtype=torch.int32).cpu().numpy() == acc).all()
    sw = (rng.random(N) * 9e-3 + 1e-3).astype(np.float32)
    bias = (rng.standard_normal(N) * 0.5).astype(np.float32)
    sx = (rng.random(M) * 0.03 + 0.01).astype(np.float32)  # per-row (dynamic) activation scales
    s_out = np.float32(0.05)
    _, want = c.qgemm_epilogue(acc, x_scale=sx if M > 1 else sx[:1], w_scale=sw, out_scale=s_out, bias=bias, div_out=True)
    kw = dict(x_scale=_dev(sx), w_scale=_dev(sw), out_scale=_dev(np.array([s_out])), bias=_dev(bias))
    _check_requant(lambda exact: ops.qgemm(_dev(a), _dev(w), exact_division=exact, **kw).cpu().numpy(), want)
    # the tensor-core small-M path computes the same thing
    _check_requant(lambda exact: ops.qgemm(_dev(a), _dev(w), exact_division=exact, path="small_m", **kw).cpu().numpy(),
                   want)


@pytest.mark.parametrize("split", [1, 2, 3, 5, 8])
def test_small_m_split_k_is_exact_and_repeatable(ops, split):
    from oracle import c
    rng = np.random.default_rng(split)
    a, w = _rand_i8(rng, (48, 1024)), _rand_i8(rng, (520, 1024))
    want = c.qgemm_acc(a, w)
    for _ in range(3):  # the scratch and its arrival counters are reused
        got = ops.qgemm(_dev(a), _dev(w), out_dtype=torch.int32, path="small_m", split_k=split).cpu().numpy()
        assert (got == want).all()


def test_unaligned_shapes_take_the_simt_path(ops):
    """K = 25 cannot be addressed by TMA (rows must be 16-byte multiples): the
    reference's known-answer shape (x [4,25], w [71,25]) still has to work."""
    from oracle import c
    assert ops.qgemm_path(4, 71, 25) == "simt"
    x = np.full((4, 25), -0.6, dtype=np.float32)
    w = np.full((71, 25), -0.8, dtype=np.float32)
    s_x, s_w, s_out = np.float32(8.333333e-3), np.float32(1.568627e-2), np.float32(1.0)
    xq = ops.quantize(_dev(x), _dev(np.array([s_x])))
    wq = ops.quantize(_dev(w), _dev(np.array([s_w])))
    assert (xq.cpu().numpy() == c.quantize(x, s_x)).all()
    q = ops.qgemm(xq, wq, x_scale=_dev(np.array([s_x])), w_scale=_dev(np.array([s_w])),
                  out_scale=_dev(np.array([s_out])), fold_out_scale=True)
    y = ops.dequantize(q, _dev(np.array([s_out])))
    assert (y.cpu().numpy() == 12.0).all()  # tao_compiler/mlir/disc/tests/pdll/qgemm.cc:24-42


@pytest.mark.parametrize("M,K,N", [(1, 768, 768), (64, 768, 3072), (333, 3072, 768), (1024, 768, 768)])
@pytest.mark.parametrize("bias_kind", ["f32", "i8", None])
def test_reference_epilogue_int8(ops, M, K, N, bias_kind):
    """ral_pdll_qgemm: sat(rne(acc * (s_x * s_w / s_out) + bias)) (config 1 scales)."""
    from oracle import c
    rng = np.random.default_rng(M + K + N)
    a, w = _rand_i8(rng, (M, K)), _rand_i8(rng, (N, K))
    s_x, s_w, s_out = np.float32(0.02), np.float32(0.004), np.float32(0.05)
    bias = None
    if bias_kind == "f32":
        bias = (rng.standard_normal(N) * 20).astype(np.float32)
    elif bias_kind == "i8":
        bias = _rand_i8(rng, N)
    _, want = c.qgemm_epilogue(c.qgemm_acc(a, w), x_scale=s_x, w_scale=s_w, out_scale=s_out, bias=bias,
                               fold_out=True)
    got = ops.qgemm(_dev(a), _dev(w), x_scale=_dev(np.array([s_x])), w_scale=_dev(np.array([s_w])),
                    out_scale=_dev(np.array([s_out])), bias=None if bias is None else _dev(bias),
                    fold_out_scale=True).cpu().numpy()
    assert (got == want).all()
    assert np.abs(got.astype(int)).max() > 100  # the case exercises saturation too


@pytest.mark.parametrize("M", [7, 200])
def test_per_channel_folded_form(ops, M):
    """ral_pdll_qgemm_per_channel: every scale operand has N entries, int8 bias."""
    from oracle import c
    rng = np.random.default_rng(5)
    K, N = 256, 192
    a, w = _rand_i8(rng, (M, K)), _rand_i8(rng, (N, K))
    sx = (rng.random(N) * 0.02 + 0.01).astype(np.float32)
    sw = (rng.random(N) * 9e-3 + 1e-3).astype(np.float32)
    so = (rng.random(N) * 0.05 + 0.02).astype(np.float32)
    bias = _rand_i8(rng, N)
    _, want = c.qgemm_epilogue(c.qgemm_acc(a, w), x_scale=sx, w_scale=sw, out_scale=so, bias=bias,
                               fold_out=True, x_per_col=True)
    got = ops.qgemm(_dev(a), _dev(w), x_scale=_dev(sx), w_scale=_dev(sw), out_scale=_dev(so), bias=_dev(bias),
                    fold_out_scale=True, x_scale_per_col=True).cpu().numpy()
    assert (got == want).all()


@pytest.mark.parametrize("M,K,N", [(7, 768, 768), (64, 768, 3072), (333, 768, 3072), (1024, 3072, 768)])
@pytest.mark.parametrize("act", [None, "gelu", "silu"])
def test_fused_epilogue_fp16_and_requant(ops, M, K, N, act):
    """Config 1: per-tensor s_x = 0.02, per-channel s_w in [1e-3, 1e-2], fp32 bias;
    fp16 dequantized output and int8 requantized at 0.05."""
    from oracle import c
    rng = np.random.default_rng(M * 3 + N)
    a, w = _rand_i8(rng, (M, K)), _rand_i8(rng, (N, K))
    sw = (rng.random(N) * 9e-3 + 1e-3).astype(np.float32)
    bias = (rng.standard_normal(N) * 0.01).astype(np.float32)
    s_x, s_out = np.float32(0.02), np.float32(0.05)
    acc = c.qgemm_acc(a, w)
    f_want, _ = c.qgemm_epilogue(acc, x_scale=s_x, w_scale=sw, bias=bias, act=act)
    _, q_want = c.qgemm_epilogue(acc, x_scale=s_x, w_scale=sw, out_scale=s_out, bias=bias, act=act, div_out=True)
    kw = dict(x_scale=_dev(np.array([s_x])), w_scale=_dev(sw), bias=_dev(bias), act=act)
    f16 = ops.qgemm(_dev(a), _dev(w), out_dtype=torch.float16, **kw).float().cpu().numpy()
    f32 = ops.qgemm(_dev(a), _dev(w), out_dtype=torch.float32, **kw).cpu().numpy()
    assert np.allclose(f32, f_want, rtol=RTOL, atol=ATOL)
    finite = np.abs(f_want) < 60000
    assert np.allclose(f16[finite], f_want[finite], rtol=RTOL, atol=ATOL)
    # with an activation libdevice's erf / exp stand against libm's: one level allowed in the exact form too
    _check_requant(lambda exact: ops.qgemm(_dev(a), _dev(w), out_scale=_dev(np.array([s_out])), exact_division=exact,
                                           **kw).cpu().numpy(), q_want, exact_ok=act is None)
    if act is None:
        assert (f32 == f_want).all()


@pytest.mark.parametrize("M", [5, 150])
def test_per_row_dynamic_scales(ops, M):
    """Per-token activation scales (config 4): acc * s_x[m] * s_w[n] + bias."""
    from oracle import c
    rng = np.random.default_rng(M)
    K, N = 512, 320
    x = (rng.standard_normal((M, K)) * rng.random((M, 1)) * 4).astype(np.float32)
    w = _rand_i8(rng, (N, K))
    sw = (rng.random(N) * 9e-3 + 1e-3).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    xq, sx = ops.dynamic_quantize(_dev(x))
    xq_want, sx_want = c.dynamic_quantize(x)
    assert (xq.cpu().numpy() == xq_want).all() and (sx.cpu().numpy() == sx_want).all()
    want, _ = c.qgemm_epilogue(c.qgemm_acc(xq_want, w), x_scale=sx_want, w_scale=sw, bias=bias)
    got = ops.qgemm(xq, _dev(w), x_scale=sx, w_scale=_dev(sw), bias=_dev(bias), out_dtype=torch.float32)
    assert (got.cpu().numpy() == want).all()


def test_fake_quant_golden_within_one_lsb(ops, golden):
    """The reference's e2e golden (eager fake-quant linear): atol = output scale
    (pytorch_blade/tests/disc/pdl/test_e2e/test_quantization.py:408)."""
    for tag in ("r2", "r3"):
        x, w, b, s, y = [golden[f"fq_linear_{tag}_{k}"] for k in ("x", "w", "b", "scales", "y")]
        sc = [_dev(np.array([v], dtype=np.float32)) for v in s]
        xq = ops.quantize(_dev(x), sc[0])
        wq = ops.quantize(_dev(w), sc[1])
        q = ops.qgemm(xq, wq, x_scale=sc[0], w_scale=sc[1], out_scale=sc[2],
                      bias=_dev((b / s[2]).astype(np.float32)), fold_out_scale=True)
        got = ops.dequantize(q, sc[2]).cpu().numpy()
        assert got.shape == y.shape
        assert np.abs(got - y).max() <= s[2] * 1.0001


def test_empty_and_degenerate(ops):
    a = torch.zeros((0, 64), dtype=torch.int8, device="cuda")
    w = torch.ones((32, 64), dtype=torch.int8, device="cuda")
    assert ops.qgemm(a, w, out_dtype=torch.int32).shape == (0, 32)
    # extreme values: -128 * -128 * K stays inside int32
    a = torch.full((130, 4096), -128, dtype=torch.int8, device="cuda")
    w = torch.full((144, 4096), -128, dtype=torch.int8, device="cuda")
    assert (ops.qgemm(a, w, out_dtype=torch.int32) == 128 * 128 * 4096).all()
    assert (ops.qgemm(a[:3], w, out_dtype=torch.int32) == 128 * 128 * 4096).all()


@pytest.mark.parametrize("M,K,N", [(4096, 4096, 4096), (16384, 4096, 11008), (64, 4096, 11008)])
def test_full_size_checksums(ops, M, K, N):
    """At benchmark sizes the oracle is too slow; two size-independent identities
    cover every output: row sums  sum_n acc[m, n] = a[m, :] . (sum_n w[n, :])  and
    column sums  sum_m acc[m, n] = (sum_m a[m, :]) . w[n, :]  (exact in int64),
    plus 32 full rows against the oracle."""
    from oracle import c
    rng = np.random.default_rng(M + N)
    a, w = _rand_i8(rng, (M, K)), _rand_i8(rng, (N, K))
    acc = ops.qgemm(_dev(a), _dev(w), out_dtype=torch.int32)
    row_sum = acc.sum(dim=1, dtype=torch.int64).cpu().numpy()
    col_sum = acc.sum(dim=0, dtype=torch.int64).cpu().numpy()
    a64, w64 = a.astype(np.int64), w.astype(np.int64)
    assert (row_sum == a64 @ w64.sum(axis=0)).all()
    assert (col_sum == w64 @ a64.sum(axis=0)).all()
    rows = rng.choice(M, size=min(32, M), replace=False)
    assert (acc[torch.from_numpy(rows).cuda()].cpu().numpy() == c.qgemm_acc(a[rows], w)).all()


@pytest.mark.parametrize("M,g,slab,N", [(64, 2, 2048, 520), (7, 4, 1376, 264), (300, 4, 512, 392), (1024, 2, 5504, 256),
                                        (2048, 8, 128, 1024), (130, 3, 272, 72), (4, 2, 24, 10)])
@pytest.mark.parametrize("path", [None, "tiled", "pair", "skinny", "simt"])
def test_gathered_activation_layout(ops, M, g, slab, N, path):
    """The activation given as [g, M, K / g] column slabs (what an all-gather of
    column-parallel outputs leaves) multiplies exactly like the row-major
    matrix, on every path that accepts it, slab widths that are not multiples
    of the 128-byte K block included."""
    from oracle import c
    K = g * slab
    if path in ("tiled", "pair", "skinny") and slab % 16:
        pytest.skip("TMA paths need 16-byte multiples")
    rng = np.random.default_rng(M + g + slab + N)
    a, w = _rand_i8(rng, (M, K)), _rand_i8(rng, (N, K))
    gathered = np.ascontiguousarray(a.reshape(M, g, slab).transpose(1, 0, 2))
    want = c.qgemm_acc(a, w)
    got = ops.qgemm(_dev(gathered), _dev(w), out_dtype=torch.int32, path=path, a_gathered=True).cpu().numpy()
    assert got.shape == (M, N)
    assert (got == want).all()
    sw = (rng.random(N) * 9e-3 + 1e-3).astype(np.float32)
    bias = (rng.standard_normal(N) * 0.5).astype(np.float32)
    sx = (rng.random(M) * 0.03 + 0.01).astype(np.float32)
    s_out = np.float32(0.05)
    _, want8 = c.qgemm_epilogue(want, x_scale=sx, w_scale=sw, out_scale=s_out, bias=bias, div_out=True)
    _check_requant(lambda exact: ops.qgemm(_dev(gathered), _dev(w), x_scale=_dev(sx), w_scale=_dev(sw), bias=_dev(bias),
                                           out_scale=_dev(np.array([s_out])), path=path, a_gathered=True,
                                           exact_division=exact).cpu().numpy(), want8)


@pytest.mark.parametrize("M,K,N", [(1, 1024, 520), (7, 4096, 1000), (24, 2048, 392), (100, 768, 3072)])
def test_early_weight_fetch_orders_itself(ops, M, K, N):
    """weights_static lets the few-row kernels request the weight before the
    kernel in front of them has finished; activations, scales and the output
    are only touched after it has.  A chain in which each linear's activation
    is written by the kernel right before it, repeated back to back, must give
    the same bytes as the same chain with a synchronize between the steps."""
    gen = torch.Generator(device="cuda").manual_seed(M + N)
    w1 = torch.randint(-127, 128, (N, K), dtype=torch.int8, device="cuda", generator=gen)
    w2 = torch.randint(-127, 128, (K, N), dtype=torch.int8, device="cuda", generator=gen)
    sw1 = torch.rand(N, device="cuda", generator=gen) * 9e-3 + 1e-3
    sw2 = torch.rand(K, device="cuda", generator=gen) * 9e-3 + 1e-3
    x0 = torch.randn(M, K, device="cuda", generator=gen).half()
    torch.cuda.synchronize()

    def chain(sync):
        x = x0
        outs = []
        for _ in range(6):
            q, s = ops.dynamic_quantize(x)                       # writes the activation and its scales
            h = ops.qgemm(q, w1, x_scale=s, w_scale=sw1, out_dtype=torch.float16, weights_static=True)
            if sync:
                torch.cuda.synchronize()
            q2, s2 = ops.dynamic_quantize(h)
            x = ops.qgemm(q2, w2, x_scale=s2, w_scale=sw2, out_dtype=torch.float16, weights_static=True)
            x = (x.float() / x.float().abs().amax().clamp_min(1e-3)).half()  # keep the chain in range
            if sync:
                torch.cuda.synchronize()
            outs.append(x)
        torch.cuda.synchronize()
        return outs

    want = chain(True)
    for _ in range(3):
        got = chain(False)
        assert all(torch.equal(a.view(torch.int16), b.view(torch.int16)) for a, b in zip(got, want))
        assert all(torch.isfinite(a).all() for a in got)
    # without the promise a weight written by the previous kernel is still read correctly
    w_late = torch.empty_like(w1)
    for _ in range(3):
        w_late.copy_(w1)  # a device-side copy kernel right in front of the linear
        q, s = ops.dynamic_quantize(x0)
        a = ops.qgemm(q, w_late, x_scale=s, w_scale=sw1, out_dtype=torch.float16)
        w_late.zero_()
        b = ops.qgemm(q, w1, x_scale=s, w_scale=sw1, out_dtype=torch.float16)
        assert torch.equal(a, b)
