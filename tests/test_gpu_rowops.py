"""Parity of the bandwidth kernels (quantize / dequantize / LayerNorm / RMSNorm /
softmax) against the CPU oracle and the eager-torch goldens (B200 only).

int8 results are bit-exact; floating-point results use the tolerance of the
reference's own op tests for fp32 (rtol 1e-6, atol 1e-3) and rtol 1e-2 /
atol 1e-3 for fp16 data.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    assert torch.cuda.is_available()
    from bladedisc_b200 import ops as o
    return o


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _one_level(q, want, share=1e-3):
    """int8 results of the quantization fused behind a row operation use the reciprocal form: at most one
    level from the divide-based formula, and that on a small share of the values only."""
    d = np.abs(q.cpu().numpy().astype(np.int32) - np.asarray(want).astype(np.int32))
    assert d.max() <= 1 and (d > 0).mean() <= share, f"max {d.max()}, share off by one {(d > 0).mean():.2e}"


@pytest.mark.parametrize("shape", [(8, 128, 768), (1,), (17,), (5, 33), (1024, 3072), (3, 1, 16)])
@pytest.mark.parametrize("zp", [None, 3])
def test_quantize_per_tensor_bit_exact(ops, shape, zp):
    from oracle import c
    rng = np.random.default_rng(len(shape) + (zp or 0))
    x = (rng.standard_normal(shape) * 3).astype(np.float32)
    x.flat[0] = 1e9
    s = np.float32(np.abs(x[np.abs(x) < 1e8]).max() / 127) if x.size > 1 else np.float32(0.5)
    zpa = None if zp is None else np.array([zp], dtype=np.int32)
    want = c.quantize(x, s, zero_point=zpa)
    got = ops.quantize(_dev(x), _dev(np.array([s])), None if zpa is None else _dev(zpa))
    assert (got.cpu().numpy() == want).all()
    # ties: multiples of half a step round to even
    t = (np.arange(-300, 300, dtype=np.float32) * 0.5 * s).astype(np.float32)
    assert (ops.quantize(_dev(t), _dev(np.array([s]))).cpu().numpy() == c.quantize(t, s)).all()


def test_quantize_fp16_input_and_per_axis(ops):
    from oracle import c
    rng = np.random.default_rng(0)
    x = (rng.standard_normal((6, 40, 24)) * 2).astype(np.float16)
    s = np.float32(0.031)
    got = ops.quantize(_dev(x), _dev(np.array([s])))
    assert (got.cpu().numpy() == c.quantize(x.astype(np.float32), s)).all()
    for axis in (0, 1, 2):
        sc = (rng.random(x.shape[axis]) * 0.05 + 0.01).astype(np.float32)
        zp = rng.integers(-5, 6, x.shape[axis]).astype(np.int32)
        xf = x.astype(np.float32)
        want = c.quantize(xf, sc, zero_point=zp, axis=axis)
        got = ops.quantize(_dev(xf), _dev(sc), _dev(zp), axis=axis)
        assert (got.cpu().numpy() == want).all()
        deq = ops.dequantize(got, _dev(sc), _dev(zp), axis=axis)
        assert (deq.cpu().numpy() == c.dequantize(want, sc, zero_point=zp, axis=axis)).all()


@pytest.mark.parametrize("n", [1, 15, 16, 4097, 1 << 20])
def test_dequantize_per_tensor(ops, n):
    from oracle import c
    rng = np.random.default_rng(n)
    q = rng.integers(-128, 128, n, dtype=np.int8)
    s, zp = np.float32(0.0173), np.array([-4], dtype=np.int32)
    got = ops.dequantize(_dev(q), _dev(np.array([s])), _dev(zp))
    assert (got.cpu().numpy() == c.dequantize(q, s, zero_point=zp)).all()
    h = ops.dequantize(_dev(q), _dev(np.array([s])), _dev(zp), dtype=torch.float16)
    assert np.allclose(h.float().cpu().numpy(), c.dequantize(q, s, zero_point=zp), rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("rows,cols", [(1, 8), (7, 768), (333, 1024), (64, 4096), (5, 11008), (9, 100), (3, 16384)])
@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_dynamic_quantize(ops, rows, cols, dtype):
    from oracle import c
    rng = np.random.default_rng(rows + cols)
    x = (rng.standard_normal((rows, cols)) * rng.random((rows, 1)) * 5).astype(dtype)
    x[0] = 0  # an all-zero row must not divide by zero
    q, s = ops.dynamic_quantize(_dev(x))
    qw, sw = c.dynamic_quantize(x.astype(np.float32))
    assert (s.cpu().numpy() == sw).all()
    _one_level(q, qw)
    assert (q.cpu().numpy()[0] == 0).all()
    if rows > 1:
        assert np.abs(q.cpu().numpy()[1:]).max(axis=1).min() == 127  # every row's largest magnitude lands on the last level


def test_layernorm_golden_fp32(ops, golden):
    g = golden
    y = ops.layernorm(_dev(g["ln_x"]), _dev(g["ln_gamma"]), _dev(g["ln_beta"]), eps=1e-5)
    assert np.allclose(y.cpu().numpy(), g["ln_y"], rtol=1e-6, atol=1e-3)


@pytest.mark.parametrize("rows,cols", [(1, 768), (37, 768), (1000, 1024), (16, 4096), (5, 100), (3, 8192), (2, 12000)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("residual", [False, True])
def test_layernorm_vs_oracle(ops, rows, cols, dtype, residual):
    from oracle import c
    rng = np.random.default_rng(rows * 7 + cols)
    x = torch.from_numpy((rng.standard_normal((rows, cols)) * 2 + 0.3).astype(np.float32)).to(dtype)
    r = torch.from_numpy(rng.standard_normal((rows, cols)).astype(np.float32)).to(dtype)
    gm = torch.from_numpy(rng.standard_normal(cols).astype(np.float32)).to(dtype)
    bt = torch.from_numpy(rng.standard_normal(cols).astype(np.float32)).to(dtype)
    want, _ = c.norm(x.float().numpy(), gm.float().numpy(), bt.float().numpy(),
                     residual=r.float().numpy() if residual else None, eps=1e-5)
    got = ops.layernorm(x.cuda(), gm.cuda(), bt.cuda(), eps=1e-5, residual=r.cuda() if residual else None)
    if dtype == torch.float32:
        assert np.allclose(got.cpu().numpy(), want, rtol=1e-6, atol=1e-3)
    else:
        assert np.allclose(got.float().cpu().numpy(), want, rtol=1e-2, atol=1e-2)


def test_layernorm_quantized_second_output(ops):
    """The int8 copy is quantize(y) of the stored y in the reciprocal form: within one level of the divide."""
    from oracle import c
    rng = np.random.default_rng(1)
    x = torch.from_numpy(rng.standard_normal((130, 768)).astype(np.float32)).half().cuda()
    r = torch.from_numpy(rng.standard_normal((130, 768)).astype(np.float32)).half().cuda()
    gm = torch.ones(768, dtype=torch.float16, device="cuda")
    bt = torch.zeros(768, dtype=torch.float16, device="cuda")
    s = np.float32(4.0 / 127)
    y, q = ops.layernorm_quant(x, gm, bt, _dev(np.array([s])), residual=r)
    _one_level(q, c.quantize(y.float().cpu().numpy(), s))
    y2 = ops.layernorm(x, gm, bt, residual=r)
    assert torch.equal(y, y2)


@pytest.mark.parametrize("cols", [4096, 768, 11008])
def test_rmsnorm_sum_and_dynamic_quant(ops, cols):
    from oracle import c
    rng = np.random.default_rng(cols)
    x = torch.from_numpy(rng.standard_normal((19, cols)).astype(np.float32)).half()
    r = torch.from_numpy(rng.standard_normal((19, cols)).astype(np.float32)).half()
    gm = torch.from_numpy((rng.random(cols) + 0.5).astype(np.float32)).half()
    y, s = ops.rmsnorm(x.cuda(), gm.cuda(), eps=1e-6, residual=r.cuda(), return_sum=True)
    assert torch.equal(s.cpu(), (x.float() + r.float()).half())
    want, _ = c.norm(s.float().cpu().numpy(), gm.float().numpy(), eps=1e-6, rms=True)
    assert np.allclose(y.float().cpu().numpy(), want, rtol=1e-2, atol=1e-2)
    q, rs, s2 = ops.rmsnorm_dynamic_quant(x.cuda(), gm.cuda(), eps=1e-6, residual=r.cuda())
    assert torch.equal(s2, s)
    qw, sw = c.dynamic_quantize(y.float().cpu().numpy())
    assert (rs.cpu().numpy() == sw).all()
    _one_level(q, qw)


def test_softmax_golden_fp32(ops, golden):
    g = golden
    y = ops.softmax(_dev(g["sm_x"]))
    assert np.allclose(y.cpu().numpy(), g["sm_y"], rtol=1e-6, atol=1e-3)
    ly = ops.softmax(_dev(g["sm_x"]), log=True)
    assert np.allclose(ly.cpu().numpy(), g["sm_logy"], rtol=1e-6, atol=1e-3)


@pytest.mark.parametrize("cols", [16, 37, 128, 333, 512, 1000, 2048])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_softmax_masked_lengths(ops, cols, dtype):
    """Padded-mask attention scores: [batch, heads, L, L] with a valid length per sequence."""
    from oracle import c
    rng = np.random.default_rng(cols)
    B, H, L = 3, 2, min(cols, 24)
    x = torch.from_numpy((rng.standard_normal((B, H, L, cols)) * 4).astype(np.float32)).to(dtype)
    lens = np.array([cols, max(1, cols // 3), 1], dtype=np.int32)
    want = c.softmax(x.float().numpy(), scale=0.125, lens=lens)
    got = ops.softmax(x.cuda(), scale=0.125, lens=_dev(lens)).float().cpu().numpy()
    tol = dict(rtol=1e-6, atol=1e-3) if dtype == torch.float32 else dict(rtol=1e-2, atol=1e-3)
    assert np.allclose(got, want, **tol)
    assert (got[1][..., lens[1]:] == 0).all()
    # additive mask form
    mask = np.where(np.arange(cols)[None, :] < lens[:, None], 0.0, -10000.0).astype(np.float32)
    want_m = c.softmax(x.float().numpy(), scale=0.125, mask=mask)
    got_m = ops.softmax(x.cuda(), scale=0.125, mask=torch.from_numpy(mask).to(dtype).cuda()).float().cpu().numpy()
    assert np.allclose(got_m, want_m, **tol)


def test_rows_kernel_limits(ops):
    x = torch.zeros((2, 20000), device="cuda")
    with pytest.raises(RuntimeError, match="16384"):
        ops.softmax(x)
    assert ops.softmax(torch.zeros((0, 8), device="cuda")).shape == (0, 8)
