"""Weight-only quantized linear (ral_pdll_weight_only_qgemm) on B200 against the C oracle."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(m, k, n, seed, dtype, with_bias=True, zp_kind="128"):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((m, k)).astype(dtype)
    w = rng.integers(0, 256, (k, n), dtype=np.uint8)
    scale = (rng.random(n) * 0.02 + 0.002).astype(dtype)
    bias = rng.standard_normal(n).astype(dtype) if with_bias else None
    zp = {"128": np.full(n, 128, np.int32), "random": rng.integers(0, 256, n).astype(np.int32), "none": None}[zp_kind]
    return x, w, scale, zp, bias


def _check(out, x, w, scale, zp, bias, dtype):
    """fp32 sums in another order than the oracle's double: a few fp32 ulps of the sum of magnitudes,
    plus the rounding of the result to its type."""
    from oracle import c
    want = c.weight_only_qgemm(x, w, scale, zp, bias)
    z = 0 if zp is None else zp
    mag = (np.abs(x.astype(np.float32)) @ np.abs(w.astype(np.float32) - z)) * np.abs(scale.astype(np.float32))
    tol = 4e-6 * mag + 1e-6
    if dtype == np.float16:
        tol = tol + np.abs(want) * 2.0 ** -10 + 1e-7
    got = out.float().cpu().numpy()
    assert np.isfinite(got).all()
    bad = np.abs(got - want) > tol
    assert not bad.any(), (int(bad.sum()), float(np.abs(got - want).max()))


def _run(x, w, scale, zp, bias, path=None):
    from bladedisc_b200 import ops
    d = lambda a: None if a is None else torch.from_numpy(a).cuda()
    out = ops.weight_only_qgemm(d(x), d(w), d(scale), d(zp), d(bias), path=path)
    assert ops.kernel_status() == 0, "a bounded wait of a kernel ran out"
    return out


@pytest.mark.parametrize("m", [1, 2, 3, 4, 5, 8, 13, 16])
@pytest.mark.parametrize("dtype", [np.float16, np.float32])
def test_few_rows_match_oracle(m, dtype):
    """Every row tile (1, 2, 4, 8, 16) with and without padding rows; k split over blocks."""
    args = _case(m, 1024, 768, m, dtype)
    _check(_run(*args), *args, dtype)


@pytest.mark.parametrize("shape", [(1, 4096, 4096), (4, 4096, 11008), (8, 11008, 4096), (33, 512, 256), (2, 100, 264),
                                   (1, 64, 8), (4, 7, 16), (16, 1000, 132)])
def test_shapes_match_oracle(shape):
    """7B-shaped decode linears, more than 16 rows (groups of 16), k not a multiple of the chunk,
    narrow outputs, N a multiple of 4 only."""
    m, k, n = shape
    args = _case(m, k, n, k + n, np.float16, with_bias=(n % 16 == 0), zp_kind="random" if k < 2000 else "128")
    _check(_run(*args), *args, np.float16)


@pytest.mark.parametrize("shape", [(5, 256, 128), (16, 1024, 768), (4, 4096, 4096), (16, 4096, 11008), (64, 4096, 4096),
                                   (100, 512, 256), (128, 1024, 384), (129, 2048, 1024), (300, 1000, 144), (7, 72, 16),
                                   (1, 64, 16), (2048, 512, 512), (2400, 256, 4096), (2305, 128, 4096)])
@pytest.mark.parametrize("zp_kind", ["random", "none"])
def test_tensor_core_path_matches_oracle(shape, zp_kind):
    """The tensor-core kernel, forced: one and several row blocks, k split over clusters of every size the
    planner picks, k and channel tails (k not a multiple of 64, N a multiple of 16 only), with and without
    zero points and bias; the last two shapes are long enough for two row tiles per block (2400 rows end in a
    block whose second tile is empty, 2305 in one with a single row)."""
    m, k, n = shape
    args = _case(m, k, n, m + k + n, np.float16, with_bias=(zp_kind == "random"), zp_kind=zp_kind)
    _check(_run(*args, path="tensor"), *args, np.float16)


def test_tensor_core_path_is_repeatable_and_refuses_what_it_cannot_take():
    from bladedisc_b200 import ops
    args = _case(16, 4096, 1024, 5, np.float16, zp_kind="random")
    a = _run(*args, path="tensor")
    for _ in range(3):                       # partial tiles are added in rank order: bit-identical between runs
        assert torch.equal(_run(*args, path="tensor"), a)
    b = _run(*args, path="stream")
    assert torch.allclose(a.float(), b.float(), rtol=2e-3, atol=2e-3)  # two summation orders of the same products
    x32 = torch.zeros(8, 64, dtype=torch.float32, device="cuda")
    w = torch.zeros(64, 16, dtype=torch.uint8, device="cuda")
    with pytest.raises(RuntimeError, match="tensor cores"):
        ops.weight_only_qgemm(x32, w, torch.ones(16, device="cuda"), path="tensor")          # fp32 activations
    x16 = torch.zeros(8, 64, dtype=torch.float16, device="cuda")
    w20 = torch.zeros(64, 20, dtype=torch.uint8, device="cuda")
    with pytest.raises(RuntimeError, match="tensor cores"):
        ops.weight_only_qgemm(x16, w20, torch.ones(20, dtype=torch.float16, device="cuda"), path="tensor")  # N % 16


@pytest.mark.parametrize("shape", [(2, 3, 5), (1, 17, 3), (6, 130, 250), (3, 64, 1001)])
def test_unaligned_shapes_take_the_simple_kernel(shape):
    """The reference's own test shape (K = 3, N = 5) and other outputs that are not a multiple of 4."""
    m, k, n = shape
    for dtype in (np.float32, np.float16):
        args = _case(m, k, n, 9, dtype, zp_kind="random")
        _check(_run(*args), *args, dtype)


def test_no_zero_point_no_bias_and_repeatability():
    args = _case(4, 2048, 1024, 3, np.float16, with_bias=False, zp_kind="none")
    a = _run(*args)
    _check(a, *args, np.float16)
    for _ in range(3):                       # partials are added in k order: bit-identical between runs
        assert torch.equal(_run(*args), a)


def test_errors_and_empty():
    from bladedisc_b200 import ops
    x = torch.zeros(2, 8, dtype=torch.float16, device="cuda")
    w = torch.zeros(8, 16, dtype=torch.uint8, device="cuda")
    s = torch.ones(16, dtype=torch.float16, device="cuda")
    with pytest.raises(ValueError):
        ops.weight_only_qgemm(x, torch.zeros(9, 16, dtype=torch.uint8, device="cuda"), s)
    with pytest.raises(TypeError):
        ops.weight_only_qgemm(x, w.to(torch.int8), s)
    with pytest.raises(TypeError):
        ops.weight_only_qgemm(x, w, s.float())
    assert ops.weight_only_qgemm(x[:0], w, s).shape == (0, 16)
    # zero weights minus zero point 0: exactly the bias
    b = torch.arange(16, dtype=torch.float16, device="cuda")
    assert torch.equal(ops.weight_only_qgemm(x + 1, w, s, None, b), b.expand(2, 16))


@pytest.mark.parametrize("rank3", [False, True])
@pytest.mark.parametrize("with_bias", [False, True])
def test_custom_call(rank3, with_bias):
    """ral_pdll_weight_only_qgemm through the dispatcher, operand order of the reference's pattern
    (weight_only_qgemm.pdll:27 and :90); result allocated by the callee."""
    from bladedisc_b200.ral import MemRefSpec, RalContext, RalError
    m, k, n = 6, 256, 384
    x, w, scale, zp, bias = _case(m, k, n, 21, np.float16, with_bias=with_bias)
    d = lambda a: torch.from_numpy(a).cuda()
    xin = d(x).reshape(2, 3, k) if rank3 else d(x)
    with RalContext() as ral:
        operands = [xin, d(w)] + ([d(bias)] if with_bias else []) + [d(scale), d(zp)]
        attrs = ral.attr_blob({"weight_should_be_reordered": True})
        out = ral.call("ral_pdll_weight_only_qgemm", "gpu", [("pvoid", 0)] + operands + [("pvoid", attrs)],
                       [MemRefSpec("f16", 3 if rank3 else 2)])
        assert tuple(out.shape) == ((2, 3, n) if rank3 else (m, n))
        _check(out.reshape(m, n), x, w, scale, zp, bias, np.float16)
        ral.dealloc(out)
        with pytest.raises(RalError, match="already permuted"):
            ral.call("ral_pdll_weight_only_qgemm", "gpu",
                     [("pvoid", 0)] + operands + [("pvoid", ral.attr_blob({"weight_should_be_reordered": False}))],
                     [MemRefSpec("f16", 3 if rank3 else 2)])
        with pytest.raises(RalError, match="extents disagree"):
            bad = operands[:-1] + [d(zp[:-1].copy())]
            ral.call("ral_pdll_weight_only_qgemm", "gpu", [("pvoid", 0)] + bad + [("pvoid", attrs)],
                     [MemRefSpec("f16", 3 if rank3 else 2)])
