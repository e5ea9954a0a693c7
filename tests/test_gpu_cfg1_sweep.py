"""The dynamic-shape sweep of the quantized linear, every point, through the path the library picks itself.

Configuration: int8 A [M, K] (per-tensor scale 0.02) x int8 W [N, K] (per-channel scales uniform in
[1e-3, 1e-2]), values uniform in [-127, 127], fp32 bias; M in {1, 7, 64, 333, 1024, 4096, 16384} and
(K, N) in {(768, 768), (768, 3072), (3072, 768), (4096, 4096), (4096, 11008)}; outputs fp16 dequantized and
int8 requantized at 0.05.  That is 35 shapes x 2 outputs, and the int8 output in both of its forms.

Up to 1024 rows every output element is compared with the CPU oracle.  At 4096 and 16384 rows the oracle
would take minutes, so the int32 sums are checked through two size-independent identities that touch every
element (row sums and column sums, exact in int64) and 64 sampled rows of each output are compared with
the oracle's epilogue on the oracle's own sums for those rows.

Tolerances: int32 sums bit exact; int8 with exact division bit exact; int8 in the default reciprocal form
at most one level off on under 1e-3 of the values; fp16 rtol 1e-2 / atol 1e-3 (the tolerance the reference's
end-to-end test uses is one output scale, pytorch_blade/tests/disc/pdl/test_e2e/test_quantization.py:357-460).
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

MS = [1, 7, 64, 333, 1024, 4096, 16384]
KNS = [(768, 768), (768, 3072), (3072, 768), (4096, 4096), (4096, 11008)]
S_X, S_OUT = np.float32(0.02), np.float32(0.05)
RTOL, ATOL = 1e-2, 1e-3
FULL_COMPARE_ROWS = 1024
SAMPLED_ROWS = 64


@pytest.fixture(scope="module")
def ops():
    assert torch.cuda.is_available()
    from bladedisc_b200 import ops as o
    yield o
    assert o.kernel_status() == 0, "a kernel's bounded wait ran out"


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _check_outputs(ops, a_d, w_d, sw, bias, rows, acc_rows):
    """fp16 and both int8 forms of the launch over all of `a_d`, compared on `rows` (None = all rows)."""
    from oracle import c
    kw = dict(x_scale=_dev(np.array([S_X])), w_scale=_dev(sw), bias=_dev(bias))
    so = _dev(np.array([S_OUT]))
    pick = (lambda t: t.cpu().numpy()) if rows is None else (lambda t: t[torch.from_numpy(rows).cuda()].cpu().numpy())
    f_want, _ = c.qgemm_epilogue(acc_rows, x_scale=S_X, w_scale=sw, bias=bias)
    _, q_want = c.qgemm_epilogue(acc_rows, x_scale=S_X, w_scale=sw, out_scale=S_OUT, bias=bias, div_out=True)
    f16 = pick(ops.qgemm(a_d, w_d, out_dtype=torch.float16, **kw).float())
    finite = np.abs(f_want) < 60000
    assert np.allclose(f16[finite], f_want[finite], rtol=RTOL, atol=ATOL), "fp16 output outside rtol 1e-2 / atol 1e-3"
    q_exact = pick(ops.qgemm(a_d, w_d, out_scale=so, exact_division=True, **kw))
    assert (q_exact == q_want).all(), f"int8 (exact division): {np.count_nonzero(q_exact != q_want)} mismatches"
    q = pick(ops.qgemm(a_d, w_d, out_scale=so, **kw))
    d = np.abs(q.astype(np.int32) - q_want.astype(np.int32))
    assert d.max() <= 1 and (d > 0).mean() < 1e-3, f"int8 (reciprocal form): flip rate {(d > 0).mean():.2e}, max {d.max()}"


@pytest.mark.parametrize("K,N", KNS)
@pytest.mark.parametrize("M", MS)
def test_sweep_point(ops, M, K, N):
    from oracle import c
    rng = np.random.default_rng(M * 1000003 + K * 101 + N)
    a = rng.integers(-127, 128, (M, K), dtype=np.int8)
    w = rng.integers(-127, 128, (N, K), dtype=np.int8)
    sw = (rng.random(N) * 9e-3 + 1e-3).astype(np.float32)
    bias = (rng.standard_normal(N) * 0.01).astype(np.float32)
    a_d, w_d = _dev(a), _dev(w)
    acc = ops.qgemm(a_d, w_d, out_dtype=torch.int32)
    if M <= FULL_COMPARE_ROWS:
        want = c.qgemm_acc(a, w)
        assert (acc.cpu().numpy() == want).all(), f"path {ops.qgemm_path(M, N, K)}: int32 sums differ"
        _check_outputs(ops, a_d, w_d, sw, bias, None, want)
        return
    # every element through the checksum identities ...
    a64, w64 = a.astype(np.int64), w.astype(np.int64)
    assert (acc.sum(dim=1, dtype=torch.int64).cpu().numpy() == a64 @ w64.sum(axis=0)).all(), "row sums differ"
    assert (acc.sum(dim=0, dtype=torch.int64).cpu().numpy() == w64 @ a64.sum(axis=0)).all(), "column sums differ"
    # ... and sampled rows in full, the first and the last row among them
    rows = np.unique(np.concatenate([[0, M - 1], rng.choice(M, size=SAMPLED_ROWS, replace=False)]))
    want = c.qgemm_acc(a[rows], w)
    assert (acc[torch.from_numpy(rows).cuda()].cpu().numpy() == want).all(), "sampled rows of the int32 sums differ"
    del acc
    _check_outputs(ops, a_d, w_d, sw, bias, rows, want)
