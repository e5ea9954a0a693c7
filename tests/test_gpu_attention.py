"""The fused attention kernel over packed sequences against the numpy statement of
softmax(q k^T * scale) v (oracle/np_ref.py:attention_packed) on the same f16 inputs.

Tolerances: the kernel keeps scores and sums in fp32 but hands the probabilities to the second
product as f16 (relative rounding 2^-11), so the f16 result is compared at rtol 1e-2 / atol 2e-3 and
the int8 result (quantized at a static scale, reciprocal form) may sit one level off on a small
share of the values."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    assert torch.cuda.is_available()
    from bladedisc_b200 import ops as o
    yield o
    assert o.kernel_status() == 0, "a kernel's bounded wait ran out"


def _case(lens, heads, seed):
    rng = np.random.default_rng(seed)
    tokens = int(sum(lens))
    qkv = (rng.standard_normal((tokens, 3 * heads * 64)) * 1.2).astype(np.float16)
    return qkv, tokens


@pytest.mark.parametrize("lens,heads", [
    ([128], 1), ([1], 2), ([7, 130, 64], 2), ([512], 3), ([129, 257, 385, 511, 16], 4), ([300, 45, 512, 128, 256], 12),
])
def test_attention_matches_the_formula(ops, lens, heads):
    from oracle import np_ref
    qkv, tokens = _case(lens, heads, sum(lens) + heads)
    scale = 1.0 / math.sqrt(64)
    want = np_ref.attention_packed(qkv.astype(np.float32), lens, heads, scale)
    qkv_d = torch.from_numpy(qkv).cuda()
    blocks = ops.attention_blocks(lens, heads).cuda()
    assert int(blocks[:, 3].sum()) == sum((n + 127) // 128 for n in lens)
    got = ops.attention(qkv_d, blocks, heads, scale).float().cpu().numpy()
    assert got.shape == want.shape
    assert np.isfinite(got).all()
    assert np.allclose(got, want, rtol=1e-2, atol=2e-3), f"max abs error {np.abs(got - want).max():.3e}"
    # quantized output at the scale a calibration would pick
    s_out = np.float32(np.abs(want).max() / 127)
    q = ops.attention(qkv_d, blocks, heads, scale, out_scale=torch.tensor([s_out], device="cuda")).cpu().numpy()
    q_want = np.clip(np.rint(want / s_out), -128, 127).astype(np.int32)
    d = np.abs(q.astype(np.int32) - q_want)
    assert d.max() <= 1 and (d > 0).mean() < 0.05, f"int8: max {d.max()}, share off by one {(d > 0).mean():.3f}"


@pytest.mark.parametrize("group", [4, 2, 1])
def test_attention_is_the_same_however_the_query_blocks_are_grouped(ops, group):
    """One item per 128 query rows, per pair of blocks or per sequence: the same bytes."""
    heads, scale = 3, 0.125
    lens = [512, 300, 129, 128, 40, 385]
    qkv, tokens = _case(lens, heads, 9)
    qkv_d = torch.from_numpy(qkv).cuda()
    base = ops.attention(qkv_d, ops.attention_blocks(lens, heads).cuda(), heads, scale)
    blocks = ops.attention_blocks(lens, heads, group=group)
    assert int(blocks[:, 3].max()) == group
    so = torch.tensor([0.02], device="cuda")
    assert torch.equal(ops.attention(qkv_d, blocks.cuda(), heads, scale), base)
    assert torch.equal(ops.attention(qkv_d, blocks.cuda(), heads, scale, out_scale=so),
                       ops.attention(qkv_d, ops.attention_blocks(lens, heads).cuda(), heads, scale, out_scale=so))


def test_attention_ignores_neighbouring_sequences_and_padding_rows(ops):
    """A sequence's result does not depend on what is packed around it: the rows after its end (the next
    sequence, or nothing) are masked, never read as keys."""
    heads, scale = 2, 0.125
    lens = [200, 77, 333]
    qkv, tokens = _case(lens, heads, 5)
    qkv_d = torch.from_numpy(qkv).cuda()
    full = ops.attention(qkv_d, ops.attention_blocks(lens).cuda(), heads, scale)
    t0 = 0
    for n in lens:
        alone = ops.attention(qkv_d[t0:t0 + n].contiguous(), ops.attention_blocks([n]).cuda(), heads, scale)
        assert torch.equal(alone, full[t0:t0 + n]), f"sequence of length {n} differs when packed with others"
        t0 += n


def test_attention_argument_errors(ops):
    qkv = torch.zeros((8, 3 * 64), dtype=torch.float16, device="cuda")
    with pytest.raises(ValueError):
        ops.attention_blocks([0])
    with pytest.raises(ValueError):
        ops.attention_blocks([513])
    with pytest.raises(ValueError):
        ops.attention(qkv, torch.zeros((1, 3), dtype=torch.int32, device="cuda"), 1, 0.125)
    with pytest.raises(RuntimeError):
        ops.attention(qkv, ops.attention_blocks([8]).cuda(), 1, -1.0)
