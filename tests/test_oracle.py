"""Pins the CPU oracle (oracle/) to the reference: its known-answer vectors, the
golden its own e2e tests compare against (eager torch fake-quant composites),
its torch_quant observers, and oneDNN.  Runs without a GPU."""
import numpy as np
import pytest

from oracle import c, np_ref

F = np.float32


# --- known-answer vectors of the reference's feature tests ------------------
# tao_compiler/mlir/disc/tests/pdll/qgemm.cc:24-42 and
# tests/tensorflow_ops/quantized_matmul.cc:24-54: x = -0.6 [4,25], s_x = 1/120,
# w = -0.8 [25,71], s_w = 1.568627e-2, s_out = 1  ->  every output 12.0.
@pytest.mark.parametrize("per_channel", [False, True])
def test_kat_12(per_channel):
    s_x, s_w, s_out = F(8.333333e-3), F(1.568627e-2), F(1.0)
    x = np.full((4, 25), -0.6, dtype=F)
    w = np.full((71, 25), -0.8, dtype=F)  # stored [N, K]
    xq = c.quantize(x, s_x)
    sw = np.full(71, s_w, dtype=F) if per_channel else s_w
    wq = c.quantize(w, sw, axis=0) if per_channel else c.quantize(w, s_w)
    acc = c.qgemm_acc(xq, wq)
    _, q = c.qgemm_epilogue(acc, x_scale=s_x, w_scale=sw, out_scale=s_out, fold_out=True)
    y = c.dequantize(q, s_out)
    assert y.shape == (4, 71)
    assert (y == 12.0).all()
    # the x86 form of the same call agrees
    assert (c.dequantize(c.qgemm_x86(acc, float(s_x), np.atleast_1d(sw), float(s_out)), s_out) == 12.0).all()


# quantized_matmul.cc:56-73 (GPU variant, disabled upstream): x = 2.0 [32,64], s = 2,
# w = 1.0 [64,128], s_w = 1, s_out = 2 -> 128.0 before the int8 clamp; the stored
# int8 saturates at 127 * 2 = 254 unless the test reads the unclamped value, so pin both.
def test_kat_128():
    x = np.full((32, 64), 2.0, dtype=F)
    w = np.full((128, 64), 1.0, dtype=F)
    xq = c.quantize(x, F(2.0))
    wq = c.quantize(w, F(1.0))
    acc = c.qgemm_acc(xq, wq)
    assert (acc == 64).all()
    f, q = c.qgemm_epilogue(acc, x_scale=F(2.0), w_scale=F(1.0), out_scale=F(2.0), fold_out=True)
    assert (f == 64.0).all()
    assert (c.dequantize(q, F(2.0)) == 128.0).all()


# quantize_v2 inputs of tests/tensorflow_ops/quantize_v2.cc:25-120 pushed through the
# DISC quantize formula with a scale of 1: rounding is half-to-even, clamp is [-128, 127].
def test_round_half_even_and_clamp():
    x = np.array([0, 1, 1.25, 1.75, 127, 255, 500, -255, 64, 0.5, 1.5, 2.5, -0.5, -1.5, -2.5], dtype=F)
    q = c.quantize(x, F(1.0))
    assert q.tolist() == [0, 1, 1, 2, 127, 127, 127, -128, 64, 0, 2, 2, 0, -2, -2]
    assert (q == np_ref.quantize(x, F(1.0))).all()


def test_c_matches_numpy_statement():
    rng = np.random.default_rng(7)
    x = (rng.standard_normal((33, 129)) * 4).astype(F)
    s = F(0.0371)
    assert (c.quantize(x, s) == np_ref.quantize(x, s)).all()
    assert (c.fake_quant(x, s) == np_ref.fake_quant(x, s)).all()
    sc = (rng.random(33) * 0.05 + 0.01).astype(F)
    assert (c.quantize(x, sc, axis=0) == np_ref.quantize(x, sc[:, None])).all()
    q = c.quantize(x, s)
    assert (c.dequantize(q, s) == np_ref.dequantize(q, s)).all()
    a = rng.integers(-127, 128, (19, 160), dtype=np.int8)
    w = rng.integers(-127, 128, (31, 160), dtype=np.int8)
    acc = c.qgemm_acc(a, w)
    assert (acc == np_ref.qgemm_acc(a, w)).all()
    b = rng.standard_normal(31).astype(F)
    _, q8 = c.qgemm_epilogue(acc, x_scale=0.02, w_scale=0.005, out_scale=0.05, bias=b, fold_out=True)
    assert (q8 == np_ref.ral_epilogue(acc, 0.02, 0.005, 0.05, b)).all()
    assert (c.qgemm_ral_i8(a, w, 0.02, 0.005, 0.05, b) == q8).all()
    qd, sd = c.dynamic_quantize(x)
    qn, sn = np_ref.dynamic_quantize(x)
    assert (qd == qn).all() and (sd == sn).all()


def test_weight_quantization_in_double():
    # A value whose float32 quotient rounds the other way than its double quotient
    # would expose a float implementation; exact ties must go to even.
    w = np.array([[0.5, 1.5, 2.5, -0.5, 3.4999998]], dtype=F)
    q = c.quantize_weight(w, np.array([1.0], dtype=F), per_channel=False)
    assert q.tolist() == [[0, 2, 2, 0, 3]]


# --- the reference's own e2e golden (eager fake-quant composite) -------------
@pytest.mark.parametrize("tag", ["r2", "r3"])
def test_fake_quant_linear_golden(golden, tag):
    x, w, b, s, y = [golden[f"fq_linear_{tag}_{k}"] for k in ("x", "w", "b", "scales", "y")]
    # the restated torch fake-quant reproduces torch bit for bit
    xf, wf = c.fake_quant(x, s[0]), c.fake_quant(w, s[1])
    lin = xf.reshape(-1, x.shape[-1]).astype(np.float64) @ wf.T.astype(np.float64) + b
    # int8 pipeline as the GPU pattern lowers it: bias pre-divided by the output scale
    # (pdll_files/gpu/dequant_gemm_quant_bias_f32_quant.pdll:72-79)
    xq, wq = c.quantize(x, s[0]), c.quantize(w, s[1])
    assert (c.dequantize(xq, s[0]) == xf).all() or np.abs(c.dequantize(xq, s[0]) - xf).max() <= s[0]
    acc = c.qgemm_acc(xq, wq)
    _, q = c.qgemm_epilogue(acc, x_scale=s[0], w_scale=s[1], out_scale=s[2], bias=(b / s[2]).astype(F),
                            fold_out=True)
    got = c.dequantize(q, s[2])
    # tolerance of the reference's GPU e2e test: atol = output scale (test_quantization.py:408)
    assert np.abs(got - y).max() <= s[2] * 1.0001
    # and in fact exact on this fixture
    assert (got == y).mean() > 0.999
    # x86 form (torch.equal is what the reference's x86 test demands, testing_base.py:187-190)
    q86 = c.qgemm_x86(acc, float(s[0]), np.atleast_1d(s[1]), float(s[2]), b)
    assert np.abs(c.dequantize(q86, s[2]) - y).max() <= s[2] * 1.0001
    del lin


def test_torch_quant_observer_scales(golden):
    # observer.py:146-149: symmetric scale = max(|min|, |max|) / ((qmax - qmin) / 2) = amax / 127.5
    x = golden["tq_calib"]
    amax = np.abs(x).max().astype(F)
    assert np.allclose(golden["tq_s_x"], amax / F(127.5), rtol=1e-6)
    w1 = golden["tq_w1"]
    assert np.allclose(golden["tq_s_w1"], np.abs(w1).max(axis=1) / F(127.5), rtol=1e-6)


def test_torch_quant_mlp_golden(golden):
    """The reference's quantized MLP (observers in fake-quant mode) replayed as int8."""
    g = golden
    x, w1, b1, w2, b2 = g["tq_x"], g["tq_w1"], g["tq_b1"], g["tq_w2"], g["tq_b2"]
    s_x, s_h, s_g, s_y = g["tq_s_x"], g["tq_s_h"], g["tq_s_g"], g["tq_s_y"]
    s_w1, s_w2 = g["tq_s_w1"], g["tq_s_w2"]
    xq = c.quantize(x, s_x)
    w1q = c.quantize(w1, s_w1, axis=0)
    w2q = c.quantize(w2, s_w2, axis=0)
    acc1 = c.qgemm_acc(xq, w1q)
    # fc1 -> quantize at s_h (the fc1 output observer)
    _, hq = c.qgemm_epilogue(acc1, x_scale=s_x, w_scale=s_w1, out_scale=s_h, bias=b1, div_out=True)
    h_pre = c.dequantize(hq, s_h)
    assert np.abs(h_pre - g["tq_h_pre"]).max() <= s_h[0] * 1.0001
    # gelu on the dequantized value, re-quantized at s_g
    gq = c.quantize(np_ref.gelu(h_pre), s_g)
    assert np.abs(c.dequantize(gq, s_g) - g["tq_h_act"]).max() <= s_g[0] * 1.0001 + s_h[0]
    acc2 = c.qgemm_acc(gq, w2q)
    _, yq = c.qgemm_epilogue(acc2, x_scale=s_g, w_scale=s_w2, out_scale=s_y, bias=b2, div_out=True)
    y = c.dequantize(yq, s_y)
    # end to end: a few output LSBs (errors of one LSB upstream propagate)
    assert np.abs(y - g["tq_y"]).max() <= 3 * s_y[0]
    assert np.abs(y - g["tq_y"]).mean() <= 0.25 * s_y[0]


def test_onednn_int8_linear(golden):
    """oneDNN (the library behind the reference's x86 call) vs the restatement: <= 1 LSB."""
    if "onednn_y" not in golden.files:
        pytest.skip("fixture generated without the onednn op")
    a, w, sw, b, sc, y = [golden["onednn_" + k] for k in ("a", "w", "sw", "b", "scales", "y")]
    acc = c.qgemm_acc(a, w)
    _, q = c.qgemm_epilogue(acc, x_scale=sc[0], w_scale=sw, out_scale=sc[1], bias=b, div_out=True)
    assert np.abs(q.astype(int) - y.astype(int)).max() <= 1
    q86 = c.qgemm_x86(acc, float(sc[0]), sw, float(sc[1]), b)
    assert np.abs(q86.astype(int) - y.astype(int)).max() <= 1


def test_row_ops_against_eager_torch_golden(golden):
    g = golden
    y, _ = c.norm(g["ln_x"], g["ln_gamma"], g["ln_beta"], eps=1e-5)
    # tolerance of the reference's op tests: rtol 1e-6, atol 1e-3 (testing_base.py:93-94)
    assert np.allclose(y, g["ln_y"], rtol=1e-6, atol=1e-3)
    assert np.allclose(np_ref.layernorm(g["ln_x"], g["ln_gamma"], g["ln_beta"]), g["ln_y"], rtol=1e-6, atol=1e-3)
    assert np.allclose(c.softmax(g["sm_x"]), g["sm_y"], rtol=1e-6, atol=1e-3)
    assert np.allclose(c.softmax(g["sm_x"], log=True), g["sm_logy"], rtol=1e-6, atol=1e-3)
    f, _ = c.qgemm_epilogue(np.zeros((5, 33), np.int32), bias=None, act="gelu")
    assert (f == 0).all()
    assert np.allclose(np_ref.gelu(g["gelu_x"]), g["gelu_y"], rtol=1e-6, atol=1e-3)


def test_softmax_lens_and_empty_rows():
    rng = np.random.default_rng(3)
    x = rng.standard_normal((3, 2, 5, 12)).astype(F)
    lens = np.array([12, 7, 0], dtype=np.int32)
    y = c.softmax(x, scale=0.5, lens=lens)
    assert np.allclose(y[0].sum(-1), 1.0, atol=1e-6)
    assert (y[1][..., 7:] == 0).all() and np.allclose(y[1].sum(-1), 1.0, atol=1e-6)
    assert np.allclose(y[1][..., :7], np_ref.softmax(x[1][..., :7], 0.5), atol=1e-6)


def test_rmsnorm_and_residual():
    rng = np.random.default_rng(4)
    x = rng.standard_normal((7, 64)).astype(F)
    r = rng.standard_normal((7, 64)).astype(F)
    gm = rng.standard_normal(64).astype(F)
    y, s = c.norm(x, gm, residual=r, eps=1e-6, rms=True)
    h = (x + r).astype(np.float64)
    want = h / np.sqrt((h * h).mean(-1, keepdims=True) + 1e-6) * gm
    assert np.allclose(y, want, rtol=1e-6, atol=1e-6)
    assert (s == x + r).all()


def test_decoder_glue_restatements():
    """The restatements behind the column-parallel decoder tests, pinned to their
    defining formulas in numpy / eager torch."""
    import torch
    rng = np.random.default_rng(4)
    g = (rng.standard_normal((9, 40)) * 3).astype(np.float32)
    u = (rng.standard_normal((9, 40)) * 3).astype(np.float32)
    q, s = c.gated_quantize(g, u)
    h = (g.astype(np.float64) / (1 + np.exp(-g.astype(np.float64))) * u).astype(np.float32)
    want_s = np.maximum(np.abs(h).max(axis=1) / np.float32(127), np.finfo(np.float32).eps).astype(np.float32)
    assert (s == want_s).all()
    assert (q == np.clip(np.rint(h / want_s[:, None]), -128, 127)).all()
    assert (q == torch.nn.functional.silu(torch.from_numpy(g).double()).mul(torch.from_numpy(u).double()).float()
            .div(torch.from_numpy(want_s)[:, None]).round().clamp(-128, 127).to(torch.int8).numpy()).all()
    q1, s1 = c.gated_quantize(g)
    q2, s2 = c.dynamic_quantize(g)
    assert (q1 == q2).all() and (s1 == s2).all()
    # rotary embedding against the eager elementwise form
    tokens, heads, dim = 6, 3, 16
    x = rng.standard_normal((tokens, heads, dim)).astype(np.float32)
    pos = np.array([0, 1, 5, 9, 2, 7])
    inv = 10000.0 ** (-np.arange(dim // 2, dtype=np.float32) / np.float32(dim // 2))
    ang = torch.arange(12, dtype=torch.float32)[:, None] * torch.from_numpy(inv.astype(np.float32))[None, :]
    cos_t, sin_t = ang.cos().numpy(), ang.sin().numpy()
    y = c.rope(x, pos, cos_t, sin_t)
    xt = torch.from_numpy(x)
    cs, sn = torch.from_numpy(cos_t)[pos][:, None, :], torch.from_numpy(sin_t)[pos][:, None, :]
    x1, x2 = xt[..., :dim // 2], xt[..., dim // 2:]
    want = torch.cat([x1 * cs - x2 * sn, x2 * cs + x1 * sn], dim=-1).numpy()
    assert (y == want).all()
    # the layout an all-gather of column shards leaves
    m = rng.integers(-128, 128, (5, 12), dtype=np.int8)
    lay = c.gathered_layout(m, 3)
    assert lay.shape == (3, 5, 4) and (lay[1] == m[:, 4:8]).all()
    assert (lay.transpose(1, 0, 2).reshape(5, 12) == m).all()


def test_weight_only_restatement_is_the_eager_model_the_reference_compiles():
    """F.linear over fake_quantize_per_channel_affine(weight, scale, 128, axis 0, 0, 255), the module of
    pytorch_blade/tests/disc/pdl/test_torchscipt_to_mhlo/test_quantization.py:501-618; the custom call
    receives the uint8 weight transposed to [K, N], the scales and the zero points."""
    import torch
    import torch.nn.functional as F
    torch.manual_seed(0)
    for (m, k, n, with_bias) in ((2, 3, 5, False), (2, 3, 5, True), (7, 96, 40, True), (1, 300, 17, False)):
        weight = torch.randn(n, k)
        scale = torch.rand(n) * 0.02 + 0.005
        zp = torch.full((n,), 128, dtype=torch.int32)
        bias = torch.randn(n) if with_bias else None
        x = torch.randn(m, k)
        want = F.linear(x, torch.fake_quantize_per_channel_affine(weight, scale, zp, 0, 0, 255), bias).numpy()
        q = torch.clamp(torch.round(weight / scale[:, None]) + 128, 0, 255).to(torch.uint8)     # [N, K]
        got = c.weight_only_qgemm(x.numpy(), q.t().contiguous().numpy(), scale.numpy(), zp.numpy(),
                                  None if bias is None else bias.numpy())
        bound = (np.abs(x.numpy()) @ np.abs(q.t().numpy().astype(np.float32) - 128)) * scale.numpy()
        assert np.all(np.abs(got - want) <= 2e-6 * bound + 1e-6)
    # zero points other than 128 and a missing zero point
    rng = np.random.default_rng(2)
    x = rng.standard_normal((3, 33)).astype(np.float32)
    w = rng.integers(0, 256, (33, 12), dtype=np.uint8)
    s = (rng.random(12) * 0.1).astype(np.float32)
    z = rng.integers(0, 256, 12).astype(np.int32)
    want = (x.astype(np.float64) @ (w.astype(np.float64) - z)) * s
    assert np.allclose(c.weight_only_qgemm(x, w, s, z), want, rtol=1e-6, atol=1e-6)
    assert np.allclose(c.weight_only_qgemm(x, w, s), (x.astype(np.float64) @ w.astype(np.float64)) * s, rtol=1e-6)


def test_observer_restatement_matches_the_reference_observers():
    """oracle/np_ref.py against tests/golden/observer_golden.npz, which holds what the reference's own
    MinMaxObserver / PerChannelMinMaxObserver computed (tests/golden/make_observer_golden.py)."""
    from pathlib import Path
    from oracle import np_ref
    g = np.load(Path(__file__).parent / "golden" / "observer_golden.npz")
    schemes = {"sym": (-128, 127, True, 0), "affine": (0, 255, False, 0), "affine_s8": (-128, 127, False, 0)}
    for tag, (qmin, qmax, sym, szp) in schemes.items():
        lo, hi = np_ref.observe_minmax(list(g["act_batches"]))
        assert (lo == g[f"act_{tag}_min"]).all() and (hi == g[f"act_{tag}_max"]).all()
        s, z = np_ref.minmax_qparams(lo, hi, qmin, qmax, sym, szp)
        assert (s == g[f"act_{tag}_scale"]).all() and (z == g[f"act_{tag}_zp"]).all()
    lo, hi = np_ref.observe_minmax([g["pos_x"]])
    s, z = np_ref.minmax_qparams(lo, hi, 0, 255, False)
    assert (s == g["pos_scale"]).all() and (z == g["pos_zp"]).all() and z[0] == 0      # range widened to zero
    for tag, key, axis, (qmin, qmax, sym) in (("w_ax0", "w", 0, (-128, 127, True)), ("w_ax1", "w", 1, (-128, 127, True)),
                                              ("k4_ax3", "k4", 3, (-128, 127, True)),
                                              ("w_ax0_affine", "w", 0, (0, 255, False))):
        t = g[key]
        lo, hi = np_ref.observe_minmax([t, t * np.float32(0.5) + np.float32(0.01)], ch_axis=axis)
        assert (lo == g[f"{tag}_min"]).all() and (hi == g[f"{tag}_max"]).all()
        s, z = np_ref.minmax_qparams(lo, hi, qmin, qmax, sym)
        assert (s == g[f"{tag}_scale"]).all() and (z == g[f"{tag}_zp"]).all()
    # and the scales the encoder goldens were calibrated with (same observers, other data)
    q = np.load(Path(__file__).parent / "golden" / "qpath_golden.npz")
    lo, hi = np_ref.observe_minmax(list(q["tq_calib"]))
    assert (np_ref.minmax_qparams(lo, hi)[0] == q["tq_s_x"]).all()
    lo, hi = np_ref.observe_minmax([q["tq_w1"]], ch_axis=0)
    assert (np_ref.minmax_qparams(lo, hi)[0] == q["tq_s_w1"]).all()


def test_attention_restatement_is_eager_torch_attention():
    """oracle/np_ref.py:attention_packed restates softmax(q k^T * scale) v; the reference has no single
    function for it (two library GEMMs and a generated softmax), so it is pinned to eager torch."""
    import torch
    rng = np.random.default_rng(3)
    lens, heads, d = [5, 33, 70], 3, 64
    qkv = rng.standard_normal((sum(lens), 3 * heads * d)).astype(np.float32)
    got = np_ref.attention_packed(qkv, lens, heads, 0.125)
    t0 = 0
    for n in lens:
        blk = torch.from_numpy(qkv[t0:t0 + n])
        q, k, v = (blk[:, i * heads * d:(i + 1) * heads * d].view(n, heads, d).transpose(0, 1) for i in range(3))
        want = torch.softmax(q @ k.transpose(-1, -2) * 0.125, dim=-1) @ v
        want = want.transpose(0, 1).reshape(n, heads * d).numpy()
        assert np.allclose(got[t0:t0 + n], want, rtol=1e-5, atol=1e-6)
        t0 += n
