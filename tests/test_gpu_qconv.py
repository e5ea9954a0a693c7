"""Quantized 2-D convolution on B200 against the C oracle (bit exact) and the reference's known answers."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _f(v):
    return torch.tensor(np.atleast_1d(v), dtype=torch.float32, device="cuda")


CASES = [
    # data format, input shape, kernel (out, y, x), strides, dilations, padding, explicit, per-channel
    ("NHWC", (2, 9, 8, 32), (48, 3, 3), [1], [1], "SAME", (), True),            # 16-byte gather, channels-last output
    ("NHWC", (2, 9, 8, 32), (48, 3, 3), [1, 2, 2, 1], [1], "VALID", (), False),
    ("NHWC", (3, 11, 7, 25), (8, 3, 2), [2, 1], [1, 2], "EXPLICIT", (1, 2, 2, 0), True),   # K = 150: padded, packed kernel
    ("NHWC", (1, 5, 5, 3), (5, 5, 5), [1], [1], "SAME", (), True),              # window as large as the image
    ("NHWC", (1, 4, 4, 16), (16, 1, 1), [1], [1], "VALID", (), True),           # 16 rows: few-row linear
    ("NCHW", (2, 32, 9, 8), (24, 3, 3), [1], [1], "SAME", (), True),            # strided gather, scattered output
    ("NCHW", (2, 25, 8, 8), (8, 3, 3), [1, 1, 2, 2], [1, 1, 2, 2], "VALID", (), False),
    ("NHWC", (4, 28, 28, 64), (128, 3, 3), [1], [1], "SAME", (), True),         # 3136 rows x 576: tensor-core tiles
    ("NHWC", (4, 28, 28, 64), (128, 1, 1), [1], [1], "VALID", (), True),        # pointwise: the input is the matrix, no gather
    ("NHWC", (2, 14, 14, 48), (32, 1, 1), [1], [1], "SAME", (), False),         # pointwise, SAME (no padding for a 1 x 1 window)
    ("NHWC", (2, 14, 14, 64), (32, 1, 1), [1, 2, 2, 1], [1], "VALID", (), True),  # 1 x 1 with stride 2: gathered
    # multiples of 64 channels: the linear fetches its tiles from the image (TMA im2col), no gathered matrix
    ("NHWC", (2, 14, 14, 128), (32, 3, 3), [1], [1], "SAME", (), True),          # 392 rows: the last tile runs past the batch
    ("NHWC", (4, 16, 16, 256), (64, 3, 3), [1, 2, 2, 1], [1], "SAME", (), True),  # stride 2, two channel blocks per position
    ("NHWC", (2, 20, 20, 128), (16, 3, 3), [1], [1, 2, 2, 1], "VALID", (), False),  # dilation 2
    ("NHWC", (3, 12, 10, 128), (48, 3, 2), [1, 2, 1, 1], [1], "EXPLICIT", (2, 1, 0, 1), True),  # uneven padding and strides
    ("NHWC", (2, 16, 16, 128), (32, 1, 1), [1, 2, 2, 1], [1], "VALID", (), True),  # 1 x 1 with stride 2, from the image
    ("NHWC", (2, 14, 14, 64), (32, 3, 3), [1], [1], "SAME", (), True),           # 64 channels: K blocks of 64 bytes
    ("NHWC", (2, 13, 11, 192), (24, 3, 3), [1, 2, 2, 1], [1], "SAME", (), False),  # 192 channels: three 64-byte blocks per position
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: f"{c[0]}-{'x'.join(map(str, c[1]))}-{c[5]}")
def test_matches_oracle(case):
    from bladedisc_b200 import ops
    from oracle import c
    fmt, in_shape, (o, ky, kx), strides, dilations, padding, explicit, per_channel = case
    rng = np.random.default_rng(sum(in_shape) + o)
    ci = in_shape[3] if fmt == "NHWC" else in_shape[1]
    x = rng.integers(-128, 128, in_shape, dtype=np.int8)
    w = rng.integers(-128, 128, (o, ky, kx, ci), dtype=np.int8)
    sw = (rng.random(o if per_channel else 1) * 4e-3 + 1e-3).astype(np.float32)
    s_x, s_out = np.float32(0.02), np.float32(0.11)
    pad, res, meta = ops.qconv2d_plan(fmt, in_shape, w.shape, strides, dilations, padding, explicit)
    want = c.qconv2d(x, w, s_x, sw, s_out, fmt, meta[12:14], meta[14:16], pad)
    assert want.shape == tuple(res) and np.abs(want).max() > 5 and (np.abs(want) < 127).any()
    got = ops.qconv2d(_dev(x), _dev(w), _f(s_x), _f(sw), _f(s_out), fmt, strides, dilations, padding, explicit)
    assert tuple(got.shape) == tuple(res)
    assert (got.cpu().numpy() == want).all()


def test_known_answers_through_the_custom_calls():
    """-0.6 * -0.8 over 3 x 3 x 25 = 108, over 1 x 1 x 25 = 12
    (tao_compiler/mlir/disc/tests/pdll/quantized_conv2d.cc:24-215), once through ral_pdll_qconv2d with the
    attributes of the pattern and once through ral_qconv with padding / metadata operands."""
    from bladedisc_b200 import ops
    from bladedisc_b200.ral import MemRefSpec, RalContext, RalError
    from test_qconv_plan import KATS, S_OUT, S_W, S_X, kat_operands
    with RalContext() as ral:
        zero = torch.zeros((), dtype=torch.int32, device="cuda")
        zeros8 = torch.zeros(8, dtype=torch.int32, device="cuda")
        sx, so = torch.tensor(S_X, device="cuda"), torch.tensor(S_OUT, device="cuda")
        sw = torch.full((8,), float(S_W), device="cuda")
        for fmt, in_shape, kyx, strides, dilations, padding, x_val, out_shape, want in KATS:
            xq, wq = kat_operands(fmt, in_shape, kyx, x_val)
            attrs = ral.attr_blob({"data_format": fmt, "strides": list(strides), "dilations": list(dilations),
                                   "padding": padding, "explicit_paddings": [], "weight_is_const": True})
            q = ral.call("ral_pdll_qconv2d", "gpu", [("pvoid", 0), _dev(xq), _dev(wq), sx, zero, sw, zeros8, so, zero,
                                                     ("pvoid", attrs)], [MemRefSpec("i8", 4)])
            assert tuple(q.shape) == out_shape and (q.float() * float(S_OUT) == want).all()
            ral.dealloc(q)
            # the library-call form: output preallocated, padding and metadata as host operands
            pad, res, meta = ops.qconv2d_plan(fmt, in_shape, wq.shape, strides, dilations, padding)
            out = torch.full(out_shape, 99, dtype=torch.int8, device="cuda")
            pad_h = torch.tensor(pad, dtype=torch.int32)
            meta_h = torch.tensor(meta[:16], dtype=torch.int32)
            ral.call("ral_qconv", "gpu", [("pvoid", 0), _dev(xq), _dev(wq), pad_h, sx, zero, sw, zeros8, so, zero, out,
                                          meta_h])
            assert (out.float() * float(S_OUT) == want).all()
        with pytest.raises(RalError, match="fail to generate paddings"):
            bad = ral.attr_blob({"data_format": "NHWC", "strides": [1], "dilations": [1], "padding": "FULL",
                                 "explicit_paddings": [], "weight_is_const": True})
            xq, wq = kat_operands("NHWC", (1, 2, 2, 25), (1, 1), -0.6)
            ral.call("ral_pdll_qconv2d", "gpu", [("pvoid", 0), _dev(xq), _dev(wq), sx, zero, sw, zeros8, so, zero,
                                                 ("pvoid", bad)], [MemRefSpec("i8", 4)])
        with pytest.raises(RalError, match="grouped convolution"):
            attrs = ral.attr_blob({"data_format": "NHWC", "strides": [1], "dilations": [1], "padding": "VALID",
                                   "explicit_paddings": [], "weight_is_const": True})
            ral.call("ral_pdll_qconv2d", "gpu", [("pvoid", 0), _dev(np.zeros((1, 4, 4, 8), np.int8)),
                                                 _dev(np.zeros((8, 1, 1, 4), np.int8)), sx, zero, sw, zeros8, so, zero,
                                                 ("pvoid", attrs)], [MemRefSpec("i8", 4)])


def test_empty_and_errors():
    from bladedisc_b200 import ops
    x = torch.zeros((0, 8, 8, 16), dtype=torch.int8, device="cuda")
    w = torch.zeros((4, 3, 3, 16), dtype=torch.int8, device="cuda")
    s = _f(1.0)
    assert ops.qconv2d(x, w, s, s, s).shape == (0, 6, 6, 4)
    with pytest.raises(ValueError, match="one group"):
        ops.qconv2d(torch.zeros((1, 8, 8, 16), dtype=torch.int8, device="cuda"),
                    torch.zeros((4, 3, 3, 8), dtype=torch.int8, device="cuda"), s, s, s)
    with pytest.raises(TypeError):
        ops.qconv2d(x.float(), w, s, s, s)
