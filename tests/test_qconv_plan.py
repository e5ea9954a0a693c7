"""Host-side geometry of the quantized convolution against the tables of the reference's own
self-check (tao_compiler/mlir/ral/context/common_context_impl_pdll.cc:140-305) and the oracle
against the known answers of tao_compiler/mlir/disc/tests/pdll/quantized_conv2d.cc.  No GPU."""
import ctypes
import itertools

import numpy as np
import pytest

from bladedisc_b200 import lib as L


def plan(fmt, strides, dilations, padding, explicit=(), input_sizes=(4, 16, 16, 25), weight_sizes=(8, 3, 3, 25),
         const=True):
    lib = L.load()
    arr = lambda v: (ctypes.c_int64 * max(len(v), 1))(*v)
    pad = (ctypes.c_int32 * 4)()
    res = (ctypes.c_int64 * 4)()
    meta = (ctypes.c_int32 * 17)()
    rc = lib.disc_b200_qconv2d_plan(fmt.encode(), arr(strides), len(strides), arr(dilations), len(dilations),
                                    padding.encode(), arr(explicit), len(explicit), 1 if const else 0, arr(input_sizes),
                                    arr(weight_sizes), pad, res, meta)
    if rc != 0:
        raise ValueError(lib.disc_b200_last_error_string().decode())
    return list(pad), list(res), list(meta)


STRIDES = [[1], [2, 2], [1, 2, 3, 1]]           # "strides1", "strides22", "strides1231" -> (1,1), (2,2), (2,3)
RESOLVED = [(1, 1), (2, 2), (2, 3)]


def test_metadata_table(built_lib):
    want = [
        [0, 3, 1, 2, 3, 0, 1, 2, 0, 3, 1, 2, 1, 1, 1, 1, 1], [0, 3, 1, 2, 3, 0, 1, 2, 0, 3, 1, 2, 1, 1, 2, 2, 1],
        [0, 3, 1, 2, 3, 0, 1, 2, 0, 3, 1, 2, 1, 1, 2, 3, 1], [0, 3, 1, 2, 3, 0, 1, 2, 0, 3, 1, 2, 2, 2, 1, 1, 1],
        [0, 3, 1, 2, 3, 0, 1, 2, 0, 3, 1, 2, 2, 2, 2, 2, 1], [0, 3, 1, 2, 3, 0, 1, 2, 0, 3, 1, 2, 2, 2, 2, 3, 1],
        [0, 3, 1, 2, 3, 0, 1, 2, 0, 3, 1, 2, 2, 3, 1, 1, 1], [0, 3, 1, 2, 3, 0, 1, 2, 0, 3, 1, 2, 2, 3, 2, 2, 1],
        [0, 3, 1, 2, 3, 0, 1, 2, 0, 3, 1, 2, 2, 3, 2, 3, 1]]
    got = [plan("NHWC", s, d, "VALID")[2] for s, d in itertools.product(STRIDES, STRIDES)]
    assert got == want
    # channels first: batch 0, channel 1, spatial 2, 3 (reorder check of the reference: [2, 3, 0, 1])
    assert plan("NCHW", [1], [1], "VALID", input_sizes=(4, 25, 16, 16))[2][:12] == [0, 1, 2, 3, 3, 0, 1, 2, 0, 1, 2, 3]
    assert plan("NHWC", [1], [1], "VALID", const=False)[2][16] == 0


def test_padding_and_result_shape_tables(built_lib):
    pads = [[1, 1, 1, 1], [0, 1, 0, 1], [0, 1, 1, 1], [2, 2, 2, 2], [1, 2, 1, 2], [1, 2, 2, 2], [2, 2, 3, 3], [1, 2, 2, 3],
            [1, 2, 3, 3]] + [[0, 0, 0, 0]] * 9
    shapes = [[4, 16, 16, 8], [4, 8, 8, 8], [4, 8, 6, 8], [4, 16, 16, 8], [4, 8, 8, 8], [4, 8, 6, 8], [4, 16, 16, 8],
              [4, 8, 8, 8], [4, 8, 6, 8], [4, 14, 14, 8], [4, 7, 7, 8], [4, 7, 5, 8], [4, 12, 12, 8], [4, 6, 6, 8],
              [4, 6, 4, 8], [4, 12, 10, 8], [4, 6, 5, 8], [4, 6, 4, 8]]
    i = 0
    for padding in ("SAME", "VALID"):
        for d in STRIDES:                                # dilations outer, strides inner, as the reference loops
            for s in STRIDES:
                p, r, _ = plan("NHWC", s, d, padding)
                assert p == pads[i] and r == shapes[i], (padding, s, d)
                i += 1
    explicit_shapes = [[4, 17, 21, 8], [4, 9, 11, 8], [4, 9, 7, 8], [4, 15, 19, 8], [4, 8, 10, 8], [4, 8, 7, 8],
                       [4, 15, 17, 8], [4, 8, 9, 8], [4, 8, 6, 8]]
    i = 0
    for d in STRIDES:
        for s in STRIDES:
            p, r, _ = plan("NHWC", s, d, "EXPLICIT", explicit=[0, 0, 1, 2, 3, 4, 0, 0])
            assert p == [1, 2, 3, 4] and r == explicit_shapes[i]
            i += 1
    assert plan("NHWC", [1], [1], "EXPLICIT", explicit=[1, 2, 3, 4])[0] == [1, 2, 3, 4]


def test_plan_errors(built_lib):
    for kwargs, msg in ((dict(fmt="NHW", strides=[1], dilations=[1], padding="VALID"), "spatial dims"),
                        (dict(fmt="NHWC", strides=[1, 1, 1], dilations=[1], padding="VALID"), "strides and dilations"),
                        (dict(fmt="NHWC", strides=[1], dilations=[0], padding="VALID"), "strides and dilations"),
                        (dict(fmt="NHWC", strides=[1], dilations=[1], padding="FULL"), "paddings"),
                        (dict(fmt="NHWC", strides=[1], dilations=[1], padding="EXPLICIT", explicit=[1, 2]), "explicit")):
        with pytest.raises(ValueError, match=msg):
            plan(**kwargs)


def test_workspace_query_rejects_bad_geometry(built_lib):
    lib = L.load()
    a = L.QConv2dArgs()
    a.input_sizes[:] = [16, 8, 8, 25]
    a.kernel_sizes[:] = [8, 3, 3, 25]
    a.output_sizes[:] = [16, 6, 6, 8]
    a.padding[:] = [0, 0, 0, 0]
    a.metadata[:] = [0, 3, 1, 2, 3, 0, 1, 2, 0, 3, 1, 2, 1, 1, 1, 1]
    rows, kp = 16 * 6 * 6, 240                      # 3 * 3 * 25 = 225 -> padded to 240
    assert lib.disc_b200_qconv2d_workspace_bytes(ctypes.byref(a)) == rows * kp + 8 * kp + 0 + (256 - (8 * kp) % 256) % 256
    a.output_sizes[:] = [16, 5, 6, 8]               # not what the convolution produces
    assert lib.disc_b200_qconv2d_workspace_bytes(ctypes.byref(a)) == -1
    a.output_sizes[:] = [16, 6, 6, 8]
    a.kernel_sizes[:] = [8, 3, 3, 5]                # 25 input channels over 5 per filter: groups
    assert lib.disc_b200_qconv2d_workspace_bytes(ctypes.byref(a)) == -1
    a.kernel_sizes[:] = [8, 3, 3, 25]
    a.metadata[0] = 3                               # not a permutation
    assert lib.disc_b200_qconv2d_workspace_bytes(ctypes.byref(a)) == -1


# (data format, input shape, kernel y x, attrs) -> expected value everywhere, from quantized_conv2d.cc:24-235
KATS = [("NHWC", (1, 2, 2, 25), (1, 1), [1, 1, 1, 1], [1, 1, 1, 1], "SAME", -0.6, (1, 2, 2, 8), 12.0),
        ("NHWC", (16, 8, 8, 25), (3, 3), [1, 1, 1, 1], [1, 1, 1, 1], "VALID", -0.6, (16, 6, 6, 8), 108.0),
        ("NHWC", (16, 8, 8, 25), (3, 3), [1, 2, 2, 1], [1, 2, 2, 1], "VALID", -0.6, (16, 2, 2, 8), 108.0),
        ("NHWC", (16, 8, 8, 25), (3, 3), [1, 2, 2, 1], [1, 1, 1, 1], "SAME", 0.0, (16, 4, 4, 8), 0.0),
        ("NCHW", (1, 25, 2, 2), (1, 1), [1, 1, 1, 1], [1, 1, 1, 1], "SAME", -0.6, (1, 8, 2, 2), 12.0),
        ("NCHW", (16, 25, 8, 8), (3, 3), [1, 1, 1, 1], [1, 1, 1, 1], "VALID", -0.6, (16, 8, 6, 6), 108.0),
        ("NCHW", (16, 25, 8, 8), (3, 3), [1, 1, 2, 2], [1, 1, 2, 2], "VALID", -0.6, (16, 8, 2, 2), 108.0),
        ("NCHW", (16, 25, 8, 8), (3, 3), [1, 1, 2, 2], [1, 1, 2, 2], "SAME", 0.0, (16, 8, 4, 4), 0.0)]
S_X, S_W, S_OUT = np.float32(8.333333e-3), np.float32(1.568627e-2), np.float32(1.0)


def kat_operands(fmt, in_shape, kyx, x_val):
    xq = np.full(in_shape, np.clip(np.rint(np.float32(x_val) / S_X), -128, 127), np.int8)
    wq = np.full((8,) + kyx + (25,), np.clip(np.rint(np.float32(-0.8) / S_W), -128, 127), np.int8)   # OHWI
    return xq, wq


@pytest.mark.parametrize("kat", KATS, ids=lambda k: f"{k[0]}-{k[1]}-{k[5]}")
def test_oracle_reproduces_the_reference_known_answers(built_lib, kat):
    from oracle import c
    fmt, in_shape, kyx, strides, dilations, padding, x_val, out_shape, want = kat
    pad, res, meta = plan(fmt, strides, dilations, padding, input_sizes=in_shape, weight_sizes=(8,) + kyx + (25,))
    assert tuple(res) == out_shape
    xq, wq = kat_operands(fmt, in_shape, kyx, x_val)
    q = c.qconv2d(xq, wq, S_X, np.full(8, S_W, np.float32), S_OUT, fmt, meta[12:14], meta[14:16], pad)
    assert q.shape == out_shape
    assert (q.astype(np.float32) * S_OUT == want).all()


def test_oracle_against_plain_numpy(built_lib):
    """Random operands, padding on all sides, per-channel scales: direct loops in numpy (NHWC and NCHW)."""
    from oracle import c
    rng = np.random.default_rng(0)
    x = rng.integers(-128, 128, (2, 7, 6, 5), dtype=np.int8)            # NHWC
    w = rng.integers(-128, 128, (4, 3, 2, 5), dtype=np.int8)            # OHWI
    sw = (rng.random(4) * 0.01 + 0.001).astype(np.float32)
    strides, dil, pad = (2, 1), (1, 2), (1, 2, 2, 0)
    q = c.qconv2d(x, w, 0.05, sw, 0.3, "NHWC", strides, dil, pad)
    xp = np.pad(x.astype(np.int64), ((0, 0), (pad[0], pad[1]), (pad[2], pad[3]), (0, 0)))
    oh, ow = q.shape[1], q.shape[2]
    want = np.zeros(q.shape, np.int8)
    for oy in range(oh):
        for ox in range(ow):
            patch = xp[:, oy * strides[0]: oy * strides[0] + (3 - 1) * dil[0] + 1: dil[0],
                       ox * strides[1]: ox * strides[1] + (2 - 1) * dil[1] + 1: dil[1], :]
            acc = np.einsum("nyxc,oyxc->no", patch, w.astype(np.int64))
            cs = (np.float32(0.05) * sw) / np.float32(0.3)
            want[:, oy, ox, :] = np.clip(np.rint(acc.astype(np.float32) * cs), -128, 127)
    assert (q == want).all()
    q2 = c.qconv2d(x.transpose(0, 3, 1, 2), w, 0.05, sw, 0.3, "NCHW", strides, dil, pad)
    assert (q2 == want.transpose(0, 3, 1, 2)).all()


def test_plan_equals_the_reference_functions_on_random_attributes(built_lib, ref_host):
    """The reference's own generateReorderDims / generateStrides / generateDilations / generatePadding /
    generateExplicitPaddings / generateMetadata / generateResultShape (compiled from its tree into the host
    oracle) against disc_b200_qconv2d_plan on a few thousand random attribute sets."""
    rng = np.random.default_rng(5)
    arr = lambda v: (ctypes.c_int64 * max(len(v), 1))(*[int(i) for i in v])
    checked = 0
    for _ in range(3000):
        fmt = ["NHWC", "NCHW"][rng.integers(2)]
        n, c, h, w = (int(rng.integers(1, 5)), int(rng.integers(1, 9)), int(rng.integers(1, 40)), int(rng.integers(1, 40)))
        in_sizes = (n, h, w, c) if fmt == "NHWC" else (n, c, h, w)
        kh, kw = int(rng.integers(1, 6)), int(rng.integers(1, 6))
        w_sizes = (int(rng.integers(1, 9)), kh, kw, c)
        form = int(rng.integers(3))
        pick = lambda: int(rng.integers(1, 4))
        def attr():
            a, b = pick(), pick()
            if form == 0:
                return [a]
            if form == 1:
                return [a, b]
            return [1, a, b, 1] if fmt == "NHWC" else [1, 1, a, b]
        strides, dilations = attr(), attr()
        padding = ["SAME", "VALID", "EXPLICIT"][rng.integers(3)]
        explicit = []
        if padding == "EXPLICIT":
            p4 = [int(v) for v in rng.integers(0, 4, 4)]
            explicit = p4 if rng.integers(2) else ([0, 0] + p4 + [0, 0] if fmt == "NHWC" else [0, 0, 0, 0] + p4)
        pad_r, res_r, meta_r = (ctypes.c_int32 * 4)(), (ctypes.c_int64 * 4)(), (ctypes.c_int32 * 17)()
        rc = ref_host.ref_conv_plan(fmt.encode(), arr(strides), len(strides), arr(dilations), len(dilations),
                                    padding.encode(), arr(explicit), len(explicit), 1, arr(in_sizes), arr(w_sizes), pad_r,
                                    res_r, meta_r)
        assert rc == 0
        pad, res, meta = plan(fmt, strides, dilations, padding, explicit, in_sizes, w_sizes)
        assert pad == list(pad_r) and meta == list(meta_r), (fmt, strides, dilations, padding, explicit)
        # (the shape formula is the reference's even where the window does not fit the image and it goes to
        # zero or below; the convolution call itself refuses such shapes)
        assert res == list(res_r), (fmt, in_sizes, w_sizes, strides, dilations, padding, explicit)
        checked += all(v > 0 for v in res_r)
    assert checked > 2000
