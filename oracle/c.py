"""TEST INFRASTRUCTURE: ctypes wrapper of oracle/qpath_oracle.c (numpy in, numpy out).

Each wrapper names the C function it calls; the C source cites the reference
file:line that the function restates.
"""
import ctypes
import subprocess
from ctypes import POINTER, c_float, c_int, c_int8, c_int32, c_int64, c_void_p
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_SO = _HERE / "_build" / "libqpath_oracle.so"
_lib = None

SCALE_NONE, SCALE_SCALAR, SCALE_PER_COL, SCALE_PER_ROW = 0, 1, 2, 3
BIAS_NONE, BIAS_F32, BIAS_I8 = 0, 1, 2
ACT = {None: 0, "none": 0, "gelu": 1, "silu": 2}


def build() -> Path:
    """Compiles the C restatement (gcc) if it is missing or stale."""
    src = _HERE / "qpath_oracle.c"
    if not _SO.exists() or _SO.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE)], check=True, stdout=subprocess.DEVNULL)
    return _SO


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(str(build()))
    return _lib


def _f32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


def _i32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.int32)


def _ptr(a):
    return None if a is None else a.ctypes.data_as(c_void_p)


def _axis_view(shape, axis):
    if axis is None:
        return 1, 1
    axis = axis % len(shape)
    inner = int(np.prod(shape[axis + 1:], dtype=np.int64))
    return int(shape[axis]), inner


def quantize(x, scale, zero_point=None, axis=None, qmin=-128, qmax=127):
    """oracle_quantize_f32"""
    x = _f32(x)
    scale = _f32(np.atleast_1d(scale))
    zp = _i32(np.atleast_1d(zero_point)) if zero_point is not None else None
    ch, inner = _axis_view(x.shape, axis if scale.size > 1 else None)
    q = np.empty(x.shape, dtype=np.int8)
    lib().oracle_quantize_f32(_ptr(x), c_int64(x.size), _ptr(scale), _ptr(zp), c_int64(ch), c_int64(inner),
                              c_int32(qmin), c_int32(qmax), _ptr(q))
    return q


def dequantize(q, scale, zero_point=None, axis=None):
    """oracle_dequantize_f32"""
    q = np.ascontiguousarray(q, dtype=np.int8)
    scale = _f32(np.atleast_1d(scale))
    zp = _i32(np.atleast_1d(zero_point)) if zero_point is not None else None
    ch, inner = _axis_view(q.shape, axis if scale.size > 1 else None)
    y = np.empty(q.shape, dtype=np.float32)
    lib().oracle_dequantize_f32(_ptr(q), c_int64(q.size), _ptr(scale), _ptr(zp), c_int64(ch), c_int64(inner),
                                _ptr(y))
    return y


def quantize_weight(w, scale, zero_point=None, per_channel=True, qmin=-128, qmax=127):
    """oracle_quantize_weight_f64"""
    w = _f32(w)
    scale = _f32(np.atleast_1d(scale))
    zp = _i32(np.atleast_1d(zero_point)) if zero_point is not None else None
    q = np.empty(w.shape, dtype=np.int8)
    lib().oracle_quantize_weight_f64(_ptr(w), c_int64(w.shape[0]), c_int64(w.shape[1]), _ptr(scale), _ptr(zp),
                                     c_int(1 if per_channel else 0), c_int32(qmin), c_int32(qmax), _ptr(q))
    return q


def fake_quant(x, scale, zero_point=None, axis=None, qmin=-128, qmax=127):
    """oracle_fake_quant_f32"""
    x = _f32(x)
    scale = _f32(np.atleast_1d(scale))
    zp = _i32(np.atleast_1d(zero_point)) if zero_point is not None else None
    ch, inner = _axis_view(x.shape, axis if scale.size > 1 else None)
    y = np.empty(x.shape, dtype=np.float32)
    lib().oracle_fake_quant_f32(_ptr(x), c_int64(x.size), _ptr(scale), _ptr(zp), c_int64(ch), c_int64(inner),
                                c_int32(qmin), c_int32(qmax), _ptr(y))
    return y


def qgemm_acc(a, w):
    """oracle_qgemm_acc: int32 a[M,K] . w[N,K]^T"""
    a = np.ascontiguousarray(a, dtype=np.int8)
    w = np.ascontiguousarray(w, dtype=np.int8)
    K = w.shape[1]
    a2 = a.reshape(-1, K)
    acc = np.empty((a2.shape[0], w.shape[0]), dtype=np.int32)
    lib().oracle_qgemm_acc(_ptr(a2), _ptr(w), c_int64(a2.shape[0]), c_int64(w.shape[0]), c_int64(K), _ptr(acc))
    return acc.reshape(a.shape[:-1] + (w.shape[0],))


def _kind(s, rows, cols, is_x, x_per_col=False):
    if s is None:
        return SCALE_NONE
    if s.size == 1:
        return SCALE_SCALAR
    if is_x and not x_per_col:
        assert s.size == rows
        return SCALE_PER_ROW
    assert s.size == cols
    return SCALE_PER_COL


def qgemm_epilogue(acc, x_scale=None, w_scale=None, out_scale=None, bias=None, fold_out=False,
                   div_out=False, act=None, x_per_col=False):
    """oracle_qgemm_epilogue: returns (float32 values, int8 values)."""
    acc = np.ascontiguousarray(acc, dtype=np.int32)
    N = acc.shape[-1]
    acc2 = acc.reshape(-1, N)
    M = acc2.shape[0]
    xs = _f32(np.atleast_1d(x_scale)) if x_scale is not None else None
    ws = _f32(np.atleast_1d(w_scale)) if w_scale is not None else None
    os_ = _f32(np.atleast_1d(out_scale)) if out_scale is not None else None
    bias_kind = BIAS_NONE
    b = None
    if bias is not None:
        b = np.ascontiguousarray(bias)
        if b.dtype == np.int8:
            bias_kind = BIAS_I8
        else:
            b = _f32(b)
            bias_kind = BIAS_F32
    of = np.empty((M, N), dtype=np.float32)
    oi = np.empty((M, N), dtype=np.int8)
    lib().oracle_qgemm_epilogue(_ptr(acc2), c_int64(M), c_int64(N), _ptr(xs), c_int(_kind(xs, M, N, True, x_per_col)),
                                _ptr(ws), c_int(_kind(ws, M, N, False)), _ptr(os_),
                                c_int(_kind(os_, M, N, False)), _ptr(b), c_int(bias_kind),
                                c_int(1 if fold_out else 0), c_int(1 if div_out else 0), c_int(ACT[act]),
                                _ptr(of), _ptr(oi))
    return of.reshape(acc.shape), oi.reshape(acc.shape)


def qgemm_x86(acc, s_x, s_w, s_out, bias=None):
    """oracle_qgemm_x86"""
    acc = np.ascontiguousarray(acc, dtype=np.int32)
    N = acc.shape[-1]
    acc2 = acc.reshape(-1, N)
    ws = _f32(np.atleast_1d(s_w))
    b = _f32(bias) if bias is not None else None
    out = np.empty(acc2.shape, dtype=np.int8)
    lib().oracle_qgemm_x86(_ptr(acc2), c_int64(acc2.shape[0]), c_int64(N), c_float(s_x), _ptr(ws),
                           c_int(1 if ws.size > 1 else 0), c_float(s_out), _ptr(b), _ptr(out))
    return out.reshape(acc.shape)


def qgemm_ral_i8(a, w, s_x, s_w, s_out, bias=None):
    """oracle_qgemm_ral_i8 (product + ral_pdll_qgemm epilogue in one, OpenMP when built with it)."""
    a = np.ascontiguousarray(a, dtype=np.int8)
    w = np.ascontiguousarray(w, dtype=np.int8)
    K = w.shape[1]
    a2 = a.reshape(-1, K)
    ws = _f32(np.atleast_1d(s_w))
    b = _f32(bias) if bias is not None else None
    out = np.empty((a2.shape[0], w.shape[0]), dtype=np.int8)
    lib().oracle_qgemm_ral_i8(_ptr(a2), _ptr(w), c_int64(a2.shape[0]), c_int64(w.shape[0]), c_int64(K),
                              c_float(s_x), _ptr(ws), c_int(1 if ws.size > 1 else 0), c_float(s_out),
                              _ptr(b), _ptr(out))
    return out.reshape(a.shape[:-1] + (w.shape[0],))


def dynamic_quantize(x):
    """oracle_dynamic_quantize_f32: returns (q, row_scale)."""
    x = _f32(x)
    cols = x.shape[-1]
    x2 = x.reshape(-1, cols)
    q = np.empty(x2.shape, dtype=np.int8)
    s = np.empty(x2.shape[0], dtype=np.float32)
    lib().oracle_dynamic_quantize_f32(_ptr(x2), c_int64(x2.shape[0]), c_int64(cols), _ptr(q), _ptr(s))
    return q.reshape(x.shape), s


def norm(x, gamma, beta=None, residual=None, eps=1e-5, rms=False):
    """oracle_norm_f32: returns (y, x + residual)."""
    x = _f32(x)
    cols = x.shape[-1]
    x2 = x.reshape(-1, cols)
    r = _f32(residual).reshape(-1, cols) if residual is not None else None
    g = _f32(gamma)
    b = _f32(beta) if beta is not None else None
    y = np.empty(x2.shape, dtype=np.float32)
    s = np.empty(x2.shape, dtype=np.float32)
    lib().oracle_norm_f32(_ptr(x2), _ptr(r), _ptr(g), _ptr(b), c_int64(x2.shape[0]), c_int64(cols), c_float(eps),
                          c_int(1 if rms else 0), _ptr(y), _ptr(s))
    return y.reshape(x.shape), s.reshape(x.shape)


def softmax(x, scale=1.0, lens=None, mask=None, log=False):
    """oracle_softmax_f32: lens / mask are per index of the leading axis."""
    x = _f32(x)
    cols = x.shape[-1]
    x2 = x.reshape(-1, cols)
    rows = x2.shape[0]
    rpb = rows
    ln = None
    mk = None
    if lens is not None:
        ln = _i32(lens)
        rpb = rows // x.shape[0]
    if mask is not None:
        mk = _f32(mask).reshape(-1, cols)
        rpb = rows // x.shape[0]
    y = np.empty(x2.shape, dtype=np.float32)
    lib().oracle_softmax_f32(_ptr(x2), c_int64(rows), c_int64(cols), c_int64(rpb), _ptr(ln), _ptr(mk),
                             c_float(scale), c_int(1 if log else 0), _ptr(y))
    return y.reshape(x.shape)


def gated_quantize(gate, up=None):
    """oracle_gated_quantize_f32: (q int8, row_scale) of silu(gate) * up (of gate without up)."""
    g = _f32(gate)
    u = _f32(up)
    rows, cols = g.shape
    q = np.empty((rows, cols), dtype=np.int8)
    s = np.empty(rows, dtype=np.float32)
    lib().oracle_gated_quantize_f32(_ptr(g), _ptr(u), c_int64(rows), c_int64(cols), c_int64(cols), _ptr(q), _ptr(s))
    return q, s


def rope(x, pos, cos_t, sin_t):
    """oracle_rope_f32: x [tokens, heads, dim], pos [tokens], tables [positions, dim / 2]."""
    x = _f32(x)
    tokens, heads, dim = x.shape
    p = np.ascontiguousarray(pos, dtype=np.int64)
    y = np.empty_like(x)
    lib().oracle_rope_f32(_ptr(x), _ptr(p), _ptr(_f32(cos_t)), _ptr(_f32(sin_t)), c_int64(tokens), c_int64(heads),
                          c_int64(dim), _ptr(y))
    return y


def gathered_layout(x, ranks):
    """oracle_gathered_layout: row-major [rows, cols] -> [ranks, rows, cols / ranks]."""
    x = np.ascontiguousarray(x)
    rows, cols = x.shape
    out = np.empty((ranks, rows, cols // ranks), dtype=x.dtype)
    lib().oracle_gathered_layout(_ptr(x), c_int64(rows), c_int64(cols), c_int64(ranks), c_int64(x.itemsize), _ptr(out))
    return out


def weight_only_qgemm(x, w, scale, zp=None, bias=None):
    """oracle_weight_only_qgemm_f32: x [M, K] float, w uint8 [K, N], scale / bias [N], zp int32 [N] -> float32 [M, N]."""
    x = _f32(x)
    w = np.ascontiguousarray(w, dtype=np.uint8)
    m, k = x.shape
    n = w.shape[1]
    z = None if zp is None else np.ascontiguousarray(zp, dtype=np.int32)
    out = np.empty((m, n), dtype=np.float32)
    lib().oracle_weight_only_qgemm_f32(_ptr(x), _ptr(w), _ptr(_f32(scale)), _ptr(z), _ptr(_f32(bias)), c_int64(m),
                                       c_int64(n), c_int64(k), _ptr(out))
    return out


def conv2d_roles(data_format, input_shape, weight_shape, strides, dilations, padding):
    """Geometry of a convolution by role for ``qconv2d``: input in ``data_format`` ("NHWC" | "NCHW"),
    kernel [out, y, x, in], ``strides`` / ``dilations`` = (y, x), ``padding`` = (top, bottom, left, right).
    Returns (dims9, x_stride4, w_stride4, o_stride4, conv8, output_shape)."""
    def dense(shape):
        st, s = [0] * 4, 1
        for i in range(3, -1, -1):
            st[i] = s
            s *= shape[i]
        return st
    pos = {ch: data_format.index(ch) for ch in "NCHW"}
    n, c = input_shape[pos["N"]], input_shape[pos["C"]]
    h, w = input_shape[pos["H"]], input_shape[pos["W"]]
    o, kh, kw, ci = weight_shape
    assert ci == c
    (sh, sw), (dh, dw), (pt, pb, pl, pr) = strides, dilations, padding
    oh = (h + pt + pb - ((kh - 1) * dh + 1)) // sh + 1
    ow = (w + pl + pr - ((kw - 1) * dw + 1)) // sw + 1
    out_shape = [0] * 4
    out_shape[pos["N"]], out_shape[pos["C"]], out_shape[pos["H"]], out_shape[pos["W"]] = n, o, oh, ow
    xs, os_, ws = dense(input_shape), dense(out_shape), dense(weight_shape)
    role = lambda st: [st[pos["N"]], st[pos["C"]], st[pos["H"]], st[pos["W"]]]
    return ([n, c, h, w, o, kh, kw, oh, ow], role(xs), [ws[0], ws[3], ws[1], ws[2]], role(os_),
            [sh, sw, dh, dw, pt, pb, pl, pr], tuple(out_shape))


def qconv2d(x, w, x_scale, w_scale, out_scale, data_format="NHWC", strides=(1, 1), dilations=(1, 1),
            padding=(0, 0, 0, 0)):
    """oracle_qconv2d_s8: int8 input in ``data_format``, int8 kernel [out, y, x, in] -> int8 output in ``data_format``."""
    x = np.ascontiguousarray(x, dtype=np.int8)
    w = np.ascontiguousarray(w, dtype=np.int8)
    dims, xs, ws, os_, conv, out_shape = conv2d_roles(data_format, x.shape, w.shape, strides, dilations, padding)
    out = np.zeros(out_shape, dtype=np.int8)
    ws_arr = np.ascontiguousarray(np.atleast_1d(w_scale), dtype=np.float32)
    i64 = lambda v: np.ascontiguousarray(v, dtype=np.int64)
    a = [i64(dims), i64(xs), i64(ws), i64(os_), i64(conv)]
    lib().oracle_qconv2d_s8(_ptr(x), _ptr(w), _ptr(out), *[_ptr(v) for v in a], c_float(float(x_scale)), _ptr(ws_arr),
                            c_int(1 if ws_arr.size > 1 else 0), c_float(float(out_scale)))
    return out
