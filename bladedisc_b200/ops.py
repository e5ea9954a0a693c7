"""Operators of the quantized path on torch CUDA tensors.

Every function launches hand-written sm_100a kernels through the C ABI of
libdisc_b200_ral.so on torch's current stream.  torch is used for device
memory and streams only.  Nothing here computes on the CPU and nothing falls
back to torch operators.
"""
import ctypes
import math
from typing import Optional, Tuple

import torch

from . import lib as _lib

_ACT = {None: _lib.ACT_NONE, "none": _lib.ACT_NONE, "gelu": _lib.ACT_GELU, "silu": _lib.ACT_SILU}
_OUT = {torch.int8: _lib.OUT_I8, torch.float16: _lib.OUT_F16, torch.float32: _lib.OUT_F32,
        torch.int32: _lib.OUT_I32}
_PATH = {None: _lib.PATH_AUTO, "auto": _lib.PATH_AUTO, "tiled": _lib.PATH_TILED,
         "small_m": _lib.PATH_SMALL_M, "simt": _lib.PATH_SIMT, "pair": _lib.PATH_PAIR,
         "gemv": _lib.PATH_GEMV, "skinny": _lib.PATH_SKINNY}
_scratch = {}


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _cuda(t: torch.Tensor, name: str, dtype=None) -> torch.Tensor:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor: the quantized path has no CPU implementation")
    if dtype is not None and t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")
    return t.contiguous()


def _etype(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return _lib.F32
    if t.dtype == torch.float16:
        return _lib.F16
    raise TypeError(f"float32 or float16 expected, got {t.dtype}")


def qgemm_scratch(device: torch.device, nbytes: int) -> torch.Tensor:
    """Zero-initialised scratch of the small-M path, one per (device, stream)."""
    key = (device.index, _stream())
    buf = _scratch.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.zeros(max(nbytes, 8 << 20), dtype=torch.uint8, device=device)
        _scratch[key] = buf
    return buf


def _scale_kind(s: Optional[torch.Tensor], rows: int, cols: int, what: str, x_per_col: bool) -> int:
    if s is None:
        return _lib.SCALE_NONE
    if s.numel() == 1:
        return _lib.SCALE_SCALAR
    if what == "x" and not x_per_col:
        if s.numel() != rows:
            raise ValueError(f"x_scale has {s.numel()} entries; expected 1 or one per row ({rows})")
        return _lib.SCALE_PER_ROW
    if s.numel() != cols:
        raise ValueError(f"{what}_scale has {s.numel()} entries; expected 1 or one per channel ({cols})")
    return _lib.SCALE_PER_COL


def qgemm(a: torch.Tensor, w: torch.Tensor, *, x_scale: Optional[torch.Tensor] = None,
          w_scale: Optional[torch.Tensor] = None, out_scale: Optional[torch.Tensor] = None,
          bias: Optional[torch.Tensor] = None, act: Optional[str] = None,
          out_dtype: torch.dtype = torch.int8, fold_out_scale: bool = False,
          x_scale_per_col: bool = False, path: Optional[str] = None, split_k: int = 0,
          out: Optional[torch.Tensor] = None, a_gathered: bool = False,
          weights_static: bool = False, exact_division: bool = False) -> torch.Tensor:
    """out = epilogue(a[..., K] @ w[N, K]^T) with int8 operands and int32 accumulation.

    ``fold_out_scale=True`` is the reference custom call ``ral_pdll_qgemm``:
    ``sat_s8(rne(acc * (x_scale * w_scale / out_scale) + bias))``.  Otherwise
    ``v = act(acc * x_scale * w_scale + bias)`` and int8 output divides ``v`` by
    ``out_scale`` before rounding: as a product with the correctly rounded
    reciprocal (at most one int8 level from the quotient, at rounding ties only),
    or, with ``exact_division=True``, as the IEEE quotient the reference's
    quantize computes, bit for bit.  Scales and bias are device tensors.

    ``a_gathered=True``: ``a`` is ``[g, M, K / g]``, the buffer an all-gather of
    column-parallel outputs leaves (slab ``r`` holds columns ``r * K / g ...``);
    it is consumed in place, the result is ``[M, N]``.

    ``weights_static=True`` promises that ``w`` was final before the previous
    kernel on the stream was launched (inference weights): the few-row paths
    then fetch it while that kernel still runs.
    """
    if a_gathered:
        # a block of rows of a gathered buffer ([:, m0:m1, :]) is accepted as it is
        if not a.is_cuda or a.dtype != torch.int8:
            raise TypeError("a must be a CUDA int8 tensor")
        if a.dim() == 3 and (a.stride(2) != 1 or a.stride(1) != a.shape[2]):
            a = a.contiguous()
    else:
        a = _cuda(a, "a", torch.int8)
    w = _cuda(w, "w", torch.int8)
    if a_gathered:
        if a.dim() != 3 or w.dim() != 2 or a.shape[0] * a.shape[2] != w.shape[1]:
            raise ValueError(f"shape mismatch: gathered a {tuple(a.shape)} w {tuple(w.shape)}")
    elif w.dim() != 2 or a.shape[-1] != w.shape[1]:
        raise ValueError(f"shape mismatch: a {tuple(a.shape)} w {tuple(w.shape)}")
    K = w.shape[1]
    N = w.shape[0]
    M = a.numel() // K if K else 0
    out_shape = ((a.shape[1],) if a_gathered else tuple(a.shape[:-1])) + (N,)
    if out is None:
        out = torch.empty(out_shape, dtype=out_dtype, device=a.device)
    elif out.dtype != out_dtype or not out.is_contiguous() or out.numel() != M * N:
        raise ValueError("out must be a contiguous tensor of the result's dtype and size")
    if M == 0 or N == 0:
        return out
    args = _lib.QGemmArgs()
    args.a, args.w, args.out = a.data_ptr(), w.data_ptr(), out.data_ptr()
    args.M, args.N, args.K = M, N, K
    args.lda, args.ldw, args.ldo = K, K, N
    if a_gathered:
        args.a_slabs, args.a_slab_cols, args.a_slab_stride = a.shape[0], a.shape[2], a.stride(0)
        args.lda = a.shape[2]
    args.weights_static = 1 if weights_static else 0
    keep = []
    for name, t in (("x", x_scale), ("w", w_scale), ("out", out_scale)):
        if t is not None:
            t = _cuda(t, f"{name}_scale", torch.float32)
            keep.append(t)
        kind = _scale_kind(t, M, N, name, x_scale_per_col)
        setattr(args, f"{name}_scale", _p(t))
        setattr(args, f"{name}_scale_kind", kind)
    if bias is not None:
        bias = _cuda(bias, "bias")
        if bias.dtype == torch.float32:
            args.bias_kind = _lib.BIAS_F32
        elif bias.dtype == torch.int8:
            args.bias_kind = _lib.BIAS_I8
        else:
            raise TypeError("bias must be float32 or int8")
        if bias.numel() != N:
            raise ValueError("bias must have one entry per output channel")
        args.bias = bias.data_ptr()
    args.fold_out_scale = 1 if fold_out_scale else 0
    args.div_out_scale = 1 if (out_dtype == torch.int8 and out_scale is not None and not fold_out_scale) else 0
    args.div_exact = 1 if exact_division else 0
    args.act = _ACT[act]
    args.out_dtype = _OUT[out_dtype]
    args.path = _PATH[path]
    args.split_k = split_k
    L = _lib.load()
    if M <= 128:
        need = L.disc_b200_qgemm_scratch_bytes(M, N, K)
        ws = qgemm_scratch(a.device, need)
        args.splitk_ws = ws.data_ptr()
        args.splitk_ws_bytes = ws.numel()
    _lib.check(L.disc_b200_qgemm(ctypes.byref(args), _stream()))
    return out


def qgemm_path(M: int, N: int, K: int) -> str:
    """Which kernel path an aligned (M, N, K) problem takes."""
    args = _lib.QGemmArgs()
    args.a, args.w, args.out = 16, 16, 16
    args.M, args.N, args.K, args.lda, args.ldw, args.ldo = M, N, K, K, K, N
    code = _lib.load().disc_b200_qgemm_path(ctypes.byref(args))
    return {1: "tiled", 2: "small_m", 3: "simt", 4: "pair", 5: "gemv", 6: "skinny"}[code]


def quantize(x: torch.Tensor, scale: torch.Tensor, zero_point: Optional[torch.Tensor] = None,
             axis: Optional[int] = None, qmin: int = -128, qmax: int = 127) -> torch.Tensor:
    """q = clamp(rne(x / scale + zero_point), qmin, qmax) as int8 (static scales)."""
    x = _cuda(x, "x")
    scale = _cuda(scale, "scale", torch.float32)
    if zero_point is not None:
        zero_point = _cuda(zero_point, "zero_point", torch.int32)
    q = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    channels, inner = 1, 1
    if axis is not None and scale.numel() > 1:
        axis = axis % x.dim()
        channels = x.shape[axis]
        inner = 1
        for d in x.shape[axis + 1:]:
            inner *= d
        if scale.numel() != channels:
            raise ValueError("scale must have one entry per slice along axis")
    _lib.check(_lib.load().disc_b200_quantize(x.data_ptr(), _etype(x), q.data_ptr(), x.numel(),
                                              scale.data_ptr(), _p(zero_point), channels, inner,
                                              qmin, qmax, _stream()))
    return q


def dequantize(q: torch.Tensor, scale: torch.Tensor, zero_point: Optional[torch.Tensor] = None,
               axis: Optional[int] = None, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """y = (q - zero_point) * scale."""
    q = _cuda(q, "q", torch.int8)
    scale = _cuda(scale, "scale", torch.float32)
    if zero_point is not None:
        zero_point = _cuda(zero_point, "zero_point", torch.int32)
    y = torch.empty(q.shape, dtype=dtype, device=q.device)
    channels, inner = 1, 1
    if axis is not None and scale.numel() > 1:
        axis = axis % q.dim()
        channels = q.shape[axis]
        for d in q.shape[axis + 1:]:
            inner *= d
    _lib.check(_lib.load().disc_b200_dequantize(q.data_ptr(), y.data_ptr(), _etype(y), q.numel(),
                                                scale.data_ptr(), _p(zero_point), channels, inner,
                                                _stream()))
    return y


def dynamic_quantize(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-row symmetric int8: returns (q, row_scale) with row_scale = max|row| / 127."""
    x = _cuda(x, "x")
    cols = x.shape[-1]
    rows = x.numel() // cols if cols else 0
    q = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    s = torch.empty(rows, dtype=torch.float32, device=x.device)
    _lib.check(_lib.load().disc_b200_dynamic_quantize(x.data_ptr(), _etype(x), q.data_ptr(),
                                                      s.data_ptr(), rows, cols, _stream()))
    return q, s


def _norm(x, residual, gamma, beta, eps, rms, q_scale, want_y, want_sum, want_q, dynamic_q,
          x_gathered=False):
    x = _cuda(x, "x")
    gamma = _cuda(gamma, "gamma", x.dtype)
    a = _lib.NormArgs()
    if x_gathered:  # [g, rows, cols / g] column slabs
        if x.dim() != 3:
            raise ValueError("a gathered x is [g, rows, cols / g]")
        rows, cols = x.shape[1], x.shape[0] * x.shape[2]
        a.x_slab_cols, a.x_slab_stride = x.shape[2], x.shape[1] * x.shape[2]
        shape = (rows, cols)
    else:
        cols = x.shape[-1]
        rows = x.numel() // cols if cols else 0
        shape = tuple(x.shape)
    a.x = x.data_ptr()
    a.gamma = gamma.data_ptr()
    keep = [x, gamma]
    if residual is not None:
        residual = _cuda(residual, "residual", x.dtype)
        if tuple(residual.shape) != shape:
            raise ValueError("residual must have the shape of x")
        a.residual = residual.data_ptr()
        keep.append(residual)
    if beta is not None:
        beta = _cuda(beta, "beta", x.dtype)
        a.beta = beta.data_ptr()
        keep.append(beta)
    y = s = q = rs = None
    if want_y:
        y = torch.empty(shape, dtype=x.dtype, device=x.device)
        a.y = y.data_ptr()
    if want_sum:
        s = torch.empty(shape, dtype=x.dtype, device=x.device)
        a.sum_out = s.data_ptr()
    if want_q:
        q = torch.empty(shape, dtype=torch.int8, device=x.device)
        a.q_out = q.data_ptr()
        if dynamic_q:
            rs = torch.empty(rows, dtype=torch.float32, device=x.device)
            a.q_row_scale = rs.data_ptr()
        else:
            q_scale = _cuda(q_scale, "q_scale", torch.float32)
            a.q_scale = q_scale.data_ptr()
            keep.append(q_scale)
    a.rows, a.cols, a.eps, a.type, a.rms = rows, cols, eps, _etype(x), 1 if rms else 0
    _lib.check(_lib.load().disc_b200_norm(ctypes.byref(a), _stream()))
    return y, s, q, rs


def layernorm(x, gamma, beta, eps: float = 1e-5, residual=None) -> torch.Tensor:
    """LayerNorm(x [+ residual]) over the last axis."""
    return _norm(x, residual, gamma, beta, eps, False, None, True, False, False, False)[0]


def layernorm_quant(x, gamma, beta, q_scale, eps: float = 1e-5, residual=None):
    """LayerNorm(x [+ residual]) and its int8 copy at a static scale: (y, q)."""
    y, _, q, _ = _norm(x, residual, gamma, beta, eps, False, q_scale, True, False, True, False)
    return y, q


def rmsnorm(x, gamma, eps: float = 1e-6, residual=None, return_sum: bool = False, x_gathered: bool = False):
    """RMSNorm(x [+ residual]); with return_sum also x + residual."""
    y, s, _, _ = _norm(x, residual, gamma, None, eps, True, None, True, return_sum, False, False,
                       x_gathered=x_gathered)
    return (y, s) if return_sum else y


def rmsnorm_dynamic_quant(x, gamma, eps: float = 1e-6, residual=None, x_gathered: bool = False):
    """RMSNorm(x [+ residual]) quantized per row: (q, row_scale, x + residual or None).

    ``x_gathered``: x is ``[g, rows, cols / g]``, the buffer an all-gather of
    column-parallel outputs leaves; it is read in place."""
    _, s, q, rs = _norm(x, residual, gamma, None, eps, True, None, False, residual is not None, True, True,
                        x_gathered=x_gathered)
    return q, rs, s


def _gated(gate, up, q, row_scale, pass_):
    gate = _cuda_strided(gate, "gate")
    a = _lib.GatedQuantArgs()
    a.gate, a.ld = gate.data_ptr(), gate.stride(0)
    a.rows, a.cols, a.type, a.pass_ = gate.shape[0], gate.shape[1], _etype(gate), pass_
    if up is not None:
        up = _cuda_strided(up, "up")
        if up.shape != gate.shape or up.stride(0) != gate.stride(0) or up.dtype != gate.dtype:
            raise ValueError("up must match gate in shape, row stride and dtype")
        a.up = up.data_ptr()
    a.row_scale = row_scale.data_ptr()
    if q is not None:
        a.q, a.ldq = q.data_ptr(), q.stride(0)
    _lib.check(_lib.load().disc_b200_gated_quantize(ctypes.byref(a), _stream()))


def _cuda_strided(t: torch.Tensor, name: str) -> torch.Tensor:
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor: this library has no CPU path")
    if t.dim() != 2 or t.stride(1) != 1:
        raise ValueError(f"{name} must be 2-D with unit column stride")
    return t


def quantize_rows_whole(gate: torch.Tensor, up: Optional[torch.Tensor] = None,
                        out: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Both passes in one kernel for rows that are whole on this GPU: ``(q, row_scale)``."""
    s = torch.empty(gate.shape[0], dtype=torch.float32, device=gate.device)
    if out is None:
        out = torch.empty(gate.shape, dtype=torch.int8, device=gate.device)
    elif out.dtype != torch.int8 or tuple(out.shape) != tuple(gate.shape) or out.stride(1) != 1:
        raise ValueError("out must be int8 of gate's shape with unit column stride")
    _gated(gate, up, out, s, 2)
    return out, s


def row_scale_local(gate: torch.Tensor, up: Optional[torch.Tensor] = None) -> torch.Tensor:
    """First pass of the two-pass per-row quantization of ``h = silu(gate) * up``
    (``h = gate`` without ``up``): ``max(max|h[r, :]| / 127, eps)`` over the
    columns this GPU holds.  Rows may be strided views (column halves of one buffer)."""
    s = torch.empty(gate.shape[0], dtype=torch.float32, device=gate.device)
    _gated(gate, up, None, s, 0)
    return s


def quantize_rows(gate: torch.Tensor, row_scale: torch.Tensor, up: Optional[torch.Tensor] = None,
                  out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Second pass: ``sat(rne(h / row_scale[r]))`` into ``out`` (int8, may be a strided view)."""
    row_scale = _cuda(row_scale, "row_scale", torch.float32)
    if out is None:
        out = torch.empty(gate.shape, dtype=torch.int8, device=gate.device)
    elif out.dtype != torch.int8 or tuple(out.shape) != tuple(gate.shape) or out.stride(1) != 1:
        raise ValueError("out must be int8 of gate's shape with unit column stride")
    _gated(gate, up, out, row_scale, 1)
    return out


def weight_only_qgemm(x: torch.Tensor, w: torch.Tensor, scale: torch.Tensor, zero_point: Optional[torch.Tensor] = None,
                      bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                      path: Optional[str] = None) -> torch.Tensor:
    """``x @ ((w - zero_point) * scale) + bias`` with ``w`` uint8 ``[K, N]`` (the transposed
    weight the reference's pattern hands to ``ral_pdll_weight_only_qgemm``), ``scale`` /
    ``bias`` of ``x``'s dtype (float16 or float32) ``[N]``, ``zero_point`` int32 ``[N]``.
    Dequantization happens in the kernel; sums are fp32.  ``path``: None (by shape),
    "stream" or "tensor" (fp16, 16-byte aligned operands, N a multiple of 16)."""
    x = _cuda(x, "x")
    w = _cuda(w, "w", torch.uint8)
    if w.dim() != 2 or x.shape[-1] != w.shape[0]:
        raise ValueError("w must be [K, N] with K = x.shape[-1]")
    K, N = w.shape
    M = math.prod(x.shape[:-1])
    scale = _cuda(scale, "scale", x.dtype)
    if scale.numel() != N:
        raise ValueError("one scale per output column expected")
    if zero_point is not None:
        zero_point = _cuda(zero_point, "zero_point", torch.int32)
        if zero_point.numel() != N:
            raise ValueError("one zero point per output column expected")
    if bias is not None:
        bias = _cuda(bias, "bias", x.dtype)
        if bias.numel() != N:
            raise ValueError("one bias per output column expected")
    if out is None:
        out = torch.empty(x.shape[:-1] + (N,), dtype=x.dtype, device=x.device)
    elif out.dtype != x.dtype or not out.is_contiguous() or out.numel() != M * N:
        raise ValueError("out must be contiguous, of x's dtype and [..., N]")
    L = _lib.load()
    a = _lib.WeightOnlyQGemmArgs()
    a.x, a.w, a.scale, a.zero_point, a.bias, a.out = x.data_ptr(), w.data_ptr(), scale.data_ptr(), _p(zero_point), \
        _p(bias), out.data_ptr()
    a.m, a.n, a.k, a.ldx, a.ldw, a.ldo = M, N, K, K, N, N
    a.type = _etype(x)
    a.path = {None: 0, "stream": 1, "tensor": 2}[path]
    _lib.check(L.disc_b200_weight_only_qgemm(ctypes.byref(a), _stream()))
    return out


def qconv2d_plan(data_format: str, input_shape, weight_shape, strides=(1,), dilations=(1,), padding="VALID",
                 explicit_paddings=(), weight_is_const: bool = True):
    """(padding (top, bottom, left, right), result shape, metadata) of a quantized convolution from the
    attributes of ``ral_pdll_qconv2d``; host only."""
    L = _lib.load()
    arr = lambda v: (ctypes.c_int64 * max(len(v), 1))(*[int(i) for i in v])
    pad = (ctypes.c_int32 * 4)()
    res = (ctypes.c_int64 * 4)()
    meta = (ctypes.c_int32 * 17)()
    _lib.check(L.disc_b200_qconv2d_plan(data_format.encode(), arr(strides), len(strides), arr(dilations),
                                        len(dilations), padding.encode(), arr(explicit_paddings),
                                        len(explicit_paddings), 1 if weight_is_const else 0, arr(input_shape),
                                        arr(weight_shape), pad, res, meta))
    return tuple(pad), tuple(res), tuple(meta)


def qconv2d(x: torch.Tensor, w: torch.Tensor, x_scale: torch.Tensor, w_scale: torch.Tensor, out_scale: torch.Tensor,
            data_format: str = "NHWC", strides=(1,), dilations=(1,), padding="VALID",
            explicit_paddings=()) -> torch.Tensor:
    """int8 convolution ``sat(rne(conv(x, w) * (x_scale * w_scale / out_scale)))``: ``x`` int8 in ``data_format``,
    ``w`` int8 ``[out, y, x, in]``, scales float32 CUDA tensors (``w_scale``: one value or one per output
    channel); ``padding`` "SAME" | "VALID" | "EXPLICIT" with the reference's rules."""
    x = _cuda(x, "x", torch.int8)
    w = _cuda(w, "w", torch.int8)
    if x.dim() != 4 or w.dim() != 4:
        raise ValueError("rank-4 input and kernel expected")
    x_scale, w_scale, out_scale = (_cuda(t, n, torch.float32) for t, n in
                                   ((x_scale, "x_scale"), (w_scale, "w_scale"), (out_scale, "out_scale")))
    pad, res, meta = qconv2d_plan(data_format, x.shape, w.shape, strides, dilations, padding, explicit_paddings)
    out = torch.empty(res, dtype=torch.int8, device=x.device)
    if out.numel() == 0 or x.numel() == 0:
        return out
    if w_scale.numel() not in (1, w.shape[0]):
        raise ValueError("w_scale must hold one value or one per output channel")
    L = _lib.load()
    a = _lib.QConv2dArgs()
    a.x, a.w, a.out = x.data_ptr(), w.data_ptr(), out.data_ptr()
    a.input_sizes[:] = list(x.shape)
    a.kernel_sizes[:] = list(w.shape)
    a.output_sizes[:] = list(res)
    a.padding[:] = list(pad)
    a.metadata[:] = list(meta[:16])
    a.x_scale, a.w_scale, a.out_scale = x_scale.data_ptr(), w_scale.data_ptr(), out_scale.data_ptr()
    a.w_scale_per_channel = 1 if w_scale.numel() > 1 else 0
    need = L.disc_b200_qconv2d_workspace_bytes(ctypes.byref(a))
    if need < 0:
        raise ValueError("shapes, padding and metadata do not describe a convolution (one group only)")
    work = torch.empty(need, dtype=torch.uint8, device=x.device)
    rows = out.numel() // w.shape[0]
    kp = (w.shape[1] * w.shape[2] * w.shape[3] + 15) // 16 * 16
    ws = qgemm_scratch(x.device, L.disc_b200_qgemm_scratch_bytes(rows, w.shape[0], kp))
    a.workspace, a.workspace_bytes = work.data_ptr(), need
    a.splitk_ws, a.splitk_ws_bytes = ws.data_ptr(), ws.numel()
    _lib.check(L.disc_b200_qconv2d(ctypes.byref(a), _stream()))
    return out


def softmax(x: torch.Tensor, scale: float = 1.0, lens: Optional[torch.Tensor] = None,
            mask: Optional[torch.Tensor] = None, log: bool = False) -> torch.Tensor:
    """softmax(x * scale + mask) over the last axis.

    ``lens`` (int32, one per index of the leading axis) zeroes the columns at
    and beyond the length; ``mask`` ([leading, cols], dtype of x) is added.
    """
    x = _cuda(x, "x")
    cols = x.shape[-1]
    rows = x.numel() // cols if cols else 0
    y = torch.empty_like(x)
    rpb = rows
    if lens is not None:
        lens = _cuda(lens, "lens", torch.int32)
        if lens.numel() != x.shape[0]:
            raise ValueError("one length per index of the leading axis expected")
        rpb = rows // x.shape[0]
    if mask is not None:
        mask = _cuda(mask, "mask", x.dtype)
        if mask.numel() != x.shape[0] * cols:
            raise ValueError("mask must be [leading axis, cols]")
        rpb = rows // x.shape[0]
    _lib.check(_lib.load().disc_b200_softmax(x.data_ptr(), y.data_ptr(), _etype(x), rows, cols, rpb,
                                             _p(lens), _p(mask), float(scale), 1 if log else 0,
                                             _stream()))
    return y


def attention_blocks(lens, heads: int = 12, group: int = 1) -> torch.Tensor:
    """Work list of `attention` for sequences packed one after the other (host tensor, int32 [n, 4]): one row
    {first token of the sequence, length, first query row of the item, query blocks of the item} per item.
    An item is `group` (or, at the end of a sequence, fewer) consecutive blocks of 128 query rows of a
    sequence; its thread block fetches the sequence's keys and values once.  Which size is fastest depends on
    the batch: with many more items than SMs whole-sequence items win (34 vs 43 us on 32 sequences of up to
    512 tokens), on a few sequences one block per item does (9 vs 28 us on 4 sequences).  Longer items come
    first; the kernel starts all heads of an item before the next item."""
    lens = [int(v) for v in lens]
    for n in lens:
        if n < 1 or n > 512:
            raise ValueError(f"sequence length {n} outside 1..512")
    group = max(1, min(4, int(group)))
    rows = []
    tok0 = 0
    for n in lens:
        nblk = (n + 127) // 128
        for b0 in range(0, nblk, group):
            rows.append((tok0, n, b0 * 128, min(group, nblk - b0)))
        tok0 += n
    rows.sort(key=lambda r: -(r[1] * r[3]))
    return torch.tensor(rows, dtype=torch.int32).reshape(-1, 4)


def attention(qkv: torch.Tensor, blocks: torch.Tensor, heads: int, scale: float,
              out_scale: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """softmax(q k^T * scale) v per head over packed sequences, in one kernel.

    ``qkv``: f16 [tokens, 3 * heads * 64]; ``blocks``: device copy of ``attention_blocks(lens)``.
    Returns [tokens, heads * 64]: int8 quantized at ``out_scale`` (a device scalar), f16 without it."""
    qkv = _cuda(qkv, "qkv", torch.float16)
    if qkv.dim() != 2 or qkv.shape[1] != 3 * heads * 64:
        raise ValueError(f"qkv must be [tokens, {3 * heads * 64}], got {tuple(qkv.shape)}")
    if not blocks.is_cuda or blocks.dtype != torch.int32 or blocks.dim() != 2 or blocks.shape[1] != 4:
        raise ValueError("blocks must be a CUDA int32 [n, 4] tensor (see attention_blocks)")
    tokens = qkv.shape[0]
    hidden = heads * 64
    dtype = torch.int8 if out_scale is not None else torch.float16
    if out is None:
        out = torch.empty((tokens, hidden), dtype=dtype, device=qkv.device)
    elif out.dtype != dtype or tuple(out.shape) != (tokens, hidden) or not out.is_contiguous():
        raise ValueError("out must be a contiguous [tokens, hidden] tensor of the result's dtype")
    args = _lib.AttentionArgs()
    args.qkv, args.tokens, args.ld_qkv, args.heads = qkv.data_ptr(), tokens, qkv.shape[1], heads
    blocks = blocks.contiguous()
    args.blocks, args.num_blocks, args.scale = blocks.data_ptr(), blocks.shape[0], float(scale)
    args.out, args.ld_out = out.data_ptr(), hidden
    if out_scale is not None:
        out_scale = _cuda(out_scale, "out_scale", torch.float32)
        args.out_scale = out_scale.data_ptr()
    _lib.check(_lib.load().disc_b200_attention(ctypes.byref(args), _stream()))
    return out


def rope_kv_append(qkv: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, cos: torch.Tensor,
                   sin: torch.Tensor, batch: int, seq: int, pos0: int) -> None:
    """Rotates q and k inside ``qkv`` (fp16 ``[batch * seq, 3 * heads * dim]``, q in place) and
    appends the rotated k and v to the caches ``[batch, heads, cache_len, dim]`` at ``pos0``."""
    for t, n in ((qkv, "qkv"), (k_cache, "k_cache"), (v_cache, "v_cache")):
        if not t.is_cuda or t.dtype != torch.float16 or not t.is_contiguous():
            raise ValueError(f"{n} must be a contiguous CUDA fp16 tensor")
    heads, cache_len, dim = k_cache.shape[1], k_cache.shape[2], k_cache.shape[3]
    if qkv.numel() != batch * seq * 3 * heads * dim or k_cache.shape[0] != batch or v_cache.shape != k_cache.shape:
        raise ValueError("qkv / cache shapes disagree")
    cos, sin = _cuda(cos, "cos", torch.float32), _cuda(sin, "sin", torch.float32)
    if cos.shape[0] < pos0 + seq or cos.shape[1] != dim // 2 or sin.shape != cos.shape:
        raise ValueError("cos / sin tables must be [>= pos0 + seq, dim / 2]")
    _lib.check(_lib.load().disc_b200_rope_kv_append(qkv.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                                                    cos.data_ptr(), sin.data_ptr(), batch, seq, heads, dim, pos0,
                                                    cache_len, _stream()))


def kernel_status() -> int:
    """0 unless a kernel's bounded wait ran out since the last query (synchronises)."""
    return _lib.load().disc_b200_kernel_status()
