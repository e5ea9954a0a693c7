"""TEST INFRASTRUCTURE: numpy statement of the same formulas as qpath_oracle.c,
written independently so that tests can cross-check the C restatement.
All float arithmetic is float32 unless a formula says double."""
import math

import numpy as np

f32 = np.float32


def quantize(x, scale, zero_point=0, qmin=-128, qmax=127):
    """clamp(rne(x / scale + zp)), per-tensor or broadcastable scale
    (disc_lower_quantize_and_dequantize.cc:77-93 of the reference)."""
    x = np.asarray(x, dtype=f32)
    t = (x / np.asarray(scale, dtype=f32)).astype(f32) + np.asarray(zero_point, dtype=f32)
    t = np.rint(t.astype(f32))
    return np.clip(t, qmin, qmax).astype(np.int8)


def dequantize(q, scale, zero_point=0):
    """(q - zp) * scale (disc_lower_quantize_and_dequantize.cc:131-136)."""
    return ((q.astype(np.int32) - np.asarray(zero_point, dtype=np.int32)).astype(f32)
            * np.asarray(scale, dtype=f32)).astype(f32)


def fake_quant(x, scale, zero_point=0, qmin=-128, qmax=127):
    """torch.fake_quantize_*_affine: multiply by the reciprocal, nearbyint, clamp, scale back."""
    x = np.asarray(x, dtype=f32)
    s = np.asarray(scale, dtype=f32)
    inv = (f32(1.0) / s).astype(f32)
    t = np.rint((x * inv).astype(f32)) + np.asarray(zero_point, dtype=f32)
    t = np.clip(t, qmin, qmax)
    return ((t - np.asarray(zero_point, dtype=f32)).astype(f32) * s).astype(f32)


def qgemm_acc(a, w):
    """int32 a[M,K] . w[N,K]^T (exact in int64, then checked to fit int32)."""
    acc = a.astype(np.int64) @ w.astype(np.int64).T
    assert np.abs(acc).max() < 2 ** 31
    return acc.astype(np.int32)


def ral_epilogue(acc, s_x, s_w, s_out, bias=None):
    """sat_s8(rne(fma(acc, (s_x * s_w) / s_out, bias))): quantized_gpu_kernel_impl.cc:382,418-420.
    The fused multiply-add is done in double and rounded once, which equals fmaf
    for these magnitudes (|acc| < 2^31, one rounding)."""
    cs = ((np.asarray(s_x, dtype=f32) * np.asarray(s_w, dtype=f32)).astype(f32)
          / np.asarray(s_out, dtype=f32)).astype(f32)
    b = np.zeros(acc.shape[-1], dtype=f32) if bias is None else np.asarray(bias).astype(f32)
    v = (acc.astype(np.float64) * cs.astype(np.float64) + b.astype(np.float64)).astype(f32)
    return np.clip(np.rint(v), -128, 127).astype(np.int8)


def gelu(v):
    v = np.asarray(v, dtype=f32)
    erf = np.vectorize(math.erf)
    return (f32(0.5) * v * (f32(1.0) + erf((v * f32(0.70710678118654752440)).astype(np.float64)).astype(f32))).astype(f32)


def dynamic_quantize(x):
    x = np.asarray(x, dtype=f32)
    m = np.abs(x).max(axis=-1, keepdims=True)
    s = np.maximum((m / f32(127.0)).astype(f32), np.finfo(f32).eps).astype(f32)
    q = np.clip(np.rint((x / s).astype(f32)), -128, 127).astype(np.int8)
    return q, s.reshape(-1)


def layernorm(x, gamma, beta, eps=1e-5):
    x = np.asarray(x, dtype=np.float64)
    mean = x.mean(axis=-1, keepdims=True)
    var = ((x - mean) ** 2).mean(axis=-1, keepdims=True)
    return ((x - mean) / np.sqrt(var + eps) * gamma + beta).astype(f32)


def softmax(x, scale=1.0):
    x = (np.asarray(x, dtype=f32) * f32(scale)).astype(np.float64)
    e = np.exp(x - x.max(axis=-1, keepdims=True))
    return (e / e.sum(axis=-1, keepdims=True)).astype(f32)


def observe_minmax(batches, ch_axis=None):
    """Running range of MinMaxObserver (ch_axis None) / PerChannelMinMaxObserver after the batches
    (tools/torch_quant/torch_quant/observer.py:239-245, 262-285): float32 minimum and maximum, per channel
    over every other axis."""
    lo = hi = None
    for b in batches:
        b = np.asarray(b, dtype=np.float32)
        if ch_axis is None:
            mn, mx = b.min(keepdims=True).reshape(1), b.max(keepdims=True).reshape(1)
        else:
            axes = tuple(i for i in range(b.ndim) if i != ch_axis % b.ndim)
            mn, mx = b.min(axis=axes), b.max(axis=axes)
        lo = mn if lo is None else np.minimum(lo, mn)
        hi = mx if hi is None else np.maximum(hi, mx)
    return lo.astype(np.float32), hi.astype(np.float32)


def minmax_qparams(min_val, max_val, qmin=-128, qmax=127, symmetric=True, symmetric_zero_point=0):
    """Observer._calculate_qparams (observer.py:134-165) in float32: the range widened to include zero,
    scale floored at the float32 epsilon, affine zero point = clamp(qmin - rne(lo / scale))."""
    lo = np.minimum(np.asarray(min_val, np.float32), np.float32(0))
    hi = np.maximum(np.asarray(max_val, np.float32), np.float32(0))
    eps = np.finfo(np.float32).eps
    if symmetric:
        scale = np.maximum(np.maximum(-lo, hi) / np.float32((qmax - qmin) / 2), eps).astype(np.float32)
        zp = np.full(scale.shape, symmetric_zero_point, np.int32)
    else:
        scale = np.maximum((hi - lo) / np.float32(qmax - qmin), eps).astype(np.float32)
        zp = np.clip(qmin - np.rint(lo / scale).astype(np.int32), qmin, qmax).astype(np.int32)
    return scale, zp


def attention_packed(qkv, lens, heads, scale):
    """softmax(q k^T * scale) v per sequence and head over packed sequences, float32.

    qkv: [tokens, 3 * heads * d] (q | k | v), sequences one after the other.  This is the
    arithmetic of the chain the reference's compiled encoder runs for self-attention: a batched
    GEMM (ral_gemm, stream_executor_based_impl.cc:551-637), the row softmax its compiler
    generates (lhlo_legalize_roots_to_loops.cc:1263-1289, max-subtracted) and a second GEMM.
    No reference source states the chain as one function, so this restates the defining formula;
    tests pin it to eager torch."""
    qkv = np.asarray(qkv, dtype=f32)
    hidden = qkv.shape[1] // 3
    d = hidden // heads
    out = np.empty((qkv.shape[0], hidden), dtype=f32)
    t0 = 0
    for n in (int(v) for v in lens):
        blk = qkv[t0:t0 + n]
        for h in range(heads):
            q = blk[:, h * d:(h + 1) * d]
            k = blk[:, hidden + h * d:hidden + (h + 1) * d]
            v = blk[:, 2 * hidden + h * d:2 * hidden + (h + 1) * d]
            s = (q @ k.T).astype(f32) * f32(scale)
            s = s - s.max(axis=1, keepdims=True)
            p = np.exp(s).astype(f32)
            p = p / p.sum(axis=1, keepdims=True)
            out[t0:t0 + n, h * d:(h + 1) * d] = (p @ v).astype(f32)
        t0 += n
    return out


def histc(x, lo, hi, bins):
    """Counts per bin as torch.histc computes them on the CPU (aten/src/ATen/native/cpu/HistogramKernel.cpp,
    linear interpolation), which the reference's HistogramObserver calls once per batch
    (tools/torch_quant/torch_quant/observer.py:693,712): bin (int)((x - lo) * bins / (hi - lo)) in float32,
    the last bin includes hi; values outside [lo, hi] and NaN are skipped."""
    x = np.asarray(x, dtype=f32).reshape(-1)
    lo, hi = f32(lo), f32(hi)
    x = x[(x >= lo) & (x <= hi)]
    pos = (((x - lo).astype(f32) * f32(bins)).astype(f32) / f32(hi - lo)).astype(f32).astype(np.int64)
    pos[pos == bins] = bins - 1
    return np.bincount(pos, minlength=bins).astype(np.int64)[:bins]
