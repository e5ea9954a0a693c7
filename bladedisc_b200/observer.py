"""Calibration observers whose state lives on the GPU: the counterpart of the
reference's ``MinMaxObserver`` / ``PerChannelMinMaxObserver``
(tools/torch_quant/torch_quant/observer.py:230-297) for calibrating on the device
the model runs on.  ``observe`` folds a batch into the running range with one read
of the tensor, ``qparams`` derives scale and zero point by the reference's rules
(observer.py:134-165); nothing is copied to the host in between.
"""
import math
from typing import Optional, Tuple

import torch

from . import lib as _lib
from . import ops as _ops

# (qmin, qmax, zero point of the symmetric scheme)
_RANGES = {"qint8": (-128, 127, 0), "quint8": (0, 255, 128)}


class MinMaxObserver:
    """Per-tensor range; ``dtype`` "qint8" | "quint8", symmetric or affine."""

    def __init__(self, dtype: str = "qint8", symmetric: bool = True, device: Optional[torch.device] = None):
        if dtype not in _RANGES:
            raise ValueError(f"dtype must be one of {sorted(_RANGES)}")
        if symmetric and dtype != "qint8":
            raise ValueError("Symmetric quantization requires signed dtype.")  # as the reference (observer.py:108-109)
        self.dtype, self.symmetric = dtype, symmetric
        self.device = torch.device("cuda") if device is None else device
        self.ch_axis = -1
        self.min_val = torch.full((1,), math.inf, device=self.device)
        self.max_val = torch.full((1,), -math.inf, device=self.device)
        self._scratch = None

    def _view(self, x: torch.Tensor) -> Tuple[int, int, int]:
        return 1, 1, x.numel()

    def observe(self, x: torch.Tensor) -> torch.Tensor:
        """Folds ``x`` (float32 / float16 CUDA tensor) into the running range; returns ``x``."""
        if not x.is_cuda:
            raise ValueError("x must be a CUDA tensor: the observers have no CPU implementation")
        if x.numel() == 0:
            return x
        xc = x.detach().contiguous()
        outer, channels, inner = self._view(xc)
        if self.min_val.numel() != channels:
            if not math.isinf(float(self.min_val.max())):
                raise ValueError("the number of channels changed between batches")
            self.min_val = torch.full((channels,), math.inf, device=self.device)
            self.max_val = torch.full((channels,), -math.inf, device=self.device)
        L = _lib.load()
        need = L.disc_b200_observe_minmax_scratch_floats(outer, channels, inner)
        if self._scratch is None or self._scratch.numel() < need:
            self._scratch = torch.empty(need, dtype=torch.float32, device=self.device)
        _lib.check(L.disc_b200_observe_minmax(xc.data_ptr(), _ops._etype(xc), outer, channels, inner,
                                              self.min_val.data_ptr(), self.max_val.data_ptr(),
                                              self._scratch.data_ptr(), self._scratch.numel(), _ops._stream()))
        return x

    __call__ = observe

    def qparams(self) -> Tuple[torch.Tensor, torch.Tensor]:
        """(scale float32, zero point int32), one entry per channel (one in all per tensor)."""
        qmin, qmax, sym_zp = _RANGES[self.dtype]
        n = self.min_val.numel()
        scale = torch.empty(n, dtype=torch.float32, device=self.device)
        zp = torch.empty(n, dtype=torch.int32, device=self.device)
        _lib.check(_lib.load().disc_b200_minmax_qparams(self.min_val.data_ptr(), self.max_val.data_ptr(), n, qmin, qmax,
                                                        1 if self.symmetric else 0, sym_zp, scale.data_ptr(),
                                                        zp.data_ptr(), _ops._stream()))
        return scale, zp


class PerChannelMinMaxObserver(MinMaxObserver):
    """One range per index of ``ch_axis``."""

    def __init__(self, ch_axis: int = 0, dtype: str = "qint8", symmetric: bool = True,
                 device: Optional[torch.device] = None):
        super().__init__(dtype, symmetric, device)
        self.ch_axis = ch_axis

    def _view(self, x: torch.Tensor) -> Tuple[int, int, int]:
        axis = self.ch_axis % x.dim()
        outer = math.prod(x.shape[:axis])
        inner = math.prod(x.shape[axis + 1:])
        return outer, x.shape[axis], inner


# --------------------------------------------------------------------------- histogram observer
# The counterpart of the reference's HistogramObserver (tools/torch_quant/torch_quant/observer.py:447-744):
# a 2048-bin histogram of everything observed, re-gridded when a batch widens the range, and a search for the
# clipping range that minimises the expected L2 quantization error.  The pass over the tensor (range and bin
# counts) runs on the GPU; what follows works on 2048 numbers and runs on the host in numpy, with the
# element types the reference's torch expressions have (float32 tensors, double Python scalars), so that the
# state after every batch equals the reference's.

import numpy as _np

_F = _np.float32


def adjust_min_max(min_val, max_val, combined_min, combined_max, bins: int, upsample_rate: int):
    """observer.py:614-637: the combined range stretched so that old and new grids share a common fine grid."""
    min_val, max_val, cmin, cmax = _F(min_val), _F(max_val), _F(combined_min), _F(combined_max)
    span = _F(max_val - min_val)
    downsample_rate = int(_np.ceil(_F(_F(_F(cmax - cmin) * _F(upsample_rate)) / span)))
    e = _F(_F(_F(_F(downsample_rate) * span) / _F(upsample_rate)) - _F(cmax - cmin))
    start_idx = int(_np.rint(_F(_F(_F(_F(min_val - cmin) * _F(bins)) * _F(upsample_rate)) / span)))
    return cmin, _F(cmax + e), downsample_rate, start_idx


def combine_histograms(on_new_grid, old_hist, upsample_rate: int, downsample_rate: int, start_idx: int, bins: int):
    """observer.py:639-672: the old histogram spread over `upsample_rate` fine bins each, laid into the new
    range at `start_idx`, summed back into `bins` coarse bins and added to the new batch's histogram."""
    fine = _np.zeros(bins * downsample_rate, dtype=_F)
    fine[start_idx:bins * upsample_rate + start_idx] = _np.repeat(old_hist.astype(_F), upsample_rate)
    integral = _np.cumsum(fine, dtype=_np.float64)[downsample_rate - 1::downsample_rate]
    shifted = _np.zeros(bins, dtype=_F)
    shifted[1:] = integral[:-1].astype(_F)
    interpolated = (integral - shifted.astype(_np.float64)) / upsample_rate
    return (on_new_grid.astype(_F) + interpolated.astype(_F)).astype(_F)


def _quantization_error(hist, min_val: float, max_val: float, bins: int, dst_nbins: int, start_bin: int,
                        end_bin: int) -> float:
    """observer.py:488-537 with the float32 element type of its tensor expressions."""
    bin_width = (float(min_val) * -1.0 + float(max_val)) / bins
    dst_bin_width = bin_width * (end_bin - start_bin + 1) / dst_nbins
    if dst_bin_width == 0.0:
        return 0.0
    bw, dw = _F(bin_width), _F(dst_bin_width)
    src = _np.arange(bins)
    begin = ((src - start_bin).astype(_F) * bw).astype(_F)
    end = (begin + bw).astype(_F)
    hi_bin = _F(dst_nbins - 1)
    of_begin = _np.clip(_np.floor((begin / dw).astype(_F)), _F(0), hi_bin).astype(_F)
    of_end = _np.clip(_np.floor((end / dw).astype(_F)), _F(0), hi_bin).astype(_F)
    begin_center = ((of_begin + _F(0.5)) * dw).astype(_F)
    density = (hist.astype(_F) / bw).astype(_F)

    def norm(db, de):
        db, de = _np.asarray(db, dtype=_F), _np.asarray(de, dtype=_F)
        return (density * (((de * de * de).astype(_F) - (db * db * db).astype(_F)).astype(_F) / _F(3))).astype(_F)

    half = _F(dst_bin_width / 2)
    total = norm(begin - begin_center, _np.full(bins, half, dtype=_F))
    total = (total + ((of_end - of_begin - _F(1)).astype(_F) * norm(_F(-dst_bin_width / 2), half)).astype(_F)).astype(_F)
    end_center = ((of_end * dw).astype(_F) + half).astype(_F)
    total = (total + norm(_F(-dst_bin_width / 2), end - end_center)).astype(_F)
    return float(total.sum(dtype=_F))


def nonlinear_param_search(hist, min_val, max_val, bins: int, dst_nbins: int):
    """observer.py:539-598: walks the quantiles inwards from both ends in steps of 1e-5 of the mass, moving the
    side whose next step crosses more bins, while the quantization error does not grow."""
    hist = hist.astype(_F)
    min_val, max_val = _F(min_val), _F(max_val)
    bin_width = _F(_F(max_val - min_val) / _F(bins))
    total = float(hist.sum(dtype=_F))
    csum = _np.cumsum(hist, dtype=_np.float64).astype(_F)
    stepsize, alpha, beta = 1e-5, 0.0, 1.0
    start_bin, end_bin = 0, bins - 1
    norm_min = float("inf")
    while alpha < beta:
        next_alpha, next_beta = alpha + stepsize, beta - stepsize
        l, r = start_bin, end_bin
        lo_mass, hi_mass = _F(next_alpha * total), _F(next_beta * total)
        while l < end_bin and csum[l] < lo_mass:
            l += 1
        while r > start_bin and csum[r] > hi_mass:
            r -= 1
        next_start, next_end = start_bin, end_bin
        if (l - start_bin) > (end_bin - r):
            next_start, alpha = l, next_alpha
        else:
            next_end, beta = r, next_beta
        if next_start == start_bin and next_end == end_bin:
            continue
        err = _quantization_error(hist, min_val, max_val, bins, dst_nbins, next_start, next_end)
        if err > norm_min:
            break
        norm_min, start_bin, end_bin = err, next_start, next_end
    new_min = _F(min_val + _F(bin_width * _F(start_bin)))
    new_max = _F(min_val + _F(bin_width * _F(end_bin + 1)))
    return new_min, new_max


class HistogramObserver:
    """Per-tensor histogram observer; ``dtype`` "qint8" | "quint8", symmetric or affine."""

    def __init__(self, bins: int = 2048, upsample_rate: int = 128, dtype: str = "quint8", symmetric: bool = False,
                 device: Optional[torch.device] = None):
        if dtype not in _RANGES:
            raise ValueError(f"dtype must be one of {sorted(_RANGES)}")
        if symmetric and dtype != "qint8":
            raise ValueError("Symmetric quantization requires signed dtype.")
        self.bins, self.upsample_rate = bins, upsample_rate
        self.dtype, self.symmetric = dtype, symmetric
        self.device = torch.device("cuda") if device is None else device
        self.histogram = _np.zeros(bins, dtype=_F)
        self.min_val, self.max_val = _F(_np.inf), _F(-_np.inf)
        self._range = MinMaxObserver("qint8", True, self.device)

    def _aminmax(self, x: torch.Tensor):
        r = self._range
        r.min_val.fill_(math.inf)
        r.max_val.fill_(-math.inf)
        r.observe(x)
        lo_hi = torch.cat([r.min_val, r.max_val]).cpu().numpy()
        return _F(lo_hi[0]), _F(lo_hi[1])

    def _histc(self, x: torch.Tensor, lo, hi) -> "_np.ndarray":
        """Bin counts of x over [lo, hi] in `bins` bins, binned as torch.histc bins."""
        counts = torch.zeros(self.bins, dtype=torch.int32, device=self.device)
        _lib.check(_lib.load().disc_b200_observe_histogram(x.data_ptr(), _ops._etype(x), x.numel(), float(lo), float(hi),
                                                           self.bins, counts.data_ptr(), _ops._stream()))
        return counts.cpu().numpy().astype(_F)

    def observe(self, x: torch.Tensor) -> torch.Tensor:
        if not x.is_cuda:
            raise ValueError("x must be a CUDA tensor: the observers have no CPU implementation")
        if x.numel() == 0:
            return x
        xc = x.detach().contiguous()
        uninitialized = _np.isinf(self.min_val) and _np.isinf(self.max_val)
        if uninitialized or self.min_val == self.max_val:
            self.min_val, self.max_val = self._aminmax(xc)
            self.histogram = self._histc(xc, self.min_val, self.max_val)
            return x
        new_min, new_max = self._aminmax(xc)
        cmin, cmax = min(new_min, self.min_val), max(new_max, self.max_val)
        cmin, cmax, down, start = adjust_min_max(self.min_val, self.max_val, cmin, cmax, self.bins, self.upsample_rate)
        on_new_grid = self._histc(xc, cmin, cmax)
        if cmin == self.min_val and cmax == self.max_val:
            self.histogram = (on_new_grid + self.histogram).astype(_F)
        else:
            self.histogram = combine_histograms(on_new_grid, self.histogram, self.upsample_rate, down, start, self.bins)
        self.min_val, self.max_val = cmin, cmax
        return x

    __call__ = observe

    def clipping_range(self):
        """(min, max) the search settles on."""
        return nonlinear_param_search(self.histogram, self.min_val, self.max_val, self.bins, 256)

    def qparams(self) -> Tuple[torch.Tensor, torch.Tensor]:
        """(scale float32, zero point int32) by the reference's rules (observer.py:134-165) from the searched range."""
        lo, hi = self.clipping_range()
        qmin, qmax, sym_zp = _RANGES[self.dtype]
        mn = torch.tensor([lo], dtype=torch.float32, device=self.device)
        mx = torch.tensor([hi], dtype=torch.float32, device=self.device)
        scale = torch.empty(1, dtype=torch.float32, device=self.device)
        zp = torch.empty(1, dtype=torch.int32, device=self.device)
        _lib.check(_lib.load().disc_b200_minmax_qparams(mn.data_ptr(), mx.data_ptr(), 1, qmin, qmax,
                                                        1 if self.symmetric else 0, sym_zp, scale.data_ptr(),
                                                        zp.data_ptr(), _ops._stream()))
        return scale, zp
