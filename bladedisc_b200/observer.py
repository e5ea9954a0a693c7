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
