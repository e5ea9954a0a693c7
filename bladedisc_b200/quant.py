"""Offline quantization parameters: what the reference computes before run time.

Scales follow tools/torch_quant/torch_quant/observer.py:134-163 of the reference
(symmetric: ``max(|min|, |max|) / ((qmax - qmin) / 2)``, clamped below by eps);
``levels`` selects the divisor: 127.5 is torch_quant's own (qmax - qmin) / 2,
127 is the ``max|x| / 127`` rule the benchmark configurations state.
Constant weights are quantized in double precision, as the compiler folds them
(tao_compiler/mlir/disc/IR/hlo_disc_ops.cc:149-340).

This is preparation code that runs once per model (torch tensor arithmetic on
whatever device the tensors live on); it is not on the inference path.
"""
from typing import Iterable, Tuple

import torch

_EPS = torch.finfo(torch.float32).eps


def symmetric_scale(min_val: torch.Tensor, max_val: torch.Tensor, levels: float = 127.0) -> torch.Tensor:
    """Scale of a symmetric int8 quantizer from observed min / max."""
    neg = torch.minimum(min_val, torch.zeros_like(min_val))
    pos = torch.maximum(max_val, torch.zeros_like(max_val))
    amax = torch.maximum(-neg, pos)
    scale = (amax / levels).to(torch.float32)
    return torch.clamp(scale, min=_EPS)


def calibrate_per_tensor(batches: Iterable[torch.Tensor], levels: float = 127.0) -> torch.Tensor:
    """Running min / max over calibration batches -> one scale (shape [1])."""
    lo = None
    hi = None
    for b in batches:
        mn, mx = torch.aminmax(b.detach().float())
        lo = mn if lo is None else torch.minimum(lo, mn)
        hi = mx if hi is None else torch.maximum(hi, mx)
    if lo is None:
        raise ValueError("no calibration batches")
    return symmetric_scale(lo, hi, levels).reshape(1)


def per_channel_scale(w: torch.Tensor, levels: float = 127.0) -> torch.Tensor:
    """One scale per output channel (row) of a [N, K] weight."""
    mn, mx = torch.aminmax(w.detach().float(), dim=1)
    return symmetric_scale(mn, mx, levels)


def quantize_weight(w: torch.Tensor, scale: torch.Tensor, qmin: int = -128, qmax: int = 127) -> torch.Tensor:
    """int8 weight, rounded half-to-even in double precision; ``scale`` is [1] or [N]."""
    s = scale.double().reshape(-1, 1) if scale.numel() > 1 else scale.double().reshape(1, 1)
    q = torch.round(w.double() / s)
    return torch.clamp(q, qmin, qmax).to(torch.int8)


def quantize_linear(w: torch.Tensor, per_channel: bool = True, levels: float = 127.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """(int8 weight [N, K], float32 scales [N] or [1]) of a Linear weight."""
    if per_channel:
        s = per_channel_scale(w, levels)
    else:
        mn, mx = torch.aminmax(w.detach().float())
        s = symmetric_scale(mn, mx, levels).reshape(1)
    return quantize_weight(w, s), s.contiguous()
