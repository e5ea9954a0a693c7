"""Quantized linear on HOST buffers: the call a serving process makes when its
activations arrive in host memory.

The int8 weight, its scales and the bias are constants of the compiled graph
and stay resident on the device (the reference uploads constants once, too:
tao_compiler/mlir/ral/context/common_context_impl_cuda.cc:61-132).  Per call,
the activation rows are streamed host -> device, multiplied, and the result
streamed back, in row chunks over three CUDA streams so that the two copy
directions and the tensor-core work overlap.  The chunk loop runs inside the
library (``disc_b200_host_linear_run``), so a host written in another language
gets the same pipeline.  Chunks of about 2048 rows measured best for a 4096-wide
layer on PCIe Gen5: every copy carries a fixed cost of some ten microseconds, so
finer chunks lose more to that than they gain in the fill and drain of the pipe;
only the first and the last chunks of a long input are smaller.
"""
import ctypes
from typing import Optional

import torch

from . import lib as _lib
from . import ops


class HostQLinear:
    """``out_host[M, N] = ral_pdll_qgemm-style int8 linear of a_host[M, K]``.

    ``out_scale`` given: int8 output ``sat(rne((acc * s_x * s_w[n] + bias[n]) / s_out))``;
    otherwise fp16 output.  ``a_host`` and ``out_host`` should be pinned for the
    copies to be asynchronous.
    """

    def __init__(self, w_i8: torch.Tensor, w_scale: torch.Tensor, x_scale: torch.Tensor,
                 bias: Optional[torch.Tensor] = None, out_scale: Optional[torch.Tensor] = None,
                 act: Optional[str] = None, chunk_rows: int = 2048, slots: int = 3):
        if not w_i8.is_cuda:
            raise ValueError("the weight must already be resident on the device")
        self.w, self.w_scale, self.x_scale, self.bias, self.out_scale = w_i8, w_scale, x_scale, bias, out_scale
        self.act = act
        self.N, self.K = w_i8.shape
        self.chunk_rows = chunk_rows
        self.slots = slots
        self.device = w_i8.device
        self.out_dtype = torch.int8 if out_scale is not None else torch.float16
        self._L = _lib.load()
        with torch.cuda.device(self.device):
            self._h = self._L.disc_b200_host_linear_create(chunk_rows, self.K, self.N, ops._OUT[self.out_dtype], slots)
        if not self._h:
            raise RuntimeError(self._L.disc_b200_last_error_string().decode())
        args = _lib.QGemmArgs()
        args.w = w_i8.data_ptr()
        args.N, args.K, args.ldw = self.N, self.K, self.K
        args.x_scale, args.x_scale_kind = x_scale.data_ptr(), _lib.SCALE_SCALAR
        args.w_scale = w_scale.data_ptr()
        args.w_scale_kind = _lib.SCALE_PER_COL if w_scale.numel() > 1 else _lib.SCALE_SCALAR
        if bias is not None:
            args.bias, args.bias_kind = bias.data_ptr(), _lib.BIAS_F32
        if out_scale is not None:
            args.out_scale, args.out_scale_kind, args.div_out_scale = out_scale.data_ptr(), _lib.SCALE_SCALAR, 1
        args.act = ops._ACT[act]
        args.out_dtype = ops._OUT[self.out_dtype]
        self._args = args
        self.kernel_launches = 0

    def close(self):
        if self._h:
            self._L.disc_b200_host_linear_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __call__(self, a_host: torch.Tensor, out_host: torch.Tensor) -> torch.Tensor:
        M = a_host.shape[0]
        if a_host.shape[1] != self.K or out_host.shape != (M, self.N) or out_host.dtype != self.out_dtype:
            raise ValueError("host buffers do not match the layer")
        if a_host.is_cuda or out_host.is_cuda or not a_host.is_contiguous() or not out_host.is_contiguous():
            raise ValueError("a_host and out_host must be contiguous host tensors")
        stream = torch.cuda.current_stream(self.device).cuda_stream
        with torch.cuda.device(self.device):
            _lib.check(self._L.disc_b200_host_linear_run(self._h, ctypes.byref(self._args), a_host.data_ptr(),
                                                         out_host.data_ptr(), M, stream))
        self.kernel_launches += self._L.disc_b200_host_linear_chunks(self._h, M)
        return out_host

    @property
    def h2d_bytes_per_row(self) -> int:
        return self.K

    @property
    def d2h_bytes_per_row(self) -> int:
        return self.N * (1 if self.out_dtype == torch.int8 else 2)
