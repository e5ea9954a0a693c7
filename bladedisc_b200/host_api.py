"""Quantized linear on HOST buffers: the call a serving process makes when its
activations arrive in host memory.

The int8 weight, its scales and the bias are constants of the compiled graph
and stay resident on the device (the reference uploads constants once, too:
tao_compiler/mlir/ral/context/common_context_impl_cuda.cc:61-132).  Per call,
the activation rows are streamed host -> device, multiplied, and the int8
result streamed back, in row chunks over three CUDA streams so that the two
copy directions and the tensor-core work overlap.
"""
from typing import Optional

import torch

from . import ops


class HostQLinear:
    """``out_host[M, N] = ral_pdll_qgemm-style int8 linear of a_host[M, K]``.

    ``out_scale`` given: int8 output ``sat(rne((acc * s_x * s_w[n] + bias[n]) / s_out))``;
    otherwise fp16 output.  ``a_host`` and ``out_host`` should be pinned for the
    copies to be asynchronous.
    """

    def __init__(self, w_i8: torch.Tensor, w_scale: torch.Tensor, x_scale: torch.Tensor,
                 bias: Optional[torch.Tensor] = None, out_scale: Optional[torch.Tensor] = None,
                 act: Optional[str] = None, chunk_rows: int = 4096, slots: int = 3):
        if not w_i8.is_cuda:
            raise ValueError("the weight must already be resident on the device")
        self.w, self.w_scale, self.x_scale, self.bias, self.out_scale = w_i8, w_scale, x_scale, bias, out_scale
        self.act = act
        self.N, self.K = w_i8.shape
        self.chunk_rows = chunk_rows
        self.slots = slots
        self.device = w_i8.device
        self.out_dtype = torch.int8 if out_scale is not None else torch.float16
        self._a = [torch.empty((chunk_rows, self.K), dtype=torch.int8, device=self.device) for _ in range(slots)]
        self._o = [torch.empty((chunk_rows, self.N), dtype=self.out_dtype, device=self.device) for _ in range(slots)]
        self._s_in = torch.cuda.Stream(self.device)
        self._s_mm = torch.cuda.Stream(self.device)
        self._s_out = torch.cuda.Stream(self.device)
        self.kernel_launches = 0

    def __call__(self, a_host: torch.Tensor, out_host: torch.Tensor) -> torch.Tensor:
        M = a_host.shape[0]
        if a_host.shape[1] != self.K or out_host.shape != (M, self.N) or out_host.dtype != self.out_dtype:
            raise ValueError("host buffers do not match the layer")
        cur = torch.cuda.current_stream(self.device)
        for s in (self._s_in, self._s_mm, self._s_out):
            s.wait_stream(cur)
        mm_done = [None] * self.slots   # slot's activation buffer may be overwritten after this
        out_done = [None] * self.slots  # slot's result buffer may be overwritten after this
        n_chunks = (M + self.chunk_rows - 1) // self.chunk_rows
        for i in range(n_chunks):
            r0 = i * self.chunk_rows
            rows = min(self.chunk_rows, M - r0)
            k = i % self.slots
            with torch.cuda.stream(self._s_in):
                if mm_done[k] is not None:
                    self._s_in.wait_event(mm_done[k])
                self._a[k][:rows].copy_(a_host[r0:r0 + rows], non_blocking=True)
                ev_in = torch.cuda.Event()
                ev_in.record(self._s_in)
            with torch.cuda.stream(self._s_mm):
                self._s_mm.wait_event(ev_in)
                if out_done[k] is not None:
                    self._s_mm.wait_event(out_done[k])
                ops.qgemm(self._a[k][:rows], self.w, x_scale=self.x_scale, w_scale=self.w_scale,
                          out_scale=self.out_scale, bias=self.bias, act=self.act, out_dtype=self.out_dtype,
                          out=self._o[k][:rows])
                self.kernel_launches += 1
                mm_done[k] = torch.cuda.Event()
                mm_done[k].record(self._s_mm)
            with torch.cuda.stream(self._s_out):
                self._s_out.wait_event(mm_done[k])
                out_host[r0:r0 + rows].copy_(self._o[k][:rows], non_blocking=True)
                out_done[k] = torch.cuda.Event()
                out_done[k].record(self._s_out)
        cur.wait_stream(self._s_out)
        cur.wait_stream(self._s_mm)
        cur.wait_stream(self._s_in)
        return out_host

    @property
    def h2d_bytes_per_row(self) -> int:
        return self.K

    @property
    def d2h_bytes_per_row(self) -> int:
        return self.N * (1 if self.out_dtype == torch.int8 else 2)
