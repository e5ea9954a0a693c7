"""Running a DISC-compiled executable on this runtime: what torch_blade's
``RalContext`` does with an engine (pytorch_blade/pytorch_blade/compiler/mlir/
runtime/ral_context.cpp:104-166 load, :185-240 outputs, :293-321 execute).

The shared object is opened, its entry point ``main`` found, its metadata file
attached to a fresh context; every run makes an execution context, binds the
inputs, calls the entry with {execution context, this library's dispatcher} and
collects what the program sent as outputs.  The work is done by the library
(``disc_b200_executable_*``); this class only moves tensors in and out.
"""
import ctypes
from typing import List, Optional, Sequence, Tuple

import numpy as np

from . import lib as _lib
from .metadata import TAG_NUMPY


class BufferRef(ctypes.Structure):
    _fields_ = [("data", ctypes.c_void_p), ("rank", ctypes.c_int32), ("sizes", ctypes.POINTER(ctypes.c_int64))]


class ExecutableError(RuntimeError):
    pass


class Executable:
    """``outputs``: one (element tag, "cuda" | "cpu") per output of the program, the
    information the reference keeps in its engine state
    (``EngineState::outputs``, ral_context.cpp:196-205)."""

    def __init__(self, so_path, metadata_path=None, outputs: Sequence[Tuple[str, str]] = (),
                 device: Optional[int] = None):
        self._L = _lib.load()
        self.outputs = list(outputs)
        self.device = device
        opts = None
        self._keep = []
        if device is not None:
            import torch
            o = _lib.ContextOptions()
            o.device = device
            o.stream = torch.cuda.current_stream(device).cuda_stream
            opts = ctypes.byref(o)
            self._keep.append(o)
        self.handle = self._L.disc_b200_executable_open(str(so_path).encode(),
                                                        str(metadata_path).encode() if metadata_path else None, opts)
        if not self.handle:
            raise ExecutableError(self._L.disc_b200_last_error_string().decode())
        self.context = self._L.disc_b200_executable_context(self.handle)

    def close(self):
        if self.handle:
            self._L.disc_b200_executable_close(self.handle)
            self.handle = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def run(self, inputs: Sequence) -> List:
        """Inputs: contiguous CUDA torch tensors or numpy arrays (host inputs).
        Returns a CUDA tensor per "cuda" output and a numpy array per "cpu" output,
        each a copy that the caller owns."""
        refs = (BufferRef * max(len(inputs), 1))()
        keep = []
        for i, t in enumerate(inputs):
            if isinstance(t, np.ndarray):
                a = t if t.flags.c_contiguous else np.ascontiguousarray(t)   # (ascontiguousarray makes rank 0 rank 1)
                ptr, shape = a.ctypes.data, a.shape
            else:
                a = t.contiguous()
                ptr, shape = a.data_ptr(), tuple(a.shape)
            sizes = (ctypes.c_int64 * max(len(shape), 1))(*shape)
            keep.append((a, sizes))
            refs[i].data = ptr
            refs[i].rank = len(shape)
            refs[i].sizes = sizes
        L = self._L
        ex = L.disc_b200_executable_run(self.handle, len(inputs), ctypes.cast(refs, ctypes.c_void_p))
        if not ex:
            msg = L.disc_b200_last_error_string().decode()
            L.tao_ral_clear_error(self.context)
            raise ExecutableError(msg)
        # Copy every output first and release the buffers this host now owns afterwards: a later
        # output may be the same buffer under a second name (it is then reported as not owned).
        release = []
        try:
            return [self._collect(ex, k, tag, where, release) for k, (tag, where) in enumerate(self.outputs)]
        finally:
            for kind, ptr in release:
                if kind == 1:
                    L.disc_b200_exec_free_output(self.context, ptr)
                else:
                    L.disc_b200_exec_free_host_output(ptr)
            L.disc_b200_exec_destroy(ex)

    def _collect(self, ex, k: int, tag: str, where: str, release: list):
        L = self._L
        data = ctypes.c_void_p()
        rank = ctypes.c_int32()
        sizes = (ctypes.c_int64 * 8)()
        owned = ctypes.c_int32()
        if L.disc_b200_exec_get_output(ex, k, ctypes.byref(data), ctypes.byref(rank), sizes, ctypes.byref(owned)) != 0:
            raise ExecutableError(f"the program sent no output {k}")
        if owned.value in (1, 2):
            release.append((owned.value, data))
        shape = tuple(sizes[i] for i in range(rank.value))
        n = int(np.prod(shape)) if shape else 1
        if where == "cpu":
            dt = np.dtype(TAG_NUMPY[tag])
            if not data.value or n == 0:
                return np.empty(shape, dt)
            buf = (ctypes.c_char * (n * dt.itemsize)).from_address(data.value)
            return np.frombuffer(buf, dtype=dt).reshape(shape).copy()
        import torch
        from .ral import _TAG_DTYPE, _tensor_from_ptr
        dtype = _TAG_DTYPE[tag]
        if not data.value or n == 0:
            return torch.empty(shape, dtype=dtype, device=f"cuda:{self.device}")
        out = _tensor_from_ptr(data.value, shape, dtype, self.device).clone()
        torch.cuda.current_stream(self.device).synchronize()   # the clone has read the buffer before it may be freed
        return out
