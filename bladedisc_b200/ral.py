"""Host glue for the RAL custom-call ABI: what a DISC-compiled ``main`` and
torch_blade's ``RalContext`` do, written out in Python.

``RalContext`` owns one library context per (device, stream) and makes one
execution context per run, as pytorch_blade/pytorch_blade/compiler/mlir/runtime/
ral_context.cpp:243-321 does.  ``RalContext.call`` mangles the api name from
the argument kinds and packs the arguments into the ``void**`` layout that
generated code uses (tao_compiler/mlir/disc/transforms/disc_to_llvm.cc:302-365;
unpacked by tao_compiler/mlir/ral/ral_helper.h:160-236): one slot per scalar,
3 + 2N slots per rank-N memref, then the result slots.
"""
import ctypes
import struct
from ctypes import c_bool, c_char_p, c_int32, c_int64, c_void_p
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch

from . import lib as _lib

_DTYPE_TAG = {torch.int8: "i8", torch.float32: "f32", torch.float16: "f16", torch.int32: "i32",
              torch.int64: "i64", torch.bool: "i1", torch.bfloat16: "bf16", torch.uint8: "ui8"}
_TAG_DTYPE = {v: k for k, v in _DTYPE_TAG.items()}


@dataclass
class MemRefSpec:
    """A result type: element tag ("i8", "f16", ...) and rank."""
    tag: str
    rank: int

    def mangled(self) -> str:
        return f"m{self.rank}d{self.tag}"


class PackedMemRef:
    """Storage for one memref descriptor plus the slot pointers into it."""

    def __init__(self, rank: int):
        self.rank = rank
        n = 3 + 2 * rank
        self.words = (c_int64 * n)()  # base, data, offset, sizes, strides (all 8 bytes wide)

    @classmethod
    def from_tensor(cls, t: Optional[torch.Tensor], rank: Optional[int] = None):
        if t is None:
            m = cls(rank or 0)
            return m
        m = cls(t.dim())
        ptr = t.data_ptr()
        m.words[0] = ptr
        m.words[1] = ptr
        m.words[2] = 0
        for i, s in enumerate(t.shape):
            m.words[3 + i] = s
        for i, s in enumerate(t.stride()):
            m.words[3 + t.dim() + i] = s
        return m

    def slots(self) -> List[int]:
        base = ctypes.addressof(self.words)
        return [base + 8 * i for i in range(3 + 2 * self.rank)]

    @property
    def data(self) -> int:
        return self.words[1]

    @property
    def sizes(self) -> Tuple[int, ...]:
        return tuple(self.words[3 + i] for i in range(self.rank))


def pack_attrs(attrs: Optional[dict]) -> bytes:
    """Serializes a flat dict into the custom_attrs wire format
    (tao_compiler/mlir/ral/context/pdll_util.cc:20-170)."""
    def s(x: str) -> bytes:
        b = x.encode()
        return struct.pack("<q", len(b)) + b

    def value(v) -> bytes:
        if isinstance(v, bool):
            return s("bool") + struct.pack("<B", 1 if v else 0)
        if isinstance(v, int):
            return s("int") + struct.pack("<q", v)
        if isinstance(v, float):
            return s("float") + struct.pack("<d", v)
        if isinstance(v, str):
            return s("str") + s(v)
        if isinstance(v, (list, tuple)) and all(isinstance(i, int) and not isinstance(i, bool) for i in v):
            return s("intArray") + struct.pack("<q", len(v)) + b"".join(struct.pack("<q", i) for i in v)
        if isinstance(v, (list, tuple)):
            return s("array") + struct.pack("<q", len(v)) + b"".join(value(i) for i in v)
        if isinstance(v, dict):
            return s("dict") + struct.pack("<q", len(v)) + b"".join(s(k) + value(x) for k, x in v.items())
        if hasattr(v, "dtype") and hasattr(v, "tobytes"):  # numpy array -> denseElementsAttr
            kind = {"i": "int", "u": "uint", "f": "float"}[v.dtype.kind]
            raw = v.tobytes()
            return (s("denseElementsAttr") + s(kind) + struct.pack("<I", v.dtype.itemsize * 8) +
                    struct.pack("<q", v.ndim) + b"".join(struct.pack("<q", d) for d in v.shape) +
                    struct.pack("<B", 0) + struct.pack("<q", len(raw)) + raw)
        raise TypeError(f"cannot serialize attribute of type {type(v)}")

    return value(dict(attrs or {}))


class RalError(RuntimeError):
    pass


class RalContext:
    """One RAL context on the current device and stream."""

    def __init__(self, device: Optional[int] = None, use_torch_allocator: bool = True,
                 nccl_comm: Optional[int] = None, comm_stream: Optional[int] = None):
        self._L = _lib.load()
        if not torch.cuda.is_available():
            raise RuntimeError("RalContext needs a CUDA device: there is no CPU implementation")
        self.device = torch.cuda.current_device() if device is None else device
        self.stream = torch.cuda.current_stream(self.device).cuda_stream
        opts = _lib.ContextOptions()
        opts.device = self.device
        opts.stream = self.stream
        if use_torch_allocator:
            dev, stream = self.device, self.stream

            # torch's caching allocator as the RAL allocator, as torch_blade does
            # (ral_context.cpp:251-266).
            def _alloc(_user, nbytes):
                return torch.cuda.caching_allocator_alloc(nbytes, dev, stream)

            def _free(_user, ptr):
                if ptr:
                    torch.cuda.caching_allocator_delete(ptr)

            self._alloc_cb = _lib.ALLOC_FN(_alloc)
            self._free_cb = _lib.FREE_FN(_free)
            opts.gpu_alloc = self._alloc_cb
            opts.gpu_free = self._free_cb
        # communicator (tp.Communicator.handle) and stream for the collective calls
        opts.nccl_comm = nccl_comm
        opts.comm_stream = comm_stream
        self._opts = opts
        self.handle = self._L.disc_b200_context_create(ctypes.byref(opts))
        self.exec_handle = None
        self._attr_blobs = {}

    # ------------------------------------------------------------ lifetime
    def begin(self):
        if self.exec_handle:
            self._L.disc_b200_exec_destroy(self.exec_handle)
        self.exec_handle = self._L.disc_b200_exec_create(self.handle)
        return self

    def end(self):
        if self.exec_handle:
            self._L.disc_b200_exec_destroy(self.exec_handle)
            self.exec_handle = None

    def close(self):
        self.end()
        if self.handle:
            self._L.disc_b200_context_destroy(self.handle)
            self.handle = None

    def __enter__(self):
        return self.begin()

    def __exit__(self, *exc):
        self.close()

    # -------------------------------------------------------------- errors
    def last_error(self) -> Tuple[int, str]:
        msg = c_char_p()
        code = self._L.tao_ral_last_error(self.handle, ctypes.byref(msg))
        return code, (msg.value or b"").decode()

    def clear_error(self):
        self._L.tao_ral_clear_error(self.handle)

    def _raise_if_error(self):
        code, msg = self.last_error()
        if code != 0:
            self.clear_error()
            raise RalError(msg)

    # --------------------------------------------------------------- calls
    def attr_blob(self, attrs: Optional[dict]) -> int:
        """Address of a serialized attribute dict, kept alive and reused so that
        the library's per-address parse cache stays valid."""
        data = pack_attrs(attrs)
        buf = self._attr_blobs.get(data)
        if buf is None:
            buf = ctypes.create_string_buffer(data, len(data))
            self._attr_blobs[data] = buf
        return ctypes.addressof(buf)

    def call(self, api: str, device: str, args: Sequence, results: Sequence[MemRefSpec] = (),
             scalar_result: Optional[str] = None, raw: bool = False):
        """Calls ``api`` through tao_ral_call_impl.

        ``args`` entries: torch tensors (memrefs), ``("pvoid", int)``,
        ``("i64", int)``, ``("i32", int)``, ``("i1", bool)``, or ``("m<N>d<tag>", None)``
        for a null memref.  The leading context argument is added here.
        Returns torch tensors that view the returned device buffers (rank-N
        results) without taking ownership; with ``raw`` the packed memref
        descriptors themselves (results in host memory).
        """
        if not self.exec_handle:
            self.begin()
        keep = []
        slots: List[int] = []
        tags: List[str] = ["pvoid"]
        ctx_slot = c_void_p(self.exec_handle)
        keep.append(ctx_slot)
        slots.append(ctypes.addressof(ctx_slot))
        for a in args:
            if isinstance(a, torch.Tensor):
                m = PackedMemRef.from_tensor(a)
                keep.append((m, a))
                slots.extend(m.slots())
                tags.append(f"m{a.dim()}d{_DTYPE_TAG[a.dtype]}")
            else:
                tag, val = a
                if tag.startswith("m") and "d" in tag:
                    rank = int(tag[1:tag.index("d")])
                    m = PackedMemRef(rank)
                    keep.append(m)
                    slots.extend(m.slots())
                elif tag in ("pvoid", "ppvoid"):
                    c = c_void_p(val)
                    keep.append(c)
                    slots.append(ctypes.addressof(c))
                elif tag == "i64":
                    c = c_int64(val)
                    keep.append(c)
                    slots.append(ctypes.addressof(c))
                elif tag == "i32":
                    c = c_int32(val)
                    keep.append(c)
                    slots.append(ctypes.addressof(c))
                elif tag == "i1":
                    c = c_bool(val)
                    keep.append(c)
                    slots.append(ctypes.addressof(c))
                else:
                    raise ValueError(f"unknown argument tag {tag}")
                tags.append(tag)
        outs = []
        if scalar_result == "pvoid":
            r = c_void_p(0)
            keep.append(r)
            slots.append(ctypes.addressof(r))
            ret_tag = "pvoid"
        elif results:
            for spec in results:
                m = PackedMemRef(spec.rank)
                outs.append((spec, m))
                # A returned memref is written as one struct through one slot.
                slots.append(ctypes.addressof(m.words))
            ret_tag = "_".join(s.mangled() for s in results)
        else:
            ret_tag = "void"
        name = f"{api}___{device}___{'_'.join(tags)}___{ret_tag}"
        arr = (c_void_p * len(slots))(*slots)
        name_buf = ctypes.create_string_buffer(name.encode())
        self._L.tao_ral_call_impl(self.exec_handle, ctypes.cast(name_buf, c_void_p), arr)
        self._raise_if_error()
        if scalar_result == "pvoid":
            return r.value
        if raw:
            return [m for _, m in outs]
        tensors = [self._view(spec, m) for spec, m in outs]
        if not results:
            return None
        return tensors[0] if len(tensors) == 1 else tuple(tensors)

    def _view(self, spec: MemRefSpec, m: PackedMemRef) -> Optional[torch.Tensor]:
        shape = m.sizes
        dtype = _TAG_DTYPE[spec.tag]
        numel = 1
        for s in shape:
            numel *= s
        if m.data == 0 or numel == 0:
            return torch.empty(shape, dtype=dtype, device=f"cuda:{self.device}")
        return _tensor_from_ptr(m.data, shape, dtype, self.device)

    # ----------------------------------------------------------- constants
    def load_metadata(self, path: str):
        """Attaches the metadata file of a compiled executable (its constants);
        the reference does this when it builds the context from the artefact
        (BaseContextOption::metadata_file_path, tao_compiler/mlir/ral/context/base/base_context.cc:30-52)."""
        if self._L.disc_b200_context_load_metadata(self.handle, str(path).encode()) != 0:
            raise RalError(self._L.disc_b200_last_error_string().decode())

    def const(self, unique_name: str, index: int, tag: str, rank: int, device: str = "gpu"):
        """``ral_const``: the constant ``unique_name`` as a device tensor
        (``device="gpu"``) or as a numpy copy of the host constant (``"cpu"``)."""
        name = ctypes.create_string_buffer(unique_name.encode())
        args = [("pvoid", 0), ("pvoid", ctypes.addressof(name)), ("i32", index)]
        spec = MemRefSpec(tag, rank)
        if device == "gpu":
            return self.call("ral_const", "gpu", args, results=[spec])
        import numpy as np
        from .metadata import TAG_NUMPY
        (m,) = self.call("ral_const", "cpu", args, results=[spec], raw=True)
        dt = np.dtype(TAG_NUMPY[tag])
        n = 1
        for d in m.sizes:
            n *= d
        if m.data == 0 or n == 0:
            return np.empty(m.sizes, dt)
        buf = (ctypes.c_char * (n * dt.itemsize)).from_address(m.data)
        return np.frombuffer(buf, dtype=dt).reshape(m.sizes).copy()

    def dealloc(self, t_or_ptr):
        ptr = t_or_ptr.data_ptr() if isinstance(t_or_ptr, torch.Tensor) else int(t_or_ptr)
        self.call("dealloc", "gpu", [("pvoid", ptr)])


class _CudaArray:
    """Minimal __cuda_array_interface__ carrier so torch can view a raw pointer."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr,
                                         "data": (ptr, False), "version": 2}


_TYPESTR = {torch.int8: "|i1", torch.uint8: "|u1", torch.float32: "<f4", torch.float16: "<f2",
            torch.int32: "<i4", torch.int64: "<i8", torch.bool: "|b1"}


def _tensor_from_ptr(ptr: int, shape, dtype, device: int) -> torch.Tensor:
    return torch.as_tensor(_CudaArray(ptr, shape, _TYPESTR[dtype]), device=f"cuda:{device}")
