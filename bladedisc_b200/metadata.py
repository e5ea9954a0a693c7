"""The metadata file that travels with a DISC executable: its constants (for the
quantized path the int8 weights, scale vectors and biases) by unique name.

Format and naming are the reference's (tao_compiler/mlir/ral/ral_metadata.cc:65-167;
unique names "<id>_<type tag>_<d0xd1x...>" parsed by
tao_compiler/mlir/ral/context/common_context_impl.cc:217-237); reading, decoding
and the upload happen inside the library (``RalContext.load_metadata`` and the
``ral_const`` custom call).  This module is the writer side and the name helpers.
"""
import ctypes
from typing import Iterable, Sequence, Tuple

import numpy as np

from . import lib as _lib

# element type tags of memref operands (the call's types), by numpy dtype
TAG_NUMPY = {"i1": np.bool_, "i8": np.int8, "ui8": np.uint8, "i16": np.int16, "ui16": np.uint16,
             "i32": np.int32, "ui32": np.uint32, "i64": np.int64, "f16": np.float16, "f32": np.float32,
             "f64": np.float64}


def const_name(uid, array_or_tag, shape: Sequence[int] = None) -> str:
    """Unique name of a constant: ``const_name(3, w)`` or ``const_name(3, "i8", (4096, 4096))``.

    The compiler writes ``<md5 of the data>_<i|f><bits>_<d0xd1x...>``
    (tao_compiler/mlir/disc/transforms/disc_convert_const_to_ral.cc:53-80): every integer type, signed or
    not, is ``i<bits>``, every float ``f<bits>``; the runtime reads the element width from the digits."""
    if isinstance(array_or_tag, str):
        tag = array_or_tag
    else:
        a = np.asarray(array_or_tag)
        bits = 1 if a.dtype == np.bool_ else a.dtype.itemsize * 8
        tag, shape = f"{'f' if a.dtype.kind == 'f' else 'i'}{bits}", a.shape
    return f"{uid}_{tag}_{'x'.join(str(int(d)) for d in shape)}"


def name_info(unique_name: str) -> Tuple[Tuple[int, ...], int]:
    """(shape, bytes per element) encoded in a unique name; ValueError if it has none."""
    L = _lib.load()
    rank = ctypes.c_int32()
    sizes = (ctypes.c_int64 * 8)()
    width = ctypes.c_int64()
    if L.disc_b200_const_name_info(unique_name.encode(), ctypes.byref(rank), sizes, ctypes.byref(width)) != 0:
        raise ValueError(f"unexpected const unique_name format: {unique_name}")
    return tuple(sizes[i] for i in range(rank.value)), width.value


def write_metadata(path, consts: Iterable[Tuple[str, bool, object]]):
    """Writes ``consts`` = (unique name, is_host, array or bytes) entries.  An
    array shorter than the shape in its name is a splat (one element repeated)."""
    L = _lib.load()
    names, hosts, blobs = [], [], []
    for name, is_host, value in consts:
        data = value if isinstance(value, (bytes, bytearray)) else np.ascontiguousarray(value).tobytes()
        names.append(name.encode())
        hosts.append(1 if is_host else 0)
        blobs.append(bytes(data))
    n = len(names)
    c_names = (ctypes.c_char_p * n)(*names)
    c_hosts = (ctypes.c_int32 * n)(*hosts)
    bufs = [ctypes.create_string_buffer(b, len(b)) for b in blobs]
    c_data = (ctypes.c_void_p * n)(*[ctypes.addressof(b) for b in bufs])
    c_bytes = (ctypes.c_int64 * n)(*[len(b) for b in blobs])
    if L.disc_b200_metadata_write(str(path).encode(), n, c_names, c_hosts, c_data, c_bytes) != 0:
        raise RuntimeError(L.disc_b200_last_error_string().decode())
