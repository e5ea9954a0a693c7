"""Damaged inputs to the two parsers that read bytes from outside: attribute blobs (with their length given)
and metadata files.  Truncations, flipped bytes and insertions must be refused or parsed, never crash."""
import ctypes

import numpy as np

from bladedisc_b200 import lib as L
from bladedisc_b200 import metadata as M
from bladedisc_b200.ral import pack_attrs


def _damage(rng, data: bytes) -> bytes:
    b = bytearray(data)
    kind = rng.integers(3)
    if kind == 0:
        b = b[: rng.integers(0, len(b))]
    elif kind == 1:
        for _ in range(rng.integers(1, 8)):
            b[rng.integers(len(b))] = rng.integers(256)
    else:
        i = rng.integers(len(b))
        b[i:i] = bytes(rng.integers(0, 256, rng.integers(1, 9), dtype=np.uint8))
    return bytes(b)


def test_damaged_attribute_blobs(built_lib):
    lib = L.load()
    good = pack_attrs({"a": 1, "b": "xyz", "c": [1, 2, 3], "d": [1.5, "q"], "e": True,
                       "f": np.arange(6, dtype=np.float32).reshape(2, 3), "g": {"h": 2}})
    out = ctypes.create_string_buffer(1 << 16)
    assert lib.disc_b200_attrs_describe_bounded(good, len(good), out, 1 << 16) > 0
    assert lib.disc_b200_attrs_describe_bounded(good, len(good) - 1, out, 1 << 16) == -1     # one byte short
    rng = np.random.default_rng(1)
    parsed = 0
    for _ in range(4000):
        blob = _damage(rng, good)
        buf = ctypes.create_string_buffer(blob, max(len(blob), 1))
        parsed += lib.disc_b200_attrs_describe_bounded(buf, len(blob), out, 1 << 16) >= 0
    assert 0 < parsed < 4000
    # lengths that no attribute can have are refused before anything is read through them
    huge = (8).to_bytes(8, "little") + b"intArray" + (1 << 40).to_bytes(8, "little")
    assert lib.disc_b200_attrs_describe(huge + b"\0" * 64, out, 1 << 16) == -1
    long_type = (1 << 20).to_bytes(8, "little") + b"x" * 64
    assert lib.disc_b200_attrs_describe(long_type, out, 1 << 16) == -1


def test_damaged_metadata_files(built_lib, tmp_path):
    from test_metadata import _host_const
    lib = L.load()
    good = tmp_path / "good"
    M.write_metadata(good, [("0_f32_8", True, np.arange(8, dtype=np.float32)), ("1_i8_4x4", False, np.arange(16, dtype=np.int8)),
                            ("2_f32_", True, np.float32(1.5))])
    data = good.read_bytes()
    rng = np.random.default_rng(0)
    loaded = 0
    bad = tmp_path / "bad"
    for _ in range(600):
        bad.write_bytes(_damage(rng, data))
        c = lib.disc_b200_context_create(None)
        e = lib.disc_b200_exec_create(c)
        if lib.disc_b200_context_load_metadata(c, str(bad).encode()) == 0:
            loaded += 1
            for name, idx, rank in (("0_f32_8", 0, 1), ("2_f32_", 2, 0)):       # whatever they decode to: no crash
                _host_const(lib, c, e, name, idx, rank)
                lib.tao_ral_clear_error(c)
        lib.disc_b200_exec_destroy(e)
        lib.disc_b200_context_destroy(c)
    assert 0 < loaded < 600
