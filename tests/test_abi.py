"""The drop-in boundary without a GPU: the shared library loads, exports every
symbol the header declares, registers the reference's custom-call names, and
packs / parses the type-erased arguments the way the reference does."""
import ctypes
import re
import struct
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "disc_b200_ral.h"


def _declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    names = set(re.findall(r"\b((?:tao_ral|disc_b200)_[a-z0-9_]+)\s*\(", text))
    # typedef'd callback types are not functions
    return sorted(n for n in names if not n.endswith("_fn"))


def test_library_loads_and_exports_every_declared_symbol(built_lib):
    from bladedisc_b200 import lib as L
    lib = L.load()
    declared = _declared_functions()
    assert len(declared) >= 20
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    assert sorted(L.SIGNATURES) == declared, "lib.py must type exactly the declared functions"
    entry = ctypes.c_char_p.in_dll(lib, "kMlirLoweredEntry")
    assert entry.value == b"main"  # tao_compiler/mlir/ral/ral_api.cc:29
    assert b"sm_100a" in lib.disc_b200_version()


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from bladedisc_b200 import lib as L
    monkeypatch.setattr(L, "_lib", None)
    monkeypatch.setattr(L, "_LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        L.load()


def test_ops_refuse_cpu_tensors(built_lib):
    import torch
    from bladedisc_b200 import ops
    with pytest.raises(ValueError, match="no CPU implementation"):
        ops.quantize(torch.zeros(4, 4), torch.ones(1))
    with pytest.raises(ValueError, match="no CPU implementation"):
        ops.qgemm(torch.zeros(4, 16, dtype=torch.int8), torch.zeros(8, 16, dtype=torch.int8))


def test_registry_holds_reference_names(built_lib, ref_ral):
    """Names mangled by the reference's own TaoRalApiFuncNameHelper
    (tao_compiler/mlir/ral/ral_helper.h:135-152) for its signatures are all
    registered here, character for character."""
    from bladedisc_b200 import lib as L
    lib = L.load()
    n = ref_ral.ref_num_names()
    assert n >= 20
    for i in range(n):
        name = ref_ral.ref_name(i)
        assert lib.disc_b200_registry_has(name) == 1, name.decode()


def test_registry_lists_new_calls(built_lib):
    from bladedisc_b200 import lib as L
    lib = L.load()
    names = [lib.disc_b200_registry_name(i).decode() for i in range(lib.disc_b200_registry_size())]
    apis = {n.split("___")[0] for n in names}
    for api in ("ral_pdll_qgemm", "ral_pdll_qgemm_per_channel", "ral_qgemm", "disc_b200_qgemm",
                "disc_b200_quantize", "disc_b200_dynamic_quantize", "disc_b200_dequantize",
                "disc_b200_layernorm", "disc_b200_add_layernorm", "disc_b200_add_layernorm_quant",
                "disc_b200_rmsnorm", "disc_b200_softmax", "disc_b200_masked_softmax",
                "ral_all_gather", "ral_all_reduce", "ral_async_collective_done", "disc_b200_qgemm_all_gather",
                "alloc", "dealloc", "ral_recv_input", "ral_send_output"):
        assert api in apis
    # bare api names resolve too (first registration keeps the nickname: ral_helper.cc:43-51)
    assert lib.disc_b200_registry_has(b"ral_pdll_qgemm") == 1
    assert lib.disc_b200_registry_has(b"no_such_call") == 0


def _slots_for_qgemm():
    """A packed ral_pdll_qgemm call built by bladedisc_b200.ral's packer, with fake pointers."""
    from bladedisc_b200.ral import PackedMemRef
    keep = []

    def memref(rank, ptr, sizes):
        m = PackedMemRef(rank)
        m.words[0], m.words[1], m.words[2] = ptr, ptr + 64, 3
        stride = 1
        for i in range(rank - 1, -1, -1):
            m.words[3 + i] = sizes[i]
            m.words[3 + rank + i] = stride
            stride *= sizes[i]
        keep.append(m)
        return m

    ctx = ctypes.c_void_p(0)
    stream = ctypes.c_void_p(0)
    attrs = ctypes.c_void_p(0xABC0)
    mems = [memref(2, 0x10000, (5, 32)), memref(2, 0x20000, (48, 32)), memref(1, 0x30000, (48,)),
            memref(0, 0x40000, ()), memref(0, 0x41000, ()), memref(0, 0x42000, ()),
            memref(0, 0x43000, ()), memref(0, 0x44000, ()), memref(0, 0x45000, ())]
    result = PackedMemRef(2)
    slots = [ctypes.addressof(ctx), ctypes.addressof(stream)]
    for m in mems:
        slots.extend(m.slots())
    slots.append(ctypes.addressof(attrs))
    slots.append(ctypes.addressof(result.words))
    keep.extend([ctx, stream, attrs, result])
    expected = [0]  # stream handle
    for m in mems:
        expected.extend(int(w) for w in m.words)
    expected.append(0xABC0)
    return slots, expected, result, keep


def test_packing_is_what_the_reference_dispatcher_unpacks(ref_ral):
    """One packed call through the reference's tao_ral_call_impl: its unpacking
    (ral_helper.h:160-208) must recover exactly what our packer stored, and its
    return convention (whole struct through the last slot, :206) must fill ours."""
    slots, expected, result, keep = _slots_for_qgemm()
    arr = (ctypes.c_void_p * len(slots))(*slots)
    name = (b"ral_pdll_qgemm___gpu___pvoid_pvoid_m2di8_m2di8_m1df32_m0df32_m0di32_m0df32_m0di32_"
            b"m0df32_m0di32_pvoid___m2di8")
    n = ref_ral.ref_dispatch(name, arr)
    got = [ref_ral.ref_recorded(i) for i in range(n)]
    assert got[0] != 0          # the context the dispatcher put in
    assert got[1:] == expected
    assert (result.words[0], result.words[1], result.words[2]) == (0x1000, 0x1040, 7)
    assert result.sizes == (100, 101)
    assert (result.words[5], result.words[6]) == (200, 201)


def test_attr_blob_roundtrip(built_lib):
    """Fixture values of the reference's own parser test
    (tao_compiler/mlir/ral/context/common_context_impl_pdll.cc:31-80)."""
    from bladedisc_b200 import lib as L
    from bladedisc_b200.ral import pack_attrs
    lib = L.load()
    attrs = {
        "name": "disc.custom_call.test.tf_fused_add_mul",
        "trueBoolAttr": True,
        "falseBoolAttr": False,
        "int127": 127,
        "intNegative123456": -123456,
        "float0_001": 0.001,
        "intArray3int128intNegative32int0": [128, -32, 0],
        "array2strtest0strtest1": ["test0", "test1"],
        "array3float0_001float23_0floatNegative0_5": [0.001, 23.0, -0.5],
        "array5intNegative5floatNegative0_5strtestint30float0_5": [-5, -0.5, "test", 30, 0.5],
    }
    blob = pack_attrs(attrs)
    out = ctypes.create_string_buffer(4096)
    n = lib.disc_b200_attrs_describe(blob, out, 4096)
    assert n > 0
    text = out.value.decode()
    assert 'name: "disc.custom_call.test.tf_fused_add_mul"' in text
    assert "trueBoolAttr: true" in text and "falseBoolAttr: false" in text
    assert "int127: 127" in text and "intNegative123456: -123456" in text
    assert "float0_001: 0.001" in text
    assert "intArray3int128intNegative32int0: [128, -32, 0]" in text
    assert 'array2strtest0strtest1: ["test0", "test1"]' in text
    assert 'array5intNegative5floatNegative0_5strtestint30float0_5: [-5, -0.5, "test", 30, 0.5]' in text
    # an empty dict still serialises to a non-empty blob: "dict" + 0 entries
    empty = pack_attrs({})
    assert empty == struct.pack("<q", 4) + b"dict" + struct.pack("<q", 0)
    assert lib.disc_b200_attrs_describe(empty, out, 4096) == 2 and out.value == b"{}"
    # dense elements, splat expanded to the full tensor
    def s(x):
        return struct.pack("<q", len(x)) + x
    dense = (s(b"dict") + struct.pack("<q", 1) + s(b"rank1UI8DenseAttr") + s(b"denseElementsAttr") + s(b"uint") +
             struct.pack("<I", 8) + struct.pack("<q", 1) + struct.pack("<q", 3) + b"\x01" + s(b"\x07"))
    assert lib.disc_b200_attrs_describe(dense, out, 4096) > 0
    assert out.value == b"{rank1UI8DenseAttr: dense<uint8[3]:3B>}"
    # the attributes of a collective call as the Python writer serialises them
    # (replica_groups is a dense [groups, ranks per group] tensor: collective.cu.cc:236-237)
    import numpy as np
    coll = pack_attrs({"all_gather_dim": 1, "replica_groups": np.arange(8, dtype=np.int64).reshape(2, 4),
                       "is_async": True, "async_token_key": 3})
    assert lib.disc_b200_attrs_describe(coll, out, 4096) > 0
    text = out.value.decode()
    assert "all_gather_dim: 1" in text and "is_async: true" in text and "async_token_key: 3" in text
    assert "replica_groups: dense<int64[2x4]:64B>" in text
    # garbage is rejected, not trusted
    assert lib.disc_b200_attrs_describe(struct.pack("<q", 3) + b"xyz", out, 4096) == -1
    assert lib.disc_b200_attrs_describe(struct.pack("<q", -5), out, 4096) == -1


def test_dispatcher_error_convention_without_gpu(built_lib):
    """Unknown api names are recorded, first error wins, nothing aborts
    (the reference logs FATAL instead: tao_compiler/mlir/ral/ral_context.cc:185-191)."""
    from bladedisc_b200 import lib as L
    lib = L.load()
    ctx = lib.disc_b200_context_create(None)
    ex = lib.disc_b200_exec_create(ctx)
    msg = ctypes.c_char_p()
    assert lib.tao_ral_last_error(ctx, ctypes.byref(msg)) == 0
    slot = ctypes.c_void_p(ex)
    arr = (ctypes.c_void_p * 1)(ctypes.addressof(slot))
    name = ctypes.create_string_buffer(b"ral_unknown___gpu___pvoid___void")
    lib.tao_ral_call_impl(ex, ctypes.cast(name, ctypes.c_void_p), arr)
    assert lib.tao_ral_last_error(ctx, ctypes.byref(msg)) != 0
    assert b"ral_unknown___gpu___pvoid___void not found" in msg.value
    name2 = ctypes.create_string_buffer(b"other___gpu___pvoid___void")
    lib.tao_ral_call_impl(ex, ctypes.cast(name2, ctypes.c_void_p), arr)
    lib.tao_ral_last_error(ex, ctypes.byref(msg))  # the execution handle is accepted too
    assert b"ral_unknown" in msg.value  # first error kept
    lib.tao_ral_clear_error(ctx)
    assert lib.tao_ral_last_error(ctx, ctypes.byref(msg)) == 0
    # input binding and recv_input are host-only logic
    sizes = (ctypes.c_int64 * 2)(3, 5)
    assert lib.disc_b200_exec_bind_input(ex, 0, 0x5000, 2, sizes) == 0
    from bladedisc_b200.ral import PackedMemRef
    idx = ctypes.c_int64(0)
    res = PackedMemRef(2)
    arr = (ctypes.c_void_p * 3)(ctypes.addressof(slot), ctypes.addressof(idx), ctypes.addressof(res.words))
    name3 = ctypes.create_string_buffer(b"ral_recv_input___cpu___pvoid_i64___m2df32")
    lib.tao_ral_call_impl(ex, ctypes.cast(name3, ctypes.c_void_p), arr)
    assert lib.tao_ral_last_error(ctx, ctypes.byref(msg)) == 0
    assert res.data == 0x5000 and res.sizes == (3, 5) and (res.words[5], res.words[6]) == (5, 1)
    idx.value = 9
    lib.tao_ral_call_impl(ex, ctypes.cast(name3, ctypes.c_void_p), arr)
    assert lib.tao_ral_last_error(ctx, ctypes.byref(msg)) != 0 and b"invalid input index" in msg.value
    lib.disc_b200_exec_destroy(ex)
    lib.disc_b200_context_destroy(ctx)


def test_attr_cache_follows_the_bytes_at_an_address(built_lib):
    """Parsed attributes are cached by blob address, as the reference does for the constant blobs of an
    executable (tao_compiler/mlir/ral/context/pdll_util.h:190-220); a host that rebuilds a blob in place
    gets the new content.  Driven through ral_pdll_qconv2d, whose attribute errors surface before any
    device work, so this runs without a GPU."""
    from bladedisc_b200 import lib as L
    from bladedisc_b200.ral import PackedMemRef, pack_attrs
    lib = L.load()
    ctx = lib.disc_b200_context_create(None)
    ex = lib.disc_b200_exec_create(ctx)
    buf = ctypes.create_string_buffer(512)

    def call(attrs):
        blob = pack_attrs(attrs)
        ctypes.memset(buf, 0, 512)
        ctypes.memmove(buf, blob, len(blob))
        slot, stream, pattrs = ctypes.c_void_p(ex), ctypes.c_void_p(0), ctypes.c_void_p(ctypes.addressof(buf))
        x, w = PackedMemRef(4), PackedMemRef(4)
        for m, shape in ((x, (1, 4, 4, 8)), (w, (4, 1, 1, 8))):
            m.words[0] = m.words[1] = 0x1000               # never dereferenced on the error paths
            for i, d in enumerate(shape):
                m.words[3 + i] = d
        s0, z0, s1, z1 = PackedMemRef(0), PackedMemRef(0), PackedMemRef(1), PackedMemRef(1)
        s1.words[3] = z1.words[3] = 4
        res = PackedMemRef(4)
        slots = [ctypes.addressof(slot), ctypes.addressof(stream)]
        for m in (x, w, s0, z0, s1, z1, s0, z0):
            slots.extend(m.slots())
        slots += [ctypes.addressof(pattrs), ctypes.addressof(res.words)]
        arr = (ctypes.c_void_p * len(slots))(*slots)
        name = ctypes.create_string_buffer(
            b"ral_pdll_qconv2d___gpu___pvoid_pvoid_m4di8_m4di8_m0df32_m0di32_m1df32_m1di32_m0df32_m0di32_pvoid___m4di8")
        lib.tao_ral_call_impl(ex, ctypes.cast(name, ctypes.c_void_p), arr)
        msg = ctypes.c_char_p()
        code = lib.tao_ral_last_error(ctx, ctypes.byref(msg))
        text = (msg.value or b"").decode()
        lib.tao_ral_clear_error(ctx)
        return code, text

    base = {"data_format": "NHWC", "strides": [1], "dilations": [1], "padding": "VALID", "explicit_paddings": [],
            "weight_is_const": True}
    code, text = call(dict(base, padding="FULL"))
    assert code != 0 and "fail to generate paddings" in text
    code, text = call(dict(base, padding="FULL"))                  # same bytes: served from the cache
    assert code != 0 and "fail to generate paddings" in text
    code, text = call(dict(base, data_format="NHW"))               # other bytes at the same address
    assert code != 0 and "fail to generate spatial dims" in text
    code, text = call(dict(base, strides=[1, 2, 3]))
    assert code != 0 and "fail to generate strides and dilations" in text
    lib.disc_b200_exec_destroy(ex)
    lib.disc_b200_context_destroy(ctx)


def test_attribute_blobs_read_the_same_by_the_reference_parser(built_lib, ref_ral):
    """pack_attrs (the writer hosts and tests use) and this library's parser against the reference's own
    parser (tao_compiler/mlir/ral/context/pdll_util.cc, compiled into oracle/_ref): both must make the
    same of every blob, the dense-tensor splat included."""
    import numpy as np
    from bladedisc_b200 import lib as L
    from bladedisc_b200.ral import pack_attrs
    lib = L.load()
    ref_ral.ref_attrs_describe.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int]

    def both(blob):
        buf = ctypes.create_string_buffer(blob, len(blob))
        mine, theirs = ctypes.create_string_buffer(8192), ctypes.create_string_buffer(8192)
        n1 = lib.disc_b200_attrs_describe(buf, mine, 8192)
        n2 = ref_ral.ref_attrs_describe(ctypes.addressof(buf), theirs, 8192)
        return n1, mine.value.decode(), n2, theirs.value.decode()

    cases = [
        {},
        {"activation": "gelu", "requant": True, "per_channel": False},
        {"name": "disc.custom_call.test.tf_fused_add_mul", "trueBoolAttr": True, "falseBoolAttr": False, "int127": 127,
         "intNegative123456": -123456, "float0_001": 0.001, "intArray3int128intNegative32int0": [128, -32, 0],
         "array2strtest0strtest1": ["test0", "test1"], "array3float0_001float23_0floatNegative0_5": [0.001, 23.0, -0.5],
         "array5intNegative5floatNegative0_5strtestint30float0_5": [-5, -0.5, "test", 30, 0.5]},
        {"data_format": "NHWC", "strides": [1, 2, 2, 1], "dilations": [1, 1, 1, 1], "padding": "SAME",
         "explicit_paddings": [], "weight_is_const": True},
        {"all_gather_dim": 1, "replica_groups": np.arange(8, dtype=np.int64).reshape(2, 4), "is_async": True,
         "async_token_key": 3, "reduction_kind": "max"},
        {"weight_should_be_reordered": True, "nested": {"a": 1, "b": [1.5, "x"]},
         "f32": np.array([[1.5, -2.0]], dtype=np.float32), "u8": np.arange(5, dtype=np.uint8)},
    ]
    for attrs in cases:
        n1, mine, n2, theirs = both(pack_attrs(attrs))
        assert n1 > 0 and n1 == n2 and mine == theirs, (mine, theirs)

    def s(x):
        return struct.pack("<q", len(x)) + x
    # a splat written by hand (the Python writer always stores every element): one element for a [3, 2] tensor
    splat = (s(b"dict") + struct.pack("<q", 1) + s(b"w") + s(b"denseElementsAttr") + s(b"float") + struct.pack("<I", 32) +
             struct.pack("<q", 2) + struct.pack("<q", 3) + struct.pack("<q", 2) + b"\x01" + s(struct.pack("<f", -0.01)))
    n1, mine, n2, theirs = both(splat)
    assert mine == theirs == "{w: dense<float32[3x2]:24B>}"
