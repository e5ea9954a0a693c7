"""The constants path of a compiled executable on the host: the metadata file
(reader, writer, both directions against the reference's own emitter/loader when
it was built here) and the ``ral_const`` custom call for host constants.  No GPU:
device constants are covered by the GPU suite."""
import ctypes

import numpy as np
import pytest

from bladedisc_b200 import lib as L
from bladedisc_b200 import metadata as M
from bladedisc_b200.ral import PackedMemRef


def _host_const(lib, ctx, ex, name, index, rank, tag="f32"):
    """ral_const on "cpu" through tao_ral_call_impl, packed by hand (no torch, no GPU)."""
    slot = ctypes.c_void_p(ex)
    stream = ctypes.c_void_p(0)
    cname = ctypes.create_string_buffer(name.encode())
    pname = ctypes.c_void_p(ctypes.addressof(cname))
    idx = ctypes.c_int32(index)
    res = PackedMemRef(rank)
    arr = (ctypes.c_void_p * 5)(ctypes.addressof(slot), ctypes.addressof(stream), ctypes.addressof(pname),
                                ctypes.addressof(idx), ctypes.addressof(res.words))
    api = ctypes.create_string_buffer(f"ral_const___cpu___pvoid_pvoid_pvoid_i32___m{rank}d{tag}".encode())
    lib.tao_ral_call_impl(ex, ctypes.cast(api, ctypes.c_void_p), arr)
    msg = ctypes.c_char_p()
    code = lib.tao_ral_last_error(ctx, ctypes.byref(msg))
    return code, (msg.value or b"").decode(), res


def _array(res, dtype):
    n = int(np.prod(res.sizes)) if res.sizes else 1
    dt = np.dtype(dtype)
    buf = (ctypes.c_char * (n * dt.itemsize)).from_address(res.data)
    return np.frombuffer(buf, dtype=dt).reshape(res.sizes).copy()


@pytest.fixture
def ctx(built_lib):
    lib = L.load()
    c = lib.disc_b200_context_create(None)
    e = lib.disc_b200_exec_create(c)
    yield lib, c, e
    lib.disc_b200_exec_destroy(e)
    lib.disc_b200_context_destroy(c)


def test_names(built_lib):
    w = np.zeros((4096, 11008), np.int8)
    assert M.const_name(7, w) == "7_i8_4096x11008"
    assert M.name_info("7_i8_4096x11008") == ((4096, 11008), 1)
    assert M.name_info("0_f32_") == ((), 4)          # rank 0: empty shape field
    assert M.name_info("12_i1_3") == ((3,), 1)       # sub-byte widths take one byte
    assert M.name_info("5_ui8_2x3x4") == ((2, 3, 4), 1)
    assert M.name_info("5_f16_8") == ((8,), 2)
    assert M.name_info("5_i64_1x1") == ((1, 1), 8)
    for bad in ("", "abc", "1_f32", "1_f32_2x", "1_f32_x2", "1_f_2", "1_f32_2_3", "1_f32_2xa"):
        with pytest.raises(ValueError):
            M.name_info(bad)


def test_host_constants_round_trip(ctx, tmp_path):
    lib, c, e = ctx
    rng = np.random.default_rng(0)
    scale = rng.standard_normal(768).astype(np.float32)
    bias = rng.standard_normal((2, 3, 5)).astype(np.float32)
    shape = np.array([4, 128, 768], np.int64)
    path = tmp_path / "model.so.pbtxt"
    M.write_metadata(path, [
        (M.const_name(0, scale), True, scale),
        (M.const_name(1, bias), True, bias),
        (M.const_name(2, shape), True, shape),
        ("3_f32_", True, np.float32(0.125)),
        ("4_f32_6x2", True, np.float32(-3.5)),              # splat: one element for 12
        (M.const_name(5, scale), False, scale),             # a device constant: not visible on "cpu"
    ])
    assert lib.disc_b200_context_load_metadata(c, str(path).encode()) == 0
    code, msg, r = _host_const(lib, c, e, M.const_name(0, scale), 0, 1)
    assert code == 0, msg
    assert r.sizes == (768,) and np.array_equal(_array(r, np.float32), scale)
    first = r.data
    code, msg, r = _host_const(lib, c, e, M.const_name(1, bias), 1, 3)
    assert code == 0 and r.sizes == (2, 3, 5) and np.array_equal(_array(r, np.float32), bias)
    assert (r.words[6], r.words[7], r.words[8]) == (15, 5, 1)      # dense row-major strides
    code, msg, r = _host_const(lib, c, e, M.const_name(2, shape), 2, 1, "i64")
    assert code == 0 and np.array_equal(_array(r, np.int64), shape)
    code, msg, r = _host_const(lib, c, e, "3_f32_", 3, 0)
    assert code == 0 and _array(r, np.float32) == np.float32(0.125)
    code, msg, r = _host_const(lib, c, e, "4_f32_6x2", 4, 2)
    assert code == 0 and np.array_equal(_array(r, np.float32), np.full((6, 2), -3.5, np.float32))
    # the second request is served from the store: same buffer, by index (the name is not read)
    code, msg, r = _host_const(lib, c, e, "ignored", 0, 1)
    assert code == 0 and r.data == first
    # and by name when the index is new
    code, msg, r = _host_const(lib, c, e, M.const_name(0, scale), 77, 1)
    assert code == 0 and r.data == first


def test_errors_are_recorded_not_fatal(ctx, tmp_path):
    lib, c, e = ctx
    code, msg, r = _host_const(lib, c, e, "0_f32_4", 0, 1)
    assert code != 0 and "no metadata file" in msg and r.data == 0
    lib.tao_ral_clear_error(c)
    assert lib.disc_b200_context_load_metadata(c, str(tmp_path / "missing").encode()) != 0
    assert b"cannot open" in lib.disc_b200_last_error_string()
    junk = tmp_path / "junk"
    junk.write_bytes(b"\x00" * 64)
    assert lib.disc_b200_context_load_metadata(c, str(junk).encode()) != 0
    assert b"bad magic" in lib.disc_b200_last_error_string()
    path = tmp_path / "m"
    M.write_metadata(path, [("0_f32_4", True, np.arange(4, dtype=np.float32)),
                            ("1_f32_4", False, np.arange(4, dtype=np.float32))])
    # a truncated copy is refused as a whole
    cut = tmp_path / "cut"
    cut.write_bytes(path.read_bytes()[:40] + path.read_bytes()[-8:])
    assert lib.disc_b200_context_load_metadata(c, str(cut).encode()) != 0
    assert b"truncated" in lib.disc_b200_last_error_string()
    assert lib.disc_b200_context_load_metadata(c, str(path).encode()) == 0
    code, msg, r = _host_const(lib, c, e, "1_f32_4", 1, 1)          # device-only constant
    assert code != 0 and "not found" in msg
    lib.tao_ral_clear_error(c)
    code, msg, r = _host_const(lib, c, e, "0_f32_4", 0, 2)          # rank of the call != rank in the name
    assert code != 0 and "unexpected shape string in unique_name" in msg
    lib.tao_ral_clear_error(c)
    with pytest.raises(RuntimeError, match="duplicated key"):
        M.write_metadata(tmp_path / "dup", [("0_f32_1", True, np.float32(1)), ("0_f32_1", True, np.float32(2))])


def test_files_are_interchangeable_with_the_reference(ctx, ref_ral, tmp_path):
    """Written by the reference's emitter -> read by this library; written here ->
    read by the reference's loader (tao_compiler/mlir/ral/ral_metadata.cc)."""
    lib, c, e = ctx
    ref_ral.ref_metadata_write.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.POINTER(ctypes.c_char_p),
                                           ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_char_p)]
    ref_ral.ref_metadata_get.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_int, ctypes.c_char_p,
                                         ctypes.c_int64]
    ref_ral.ref_metadata_get.restype = ctypes.c_int64
    rng = np.random.default_rng(1)
    w = rng.integers(-128, 128, (48, 32), dtype=np.int8)
    s = rng.standard_normal(48).astype(np.float32)
    names = [M.const_name(0, w), M.const_name(1, s), "2_i32_3"]
    # the compiler emits upper-case hex; an odd number of digits means a leading half byte
    hexes = [w.tobytes().hex().upper(), s.tobytes().hex().upper(), "7000000"]
    theirs = tmp_path / "theirs"
    n = len(names)
    rc = ref_ral.ref_metadata_write(str(theirs).encode(), n, (ctypes.c_char_p * n)(*[x.encode() for x in names]),
                                    (ctypes.c_int * n)(1, 1, 1), (ctypes.c_char_p * n)(*[h.encode() for h in hexes]))
    assert rc == 0
    assert lib.disc_b200_context_load_metadata(c, str(theirs).encode()) == 0
    code, msg, r = _host_const(lib, c, e, names[0], 0, 2, "i8")
    assert code == 0, msg
    assert np.array_equal(_array(r, np.int8), w)
    code, msg, r = _host_const(lib, c, e, names[1], 1, 1)
    assert code == 0 and np.array_equal(_array(r, np.float32), s)
    code, msg, r = _host_const(lib, c, e, names[2], 2, 1, "i32")
    assert code == 0 and np.array_equal(_array(r, np.int32), np.array([7, 7, 7], np.int32))   # 07 00 00 00 splat
    ours = tmp_path / "ours"
    M.write_metadata(ours, [(names[0], False, w), (names[1], True, s)])
    buf = ctypes.create_string_buffer(1 << 16)
    got = ref_ral.ref_metadata_get(str(ours).encode(), names[0].encode(), 0, buf, len(buf))
    assert got == 2 * w.size and bytes.fromhex(buf.raw[:got].decode()) == w.tobytes()
    got = ref_ral.ref_metadata_get(str(ours).encode(), names[1].encode(), 1, buf, len(buf))
    assert got == 8 * s.size and bytes.fromhex(buf.raw[:got].decode()) == s.tobytes()
    assert ref_ral.ref_metadata_get(str(ours).encode(), names[0].encode(), 1, buf, len(buf)) == -2
    # byte-identical files for the same constants in the same order
    same = tmp_path / "same"
    M.write_metadata(same, [(names[0], True, w), (names[1], True, s), (names[2], True, bytes.fromhex("07000000"))])
    assert same.read_bytes()[:8] == theirs.read_bytes()[:8] and same.read_bytes()[-8:] == theirs.read_bytes()[-8:]
    M.write_metadata(same, [(names[0], True, w), (names[1], True, s)])
    rc = ref_ral.ref_metadata_write(str(theirs).encode(), 2, (ctypes.c_char_p * 2)(*[x.encode() for x in names[:2]]),
                                    (ctypes.c_int * 2)(1, 1), (ctypes.c_char_p * 2)(*[h.encode() for h in hexes[:2]]))
    assert rc == 0 and same.read_bytes() == theirs.read_bytes()


def test_contexts_can_share_the_constants_of_one_file(built_lib, tmp_path, monkeypatch):
    """The process-level store of the reference (common_context_impl.cc:152-185): contexts that attach
    the same file share decoded constants, which live until the last of them is gone."""
    lib = L.load()
    scale = np.linspace(0.5, 2.0, 48).astype(np.float32)
    path = tmp_path / "shared.pbtxt"
    M.write_metadata(path, [(M.const_name(0, scale), True, scale)])
    name = M.const_name(0, scale)

    def attach(share):
        c = lib.disc_b200_context_create(None)
        e = lib.disc_b200_exec_create(c)
        f = lib.disc_b200_context_share_metadata if share else lib.disc_b200_context_load_metadata
        assert f(c, str(path).encode()) == 0
        return c, e

    def drop(c, e):
        lib.disc_b200_exec_destroy(e)
        lib.disc_b200_context_destroy(c)

    c1, e1 = attach(True)
    c2, e2 = attach(True)
    c3, e3 = attach(False)                                   # a private store next to them
    _, _, r1 = _host_const(lib, c1, e1, name, 0, 1)
    _, _, r2 = _host_const(lib, c2, e2, name, 0, 1)
    _, _, r3 = _host_const(lib, c3, e3, name, 0, 1)
    assert r1.data == r2.data and r3.data != r1.data         # one copy for the sharing contexts
    assert np.array_equal(_array(r2, np.float32), scale) and np.array_equal(_array(r3, np.float32), scale)
    drop(c1, e1)                                             # the store outlives the context that filled it
    code, msg, again = _host_const(lib, c2, e2, name, 0, 1)
    assert code == 0 and again.data == r2.data and np.array_equal(_array(again, np.float32), scale)
    c4, e4 = attach(True)                                    # a later context joins the live store
    _, _, r4 = _host_const(lib, c4, e4, "by index only", 0, 1)
    assert r4.data == r2.data
    drop(c2, e2)
    drop(c4, e4)
    drop(c3, e3)
    c5, e5 = attach(True)                                    # everything released: a fresh store decodes again
    code, msg, r5 = _host_const(lib, c5, e5, name, 0, 1)
    assert code == 0 and np.array_equal(_array(r5, np.float32), scale)
    drop(c5, e5)
    # the reference's environment switch routes the plain call to the shared store
    monkeypatch.setenv("DISC_USE_GLOBAL_CONST_STORE", "True")
    c6, e6 = attach(False)
    c7, e7 = attach(False)
    assert _host_const(lib, c6, e6, name, 0, 1)[2].data == _host_const(lib, c7, e7, name, 0, 1)[2].data
    drop(c6, e6)
    drop(c7, e7)
    assert lib.disc_b200_context_share_metadata(None, b"x") != 0
    c8 = lib.disc_b200_context_create(None)
    assert lib.disc_b200_context_share_metadata(c8, str(tmp_path / "missing").encode()) != 0
    assert b"cannot open" in lib.disc_b200_last_error_string()
    lib.disc_b200_context_destroy(c8)


def test_host_constants_equal_the_reference_runtime(ctx, ref_host, ref_ral, tmp_path):
    """Every kind of constant through the reference's own ral_const on "cpu" (its host runtime compiled into
    oracle/_ref/libref_host.so) and through this library's: same bytes, same shape.  Element widths from the
    tag, rank 0, sub-byte types, splats and a value with an odd number of hex digits."""
    ref = ref_host
    ref.ref_host_const.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_char_p, ctypes.c_int32, ctypes.c_int,
                                   ctypes.c_int, ctypes.c_void_p, ctypes.c_int64, ctypes.POINTER(ctypes.c_int64),
                                   ctypes.c_char_p, ctypes.c_int]
    lib, c, e = ctx
    rng = np.random.default_rng(8)
    consts = [
        ("0_f32_6x7", "f32", np.float32, rng.standard_normal((6, 7)).astype(np.float32)),
        ("1_i8_3x5x2", "i8", np.int8, rng.integers(-128, 128, (3, 5, 2), dtype=np.int8)),
        ("2_i64_", "i64", np.int64, np.array(-123456789012, np.int64)),                 # rank 0
        ("3_i1_9", "i1", np.bool_, rng.integers(0, 2, 9).astype(np.bool_)),             # one byte per element
        ("4_i8_4", "ui8", np.uint8, np.array([0, 1, 254, 255], np.uint8)),       # unsigned: the name says i8 too
        ("5_f64_2x2", "f64", np.float64, rng.standard_normal((2, 2))),
        ("6_i32_5x3", "i32", np.int32, np.int32(-7)),                                   # splat
        ("7_f32_1x2x3x4", "f32", np.float32, rng.standard_normal((1, 2, 3, 4)).astype(np.float32)),
    ]
    path = tmp_path / "kinds"
    M.write_metadata(path, [(name, True, value) for name, _, _, value in consts])
    # one more, written by the reference's emitter because the hex has an odd number of digits: 0x7 then 3 zero bytes
    odd = tmp_path / "odd"
    ref_ral.ref_metadata_write.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.POINTER(ctypes.c_char_p),
                                           ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_char_p)]
    assert ref_ral.ref_metadata_write(str(odd).encode(), 1, (ctypes.c_char_p * 1)(b"0_i32_2"), (ctypes.c_int * 1)(1),
                                      (ctypes.c_char_p * 1)(b"7000000")) == 0

    def theirs(meta, name, tag, dtype, rank, index):
        out = np.zeros(64, np.float64)
        sizes = (ctypes.c_int64 * 8)()
        err = ctypes.create_string_buffer(256)
        call = f"ral_const___cpu___pvoid_pvoid_pvoid_i32___m{rank}d{tag}".encode()
        rc = ref.ref_host_const(str(meta).encode(), call, name.encode(), index, rank, np.dtype(dtype).itemsize,
                                out.ctypes.data, out.nbytes, sizes, err, 256)
        assert rc == 0, err.value
        shape = tuple(sizes[d] for d in range(rank))
        n = int(np.prod(shape)) if shape else 1
        return np.frombuffer(out.tobytes()[: n * np.dtype(dtype).itemsize], dtype=dtype).reshape(shape)

    assert lib.disc_b200_context_load_metadata(c, str(path).encode()) == 0
    for index, (name, tag, dtype, value) in enumerate(consts):
        shape, _ = M.name_info(name)
        want = theirs(path, name, tag, dtype, len(shape), index)
        code, msg, r = _host_const(lib, c, e, name, index, len(shape), tag)
        assert code == 0, msg
        got = _array(r, dtype)
        assert got.shape == want.shape == shape and got.tobytes() == want.tobytes(), name
        assert np.array_equal(got, np.broadcast_to(value, shape))
    assert lib.disc_b200_context_load_metadata(c, str(odd).encode()) == 0
    want = theirs(odd, "0_i32_2", "i32", np.int32, 1, 0)
    code, msg, r = _host_const(lib, c, e, "0_i32_2", 0, 1, "i32")
    assert code == 0 and np.array_equal(_array(r, np.int32), want) and list(want) == [7, 7]


def test_a_name_that_claims_an_impossible_shape_is_refused(ctx, tmp_path):
    lib, c, e = ctx
    name = "0_f32_1099511627776x1099511627776"          # 2^80 elements: the product must not be trusted
    path = tmp_path / "huge"
    M.write_metadata(path, [(name, True, np.float32(1.0))])
    assert lib.disc_b200_context_load_metadata(c, str(path).encode()) == 0
    code, msg, r = _host_const(lib, c, e, name, 0, 2)
    assert code != 0 and "larger than 1 TiB" in msg and r.data == 0
