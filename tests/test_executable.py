"""Loading and running a compiled executable without a GPU: a hand-written stand-in
for the compiler's shared object (tests/fake_executable/program.c, host program)
goes through dlopen -> "main" -> dispatcher -> recv_input / ral_const / alloc /
send_output, as the reference's RalContext drives a real one."""
import ctypes
import subprocess
from pathlib import Path

import numpy as np
import pytest

from bladedisc_b200 import metadata as M

SRC = Path(__file__).parent / "fake_executable" / "program.c"


def build_program(tmp_path, host, variant: int = 1, extra=()):
    """host: the host program (variant 1, 2 or 3); else the GPU program."""
    define = [] if not host else [{1: "-DHOST_PROGRAM", 2: "-DHOST_PROGRAM2", 3: "-DHOST_PROGRAM3"}[variant]]
    define += list(extra)
    so = tmp_path / (f"host_program{variant}.so" if host else "gpu_program.so")
    cmd = ["gcc", "-shared", "-fPIC", "-O1", "-Wno-main"] + define + ["-o", str(so), str(SRC)]
    subprocess.run(cmd, check=True)
    return so


def test_host_program_runs_through_the_dispatcher(built_lib, tmp_path):
    from bladedisc_b200.executable import Executable, ExecutableError
    so = build_program(tmp_path, host=True)
    c = np.arange(8, dtype=np.float32) * 0.5
    meta = tmp_path / "meta"
    M.write_metadata(meta, [("0_f32_8", True, c)])
    outs = [("f32", "cpu")] * 3
    with Executable(so, meta, outs) as exe:
        for seed in range(3):                       # one context, several executions
            x = np.random.default_rng(seed).standard_normal(8).astype(np.float32)
            y, c_out, x_out = exe.run([x])
            assert np.array_equal(y, x + c) and np.array_equal(c_out, c) and np.array_equal(x_out, x)
        short = np.ones(5, np.float32)              # dynamic shape: the program sizes its result from the input
        assert exe.run([short])[0].shape == (5,)
        # wrong rank for the compiled signature: reported, and the executable stays usable
        with pytest.raises(ExecutableError, match="input rank does not match"):
            exe.run([np.ones((2, 4), np.float32)])
        with pytest.raises(ExecutableError, match="invalid input index"):
            exe.run([])
        assert np.array_equal(exe.run([x])[0], x + c)
    # the constant is missing from the file: first error kept, later calls skipped, no crash
    M.write_metadata(meta, [("9_f32_8", True, c)])
    with Executable(so, meta, outs) as exe:
        with pytest.raises(ExecutableError, match="0_f32_8 not found in metadata file"):
            exe.run([x])


def test_open_errors(built_lib, tmp_path):
    from bladedisc_b200.executable import Executable, ExecutableError
    with pytest.raises(ExecutableError, match="executable_open"):
        Executable(tmp_path / "nothing.so")
    # a shared object without the entry point
    src = tmp_path / "empty.c"
    src.write_text("int not_main(void) { return 0; }\n")
    so = tmp_path / "empty.so"
    subprocess.run(["gcc", "-shared", "-fPIC", "-o", str(so), str(src)], check=True)
    with pytest.raises(ExecutableError, match='no entry point "main"'):
        Executable(so)
    good = build_program(tmp_path, host=True)
    with pytest.raises(ExecutableError, match="cannot open"):
        Executable(good, tmp_path / "no_such_metadata")


def test_output_ownership_codes(built_lib, tmp_path):
    """owned = 2 for a host buffer the program allocated, 0 for a constant, an input and a second name."""
    from bladedisc_b200 import lib as L
    from bladedisc_b200.executable import BufferRef
    lib = L.load()
    so = build_program(tmp_path, host=True)
    meta = tmp_path / "meta"
    M.write_metadata(meta, [("0_f32_8", True, np.zeros(8, np.float32))])
    exe = lib.disc_b200_executable_open(str(so).encode(), str(meta).encode(), None)
    assert exe
    x = np.ones(8, np.float32)
    sizes = (ctypes.c_int64 * 1)(8)
    ref = BufferRef(x.ctypes.data, 1, sizes)
    ex = lib.disc_b200_executable_run(exe, 1, ctypes.addressof(ref))
    assert ex
    got = []
    for k in range(4):
        data, rank, owned = ctypes.c_void_p(), ctypes.c_int32(), ctypes.c_int32()
        s8 = (ctypes.c_int64 * 8)()
        assert lib.disc_b200_exec_get_output(ex, k, ctypes.byref(data), ctypes.byref(rank), s8, ctypes.byref(owned)) == 0
        got.append((owned.value, rank.value, s8[0], data.value))
    # out3 is out0's buffer under a second name: the earlier output owns it
    assert [g[0] for g in got] == [2, 0, 0, 0] and all(g[1:3] == (1, 8) for g in got[:3])
    assert got[3][1:3] == (2, 1) and got[3][3] == got[0][3]
    assert got[2][3] == x.ctypes.data
    assert lib.disc_b200_exec_get_output(ex, 4, None, None, None, None) != 0
    lib.disc_b200_exec_destroy(ex)
    lib.disc_b200_exec_free_host_output(got[0][3])
    lib.disc_b200_executable_close(exe)


def test_device_image_selection(built_lib):
    """The reference's table (tao_compiler/mlir/ral/context/common_context_impl.cc:209-215,
    cuda_context_impl.cc:375-395): one image -> it; several -> sm_70/75/80/86 take 1..4 when
    present, everything else (sm_60, Hopper, Blackwell) the PTX-bearing image 0."""
    from bladedisc_b200 import lib as L
    sel = L.load().disc_b200_select_device_image
    assert sel(0, 10, 0) == -1 and sel(-3, 8, 0) == -1
    assert sel(1, 8, 0) == 0 and sel(1, 10, 0) == 0
    assert [sel(5, *cc) for cc in ((7, 0), (7, 5), (8, 0), (8, 6))] == [1, 2, 3, 4]
    assert [sel(5, *cc) for cc in ((6, 0), (6, 1), (8, 9), (9, 0), (10, 0), (12, 0))] == [0] * 6
    assert sel(3, 8, 0) == 0 and sel(3, 7, 5) == 2       # an index past the images falls back to 0
    assert sel(4, 8, 6) == 0 and sel(4, 8, 0) == 3


def test_kernel_launch_without_a_driver_reports(built_lib):
    """No GPU here: an empty launch is skipped silently, a real one is reported, nothing aborts."""
    from bladedisc_b200 import lib as L
    lib = L.load()
    try:
        ctypes.CDLL("libcuda.so.1")
        pytest.skip("a CUDA driver is installed on this host")
    except OSError:
        pass
    c = lib.disc_b200_context_create(None)
    e = lib.disc_b200_exec_create(c)
    name = b"ral_kernel_launch___gpu___pvoid_ppvoid_i64_pvoid_i64_i64_i64_i64_i64_i64_i32_pvoid_i32_ppvoid___void"

    def launch(grid_x):
        slot = ctypes.c_void_p(e)
        image = ctypes.create_string_buffer(b"\x00" * 64)
        blobs = (ctypes.c_void_p * 1)(ctypes.addressof(image))
        pblobs = ctypes.c_void_p(ctypes.addressof(blobs))
        nblobs = ctypes.c_int64(1)
        kname = ctypes.create_string_buffer(b"axpb")
        pname = ctypes.c_void_p(ctypes.addressof(kname))
        dims = [ctypes.c_int64(v) for v in (grid_x, 1, 1, 128, 1, 1)]
        smem, nargs = ctypes.c_int32(0), ctypes.c_int32(0)
        stream, params = ctypes.c_void_p(0), ctypes.c_void_p(0)
        vals = [slot, pblobs, nblobs, pname] + dims + [smem, stream, nargs, params]
        arr = (ctypes.c_void_p * len(vals))(*[ctypes.addressof(v) for v in vals])
        buf = ctypes.create_string_buffer(name)
        lib.tao_ral_call_impl(e, ctypes.cast(buf, ctypes.c_void_p), arr)
        msg = ctypes.c_char_p()
        return lib.tao_ral_last_error(c, ctypes.byref(msg)), (msg.value or b"").decode()

    assert launch(0) == (0, "")
    code, msg = launch(4)
    assert code != 0 and "CUDA driver unavailable" in msg
    lib.disc_b200_exec_destroy(e)
    lib.disc_b200_context_destroy(c)


def test_inc_ref_keeps_a_host_buffer_alive_for_its_other_name(built_lib):
    """alloc -> inc_ref (reshape [6] -> [2, 3]) -> dealloc of the first name: the buffer is still
    this execution's (cpu_context_impl.cc:234-330); without the inc_ref the same dealloc releases it.
    An alias of an input counts nothing; a pointer nobody knows is an error."""
    from bladedisc_b200 import lib as L
    from bladedisc_b200.ral import PackedMemRef
    lib = L.load()
    ctx = lib.disc_b200_context_create(None)

    def call(ex, name, slots):
        arr = (ctypes.c_void_p * len(slots))(*slots)
        buf = ctypes.create_string_buffer(name)
        lib.tao_ral_call_impl(ex, ctypes.cast(buf, ctypes.c_void_p), arr)
        msg = ctypes.c_char_p()
        return lib.tao_ral_last_error(ctx, ctypes.byref(msg)), (msg.value or b"").decode()

    def run(with_inc_ref):
        ex = lib.disc_b200_exec_create(ctx)
        slot, stream = ctypes.c_void_p(ex), ctypes.c_void_p(0)
        nbytes, p = ctypes.c_uint64(24), ctypes.c_void_p(0)
        assert call(ex, b"alloc___cpu___pvoid_i64___pvoid", [ctypes.addressof(slot), ctypes.addressof(nbytes),
                                                             ctypes.addressof(p)])[0] == 0 and p.value
        flat = PackedMemRef(1)
        flat.words[0] = flat.words[1] = p.value
        flat.words[3], flat.words[4] = 6, 1
        view = PackedMemRef(2)
        if with_inc_ref:
            shape = (ctypes.c_int64 * 2)(2, 3)
            sm = PackedMemRef(1)
            sm.words[0] = sm.words[1] = ctypes.addressof(shape)
            sm.words[3], sm.words[4] = 2, 1
            code, msg = call(ex, b"inc_ref___cpu___pvoid_pvoid_m1df32_m1di64___m2df32",
                             [ctypes.addressof(slot), ctypes.addressof(stream)] + flat.slots() + sm.slots() +
                             [ctypes.addressof(view.words)])
            assert code == 0, msg
            assert view.data == p.value and view.sizes == (2, 3) and (view.words[5], view.words[6]) == (3, 1)
        assert call(ex, b"dealloc___cpu___pvoid_pvoid___void", [ctypes.addressof(slot), ctypes.addressof(p)])[0] == 0
        # what the execution still owns shows in the ownership code of an output
        idx = ctypes.c_int64(0)
        out = PackedMemRef(2)
        out.words[0] = out.words[1] = p.value
        out.words[3], out.words[4], out.words[5], out.words[6] = 2, 3, 3, 1
        assert call(ex, b"ral_send_output___cpu___pvoid_i64_m2df32___void",
                    [ctypes.addressof(slot), ctypes.addressof(idx)] + out.slots())[0] == 0
        owned = ctypes.c_int32(-1)
        assert lib.disc_b200_exec_get_output(ex, 0, None, None, None, ctypes.byref(owned)) == 0
        lib.disc_b200_exec_destroy(ex)
        if owned.value == 2:
            lib.disc_b200_exec_free_host_output(p)
        return owned.value

    assert run(with_inc_ref=True) == 2       # still owned: the second name keeps it
    assert run(with_inc_ref=False) == 0      # released by the dealloc
    # an input may be aliased freely; an unknown pointer may not
    ex = lib.disc_b200_exec_create(ctx)
    slot, stream = ctypes.c_void_p(ex), ctypes.c_void_p(0)
    sizes = (ctypes.c_int64 * 1)(4)
    assert lib.disc_b200_exec_bind_input(ex, 0, 0x7000, 1, sizes) == 0
    for ptr, ok in ((0x7000, True), (0x9000, False)):
        m, res = PackedMemRef(1), PackedMemRef(1)
        m.words[0] = m.words[1] = ptr
        m.words[3], m.words[4] = 4, 1
        code, msg = call(ex, b"inc_ref___gpu___pvoid_pvoid_m1di8___m1di8",
                         [ctypes.addressof(slot), ctypes.addressof(stream)] + m.slots() + [ctypes.addressof(res.words)])
        assert (code == 0) == ok, msg
        if ok:
            assert res.data == ptr and res.sizes == (4,)
        else:
            assert "neither an input, a constant nor owned" in msg
    lib.disc_b200_exec_destroy(ex)
    lib.disc_b200_context_destroy(ctx)


def test_the_same_program_on_the_reference_runtime_and_on_this_one(built_lib, ref_host, tmp_path):
    """One compiled shared object, two runtimes: the reference's own host runtime (BaseCpuContext with its
    constants, host buffers, reshape and input / output binding, compiled from the reference tree into
    oracle/_ref/libref_host.so) and this library.  Same inputs and metadata file -> same outputs, shapes and
    aliasing."""
    from bladedisc_b200.executable import Executable, ExecutableError
    ref = ref_host
    program = build_program(tmp_path, host=True)
    rng = np.random.default_rng(3)
    const = rng.standard_normal(8).astype(np.float32)
    meta = tmp_path / "meta"
    M.write_metadata(meta, [("0_f32_8", True, const)])
    meta_splat = tmp_path / "meta_splat"
    M.write_metadata(meta_splat, [("0_f32_8", True, np.float32(0.375))])          # one element for eight

    def run_ref(x, metadata):
        n_out = 4
        bufs = [np.zeros(64, np.float32) for _ in range(n_out)]
        in_data = (ctypes.c_void_p * 1)(x.ctypes.data)
        in_rank = (ctypes.c_int32 * 1)(x.ndim)
        in_sizes = (ctypes.c_int64 * 8)(*x.shape)
        out_ptrs = (ctypes.c_void_p * n_out)(*[b.ctypes.data for b in bufs])
        caps = (ctypes.c_int64 * n_out)(*[b.nbytes for b in bufs])
        widths = (ctypes.c_int32 * n_out)(*([4] * n_out))
        ranks, owned, alias = (ctypes.c_int32 * n_out)(), (ctypes.c_int32 * n_out)(), (ctypes.c_int32 * n_out)()
        sizes = (ctypes.c_int64 * (8 * n_out))()
        err = ctypes.create_string_buffer(512)
        rc = ref.ref_host_run(str(program).encode(), str(metadata).encode(), 1, in_data, in_rank, in_sizes, n_out,
                              out_ptrs, caps, widths, ranks, sizes, owned, alias, err, 512)
        if rc != 0:
            return rc, err.value.decode(), None
        outs = []
        for i in range(n_out):
            shape = tuple(sizes[8 * i + d] for d in range(ranks[i]))
            outs.append((bufs[i][:int(np.prod(shape))].reshape(shape).copy(), owned[i], alias[i]))
        return 0, "", outs

    for metadata, want_c in ((meta, const), (meta_splat, np.full(8, 0.375, np.float32))):
        for n in (8, 5):                                    # the program sizes its result from the input
            x = rng.standard_normal(n).astype(np.float32)
            rc, msg, theirs = run_ref(x, metadata)
            assert rc == 0, msg
            with Executable(program, metadata, [("f32", "cpu")] * 4) as exe:
                ours = exe.run([x])
            for (t, _, _), o in zip(theirs, ours):
                assert t.shape == o.shape and np.array_equal(t, o)
            assert np.array_equal(ours[0], x + want_c[:n]) and ours[3].shape == (1, n)
            assert theirs[2][2] == 0 and theirs[1][2] == -1  # out2 is input 0 itself, out1 (the constant) is not
    # The constant is missing from the file: here an error that names it.  (The reference records the same
    # message and then reads through the pointer it did not get, common_context_impl.cc:309-315, so that
    # case is not run on it.)
    other = tmp_path / "other"
    M.write_metadata(other, [("9_f32_8", True, const)])
    x = np.ones(8, np.float32)
    with Executable(program, other, [("f32", "cpu")] * 4) as exe:
        with pytest.raises(ExecutableError, match="0_f32_8 not found in metadata file"):
            exe.run([x])


def test_second_program_on_both_runtimes(built_lib, ref_host, tmp_path):
    """Rank-3 and rank-0 inputs, a persistent host buffer as an output, an input under a new shape and a
    scalar under a second name: the reference's host runtime and this library agree on every output, and
    this library reports who owns what (persistent buffer: nobody; scalar: the first output; input: nobody)."""
    from bladedisc_b200 import lib as L
    from bladedisc_b200.executable import BufferRef, Executable
    program = build_program(tmp_path, host=True, variant=2)
    meta = tmp_path / "no_constants"
    M.write_metadata(meta, [])                      # the reference's context wants a metadata file, even an empty one
    rng = np.random.default_rng(12)
    elem = [8, 8, 4, 8]
    dtypes = [np.int64, np.int64, np.float32, np.int64]
    for shape, scalar in (((2, 3, 4), 41), ((1, 5, 1), -7)):
        x = rng.standard_normal(shape).astype(np.float32)
        s = np.array(scalar, np.int64)
        bufs = [np.zeros(256, np.uint8) for _ in range(4)]
        in_data = (ctypes.c_void_p * 2)(x.ctypes.data, s.ctypes.data)
        in_rank = (ctypes.c_int32 * 2)(3, 0)
        in_sizes = (ctypes.c_int64 * 16)(*(list(shape) + [0] * 5 + [0] * 8))
        out_ptrs = (ctypes.c_void_p * 4)(*[b.ctypes.data for b in bufs])
        caps = (ctypes.c_int64 * 4)(*[b.nbytes for b in bufs])
        widths = (ctypes.c_int32 * 4)(*elem)
        ranks, owned, alias = (ctypes.c_int32 * 4)(), (ctypes.c_int32 * 4)(), (ctypes.c_int32 * 4)()
        sizes = (ctypes.c_int64 * 32)()
        err = ctypes.create_string_buffer(512)
        rc = ref_host.ref_host_run(str(program).encode(), str(meta).encode(), 2, in_data, in_rank, in_sizes, 4, out_ptrs, caps, widths,
                                   ranks, sizes, owned, alias, err, 512)
        assert rc == 0, err.value
        theirs = []
        for i in range(4):
            shp = tuple(sizes[8 * i + d] for d in range(ranks[i]))
            n = int(np.prod(shp)) if shp else 1
            theirs.append(np.frombuffer(bufs[i].tobytes()[: n * elem[i]], dtype=dtypes[i]).reshape(shp))
        with Executable(program, None, [("i64", "cpu"), ("i64", "cpu"), ("f32", "cpu"), ("i64", "cpu")]) as exe:
            ours = exe.run([x, s])
        for t, o in zip(theirs, ours):
            assert t.shape == o.shape and np.array_equal(t, o)
        assert list(ours[0]) == list(shape) and int(ours[1]) == scalar + 1 == int(ours[3])
        assert ours[2].shape == (shape[0] * shape[1], shape[2]) and np.array_equal(ours[2].ravel(), x.ravel())
        assert alias[2] == 0 and alias[0] == alias[1] == alias[3] == -1       # the reference sees out2 as input 0 too
    # ownership as this library reports it
    lib = L.load()
    exe = lib.disc_b200_executable_open(str(program).encode(), None, None)
    x = np.zeros((2, 2, 2), np.float32)
    s = np.array(1, np.int64)
    sizes3 = (ctypes.c_int64 * 3)(2, 2, 2)
    refs = (BufferRef * 2)(BufferRef(x.ctypes.data, 3, sizes3), BufferRef(s.ctypes.data, 0, None))
    ex = lib.disc_b200_executable_run(exe, 2, ctypes.cast(refs, ctypes.c_void_p))
    assert ex
    codes, ptrs = [], []
    for k in range(4):
        data, owned = ctypes.c_void_p(), ctypes.c_int32()
        assert lib.disc_b200_exec_get_output(ex, k, ctypes.byref(data), None, None, ctypes.byref(owned)) == 0
        codes.append(owned.value)
        ptrs.append(data.value)
    assert codes == [0, 2, 0, 0] and ptrs[2] == x.ctypes.data and ptrs[3] == ptrs[1]
    lib.disc_b200_exec_destroy(ex)
    lib.disc_b200_exec_free_host_output(ptrs[1])
    lib.disc_b200_executable_close(exe)


def test_attributes_and_tuple_results_on_both_runtimes(built_lib, ref_host, tmp_path):
    """The reference's own custom_call_v2 test kernels (tao_compiler/mlir/ral/context/common_context_impl_pdll.cc)
    on its runtime, the same-named calls of this library on ours, driven by one program whose attribute blob was
    written by pack_attrs.  The reference's kernel checks every value of its fixture (and, in its host build, runs
    its convolution-geometry self-check) before it computes, so finishing at all vouches for the writer; equal
    outputs vouch for the result-slot convention of a call that returns a tuple."""
    from bladedisc_b200.executable import Executable
    from bladedisc_b200.ral import pack_attrs
    fixture = {
        "name": "disc.custom_call.test.tf_fused_add_mul", "trueBoolAttr": True, "falseBoolAttr": False, "int127": 127,
        "intNegative123456": -123456, "float0_001": 0.001, "intArray3int128intNegative32int0": [128, -32, 0],
        "array2strtest0strtest1": ["test0", "test1"], "array3float0_001float23_0floatNegative0_5": [0.001, 23.0, -0.5],
        "array5intNegative5floatNegative0_5strtestint30float0_5": [-5, -0.5, "test", 30, 0.5],
        "rank0I64DenseAttr": np.array(1, np.int64), "rank1UI8DenseAttr": np.array([1], np.uint8),
        "rank2Shape2x3SplatBoolDenseAttr": np.ones((2, 3), np.int8),
        "rank2Shape2x3SplatFloatDenseAttr": np.full((2, 3), -0.01, np.float32),
        "data_format_nhwc": "NHWC", "data_format_nchw": "NCHW", "padding_same": "SAME", "padding_valid": "VALID",
        "strides1": [1], "strides22": [2, 2], "strides1231": [1, 2, 3, 1],
        "dilations1": [1], "dilations22": [2, 2], "dilations1231": [1, 2, 3, 1],
        "explicit_paddings": [0, 0, 1, 2, 3, 4, 0, 0],
    }
    blob = pack_attrs(fixture)
    header = tmp_path / "attrs_blob.h"
    header.write_text("static const unsigned char attrs_blob[] = {" + ", ".join(str(b) for b in blob) + "};\n")
    program = build_program(tmp_path, host=True, variant=3, extra=[f'-DATTRS_BLOB_H="{header}"'])
    meta = tmp_path / "no_constants"
    M.write_metadata(meta, [])
    rng = np.random.default_rng(21)
    a = rng.standard_normal((3, 5)).astype(np.float32)
    b = rng.standard_normal((3, 5)).astype(np.float32)
    bufs = [np.zeros(64, np.float32) for _ in range(3)]
    in_data = (ctypes.c_void_p * 2)(a.ctypes.data, b.ctypes.data)
    in_rank = (ctypes.c_int32 * 2)(2, 2)
    in_sizes = (ctypes.c_int64 * 16)(3, 5, 0, 0, 0, 0, 0, 0, 3, 5, 0, 0, 0, 0, 0, 0)
    out_ptrs = (ctypes.c_void_p * 3)(*[x.ctypes.data for x in bufs])
    caps = (ctypes.c_int64 * 3)(*[x.nbytes for x in bufs])
    widths = (ctypes.c_int32 * 3)(4, 4, 4)
    ranks, owned, alias = (ctypes.c_int32 * 3)(), (ctypes.c_int32 * 3)(), (ctypes.c_int32 * 3)()
    sizes = (ctypes.c_int64 * 24)()
    err = ctypes.create_string_buffer(512)
    rc = ref_host.ref_host_run(str(program).encode(), str(meta).encode(), 2, in_data, in_rank, in_sizes, 3, out_ptrs, caps,
                               widths, ranks, sizes, owned, alias, err, 512)
    assert rc == 0, err.value
    theirs = [bufs[i][:15].reshape(3, 5).copy() for i in range(3)]
    assert all((ranks[i], sizes[8 * i], sizes[8 * i + 1]) == (2, 3, 5) for i in range(3))
    with Executable(program, None, [("f32", "cpu")] * 3) as exe:
        ours = exe.run([a, b])
    for t, o in zip(theirs, ours):
        assert np.array_equal(t, o)
    assert np.array_equal(ours[1], a + b) and np.array_equal(ours[0], (a + b) * (a + b)) and np.array_equal(ours[2], ours[0])


def test_concurrent_executions_share_one_context(built_lib, tmp_path):
    """One context, one execution context per inference, several threads at once
    (the reference's threading contract: tao_compiler/mlir/ral/ral_context.cc:83-93)."""
    import threading
    from bladedisc_b200.executable import Executable
    program = build_program(tmp_path, host=True)
    const = np.linspace(0, 1, 8).astype(np.float32)
    meta = tmp_path / "meta"
    M.write_metadata(meta, [("0_f32_8", True, const)])
    wrong = []
    with Executable(program, meta, [("f32", "cpu")] * 4) as exe:
        def worker(seed):
            rng = np.random.default_rng(seed)
            for _ in range(100):
                n = int(rng.integers(1, 9))
                x = rng.standard_normal(n).astype(np.float32)
                y, c, same, view = exe.run([x])
                if not (np.array_equal(y, x + const[:n]) and np.array_equal(same, x) and view.shape == (1, n)):
                    wrong.append(seed)
        threads = [threading.Thread(target=worker, args=(s,)) for s in range(4)]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
    assert not wrong
