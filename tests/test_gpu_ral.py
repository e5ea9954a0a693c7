"""The custom calls driven the way a DISC-compiled executable drives them:
mangled name + type-erased argument array through tao_ral_call_impl (B200 only)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture()
def ral():
    from bladedisc_b200.ral import RalContext
    ctx = RalContext()
    ctx.begin()
    yield ctx
    ctx.close()


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _scalar(v, dtype=np.float32):
    return torch.tensor(v, dtype=torch.float32 if dtype == np.float32 else torch.int32, device="cuda")


def _qgemm_args(x, w, bias, s_x, s_w, s_out, attrs_ptr):
    zero = _scalar(0, np.int32)
    return [("pvoid", 0), x, w, bias, _scalar(s_x), zero, _scalar(s_w), zero, _scalar(s_out), zero,
            ("pvoid", attrs_ptr)]


def test_reference_known_answer_through_the_dispatcher(ral):
    """x = -0.6 [4,25], w = -0.8 [71,25] -> 12.0 everywhere
    (tao_compiler/mlir/disc/tests/pdll/qgemm.cc:24-42), as quantize -> ral_pdll_qgemm -> dequantize."""
    from bladedisc_b200.ral import MemRefSpec
    s_x, s_w = 8.333333e-3, 1.568627e-2
    x = torch.full((4, 25), -0.6, device="cuda")
    w = torch.full((71, 25), -0.8, device="cuda")
    empty = ral.attr_blob({})
    xq = ral.call("disc_b200_quantize", "gpu", [("pvoid", 0), x, _scalar(s_x), _scalar(0, np.int32), ("pvoid", empty)],
                  [MemRefSpec("i8", 2)])
    wq = ral.call("disc_b200_quantize", "gpu", [("pvoid", 0), w, _scalar(s_w), _scalar(0, np.int32), ("pvoid", empty)],
                  [MemRefSpec("i8", 2)])
    bias = torch.zeros(71, device="cuda")
    q = ral.call("ral_pdll_qgemm", "gpu", _qgemm_args(xq, wq, bias, s_x, s_w, 1.0, empty), [MemRefSpec("i8", 2)])
    assert q.shape == (4, 71) and q.dtype == torch.int8
    y = ral.call("disc_b200_dequantize", "gpu", [("pvoid", 0), q, _scalar(1.0), _scalar(0, np.int32), ("pvoid", empty)],
                 [MemRefSpec("f32", 2)])
    assert (y == 12.0).all()
    for t in (xq, wq, q, y):
        ral.dealloc(t)


@pytest.mark.parametrize("rank3", [False, True])
@pytest.mark.parametrize("bias_dtype", [np.float32, np.int8])
def test_pdll_qgemm_variants_match_oracle(ral, rank3, bias_dtype):
    from bladedisc_b200.ral import MemRefSpec
    from oracle import c
    rng = np.random.default_rng(3)
    shape = (2, 70, 256) if rank3 else (140, 256)
    x = rng.integers(-127, 128, shape, dtype=np.int8)
    w = rng.integers(-127, 128, (192, 256), dtype=np.int8)
    bias = (rng.standard_normal(192) * 30).astype(np.float32) if bias_dtype == np.float32 else \
        rng.integers(-127, 128, 192, dtype=np.int8)
    s_x, s_w, s_out = np.float32(0.1), np.float32(0.3), np.float32(50.0)
    _, want = c.qgemm_epilogue(c.qgemm_acc(x, w), x_scale=s_x, w_scale=s_w, out_scale=s_out, bias=bias, fold_out=True)
    q = ral.call("ral_pdll_qgemm", "gpu", _qgemm_args(_dev(x), _dev(w), _dev(bias), s_x, s_w, s_out, ral.attr_blob({})),
                 [MemRefSpec("i8", len(shape))])
    assert tuple(q.shape) == shape[:-1] + (192,)
    assert (q.cpu().numpy() == want).all()
    ral.dealloc(q)


def test_per_channel_call_and_old_style_call(ral):
    from bladedisc_b200.ral import MemRefSpec
    from oracle import c
    rng = np.random.default_rng(4)
    x = rng.integers(-127, 128, (33, 128), dtype=np.int8)
    w = rng.integers(-127, 128, (96, 128), dtype=np.int8)
    sx = np.full(96, 0.05, dtype=np.float32)
    sw = (rng.random(96) * 0.01 + 0.001).astype(np.float32)
    so = np.full(96, 0.4, dtype=np.float32)
    bias = rng.integers(-127, 128, 96, dtype=np.int8)
    zp = torch.zeros(96, dtype=torch.int32, device="cuda")
    _, want = c.qgemm_epilogue(c.qgemm_acc(x, w), x_scale=sx, w_scale=sw, out_scale=so, bias=bias, fold_out=True,
                               x_per_col=True)
    q = ral.call("ral_pdll_qgemm_per_channel", "gpu",
                 [("pvoid", 0), _dev(x), _dev(w), _dev(bias), _dev(sx), zp, _dev(sw), zp, _dev(so), zp,
                  ("pvoid", ral.attr_blob({}))], [MemRefSpec("i8", 2)])
    assert (q.cpu().numpy() == want).all()
    ral.dealloc(q)
    # ral_qgemm: caller-provided result, no bias, (tp_a, tp_b, weight_is_const) = (false, true, true)
    out = torch.empty((33, 96), dtype=torch.int8, device="cuda")
    zero = torch.tensor(0, dtype=torch.int32, device="cuda")
    f = lambda v: torch.tensor(v, dtype=torch.float32, device="cuda")
    ral.call("ral_qgemm", "gpu", [("pvoid", 0), _dev(x), _dev(w), f(0.05), zero, f(0.004), zero, f(0.4), zero, out,
                                  ("i1", False), ("i1", True), ("i1", True)])
    _, want2 = c.qgemm_epilogue(c.qgemm_acc(x, w), x_scale=np.float32(0.05), w_scale=np.float32(0.004),
                                out_scale=np.float32(0.4), fold_out=True)
    assert (out.cpu().numpy() == want2).all()


def test_fused_call_with_attrs_and_row_ops(ral):
    from bladedisc_b200.ral import MemRefSpec
    from oracle import c
    rng = np.random.default_rng(5)
    x = rng.integers(-127, 128, (2, 50, 256), dtype=np.int8)
    w = rng.integers(-127, 128, (384, 256), dtype=np.int8)
    sw = (rng.random(384) * 9e-3 + 1e-3).astype(np.float32)
    bias = (rng.standard_normal(384) * 0.01).astype(np.float32)
    s_x, s_out = np.float32(0.02), np.float32(0.05)
    attrs = ral.attr_blob({"activation": "gelu"})
    f = lambda v: torch.tensor(float(v), dtype=torch.float32, device="cuda")
    args = [("pvoid", 0), _dev(x), _dev(w), _dev(bias), f(s_x), _dev(sw), f(s_out), ("pvoid", attrs)]
    y16 = ral.call("disc_b200_qgemm", "gpu", args, [MemRefSpec("f16", 3)])
    q8 = ral.call("disc_b200_qgemm", "gpu", args, [MemRefSpec("i8", 3)])
    acc = c.qgemm_acc(x, w)
    fw, _ = c.qgemm_epilogue(acc, x_scale=s_x, w_scale=sw, bias=bias, act="gelu")
    _, qw = c.qgemm_epilogue(acc, x_scale=s_x, w_scale=sw, out_scale=s_out, bias=bias, act="gelu", div_out=True)
    assert np.allclose(y16.float().cpu().numpy(), fw, rtol=1e-2, atol=1e-3)
    assert np.abs(q8.cpu().numpy().astype(int) - qw.astype(int)).max() <= 1
    # LayerNorm(x + r) with an int8 second result: a tuple return writes one slot per element
    h = torch.from_numpy(rng.standard_normal((2, 50, 384)).astype(np.float32)).half().cuda()
    gm = torch.ones(384, dtype=torch.float16, device="cuda")
    bt = torch.zeros(384, dtype=torch.float16, device="cuda")
    ln, lq = ral.call("disc_b200_add_layernorm_quant", "gpu",
                      [("pvoid", 0), y16, h, gm, bt, f(0.03), ("pvoid", ral.attr_blob({"eps": 1e-5}))],
                      [MemRefSpec("f16", 3), MemRefSpec("i8", 3)])
    want_ln, _ = c.norm(y16.float().cpu().numpy(), np.ones(384), np.zeros(384), residual=h.float().cpu().numpy(), eps=1e-5)
    assert np.allclose(ln.float().cpu().numpy(), want_ln, rtol=1e-2, atol=1e-2)
    lq_d = np.abs(lq.cpu().numpy().astype(int) - c.quantize(ln.float().cpu().numpy(), np.float32(0.03)).astype(int))
    assert lq_d.max() <= 1 and (lq_d > 0).mean() < 1e-3  # reciprocal form of the fused quantize
    # masked softmax over [B, H, L, L]
    sc = torch.from_numpy(rng.standard_normal((2, 3, 20, 20)).astype(np.float32)).cuda()
    lens = torch.tensor([20, 11], dtype=torch.int32, device="cuda")
    p = ral.call("disc_b200_masked_softmax", "gpu", [("pvoid", 0), sc, lens, ("pvoid", ral.attr_blob({"scale": 0.5}))],
                 [MemRefSpec("f32", 4)])
    assert np.allclose(p.cpu().numpy(), c.softmax(sc.cpu().numpy(), scale=0.5, lens=lens.cpu().numpy()), atol=1e-3)
    # dynamic quantize returns (int8, row scales)
    q, rs = ral.call("disc_b200_dynamic_quantize", "gpu", [("pvoid", 0), ln, ("pvoid", ral.attr_blob({}))],
                     [MemRefSpec("i8", 3), MemRefSpec("f32", 1)])
    qw2, sw2 = c.dynamic_quantize(ln.float().cpu().numpy())
    q_d = np.abs(q.cpu().numpy().astype(int) - qw2.astype(int))
    assert q_d.max() <= 1 and (q_d > 0).mean() < 1e-3 and (rs.cpu().numpy() == sw2).all()


def test_driver_calls_and_ownership(ral):
    p = ral.call("alloc", "gpu", [("i64", 1024)], scalar_result="pvoid")
    assert p
    z = ral.call("alloc", "gpu", [("i64", 0)], scalar_result="pvoid")
    assert z  # zero-byte requests still return a pointer (cuda_context_impl.cc:265)
    src = torch.arange(256, dtype=torch.int32, device="cuda")
    ral.call("d2d_", "gpu", [("pvoid", 0), ("pvoid", src.data_ptr()), ("pvoid", p), ("i64", 1024)])
    ral.call("sync_on_stream", "gpu", [("pvoid", 0)])
    from bladedisc_b200.ral import _tensor_from_ptr
    assert torch.equal(_tensor_from_ptr(p, (256,), torch.int32, ral.device), src)
    ral.call("dealloc", "gpu", [("pvoid", p)])
    ral.call("dealloc", "gpu", [("pvoid", z)])
    ral.call("dealloc", "gpu", [("pvoid", 0)])               # null: ignored
    ral.call("dealloc", "gpu", [("pvoid", src.data_ptr())])  # not owned by this execution: ignored
    assert ral.call("ral_gpu_as_cu_stream", "gpu", [("pvoid", 0)], scalar_result="pvoid") == (ral.stream or None)


def test_errors_are_recorded_not_fatal(ral):
    from bladedisc_b200.ral import MemRefSpec, RalError
    x = torch.zeros((4, 64), dtype=torch.int8, device="cuda")
    w = torch.zeros((8, 32), dtype=torch.int8, device="cuda")  # K mismatch
    with pytest.raises(RalError, match="disagree on K"):
        ral.call("ral_pdll_qgemm", "gpu", _qgemm_args(x, w, torch.zeros(8, device="cuda"), 1, 1, 1, ral.attr_blob({})),
                 [MemRefSpec("i8", 2)])
    with pytest.raises(RalError, match="multi-stream not supported"):
        ral.call("ral_gpu_get_stream", "gpu", [("i32", 1)], scalar_result="pvoid")
    with pytest.raises(RalError, match="no device image"):
        ral.call("ral_kernel_launch", "gpu", [("ppvoid", 0), ("i64", 0), ("pvoid", 0), ("i64", 1), ("i64", 1), ("i64", 1),
                                              ("i64", 1), ("i64", 1), ("i64", 1), ("i32", 0), ("pvoid", 0), ("i32", 0),
                                              ("ppvoid", 0)])
    # empty input: early return with a null buffer and the result shape (quantized_gpu_kernel_impl.cc:347-351)
    e = torch.zeros((0, 64), dtype=torch.int8, device="cuda")
    w2 = torch.zeros((8, 64), dtype=torch.int8, device="cuda")
    q = ral.call("ral_pdll_qgemm", "gpu", _qgemm_args(e, w2, torch.zeros(8, device="cuda"), 1, 1, 1, ral.attr_blob({})),
                 [MemRefSpec("i8", 2)])
    assert tuple(q.shape) == (0, 8)


def test_constants_from_the_metadata_file(ral, tmp_path):
    """A quantized linear the way the executable runs it: weight, scales and bias
    come from the metadata file through ral_const (uploaded once, owned by the
    context), then ral_pdll_qgemm (common_context_impl_cuda.cc:61-160)."""
    from bladedisc_b200 import metadata as M
    from bladedisc_b200.ral import MemRefSpec, RalError
    from oracle import c
    rng = np.random.default_rng(11)
    x = rng.integers(-127, 128, (140, 256), dtype=np.int8)
    w = rng.integers(-127, 128, (192, 256), dtype=np.int8)
    bias = (rng.standard_normal(192) * 30).astype(np.float32)
    s_x, s_w, s_out = np.float32(0.1), np.float32(0.3), np.float32(50.0)
    zero = np.int32(0)
    consts = [(M.const_name(0, w), False, w), (M.const_name(1, bias), False, bias),
              ("2_f32_", False, s_x), ("3_f32_", False, s_w), ("4_f32_", False, s_out), ("5_i32_", False, zero),
              ("6_f16_4x8", False, np.float16(1.5)),                       # splat
              (M.const_name(7, np.zeros(2, np.int64)), True, np.array([140, 256], np.int64))]
    path = tmp_path / "model.so.pbtxt"
    M.write_metadata(path, consts)
    with pytest.raises(RalError, match="no metadata file"):
        ral.const(consts[0][0], 0, "i8", 2)
    ral.load_metadata(path)
    wd = ral.const(consts[0][0], 0, "i8", 2)
    assert wd.shape == (192, 256) and (wd.cpu().numpy() == w).all()
    assert ral.const("anything", 0, "i8", 2).data_ptr() == wd.data_ptr()   # by index: no second upload
    bd = ral.const(consts[1][0], 1, "f32", 1)
    sx, sw, so, zp = (ral.const(f"{i}_{t}_", i, t, 0) for i, t in ((2, "f32"), (3, "f32"), (4, "f32"), (5, "i32")))
    assert float(sx) == float(s_x) and int(zp) == 0
    half = ral.const("6_f16_4x8", 6, "f16", 2)
    assert half.shape == (4, 8) and (half == 1.5).all()
    assert (ral.const(consts[7][0], 7, "i64", 1, device="cpu") == [140, 256]).all()
    q = ral.call("ral_pdll_qgemm", "gpu", [("pvoid", 0), _dev(x), wd, bd, sx, zp, sw, zp, so, zp,
                                           ("pvoid", ral.attr_blob({}))], [MemRefSpec("i8", 2)])
    _, want = c.qgemm_epilogue(c.qgemm_acc(x, w), x_scale=s_x, w_scale=s_w, out_scale=s_out, bias=bias, fold_out=True)
    assert (q.cpu().numpy() == want).all()
    ral.dealloc(q)
    ral.dealloc(wd)                        # constants are persistent: a dealloc from generated code is ignored
    assert (wd.cpu().numpy() == w).all()
    with pytest.raises(RalError, match="not found in metadata file"):
        ral.const("9_f32_4", 9, "f32", 1)
    with pytest.raises(RalError, match="unexpected shape string"):
        ral.const(consts[1][0], 1, "f32", 2)


def test_compiled_executable_stand_in_runs_a_quantized_linear(tmp_path):
    """dlopen -> "main" -> dispatcher: input bound by the host, weight / bias / scales from
    the metadata file, ral_pdll_qgemm, outputs collected (ral_context.cpp:293-321).  The
    program is tests/fake_executable/program.c, written the way generated code calls."""
    from bladedisc_b200 import metadata as M
    from bladedisc_b200.executable import Executable
    from oracle import c
    from test_executable import build_program
    so = build_program(tmp_path, host=False)
    rng = np.random.default_rng(5)
    w = rng.integers(-127, 128, (192, 256), dtype=np.int8)
    bias = (rng.standard_normal(192) * 30).astype(np.float32)
    s_x, s_w, s_out = np.float32(0.1), np.float32(0.3), np.float32(50.0)
    meta = tmp_path / "meta"
    M.write_metadata(meta, [("0_i8_192x256", False, w), ("1_f32_192", False, bias), ("2_f32_", False, s_x),
                            ("3_f32_", False, s_w), ("4_f32_", False, s_out), ("5_i32_", False, np.int32(0)),
                            ("6_i64_2", True, np.array([192, 256], np.int64))])
    with Executable(so, meta, [("i8", "cuda"), ("i64", "cpu"), ("i64", "cpu")], device=torch.cuda.current_device()) as exe:
        for m in (140, 7, 1500):                     # dynamic batch: one executable, any M
            x = rng.integers(-127, 128, (m, 256), dtype=np.int8)
            q, dims, shape = exe.run([_dev(x)])
            _, want = c.qgemm_epilogue(c.qgemm_acc(x, w), x_scale=s_x, w_scale=s_w, out_scale=s_out, bias=bias,
                                       fold_out=True)
            assert (q.cpu().numpy() == want).all()
            assert list(dims) == [192, 256] and list(shape) == [m, 192]


def _nvcc_image(tmp_path, name, *flags):
    import subprocess
    from pathlib import Path
    src = Path(__file__).parent / "fake_executable" / "generated_kernel.cu"
    out = tmp_path / name
    subprocess.run(["nvcc", "-Wno-deprecated-gpu-targets", *flags, "-o", str(out), str(src)], check=True)
    return out.read_bytes()


def test_generated_kernel_launch(ral, tmp_path):
    """ral_kernel_launch: image selection, module / function cache and launch
    (cuda_context_impl.cc:348-445).  A B200 takes image 0 of a multi-image executable and
    the driver compiles its PTX; an image built for sm_100a loads directly; an image with
    only sm_80 code is refused by the driver at load time and reported as an error."""
    import ctypes
    from bladedisc_b200.ral import RalError
    ptx_image = _nvcc_image(tmp_path, "ptx.fatbin", "-fatbin", "-gencode", "arch=compute_60,code=compute_60")
    native = _nvcc_image(tmp_path, "native.cubin", "-cubin", "-gencode", "arch=compute_100a,code=sm_100a")
    ampere = _nvcc_image(tmp_path, "sm80.cubin", "-cubin", "-gencode", "arch=compute_80,code=sm_80")
    n = 100_000
    x = torch.randn(n, device="cuda")

    def mapped(images):
        """Images at fixed addresses, like the data section of an executable."""
        bufs = [ctypes.create_string_buffer(im, len(im)) for im in images]
        return bufs, (ctypes.c_void_p * len(bufs))(*[ctypes.addressof(bf) for bf in bufs])

    def launch(section, a, b, grid=None, name=b"axpb"):
        bufs, blobs = section
        y = torch.zeros(n, device="cuda")
        kname = ctypes.create_string_buffer(name)
        vals = [ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(y.data_ptr()), ctypes.c_float(a), ctypes.c_float(b),
                ctypes.c_int64(n)]
        params = (ctypes.c_void_p * len(vals))(*[ctypes.addressof(v) for v in vals])
        g = (n + 255) // 256 if grid is None else grid
        ral.call("ral_kernel_launch", "gpu",
                 [("ppvoid", ctypes.addressof(blobs)), ("i64", len(bufs)), ("pvoid", ctypes.addressof(kname)),
                  ("i64", g), ("i64", 1), ("i64", 1), ("i64", 256), ("i64", 1), ("i64", 1), ("i32", 0), ("pvoid", 0),
                  ("i32", len(vals)), ("ppvoid", ctypes.addressof(params))])
        torch.cuda.synchronize()
        return y

    one = mapped([native])
    assert torch.equal(launch(one, 2.0, 1.0), 2.0 * x + 1.0)
    assert torch.equal(launch(one, -1.0, 0.5), -1.0 * x + 0.5)                      # module and function from the cache
    five = mapped([ptx_image, ampere, ampere, ampere, ampere])                      # the layout the compiler emits
    assert torch.equal(launch(five, 3.0, 0.0), 3.0 * x)
    assert (launch(one, 2.0, 1.0, grid=0) == 0).all()                               # empty launch: skipped
    with pytest.raises(RalError, match="GetFunction 'nope'"):
        launch(one, 1.0, 0.0, name=b"nope")
    with pytest.raises(RalError, match="ModuleLoad of image 0 of 1"):
        launch(mapped([ampere]), 1.0, 0.0)
    assert torch.equal(launch(one, 2.0, 1.0), 2.0 * x + 1.0)                        # the context stays usable
