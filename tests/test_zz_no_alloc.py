"""The allocation-free small-M entry point, called through the C ABI.

Some callers of this library cannot hand the small-M quantized linear its
split-K scratch because they cannot allocate device memory where they call
it (during stream capture, inside a server whose pool owns the whole device
heap, ...).  For them `disc_b200_qgemm_small_m_noalloc` keeps the scratch in an
array built into the library.  The test checks it against the ordinary entry
point `disc_b200_qgemm` on two calls in a row (the second call sees whatever
the first left in the shared array), bit for bit: both compute exact integer
sums followed by the same epilogue.  Because both entry points end in the same
kernel, the results are also compared with the CPU oracle, differently shaped
problems are interleaved on the shared array, and the property the entry point
exists for is checked directly: device memory in use does not change across
calls after the first.

The file name sorts last on purpose: a run that stops at the first failure has
then already run every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _args(L, a, w, out, x_scale=None, w_scale=None, out_scale=None, bias=None, div_out=False, out_dtype=0, split=0,
          ws=None):
    g = L.QGemmArgs()
    M, K = a.shape
    N = w.shape[0]
    g.a, g.w, g.out = a.data_ptr(), w.data_ptr(), out.data_ptr()
    g.M, g.N, g.K, g.lda, g.ldw, g.ldo = M, N, K, K, K, N
    if x_scale is not None:
        g.x_scale, g.x_scale_kind = x_scale.data_ptr(), L.SCALE_SCALAR
    if w_scale is not None:
        g.w_scale, g.w_scale_kind = w_scale.data_ptr(), L.SCALE_PER_COL
    if out_scale is not None:
        g.out_scale, g.out_scale_kind = out_scale.data_ptr(), L.SCALE_SCALAR
    if bias is not None:
        g.bias, g.bias_kind = bias.data_ptr(), L.BIAS_F32
    g.div_out_scale = 1 if div_out else 0
    g.out_dtype = out_dtype
    g.path = L.PATH_SMALL_M
    g.split_k = split
    if ws is not None:
        g.splitk_ws, g.splitk_ws_bytes = ws.data_ptr(), ws.numel()
    return g


@pytest.mark.parametrize("M,K,N,split", [(64, 2048, 640, 4), (5, 768, 768, 0), (128, 1024, 256, 2), (16, 256, 128, 1)])
def test_noalloc_matches_regular_entry_point_twice(M, K, N, split):
    from bladedisc_b200 import lib as L
    lib = L.load()
    assert lib.disc_b200_qgemm_small_m_noalloc_capacity() == 8 << 20
    rng = np.random.default_rng(M + K + N)
    dev = "cuda"
    stream = torch.cuda.current_stream().cuda_stream
    w = torch.from_numpy(rng.integers(-127, 128, (N, K), dtype=np.int8)).to(dev)
    sw = torch.from_numpy((rng.random(N) * 9e-3 + 1e-3).astype(np.float32)).to(dev)
    bias = torch.from_numpy(rng.standard_normal(N).astype(np.float32)).to(dev)
    sx = torch.tensor([0.02], device=dev)
    so = torch.tensor([0.05], device=dev)
    ws = torch.zeros(lib.disc_b200_qgemm_scratch_bytes(M, N, K), dtype=torch.uint8, device=dev)
    for call in range(2):
        a = torch.from_numpy(rng.integers(-127, 128, (M, K), dtype=np.int8)).to(dev)
        for out_dtype, tdtype, div in ((L.OUT_I32, torch.int32, False), (L.OUT_I8, torch.int8, True),
                                       (L.OUT_F16, torch.float16, False)):
            want = torch.empty((M, N), dtype=tdtype, device=dev)
            got = torch.full((M, N), 77, dtype=tdtype, device=dev)
            kw = dict(x_scale=sx, w_scale=sw, bias=bias, out_scale=so if div else None, div_out=div,
                      out_dtype=out_dtype, split=split)
            ref_args = _args(L, a, w, want, ws=ws, **kw)
            new_args = _args(L, a, w, got, **kw)  # no scratch passed
            assert lib.disc_b200_qgemm(ctypes.byref(ref_args), stream) == 0, lib.disc_b200_last_error_string()
            assert lib.disc_b200_qgemm_small_m_noalloc(ctypes.byref(new_args), stream) == 0, \
                lib.disc_b200_last_error_string()
            torch.cuda.synchronize()
            assert torch.equal(got, want), f"call {call}, out dtype {tdtype}"
            # and against the CPU oracle, not only against the other entry point
            from oracle import c
            acc = c.qgemm_acc(a.cpu().numpy(), w.cpu().numpy())
            if out_dtype == L.OUT_I32:
                assert (got.cpu().numpy() == acc).all(), f"call {call}: accumulators differ from the oracle"
            else:
                f_want, q_want = c.qgemm_epilogue(acc, x_scale=np.float32(0.02), w_scale=sw.cpu().numpy(),
                                                  out_scale=np.float32(0.05) if div else None,
                                                  bias=bias.cpu().numpy(), div_out=div)
                if out_dtype == L.OUT_I8:
                    assert (got.cpu().numpy() == q_want).all(), f"call {call}: int8 result differs from the oracle"
                else:
                    assert np.allclose(got.float().cpu().numpy(), f_want, rtol=1e-2, atol=1e-3)
    assert lib.disc_b200_kernel_status() == 0


def test_noalloc_interleaved_shapes_share_the_array_and_allocate_nothing():
    """A large split followed by a small one (and back) on the one shared array: stale partial sums and
    counters of the other shape must not leak into a result, and no call may change the device memory in use."""
    from bladedisc_b200 import lib as L
    from oracle import c
    lib = L.load()
    rng = np.random.default_rng(99)
    dev = "cuda"
    stream = torch.cuda.current_stream().cuda_stream
    shapes = [(128, 2048, 1024, 8), (16, 512, 256, 2), (64, 4096, 384, 8), (3, 256, 128, 2)]
    ops = []
    for M, K, N, split in shapes:
        a = rng.integers(-127, 128, (M, K), dtype=np.int8)
        w = rng.integers(-127, 128, (N, K), dtype=np.int8)
        ops.append((torch.from_numpy(a).to(dev), torch.from_numpy(w).to(dev),
                    torch.empty((M, N), dtype=torch.int32, device=dev), c.qgemm_acc(a, w), split))

    def run_all():
        for a, w, out, _, split in ops:
            out.fill_(-1)
            g = _args(L, a, w, out, out_dtype=L.OUT_I32, split=split)
            assert lib.disc_b200_qgemm_small_m_noalloc(ctypes.byref(g), stream) == 0, \
                lib.disc_b200_last_error_string()

    run_all()  # the first call on a device looks up the array's address
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    alloc0 = torch.cuda.memory_allocated()
    for _ in range(3):
        run_all()
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0, "device memory in use changed across no-alloc calls"
    assert torch.cuda.memory_allocated() == alloc0
    for a, w, out, want, split in ops:
        assert (out.cpu().numpy() == want).all(), f"shape {tuple(a.shape)} x {tuple(w.shape)} split {split}"
    assert lib.disc_b200_kernel_status() == 0


def test_noalloc_rejects_what_it_cannot_hold():
    from bladedisc_b200 import lib as L
    lib = L.load()
    dev = "cuda"
    stream = torch.cuda.current_stream().cuda_stream
    # more than 128 rows: not the small-M path
    a = torch.zeros((129, 256), dtype=torch.int8, device=dev)
    w = torch.zeros((128, 256), dtype=torch.int8, device=dev)
    out = torch.zeros((129, 128), dtype=torch.int32, device=dev)
    g = _args(L, a, w, out, out_dtype=L.OUT_I32)
    assert lib.disc_b200_qgemm_small_m_noalloc(ctypes.byref(g), stream) != 0
    assert b"more than 128" in lib.disc_b200_last_error_string()
    # partial sums larger than the built-in array: 8 splits x 128 rows x 8192 channels x 4 B = 32 MiB
    a = torch.zeros((128, 1024), dtype=torch.int8, device=dev)
    w = torch.zeros((8192, 1024), dtype=torch.int8, device=dev)
    out = torch.zeros((128, 8192), dtype=torch.int32, device=dev)
    g = _args(L, a, w, out, out_dtype=L.OUT_I32, split=8)
    assert lib.disc_b200_qgemm_small_m_noalloc(ctypes.byref(g), stream) != 0
    assert b"8 MiB built-in scratch" in lib.disc_b200_last_error_string()
    # K not a multiple of 16 cannot use TMA
    a = torch.zeros((4, 40), dtype=torch.int8, device=dev)
    w = torch.zeros((16, 40), dtype=torch.int8, device=dev)
    out = torch.zeros((4, 16), dtype=torch.int32, device=dev)
    g = _args(L, a, w, out, out_dtype=L.OUT_I32)
    assert lib.disc_b200_qgemm_small_m_noalloc(ctypes.byref(g), stream) != 0
    assert b"multiples of 16" in lib.disc_b200_last_error_string()
    # the gathered (slab) activation layout belongs to other kernels: refused, not misread
    a = torch.zeros((2, 16, 128), dtype=torch.int8, device=dev)
    w = torch.zeros((128, 256), dtype=torch.int8, device=dev)
    out = torch.full((16, 128), 55, dtype=torch.int32, device=dev)
    g = _args(L, a[0], w, out, out_dtype=L.OUT_I32)
    g.K, g.lda, g.a_slabs, g.a_slab_cols, g.a_slab_stride = 256, 128, 2, 128, 16 * 128
    assert lib.disc_b200_qgemm_small_m_noalloc(ctypes.byref(g), stream) != 0
    assert b"slab" in lib.disc_b200_last_error_string()
    # row strides below the row length (0 stands for "the row length" in this ABI, so a short positive one)
    a = torch.zeros((4, 256), dtype=torch.int8, device=dev)
    out = torch.full((4, 128), 55, dtype=torch.int32, device=dev)
    for field in ("lda", "ldw", "ldo"):
        g = _args(L, a, w, out, out_dtype=L.OUT_I32)
        setattr(g, field, 16)
        assert lib.disc_b200_qgemm_small_m_noalloc(ctypes.byref(g), stream) != 0
        assert b"row stride" in lib.disc_b200_last_error_string()
    # division by a per-channel output scale exists only in folded form
    so = torch.full((128,), 0.05, device=dev)
    out8 = torch.full((4, 128), 55, dtype=torch.int8, device=dev)
    g = _args(L, a, w, out8, out_scale=so, div_out=True, out_dtype=L.OUT_I8)
    g.out_scale_kind = L.SCALE_PER_COL
    assert lib.disc_b200_qgemm_small_m_noalloc(ctypes.byref(g), stream) != 0
    assert b"folded form" in lib.disc_b200_last_error_string()
    torch.cuda.synchronize()
    assert (out == 55).all() and (out8 == 55).all()  # a refused call writes nothing
