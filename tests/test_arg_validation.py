"""Argument checks of the direct C entry points that answer before anything touches a GPU:
status code + message, never a crash.  (What needs a device is covered by the -m gpu tests.)"""
import ctypes

import pytest

from bladedisc_b200 import lib as L


@pytest.fixture(scope="module")
def lib(built_lib):
    return L.load()


def _err(lib):
    return lib.disc_b200_last_error_string().decode()


def test_weight_only_qgemm(lib):
    a = L.WeightOnlyQGemmArgs()
    a.x = a.w = a.scale = a.out = 0x1000          # never dereferenced on these paths
    a.m, a.n, a.k, a.ldx, a.ldw, a.ldo, a.type = 4, 64, 32, 32, 64, 64, L.F16
    assert lib.disc_b200_weight_only_qgemm(None, None) != 0 and "null args" in _err(lib)
    a.m = -1
    assert lib.disc_b200_weight_only_qgemm(ctypes.byref(a), None) != 0 and "negative size" in _err(lib)
    a.m = 0
    assert lib.disc_b200_weight_only_qgemm(ctypes.byref(a), None) == 0         # nothing to do
    a.m, a.w = 4, None
    assert lib.disc_b200_weight_only_qgemm(ctypes.byref(a), None) != 0 and "null operand" in _err(lib)
    a.w, a.ldw = 0x1000, 63
    assert lib.disc_b200_weight_only_qgemm(ctypes.byref(a), None) != 0 and "row stride" in _err(lib)
    a.ldw, a.type = 64, 7
    assert lib.disc_b200_weight_only_qgemm(ctypes.byref(a), None) != 0 and "element type" in _err(lib)
    # the tensor-core kernel, asked for by name, refuses what it cannot take instead of falling back
    a.type, a.path = L.F32, 2
    assert lib.disc_b200_weight_only_qgemm(ctypes.byref(a), None) != 0 and "tensor cores" in _err(lib)
    a.type, a.n, a.ldw, a.ldo = L.F16, 24, 24, 24                                  # N not a multiple of 16
    assert lib.disc_b200_weight_only_qgemm(ctypes.byref(a), None) != 0 and "tensor cores" in _err(lib)
    a.n, a.ldw, a.ldo, a.x = 64, 64, 64, 0x1008                                    # activations not 16-byte aligned
    assert lib.disc_b200_weight_only_qgemm(ctypes.byref(a), None) != 0 and "tensor cores" in _err(lib)


def _conv_args():
    a = L.QConv2dArgs()
    a.x = a.w = a.out = a.x_scale = a.w_scale = a.out_scale = 0x1000
    a.input_sizes[:] = [2, 8, 8, 16]
    a.kernel_sizes[:] = [4, 3, 3, 16]
    a.output_sizes[:] = [2, 6, 6, 4]
    a.padding[:] = [0, 0, 0, 0]
    a.metadata[:] = [0, 3, 1, 2, 3, 0, 1, 2, 0, 3, 1, 2, 1, 1, 1, 1]
    return a


def test_qconv2d(lib):
    assert lib.disc_b200_qconv2d(None, None) != 0 and "null args" in _err(lib)
    a = _conv_args()
    need = lib.disc_b200_qconv2d_workspace_bytes(ctypes.byref(a))
    # K = 144 needs no padding, the OHWI kernel no packing, the NHWC output no scatter: the gathered matrix only
    assert need == (2 * 6 * 6 * 144 + 255) // 256 * 256
    assert lib.disc_b200_qconv2d(ctypes.byref(a), None) != 0 and "workspace" in _err(lib)
    a.workspace, a.workspace_bytes = 0x1008, need   # not 256-byte aligned
    assert lib.disc_b200_qconv2d(ctypes.byref(a), None) != 0 and "misaligned" in _err(lib)
    a.workspace, a.x = 0x1000, None
    assert lib.disc_b200_qconv2d(ctypes.byref(a), None) != 0 and "null operand" in _err(lib)
    a = _conv_args()
    a.output_sizes[:] = [2, 7, 6, 4]
    assert lib.disc_b200_qconv2d(ctypes.byref(a), None) != 0 and "output shape does not match" in _err(lib)
    a = _conv_args()
    a.metadata[12] = 0                              # stride 0
    assert lib.disc_b200_qconv2d(ctypes.byref(a), None) != 0 and "invalid conv params" in _err(lib)
    a = _conv_args()
    a.kernel_sizes[:] = [4, 3, 3, 8]
    assert lib.disc_b200_qconv2d(ctypes.byref(a), None) != 0 and "grouped convolution" in _err(lib)
    a = _conv_args()
    a.input_sizes[0] = 0
    a.output_sizes[0] = 0
    assert lib.disc_b200_qconv2d(ctypes.byref(a), None) == 0                    # empty batch


def test_observers(lib):
    f = lib.disc_b200_observe_minmax
    assert lib.disc_b200_observe_minmax_scratch_floats(1, 1, 16384) == 2
    assert lib.disc_b200_observe_minmax_scratch_floats(1, 1, 16385) == 4
    assert lib.disc_b200_observe_minmax_scratch_floats(3, 5, 1 << 30) == 2 * 5 * 1024   # capped blocks per channel
    assert lib.disc_b200_observe_minmax_scratch_floats(0, 5, 7) == 0
    assert f(0x1000, L.F32, -1, 1, 4, 0x1000, 0x1000, 0x1000, 8, None) != 0 and "negative size" in _err(lib)
    assert f(0x1000, L.F32, 0, 1, 4, 0x1000, 0x1000, 0x1000, 8, None) == 0     # nothing observed
    assert f(None, L.F32, 1, 1, 4, 0x1000, 0x1000, 0x1000, 8, None) != 0 and "null operand" in _err(lib)
    assert f(0x1000, L.F32, 1, 70000, 4, 0x1000, 0x1000, 0x1000, 1 << 20, None) != 0 and "65535 channels" in _err(lib)
    assert f(0x1000, L.F32, 1, 2, 4, 0x1000, 0x1000, 0x1000, 3, None) != 0 and "scratch" in _err(lib)
    assert f(0x1000, 9, 1, 2, 4, 0x1000, 0x1000, 0x1000, 4, None) != 0 and "element type" in _err(lib)
    q = lib.disc_b200_minmax_qparams
    assert q(0x1000, 0x1000, -1, -128, 127, 1, 0, 0x1000, 0x1000, None) != 0 and "invalid channel count" in _err(lib)
    assert q(0x1000, 0x1000, 4, 5, 5, 1, 0, 0x1000, 0x1000, None) != 0 and "quantized range" in _err(lib)
    assert q(0x1000, 0x1000, 0, -128, 127, 1, 0, 0x1000, 0x1000, None) == 0
    assert q(None, 0x1000, 4, -128, 127, 1, 0, 0x1000, 0x1000, None) != 0 and "null operand" in _err(lib)


def test_weight_only_plan_invariants(lib):
    """The launch plan of the weight-only linear over a sweep of shapes: every k row is covered, blocks get whole
    steps, shared memory fits, the cluster is a portable size, and long K falls back to fewer rows per pass."""
    def plan(m, n, k, align=16, sms=148):
        out = (ctypes.c_int64 * 7)()
        rc = lib.disc_b200_weight_only_qgemm_plan(m, n, k, align, sms, out)
        return rc, list(out)

    steps = {(16, 1): 8 * 4 * 8, (16, 2): 8 * 4 * 8, (8, 4): 8 * 2 * 8, (4, 8): 8 * 1 * 16, (4, 16): 8 * 1 * 8}
    for m in (1, 2, 3, 4, 5, 8, 9, 16, 17, 100):
        for n in (8, 128, 264, 4096, 11008, 12288, 32000):
            for k in (1, 64, 100, 4096, 11008, 28672):
                for align in (4, 8, 16):
                    rc, (group, mt, c, strips, cluster, kc, smem) = plan(m, n, k, align)
                    assert rc == 0, (m, n, k, align)
                    rows = min(group, m)
                    assert group in (1, 2, 4, 8, 16) and mt >= rows and mt in (1, 2, 4, 8, 16)
                    assert c <= align and c in (4, 8, 16) and mt * c <= 64          # accumulators per lane
                    assert strips == (n + 127) // 128
                    assert cluster in (1, 2, 4, 8) and cluster * kc >= k
                    step = 8 * (c // 4) * {16: 8, 8: 8, 4: 16 if mt <= 8 else 8}[c]
                    assert kc % step == 0 and kc >= step
                    assert (cluster - 1) * kc < k or cluster == 1                   # no block without rows
                    assert smem <= 200 * 1024
                    assert smem == 4 * (mt * 128 + max(mt * kc, 8 * mt * 128))
    assert (16, 1) in steps                                                         # (documentation of the table above)
    # the 7B shapes the kernel was measured on keep 16 rows per pass and fill the GPU in one wave
    for n, k in ((4096, 4096), (11008, 4096), (4096, 11008)):
        rc, (group, mt, c, strips, cluster, kc, smem) = plan(16, n, k)
        assert group == 16 and strips * cluster <= 2 * 148
        rc, p1 = plan(1, n, k)
        assert p1[2] == 16 and 148 <= p1[3] * p1[4] <= 2 * 148
    # a 70B-sized down projection: 16 rows of 28672 / 8 activations do not fit, 8 rows do
    rc, (group, mt, *_rest) = plan(16, 8192, 28672)
    assert rc == 0 and group == 8 and mt == 8
    # K so long that a single row's chunk does not fit
    assert plan(1, 128, 1 << 22)[0] == 2
    assert plan(0, 128, 128)[0] == 1 and plan(1, 128, 128, align=3)[0] == 1


def test_attention_work_list():
    """Host-side work list of the fused attention: items of 1, 2 or 4 query blocks, longest first, every query
    block of every sequence exactly once."""
    from bladedisc_b200 import ops
    lens = [512, 16, 129, 300, 128, 1]
    for group in (1, 2, 4):
        b = ops.attention_blocks(lens, heads=12, group=group).tolist()
        starts = [0, 512, 528, 657, 957, 1085]
        seen = set()
        for tok0, n, q0, nq in b:
            i = starts.index(tok0)
            assert n == lens[i] and q0 % 128 == 0 and 1 <= nq <= group
            for blk in range(q0 // 128, q0 // 128 + nq):
                assert blk * 128 < n and (i, blk) not in seen
                seen.add((i, blk))
        assert len(seen) == sum((n + 127) // 128 for n in lens)
        cost = [n * nq for _, n, _, nq in b]
        assert cost == sorted(cost, reverse=True)
    with pytest.raises(ValueError):
        ops.attention_blocks([513])
    with pytest.raises(ValueError):
        ops.attention_blocks([0])
