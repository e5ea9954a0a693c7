"""GPU calibration observers against what the reference's observers computed
(tests/golden/observer_golden.npz) and against the numpy restatement; bit exact."""
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).parent / "golden"


def _np(t):
    return t.cpu().numpy()


def test_per_tensor_observers_match_the_reference():
    from bladedisc_b200.observer import MinMaxObserver
    g = np.load(GOLD / "observer_golden.npz")
    for tag, kwargs in (("sym", dict(dtype="qint8", symmetric=True)), ("affine", dict(dtype="quint8", symmetric=False)),
                        ("affine_s8", dict(dtype="qint8", symmetric=False))):
        ob = MinMaxObserver(**kwargs)
        for b in g["act_batches"]:
            ob(torch.from_numpy(b).cuda())
        scale, zp = ob.qparams()
        assert (_np(ob.min_val) == g[f"act_{tag}_min"]).all() and (_np(ob.max_val) == g[f"act_{tag}_max"]).all()
        assert (_np(scale) == g[f"act_{tag}_scale"]).all() and (_np(zp) == g[f"act_{tag}_zp"]).all()
    ob = MinMaxObserver(dtype="quint8", symmetric=False)
    ob(torch.from_numpy(g["pos_x"]).cuda())
    scale, zp = ob.qparams()
    assert (_np(scale) == g["pos_scale"]).all() and (_np(zp) == g["pos_zp"]).all()
    q = np.load(GOLD / "qpath_golden.npz")          # the calibration of the encoder goldens
    ob = MinMaxObserver()
    for b in q["tq_calib"]:
        ob(torch.from_numpy(b).cuda())
    assert (_np(ob.qparams()[0]) == q["tq_s_x"]).all()


def test_per_channel_observers_match_the_reference():
    from bladedisc_b200.observer import PerChannelMinMaxObserver
    g = np.load(GOLD / "observer_golden.npz")
    for tag, key, axis, kwargs in (("w_ax0", "w", 0, {}), ("w_ax1", "w", 1, {}), ("k4_ax3", "k4", 3, {}),
                                   ("w_ax0_affine", "w", 0, dict(dtype="quint8", symmetric=False))):
        t = torch.from_numpy(g[key]).cuda()
        ob = PerChannelMinMaxObserver(ch_axis=axis, **kwargs)
        ob(t)
        ob(t * 0.5 + 0.01)
        scale, zp = ob.qparams()
        assert (_np(ob.min_val) == g[f"{tag}_min"]).all() and (_np(ob.max_val) == g[f"{tag}_max"]).all()
        assert (_np(scale) == g[f"{tag}_scale"]).all() and (_np(zp) == g[f"{tag}_zp"]).all()


@pytest.mark.parametrize("shape,axis", [((1 << 22,), None), ((64, 4096), None), ((300, 1000), 0), ((300, 1000), 1),
                                        ((7, 33, 129), 1), ((5, 3, 2, 11), -1)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_large_and_ragged_tensors_match_numpy(shape, axis, dtype):
    """Many blocks per channel, strided channels, fp16 input, two batches."""
    from bladedisc_b200.observer import MinMaxObserver, PerChannelMinMaxObserver
    from oracle import np_ref
    gen = torch.Generator(device="cuda").manual_seed(len(shape) + (axis or 0) + 5)
    batches = [torch.randn(shape, device="cuda", generator=gen).to(dtype) * (i + 1) - i for i in range(2)]
    ob = MinMaxObserver() if axis is None else PerChannelMinMaxObserver(ch_axis=axis)
    for b in batches:
        assert ob(b) is b
    lo, hi = np_ref.observe_minmax([_np(b.float()) for b in batches], ch_axis=axis)
    assert (_np(ob.min_val) == lo).all() and (_np(ob.max_val) == hi).all()
    s, z = np_ref.minmax_qparams(lo, hi)
    scale, zp = ob.qparams()
    assert (_np(scale) == s).all() and (_np(zp) == z).all()


def test_edges():
    from bladedisc_b200.observer import MinMaxObserver, PerChannelMinMaxObserver
    ob = MinMaxObserver()
    scale, zp = ob.qparams()                        # nothing observed: the reference's defaults
    assert float(scale) == 1.0 and int(zp) == 0
    ob(torch.zeros(0, device="cuda"))               # an empty batch changes nothing
    assert float(ob.qparams()[0]) == 1.0
    ob(torch.zeros(5, device="cuda"))               # all zero: scale floored at the float32 epsilon
    assert float(ob.qparams()[0]) == float(np.finfo(np.float32).eps)
    with pytest.raises(ValueError, match="signed"):
        MinMaxObserver(dtype="quint8", symmetric=True)
    with pytest.raises(ValueError, match="CUDA"):
        ob(torch.zeros(4))
    pc = PerChannelMinMaxObserver(ch_axis=0)
    pc(torch.ones(3, 4, device="cuda"))
    with pytest.raises(ValueError, match="channels changed"):
        pc(torch.ones(5, 4, device="cuda"))
    with pytest.raises(TypeError):
        ob(torch.zeros(4, dtype=torch.int32, device="cuda"))


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_histogram_observer_equals_the_reference_observer(tag):
    """State after every batch (2048-bin histogram, range) and the searched clipping range, scale and zero
    point equal what the reference's own HistogramObserver held for the same batches
    (tests/golden/observer_golden.npz, written by tests/golden/make_observer_golden.py)."""
    from pathlib import Path
    from bladedisc_b200.observer import HistogramObserver
    gold = np.load(Path(__file__).parent / "golden" / "observer_golden.npz")
    for kind, kwargs in (("affine", dict(dtype="quint8", symmetric=False)), ("sym", dict(dtype="qint8", symmetric=True))):
        ob = HistogramObserver(**kwargs)
        for i in range(int(gold[f"hist_{tag}_batches"][0])):
            ob(torch.from_numpy(gold[f"hist_{tag}_batch{i}"]).cuda())
            assert (np.array([ob.min_val, ob.max_val], np.float32) == gold[f"hist_{tag}_after{i}_minmax"]).all()
            assert (ob.histogram == gold[f"hist_{tag}_after{i}_hist"]).all(), f"histogram after batch {i}"
        lo, hi = ob.clipping_range()
        assert (np.array([lo, hi], np.float32) == gold[f"hist_{tag}_{kind}_range"]).all()
        scale, zp = ob.qparams()
        assert (scale.cpu().numpy() == gold[f"hist_{tag}_{kind}_scale"]).all()
        assert (zp.cpu().numpy() == gold[f"hist_{tag}_{kind}_zp"]).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("n", [1, 1000, 4 * 1024 * 1024 + 3])
def test_histogram_kernel_counts(dtype, n):
    """The counting kernel against the numpy statement of torch.histc on large, unaligned and f16 tensors, with
    values on the range ends, outside it and NaN."""
    import ctypes
    from bladedisc_b200 import lib as L
    from bladedisc_b200 import ops
    from oracle import np_ref
    g = torch.Generator(device="cuda").manual_seed(n)
    x = (torch.randn(n + 1, generator=g, device="cuda") * 2).to(dtype)[1:]   # not 16-byte aligned
    if n > 8:
        x[:4] = torch.tensor([-3.0, 3.5, float("nan"), 100.0], dtype=dtype)
    lo, hi = np.float32(-3.0), np.float32(3.5)
    counts = torch.zeros(2048, dtype=torch.int32, device="cuda")
    for _ in range(2):   # accumulates
        L.check(L.load().disc_b200_observe_histogram(x.data_ptr(), ops._etype(x), n, float(lo), float(hi), 2048,
                                                     counts.data_ptr(), torch.cuda.current_stream().cuda_stream))
    want = np_ref.histc(x.float().cpu().numpy(), lo, hi, 2048)
    assert (counts.cpu().numpy().astype(np.int64) == 2 * want).all()
