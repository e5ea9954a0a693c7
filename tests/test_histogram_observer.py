"""Host logic of the histogram observer and the numpy statement of torch.histc, on the CPU.

The golden file holds what the reference's own HistogramObserver (tools/torch_quant/torch_quant/observer.py:447-744)
held after every calibration batch (histogram, range) and what its search settled on (clipping range, scale, zero
point).  Here the same batches go through this repository's host functions with the bin counts taken from the numpy
restatement of torch.histc; the GPU test (tests/test_gpu_observer.py) repeats it with the CUDA kernel doing the counting.
"""
import numpy as np
import pytest
import torch

GOLD = None


@pytest.fixture(scope="module")
def gold():
    from pathlib import Path
    return np.load(Path(__file__).parent / "golden" / "observer_golden.npz")


def test_histc_restatement_is_torch_histc():
    from oracle import np_ref
    rng = np.random.default_rng(0)
    for n, lo, hi, bins in ((10000, -3.0, 2.5, 2048), (5000, 0.0, 1.0, 64), (3000, -1e-3, 7.0, 2048), (100, 2.0, 2.0 + 1e-6, 16)):
        x = (rng.standard_normal(n) * (hi - lo) / 3 + (hi + lo) / 2).astype(np.float32)
        x[:7] = [lo, hi, np.nextafter(np.float32(lo), np.float32(-np.inf)), np.nextafter(np.float32(hi), np.float32(np.inf)),
                 np.nan, (lo + hi) / 2, lo + (hi - lo) / bins]
        want = torch.histc(torch.from_numpy(x), bins, min=float(np.float32(lo)), max=float(np.float32(hi))).numpy()
        got = np_ref.histc(x, lo, hi, bins)
        assert (got == want.astype(np.int64)).all(), (n, lo, hi, bins)


def _replay(gold, tag, histc):
    """Runs the observer's host logic over the golden batches; `histc(x, lo, hi)` supplies the bin counts."""
    from bladedisc_b200 import observer as O
    F = np.float32
    hist, lo, hi = np.zeros(2048, F), F(np.inf), F(-np.inf)
    for i in range(int(gold[f"hist_{tag}_batches"][0])):
        x = gold[f"hist_{tag}_batch{i}"].reshape(-1)
        if np.isinf(lo) or lo == hi:
            lo, hi = F(x.min()), F(x.max())
            hist = histc(x, lo, hi).astype(F)
        else:
            cmin, cmax = min(F(x.min()), lo), max(F(x.max()), hi)
            cmin, cmax, down, start = O.adjust_min_max(lo, hi, cmin, cmax, 2048, 128)
            new = histc(x, cmin, cmax).astype(F)
            if cmin == lo and cmax == hi:
                hist = (new + hist).astype(F)
            else:
                hist = O.combine_histograms(new, hist, 128, down, start, 2048)
            lo, hi = cmin, cmax
        assert (np.array([lo, hi], F) == gold[f"hist_{tag}_after{i}_minmax"]).all(), f"range after batch {i}"
        assert (hist == gold[f"hist_{tag}_after{i}_hist"]).all(), \
            f"histogram after batch {i}: {np.count_nonzero(hist != gold[f'hist_{tag}_after{i}_hist'])} bins differ"
    return hist, lo, hi


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_host_logic_reproduces_the_reference_observer(gold, tag):
    from bladedisc_b200 import observer as O
    from oracle import np_ref
    hist, lo, hi = _replay(gold, tag, lambda x, a, b: np_ref.histc(x, a, b, 2048))
    new_lo, new_hi = O.nonlinear_param_search(hist, lo, hi, 2048, 256)
    want = gold[f"hist_{tag}_affine_range"]
    assert (np.array([new_lo, new_hi], np.float32) == want).all(), (new_lo, new_hi, want)
    assert (gold[f"hist_{tag}_sym_range"] == want).all()   # the search does not depend on the scheme
    # scale and zero point by the reference's rule for an affine quint8 and a symmetric qint8 scheme
    eps = np.finfo(np.float32).eps
    mn, mx = min(np.float32(new_lo), np.float32(0)), max(np.float32(new_hi), np.float32(0))
    scale = max(np.float32(np.float32(mx - mn) / np.float32(255)), eps)
    zp = int(np.clip(0 - np.rint(np.float32(mn / scale)), 0, 255))
    assert np.float32(scale) == gold[f"hist_{tag}_affine_scale"][0] and zp == int(gold[f"hist_{tag}_affine_zp"][0])
    s_sym = max(np.float32(max(-mn, mx) / np.float32(127.5)), eps)
    assert np.float32(s_sym) == gold[f"hist_{tag}_sym_scale"][0] and int(gold[f"hist_{tag}_sym_zp"][0]) == 0
