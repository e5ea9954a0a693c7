"""Generates tests/golden/observer_golden.npz from the reference's own observers.

Run where the reference tree is checked out (it imports the reference's Python
front end and CPU torch):

    python tests/golden/make_observer_golden.py

Stored: seeded calibration batches together with the running min / max, scale and
zero point that the reference's MinMaxObserver / PerChannelMinMaxObserver
(tools/torch_quant/torch_quant/observer.py:230-297) hold after observing them, for
the symmetric signed, affine unsigned and per-channel schemes; and for its
HistogramObserver (observer.py:447-744) the histogram and range after every batch
and the clipping range, scale and zero point its search arrives at.
"""
import os
import sys
import types
from pathlib import Path

import numpy as np
import torch

OUT = Path(__file__).resolve().parent / "observer_golden.npz"
REF_TQ = Path(os.environ.get("DISC_REFERENCE_ROOT", "/root/reference")) / "tools" / "torch_quant"


def main():
    sys.path.insert(0, str(REF_TQ))
    for name in ("torch_quant.mnn", "torch_quant.mnn.export", "torch_quant.mnn.MNN_compression_pb2"):
        sys.modules.setdefault(name, types.ModuleType(name))  # needs `onnx`, absent here
    from torch_quant.observer import HistogramObserver, MinMaxObserver, PerChannelMinMaxObserver

    g = torch.Generator().manual_seed(77)
    out = {}
    # activations: three batches with a drifting offset, so that min, max and the zero point all move
    acts = [torch.randn(3, 50, 96, generator=g) * (1 + i) + 0.7 * i for i in range(3)]
    out["act_batches"] = torch.stack(acts).numpy()
    for tag, kwargs in (("sym", dict(dtype=torch.qint8, qscheme=torch.per_tensor_symmetric)),
                        ("affine", dict(dtype=torch.quint8, qscheme=torch.per_tensor_affine)),
                        ("affine_s8", dict(dtype=torch.qint8, qscheme=torch.per_tensor_affine))):
        ob = MinMaxObserver(**kwargs)
        ob.set_mode(observe=True, fake_quant=False)
        for a in acts:
            ob(a)
        out[f"act_{tag}_min"] = ob.min_val.reshape(1).numpy()
        out[f"act_{tag}_max"] = ob.max_val.reshape(1).numpy()
        out[f"act_{tag}_scale"] = ob.scale.reshape(1).numpy()
        out[f"act_{tag}_zp"] = ob.zero_point.reshape(1).numpy().astype(np.int32)
    # only positive values: the range is widened to include zero
    pos = torch.rand(4, 33, generator=g) + 0.25
    ob = MinMaxObserver(dtype=torch.quint8, qscheme=torch.per_tensor_affine)
    ob.set_mode(observe=True, fake_quant=False)
    ob(pos)
    out.update({"pos_x": pos.numpy(), "pos_scale": ob.scale.reshape(1).numpy(),
                "pos_zp": ob.zero_point.reshape(1).numpy().astype(np.int32)})
    # weights: per output channel (axis 0) and per input channel (axis 1) of the same matrix, and a
    # rank-4 kernel along its last axis
    w = torch.randn(40, 72, generator=g) * 0.05
    k4 = torch.randn(3, 3, 10, 6, generator=g)
    out.update({"w": w.numpy(), "k4": k4.numpy()})
    for tag, t, axis, kwargs in (("w_ax0", w, 0, dict()), ("w_ax1", w, 1, dict()),
                                 ("k4_ax3", k4, 3, dict()),
                                 ("w_ax0_affine", w, 0, dict(dtype=torch.quint8, qscheme=torch.per_channel_affine))):
        ob = PerChannelMinMaxObserver(ch_axis=axis, **kwargs)
        ob.set_mode(observe=True, fake_quant=False)
        ob(t)
        ob(t * 0.5 + 0.01)      # a second batch inside the first one's range, shifted
        out[f"{tag}_min"] = ob.min_val.numpy()
        out[f"{tag}_max"] = ob.max_val.numpy()
        out[f"{tag}_scale"] = ob.scale.numpy()
        out[f"{tag}_zp"] = ob.zero_point.numpy().astype(np.int32)
    # histogram observer (observer.py:447-744): state after every batch and the searched range at the end.
    # Case a: each batch widens the range (the old histogram is re-gridded); case b: the second and third
    # batch stay inside the first one's range; case c: a long-tailed distribution, where the search clips.
    hist_cases = {
        "a": [torch.randn(4, 300, generator=g) * (1 + 0.5 * i) + 0.3 * i for i in range(3)],
        "b": [torch.randn(2000, generator=g) * 2, torch.randn(2000, generator=g) * 0.5, torch.rand(777, generator=g)],
        "c": [torch.randn(5000, generator=g) ** 3, torch.randn(5000, generator=g) ** 3 * 0.9],
    }
    for tag, batches in hist_cases.items():
        for kind, kwargs in (("affine", dict(dtype=torch.quint8, qscheme=torch.per_tensor_affine)),
                             ("sym", dict(dtype=torch.qint8, qscheme=torch.per_tensor_symmetric))):
            ob = HistogramObserver(**kwargs)
            ob.set_mode(observe=True, fake_quant=False)
            for i, b in enumerate(batches):
                ob(b)
                if kind == "affine":
                    out[f"hist_{tag}_batch{i}"] = b.numpy()
                    out[f"hist_{tag}_after{i}_hist"] = ob.histogram.numpy().copy()
                    out[f"hist_{tag}_after{i}_minmax"] = np.array([float(ob.min_val), float(ob.max_val)], np.float32)
            new_min, new_max = ob._non_linear_param_search()
            ob._calculate()
            out[f"hist_{tag}_{kind}_range"] = np.array([float(new_min), float(new_max)], np.float32)
            out[f"hist_{tag}_{kind}_scale"] = ob.scale.reshape(1).numpy().copy()
            out[f"hist_{tag}_{kind}_zp"] = ob.zero_point.reshape(1).numpy().astype(np.int32)
        out[f"hist_{tag}_batches"] = np.array([len(batches)], np.int32)
    np.savez_compressed(OUT, **out)
    print("wrote", OUT, OUT.stat().st_size, "bytes;", len(out), "arrays")


if __name__ == "__main__":
    main()
