"""Generates tests/golden/qpath_golden.npz.

Run where the reference tree is checked out (REF_TQ below; it imports the
reference's Python front end and CPU torch):

    python tests/golden/make_golden.py

What is stored (seeded inputs together with the outputs of reference code, so
that the tests need neither the reference tree nor torch's RNG to agree):

* fq_linear_*: the golden of the reference's own quantized-linear e2e tests
  (pytorch_blade/tests/disc/pdl/test_e2e/test_quantization.py:357-460): an
  eager ``fake_quantize(x) -> F.linear(fake_quantize(w)) + bias -> fake_quantize``
  with the constants of those tests (s_x = 0.1, s_w = 0.3, s_out in {0.05, 0.1}).
* tq_*: scales computed by the reference's torch_quant observers
  (tools/torch_quant/torch_quant/observer.py) and the output of an MLP
  quantized by them (observer fake-quant mode), per-tensor activations and
  per-channel weights as torch_quant's DISC/x86 backend configures.
* ln_*, sm_*, gelu_*: eager torch layer_norm / softmax / gelu, the golden of
  pytorch_blade/tests/disc/ops/test_layer_norm.py and test_nn_ops.py.
* onednn_*: torch.ops.onednn.qlinear_pointwise (oneDNN, the library the
  reference's x86 custom call uses) on a small int8 case.
"""
import os
import sys
import types
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F

OUT = Path(__file__).resolve().parent / "qpath_golden.npz"
REF_TQ = Path(os.environ.get("DISC_REFERENCE_ROOT", "/root/reference")) / "tools" / "torch_quant"


def fq(x, s, zp=0):
    return torch.fake_quantize_per_tensor_affine(x, s, zp, -128, 127)


def main():
    g = torch.Generator().manual_seed(20240607)
    out = {}

    # ---- reference e2e golden: per-tensor fake-quant linear, rank 2 and rank 3
    for tag, shape, n, k, s_out in (("r2", (48, 64), 80, 64, 0.05), ("r3", (2, 24, 64), 64, 64, 0.1)):
        x = torch.randn(*shape, generator=g)
        w = torch.randn(n, k, generator=g)
        b = torch.randn(n, generator=g)
        s_x, s_w = 0.1, 0.3
        y = fq(F.linear(fq(x, s_x), fq(w, s_w), b), s_out)
        out[f"fq_linear_{tag}_x"] = x.numpy()
        out[f"fq_linear_{tag}_w"] = w.numpy()
        out[f"fq_linear_{tag}_b"] = b.numpy()
        out[f"fq_linear_{tag}_scales"] = np.array([s_x, s_w, s_out], dtype=np.float32)
        out[f"fq_linear_{tag}_y"] = y.numpy()

    # ---- torch_quant observers (the reference's Python front end)
    sys.path.insert(0, str(REF_TQ))
    for name in ("torch_quant.mnn", "torch_quant.mnn.export", "torch_quant.mnn.MNN_compression_pb2"):
        sys.modules.setdefault(name, types.ModuleType(name))  # needs `onnx`, absent here
    from torch_quant.observer import MinMaxObserver, PerChannelMinMaxObserver

    x = torch.randn(4, 16, 64, generator=g)
    w1 = torch.randn(96, 64, generator=g) * 0.02
    b1 = torch.randn(96, generator=g) * 0.01
    w2 = torch.randn(64, 96, generator=g) * 0.02
    b2 = torch.randn(64, generator=g) * 0.01
    calib = [torch.randn(4, 16, 64, generator=g) for _ in range(4)]

    def lin_fp(t):
        h = F.gelu(F.linear(t, w1, b1))
        return h, F.linear(h, w2, b2)

    ob_x, ob_h, ob_y = MinMaxObserver(), MinMaxObserver(), MinMaxObserver()
    ob_g = MinMaxObserver()
    ob_w1, ob_w2 = PerChannelMinMaxObserver(ch_axis=0), PerChannelMinMaxObserver(ch_axis=0)
    for ob in (ob_x, ob_h, ob_y, ob_g, ob_w1, ob_w2):
        ob.set_mode(observe=True, fake_quant=False)
    ob_w1(w1)
    ob_w2(w2)
    for c in calib:
        ob_x(c)
        pre = F.linear(c, w1, b1)
        ob_h(pre)
        hh = F.gelu(pre)
        ob_g(hh)
        ob_y(F.linear(hh, w2, b2))
    for ob in (ob_x, ob_h, ob_y, ob_g, ob_w1, ob_w2):
        ob.set_mode(observe=False, fake_quant=True)
    # x_ob -> fc1 -> fc1_ob -> gelu -> act_ob -> fc2 -> fc2_ob, as torch_quant places observers
    h_pre = ob_h(F.linear(ob_x(x), ob_w1(w1), b1))
    h_act = ob_g(F.gelu(h_pre))
    y = ob_y(F.linear(h_act, ob_w2(w2), b2))
    out.update({
        "tq_x": x.numpy(), "tq_w1": w1.numpy(), "tq_b1": b1.numpy(), "tq_w2": w2.numpy(), "tq_b2": b2.numpy(),
        "tq_calib": torch.stack(calib).numpy(),
        "tq_s_x": ob_x.scale.reshape(1).numpy(), "tq_s_h": ob_h.scale.reshape(1).numpy(),
        "tq_s_g": ob_g.scale.reshape(1).numpy(), "tq_s_y": ob_y.scale.reshape(1).numpy(),
        "tq_s_w1": ob_w1.scale.numpy(), "tq_s_w2": ob_w2.scale.numpy(),
        "tq_h_pre": h_pre.numpy(), "tq_h_act": h_act.numpy(), "tq_y": y.numpy(),
    })

    # ---- eager torch row ops
    xl = torch.randn(6, 10, 96, generator=g) * 2 + 0.5
    gamma = torch.randn(96, generator=g)
    beta = torch.randn(96, generator=g)
    out.update({"ln_x": xl.numpy(), "ln_gamma": gamma.numpy(), "ln_beta": beta.numpy(),
                "ln_y": F.layer_norm(xl, (96,), gamma, beta, 1e-5).numpy()})
    xs = torch.randn(3, 4, 20, 37, generator=g) * 3
    out.update({"sm_x": xs.numpy(), "sm_y": F.softmax(xs, dim=-1).numpy(),
                "sm_logy": F.log_softmax(xs, dim=-1).numpy()})
    xg = torch.randn(5, 33, generator=g) * 2
    out.update({"gelu_x": xg.numpy(), "gelu_y": F.gelu(xg).numpy(), "silu_y": F.silu(xg).numpy()})

    # ---- oneDNN int8 linear (x86 library path of the reference)
    try:
        a = torch.randint(-127, 128, (32, 64), dtype=torch.int8, generator=g)
        wq = torch.randint(-127, 128, (48, 64), dtype=torch.int8, generator=g)
        sw = torch.rand(48, generator=g) * 9e-3 + 1e-3
        bb = torch.randn(48, generator=g) * 0.5
        s_x, s_out = 0.02, 0.05
        packed = torch.ops.onednn.qlinear_prepack(wq.contiguous(), [32, 64])  # weight as [N, K]
        y8 = torch.ops.onednn.qlinear_pointwise(a, s_x, 0, packed, sw, torch.zeros(48, dtype=torch.int64), bb,
                                                s_out, 0, torch.int8, "none", [], "")
        out.update({"onednn_a": a.numpy(), "onednn_w": wq.numpy(), "onednn_sw": sw.numpy(),
                    "onednn_b": bb.numpy(), "onednn_scales": np.array([s_x, s_out], dtype=np.float32),
                    "onednn_y": y8.numpy()})
    except Exception as e:  # keeps the generator usable if the op signature moves
        print("onednn fixture skipped:", e)

    np.savez_compressed(OUT, **out)
    print("wrote", OUT, OUT.stat().st_size, "bytes;", len(out), "arrays")


if __name__ == "__main__":
    main()
