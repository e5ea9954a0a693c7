"""Per-kernel sweep: every (M, K, N) point of the quantized-linear configuration
and the bandwidth kernels, with achieved TOPS / GB/s and the roofline fraction.

    python -m bladedisc_b200.kernel_bench [--quick] [--json out.json] [--only a,b] [--shape M,K,N] [--eager]

Timing: CUDA events on the launching stream around `iters` back-to-back
launches after 3 warm-ups.  Operand sets rotate through copies whose total
footprint exceeds the 126 MB L2, so no launch finds its operands cached by
the previous one.  Peaks come from MEASURED_PEAKS.json when it is present.
"""
import argparse
import json
from pathlib import Path

import torch

from . import ops

ROOT = Path(__file__).resolve().parent.parent
L2_BYTES = 126 << 20
MS = [1, 7, 64, 333, 1024, 4096, 16384]
KNS = [(768, 768), (768, 3072), (3072, 768), (4096, 4096), (4096, 11008), (11008, 4096)]


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d["hbm_gbs"], 2.0 * d["bf16_tflops"], "measured"
    return 6650.0, 2.0 * 1590.0, "fallback"


EAGER = False


def time_ms(fns, iters):
    """Average ms per launch; `fns` is a list of closures over rotating operand sets.

    The launches are captured into one CUDA graph and replayed, so that the
    host's per-call overhead (tens of microseconds from Python) does not hide
    kernels that run for a few microseconds; if capture fails the launches are
    issued eagerly.
    """
    n = len(fns)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for i in range(min(3, n) + 2):
            fns[i % n]()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    graph = None
    try:
        if EAGER:
            raise RuntimeError("eager timing requested")
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for i in range(iters):
                fns[i % n]()
        graph.replay()
        torch.cuda.synchronize()
    except Exception:
        graph = None
        torch.cuda.synchronize()
    if graph is not None:
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters
    e0.record()
    for i in range(iters):
        fns[i % n]()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def copies_for(nbytes):
    return max(2, min(400, (2 * L2_BYTES + nbytes - 1) // max(nbytes, 1)))


def bench_int_mm(M, K, N, iters):
    """cuBLASLt's int8 GEMM with int32 output (torch._int_mm), the library call the reference's GPU custom call
    makes (quantized_gpu_kernel_impl.cc:130-159): the kernel to compare with, not part of this library.
    Returns microseconds per launch, or None for shapes the library call does not take."""
    if M <= 16 or K % 8 or N % 8 or not hasattr(torch, "_int_mm"):
        return None
    dev = "cuda"
    n_sets = copies_for(M * K + N * K + 4 * M * N)
    g = torch.Generator(device=dev).manual_seed(M + K + N)
    sets = [(torch.randint(-127, 128, (M, K), dtype=torch.int8, device=dev, generator=g),
             torch.randint(-127, 128, (N, K), dtype=torch.int8, device=dev, generator=g),
             torch.empty((M, N), dtype=torch.int32, device=dev)) for _ in range(n_sets)]
    try:
        fns = [(lambda a=a, w=w, o=o: torch._int_mm(a, w.t(), out=o)) for a, w, o in sets]
        return time_ms(fns, iters) * 1e3
    except Exception:
        torch.cuda.synchronize()
        return None


def bench_qgemm(M, K, N, out_dtype, hbm, tops_peak, iters, exact=False, path=None):
    dev = "cuda"
    b_out = 1 if out_dtype == torch.int8 else 2
    algo_bytes = M * K + N * K + M * N * b_out + 8 * N
    n_sets = copies_for(algo_bytes)
    g = torch.Generator(device=dev).manual_seed(M + K + N)
    sets = []
    for _ in range(n_sets):
        a = torch.randint(-127, 128, (M, K), dtype=torch.int8, device=dev, generator=g)
        w = torch.randint(-127, 128, (N, K), dtype=torch.int8, device=dev, generator=g)
        o = torch.empty((M, N), dtype=out_dtype, device=dev)
        sets.append((a, w, o))
    sw = torch.rand(N, device=dev, generator=g) * 9e-3 + 1e-3
    bias = torch.randn(N, device=dev, generator=g) * 0.01
    sx = torch.tensor([0.02], device=dev)
    so = torch.tensor([0.05], device=dev) if out_dtype == torch.int8 else None
    torch.cuda.synchronize()  # the weights are final from here on, as inference weights are
    fns = [(lambda a=a, w=w, o=o: ops.qgemm(a, w, x_scale=sx, w_scale=sw, out_scale=so, bias=bias,
                                            out_dtype=out_dtype, out=o, weights_static=True,
                                            exact_division=exact, path=path)) for a, w, o in sets]
    ms = time_ms(fns, iters)
    tops = 2.0 * M * N * K / (ms * 1e-3) / 1e12
    gbs = algo_bytes / (ms * 1e-3) / 1e9
    path = path or ops.qgemm_path(M, N, K)
    # the bound that applies: time cannot beat max(ops / tensor peak, bytes / hbm peak)
    t_tensor = 2.0 * M * N * K / (tops_peak * 1e12)
    t_hbm = algo_bytes / (hbm * 1e9)
    bound = "tensor" if t_tensor >= t_hbm else "hbm"
    frac = max(t_tensor, t_hbm) / (ms * 1e-3)
    return {"kernel": f"qgemm_{path}", "M": M, "K": K, "N": N,
            "out": str(out_dtype).split(".")[-1] + ("/exact" if exact else ""), "us": ms * 1e3,
            "tops": tops, "gbs": gbs, "bound": bound, "frac": frac, "sets": n_sets}


def bench_weight_only(M, K, N, hbm, iters, path=None):
    """Weight-only linear: algorithmic bytes = the uint8 weights once + activations in and out + per-column vectors."""
    dev = "cuda"
    algo_bytes = K * N + 2 * M * K + 2 * M * N + (2 + 4 + 2) * N
    n_sets = copies_for(algo_bytes)
    g = torch.Generator(device=dev).manual_seed(M + K + N)
    sets = []
    for _ in range(n_sets):
        x = torch.randn((M, K), dtype=torch.float16, device=dev, generator=g)
        w = torch.randint(0, 256, (K, N), dtype=torch.uint8, device=dev, generator=g)
        o = torch.empty((M, N), dtype=torch.float16, device=dev)
        sets.append((x, w, o))
    scale = (torch.rand(N, device=dev, generator=g) * 0.02 + 0.002).half()
    zp = torch.full((N,), 128, dtype=torch.int32, device=dev)
    bias = torch.randn(N, device=dev, generator=g).half()
    torch.cuda.synchronize()
    fns = [(lambda x=x, w=w, o=o: ops.weight_only_qgemm(x, w, scale, zp, bias, out=o, path=path)) for x, w, o in sets]
    ms = time_ms(fns, iters)
    gbs = algo_bytes / (ms * 1e-3) / 1e9
    return {"kernel": "weight_only_qgemm", "M": M, "K": K, "N": N, "out": "float16/" + (path or "auto"), "us": ms * 1e3,
            "tops": 2.0 * M * N * K / (ms * 1e-3) / 1e12, "gbs": gbs, "bound": "hbm", "frac": gbs / hbm, "sets": n_sets}


def bench_qconv(n, h, w, c, o, k, stride, hbm, tops_peak, iters):
    """int8 NHWC convolution, SAME padding: algorithmic bytes = input + kernel + output once."""
    dev = "cuda"
    oh, ow = (h + stride - 1) // stride, (w + stride - 1) // stride
    algo_bytes = n * h * w * c + o * k * k * c + n * oh * ow * o + 4 * o
    n_sets = copies_for(algo_bytes)
    g = torch.Generator(device=dev).manual_seed(n + h + c + o)
    xs = [torch.randint(-127, 128, (n, h, w, c), dtype=torch.int8, device=dev, generator=g) for _ in range(n_sets)]
    wt = torch.randint(-127, 128, (o, k, k, c), dtype=torch.int8, device=dev, generator=g)
    sw = torch.rand(o, device=dev, generator=g) * 4e-3 + 1e-3
    sx, so = torch.tensor([0.02], device=dev), torch.tensor([0.1], device=dev)
    torch.cuda.synchronize()
    fns = [(lambda x=x: ops.qconv2d(x, wt, sx, sw, so, "NHWC", [stride], [1], "SAME")) for x in xs]
    ms = time_ms(fns, iters)
    macs = n * oh * ow * o * k * k * c
    t_tensor = 2.0 * macs / (tops_peak * 1e12)
    t_hbm = algo_bytes / (hbm * 1e9)
    return {"kernel": "qconv2d", "M": n * oh * ow, "K": k * k * c, "N": o, "out": "int8", "us": ms * 1e3,
            "tops": 2.0 * macs / (ms * 1e-3) / 1e12, "gbs": algo_bytes / (ms * 1e-3) / 1e9,
            "bound": "tensor" if t_tensor >= t_hbm else "hbm", "frac": max(t_tensor, t_hbm) / (ms * 1e-3), "sets": n_sets}


def bench_observer(shape, axis, dtype, hbm, iters):
    """Min / max observer: one read of the tensor."""
    from bladedisc_b200.observer import MinMaxObserver, PerChannelMinMaxObserver
    dev = "cuda"
    nbytes = int(torch.tensor(shape).prod()) * (2 if dtype == torch.float16 else 4)
    n_sets = copies_for(nbytes)
    g = torch.Generator(device=dev).manual_seed(7)
    xs = [torch.randn(shape, device=dev, generator=g).to(dtype) for _ in range(n_sets)]
    ob = MinMaxObserver() if axis is None else PerChannelMinMaxObserver(ch_axis=axis)
    ob(xs[0])
    torch.cuda.synchronize()
    fns = [(lambda x=x: ob(x)) for x in xs]
    ms = time_ms(fns, iters)
    gbs = nbytes / (ms * 1e-3) / 1e9
    return {"kernel": "observe_minmax" + ("" if axis is None else f"_axis{axis}"), "rows": shape[0], "cols": shape[-1],
            "dtype": str(dtype).split(".")[-1], "us": ms * 1e3, "gbs": gbs, "frac": gbs / hbm}


def bench_rows(name, rows, cols, dtype, hbm, iters):
    dev = "cuda"
    eb = 2 if dtype == torch.float16 else 4
    E = rows * cols
    g = torch.Generator(device=dev).manual_seed(rows + cols)
    if name == "quantize":
        algo = eb * E + E
    elif name == "dynamic_quantize":
        algo = eb * E + E + 4 * rows
    elif name == "layernorm":
        algo = 2 * eb * E + 2 * eb * cols
    elif name == "add_layernorm_quant":
        algo = 3 * eb * E + E + 2 * eb * cols
    elif name == "rmsnorm_dynquant":
        algo = eb * E + E + 4 * rows + eb * cols
    elif name == "softmax":
        algo = 2 * eb * E
    elif name == "swiglu_rowscale":      # pass 0 of the two-pass quantization of silu(gate) * up
        algo = 2 * eb * E + 4 * rows
    elif name == "swiglu_quantize":      # pass 1
        algo = 2 * eb * E + E + 4 * rows
    else:
        raise ValueError(name)
    n_sets = copies_for(algo)
    if name.startswith("swiglu"):
        bufs = [torch.randn((rows, 2 * cols), device=dev, generator=g).to(dtype) for _ in range(n_sets)]
        scales = [ops.row_scale_local(b[:, :cols], b[:, cols:]) for b in bufs]
        outs = [torch.empty((rows, cols), dtype=torch.int8, device=dev) for _ in bufs]
        if name == "swiglu_rowscale":
            fns = [(lambda b=b: ops.row_scale_local(b[:, :cols], b[:, cols:])) for b in bufs]
        else:
            fns = [(lambda b=b, s=s, o=o: ops.quantize_rows(b[:, :cols], s, b[:, cols:], out=o))
                   for b, s, o in zip(bufs, scales, outs)]
        ms = time_ms(fns, iters)
        gbs = algo / (ms * 1e-3) / 1e9
        return {"kernel": name, "rows": rows, "cols": cols, "dtype": str(dtype).split(".")[-1], "us": ms * 1e3,
                "gbs": gbs, "bound": "hbm", "frac": gbs / hbm, "sets": n_sets}
    xs = [torch.randn((rows, cols), device=dev, generator=g).to(dtype) for _ in range(n_sets)]
    rs = [torch.randn((rows, cols), device=dev, generator=g).to(dtype) for _ in range(n_sets)] \
        if name == "add_layernorm_quant" else None
    gamma = torch.ones(cols, dtype=dtype, device=dev)
    beta = torch.zeros(cols, dtype=dtype, device=dev)
    s = torch.tensor([0.03], device=dev)
    if name == "quantize":
        fns = [(lambda x=x: ops.quantize(x, s)) for x in xs]
    elif name == "dynamic_quantize":
        fns = [(lambda x=x: ops.dynamic_quantize(x)) for x in xs]
    elif name == "layernorm":
        fns = [(lambda x=x: ops.layernorm(x, gamma, beta)) for x in xs]
    elif name == "add_layernorm_quant":
        fns = [(lambda x=x, r=r: ops.layernorm_quant(x, gamma, beta, s, residual=r)) for x, r in zip(xs, rs)]
    elif name == "rmsnorm_dynquant":
        fns = [(lambda x=x: ops.rmsnorm_dynamic_quant(x, gamma)) for x in xs]
    else:
        fns = [(lambda x=x: ops.softmax(x, scale=0.125)) for x in xs]
    ms = time_ms(fns, iters)
    gbs = algo / (ms * 1e-3) / 1e9
    return {"kernel": name, "rows": rows, "cols": cols, "dtype": str(dtype).split(".")[-1], "us": ms * 1e3,
            "gbs": gbs, "bound": "hbm", "frac": gbs / hbm, "sets": n_sets,
            "note": "timing includes torch's allocation of the outputs"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--quick", action="store_true", help="a few points only")
    ap.add_argument("--json", default=None)
    ap.add_argument("--only", default=None, help="comma-separated substrings: run only the cases whose kernel name contains one (qgemm, quantize, norm, softmax ...)")
    ap.add_argument("--eager", action="store_true", help="no CUDA graph (for ncu captures); few iterations")
    ap.add_argument("--shape", default=None, help="M,K,N: only this quantized-linear point (with --only qgemm)")
    ap.add_argument("--min-rows", type=int, default=0, help="quantized-linear points with at least this many rows")
    ap.add_argument("--max-rows", type=int, default=1 << 30, help="quantized-linear points with at most this many rows")
    ap.add_argument("--path", default=None, help="force a quantized-linear path (tiled, pair, skinny, small_m, gemv)")
    ap.add_argument("--woq-path", default=None, help="weight-only linear: stream or tensor (default: both up to 16 rows, the library's choice above)")
    ap.add_argument("--exact", action="store_true", help="also time int8 output with the exact-division epilogue")
    ap.add_argument("--int-mm", action="store_true", help="also time cuBLASLt int8 -> int32 (torch._int_mm) per point")
    args = ap.parse_args()
    global EAGER
    EAGER = args.eager
    only = [o for o in (args.only or "").split(",") if o]
    hbm, tops_peak, src = peaks()
    out = {"peaks": {"hbm_gbs": hbm, "int8_tops": tops_peak, "source": src}, "rows": []}
    ms_list = [7, 64, 4096] if args.quick else MS
    kns = [(768, 3072), (4096, 4096)] if args.quick else KNS
    if args.shape:
        m, k, n = (int(v) for v in args.shape.split(","))
        ms_list, kns = [m], [(k, n)]
    print(f"# peaks ({src}): HBM {hbm:.0f} GB/s, int8 tensor {tops_peak:.0f} TOPS (2 x bf16)")
    print(f"{'kernel':<16}{'M':>6}{'K':>6}{'N':>7}{'out':>14}{'us':>10}{'TOPS':>9}{'GB/s':>9}{'bound':>8}{'frac':>7}"
          + (f"{'int_mm us':>11}{'vs':>6}" if args.int_mm else ""))
    ms_list = [m for m in ms_list if args.min_rows <= m <= args.max_rows]
    for K, N in kns:
        for M in ms_list:
            if only and "qgemm" not in only:
                continue
            iters = 200 if M <= 1024 else 30
            if args.eager:
                iters = 3
            lib_us = bench_int_mm(M, K, N, iters) if args.int_mm else None
            for od, exact in ((torch.int8, False), (torch.int8, True), (torch.float16, False)):
                if exact and not args.exact:
                    continue
                r = bench_qgemm(M, K, N, od, hbm, tops_peak, iters, exact, args.path)
                if lib_us:
                    r["int_mm_us"] = lib_us
                out["rows"].append(r)
                print(f"{r['kernel']:<16}{M:>6}{K:>6}{N:>7}{r['out']:>14}{r['us']:>10.2f}{r['tops']:>9.1f}{r['gbs']:>9.0f}"
                      f"{r['bound']:>8}{r['frac']:>7.2f}"
                      + (f"{lib_us:>11.2f}{lib_us / r['us']:>6.2f}" if lib_us else ""), flush=True)
    if not only or any("weight_only" in o for o in only):
        wo_ms = [1, 4, 16] if args.quick else [1, 2, 4, 8, 16, 64, 256, 2048]
        wo_kns = [(4096, 4096)] if args.quick else [(4096, 4096), (4096, 11008), (11008, 4096), (4096, 12288)]
        if args.shape:
            wo_ms, wo_kns = ms_list, kns
        for K, N in wo_kns:
            for M in wo_ms:
                for wpath in ([args.woq_path] if args.woq_path else ([None] if M > 16 else ["stream", "tensor"])):
                    r = bench_weight_only(M, K, N, hbm, 3 if args.eager else (100 if M <= 256 else 20), wpath)
                    out["rows"].append(r)
                    print(f"{r['kernel']:<18}{M:>5}{K:>6}{N:>7}{r['out']:>16}{r['us']:>10.2f}{r['tops']:>9.1f}{r['gbs']:>9.0f}"
                          f"{r['bound']:>8}{r['frac']:>7.2f}", flush=True)
    if only and any("qconv" in o for o in only):
        # (batch, height, width, channels in, channels out, window, stride): ResNet-50-shaped layers
        for n, h, w, c, o, k, st in ((32, 56, 56, 64, 64, 3, 1), (32, 28, 28, 128, 128, 3, 1), (32, 14, 14, 256, 256, 3, 1),
                                     (32, 56, 56, 64, 256, 1, 1), (32, 56, 56, 256, 128, 1, 2)):
            r = bench_qconv(n, h, w, c, o, k, st, hbm, tops_peak, 3 if args.eager else 30)
            out["rows"].append(r)
            print(f"{r['kernel']:<16}{r['M']:>7}{r['K']:>6}{r['N']:>6}{r['out']:>9}{r['us']:>10.2f}{r['tops']:>9.1f}{r['gbs']:>9.0f}"
                  f"{r['bound']:>8}{r['frac']:>7.2f}", flush=True)
    if only and any("observe" in o for o in only):
        for shape, axis, dt in (((16384, 4096), None, torch.float16), ((16384, 4096), None, torch.float32),
                                ((4096, 4096), 0, torch.float32), ((16384, 768), 1, torch.float16)):
            r = bench_observer(shape, axis, dt, hbm, 3 if args.eager else 50)
            out["rows"].append(r)
            print(f"{r['kernel']:<22}{r['rows']:>8}{r['cols']:>7}{r['dtype']:>9}{r['us']:>10.2f}{r['gbs']:>9.0f}{r['frac']:>7.2f}",
                  flush=True)
    row_cases = [("quantize", 16384, 768, torch.float32), ("quantize", 16384, 3072, torch.float16),
                 ("dynamic_quantize", 16384, 4096, torch.float16), ("layernorm", 16384, 768, torch.float16),
                 ("add_layernorm_quant", 16384, 768, torch.float16), ("add_layernorm_quant", 32768, 1024, torch.float16),
                 ("rmsnorm_dynquant", 16384, 4096, torch.float16), ("softmax", 32 * 12 * 512, 512, torch.float16),
                 ("softmax", 196608, 128, torch.float16),
                 ("swiglu_rowscale", 16384, 11008, torch.float16), ("swiglu_quantize", 16384, 11008, torch.float16)]
    if args.quick:
        row_cases = row_cases[:1] + row_cases[3:5] + row_cases[7:8]
    print(f"{'kernel':<22}{'rows':>8}{'cols':>7}{'dtype':>9}{'us':>10}{'GB/s':>9}{'frac':>7}")
    for name, rows, cols, dt in row_cases:
        if only and not any(o in name for o in only):
            continue
        r = bench_rows(name, rows, cols, dt, hbm, 3 if args.eager else 50)
        out["rows"].append(r)
        print(f"{name:<22}{rows:>8}{cols:>7}{r['dtype']:>9}{r['us']:>10.2f}{r['gbs']:>9.0f}{r['frac']:>7.2f}", flush=True)
    st = ops.kernel_status()
    print("kernel_status", st)
    if args.json:
        Path(args.json).write_text(json.dumps(out, indent=1))


if __name__ == "__main__":
    main()
