"""Benchmark of the quantized-linear hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one int8 quantized linear over one batch of M activation rows
(the dynamic-shape sweep's largest square point: M = 16384, K = 4096, N = 4096, per-channel
weight scales, fp32 bias, int8 output requantized at 0.05).  With N > 1 ranks
(torchrun) every rank runs the same step on its own rows: the rows of a linear
are independent, so there is no collective and the scaling is "weak".

Prints one JSON line (rank 0).  `value` is device-timed with inputs resident in
HBM; `e2e` is the same metric through the host-buffer API with the host<->device
copies inside the timed region.  `--impl reference` times the CPU stand-in for
the reference's x86 path (oneDNN int8 linear) on the host cores.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

M_ROWS, K_DIM, N_DIM = 16384, 4096, 4096
S_X, S_OUT = 0.02, 0.05
NOMINAL_INT8_TOPS = 4500.0
# dram__bytes_read.sum + dram__bytes_write.sum of one qgemm_pair_kernel launch at the
# bench shape, from the ncu capture summarised under profiles/ (captured at rows=8192: 60.4 MB;
# the activation and output terms scaled by the row count, the weight term kept).
NCU_DRAM_BYTES_PER_LAUNCH = 1.04e8
VERIFY_ROWS = 64


def _args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--rows", type=int, default=M_ROWS, help="activation rows per rank and step")
    ap.add_argument("--skip-cpu-baseline", action="store_true")
    ap.add_argument("--skip-encoder", action="store_true", help="qlinear workload: leave out the BERT-base record")
    ap.add_argument("--shard-of", type=int, default=None,
                    help="encoder workloads on one GPU: run the share rank 0 of this many ranks would get")
    ap.add_argument("--layers", type=int, default=32, help="decoder layers of the llama7b workload")
    ap.add_argument("--tp-row-blocks", type=int, default=None,
                    help="llama7b workload: row blocks per column-parallel linear (gather of one block overlaps "
                         "the next block's GEMM); default: the library's")
    ap.add_argument("--profile", action="store_true",
                    help="for ncu captures: only warm-up and timed steps (no clock hold, e2e or CPU legs)")
    ap.add_argument("--workload", default="qlinear", choices=["qlinear", "bert_base", "bert_large", "llama7b"],
                    help="qlinear (default, configuration 1) or a W8A8 encoder forward (configurations 2 / 3)")
    return ap.parse_args()


def _peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d.get("hbm_gbs"), "bf16": d.get("bf16_tflops"),
                "bf16_sustained": d.get("bf16_tflops_sustained") or d.get("bf16_tflops"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) in a thread while the
    GPU is under load; falls back to polling nvidia-smi."""
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.mask = 0
        self.max_mhz = None
        self._stop = threading.Event()
        self.thread = None
        self.how = None

    def _nvml_loop(self, nv, h):
        while not self._stop.is_set():
            try:
                self.samples.append(float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)))
                self.mask |= int(nv.nvmlDeviceGetCurrentClocksEventReasons(h))
            except Exception:
                pass
            time.sleep(0.01)

    def _smi_loop(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        bits = [0x8, 0x40, 0x20, 0x4]
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-i",
                                      str(self.index)], capture_output=True, text=True, timeout=10).stdout
                parts = [p.strip() for p in out.strip().split(",")]
                self.samples.append(float(parts[0]))
                self.max_mhz = float(parts[1])
                for b, v in zip(bits, parts[2:6]):
                    if v.lower().startswith("active"):
                        self.mask |= b
            except Exception:
                time.sleep(0.05)

    def start(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            uuid = None
            try:
                import torch
                uuid = str(torch.cuda.get_device_properties(self.index).uuid)
            except Exception:
                pass
            h = None
            if uuid:
                for i in range(nv.nvmlDeviceGetCount()):
                    cand = nv.nvmlDeviceGetHandleByIndex(i)
                    u = nv.nvmlDeviceGetUUID(cand)
                    u = u.decode() if isinstance(u, bytes) else u
                    if uuid in u:
                        h = cand
            if h is None:
                h = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            self.how = "nvml"
            self.thread = threading.Thread(target=self._nvml_loop, args=(nv, h), daemon=True)
        except Exception:
            self.how = "nvidia-smi"
            self.thread = threading.Thread(target=self._smi_loop, daemon=True)
        self.thread.start()

    def stop(self):
        self._stop.set()
        if self.thread:
            self.thread.join(timeout=15)
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(n for b, n in self.REASONS.items() if self.mask & b),
                "samples": len(s), "how": self.how}


def _make_problem(torch, rows, device, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    a = torch.randint(-127, 128, (rows, K_DIM), dtype=torch.int8, generator=g)
    w = torch.randint(-127, 128, (N_DIM, K_DIM), dtype=torch.int8, generator=g)
    w_scale = torch.rand(N_DIM, generator=g) * 9e-3 + 1e-3
    bias = torch.randn(N_DIM, generator=g) * 0.01
    return a, w, w_scale, bias


def _cpu_onednn(torch, a, w, w_scale, bias, seconds, threads):
    """oneDNN int8 linear (prepacked weight), the library behind the reference's x86 custom call
    (tao_compiler/mlir/ral/context/common_context_impl_quantization.cc:1268-1400)."""
    torch.set_num_threads(threads)
    packed = torch.ops.onednn.qlinear_prepack(w.contiguous(), list(a.shape))
    zp = torch.zeros(w.shape[0], dtype=torch.int64)

    def run():
        return torch.ops.onednn.qlinear_pointwise(a, S_X, 0, packed, w_scale, zp, bias, S_OUT, 0, torch.int8,
                                                  "none", [], "")
    run()
    n, t0 = 0, time.perf_counter()
    while True:
        run()
        n += 1
        dt = time.perf_counter() - t0
        if dt >= seconds:
            break
    return dt / n


def _cpu_oracle_port(a, w, w_scale, bias, seconds):
    from oracle import c
    a, w = a.numpy(), w.numpy()
    c.qgemm_ral_i8(a[:8], w, S_X, w_scale.numpy(), S_OUT, bias.numpy())
    n, t0 = 0, time.perf_counter()
    while True:
        c.qgemm_ral_i8(a, w, S_X, w_scale.numpy(), S_OUT, bias.numpy())
        n += 1
        dt = time.perf_counter() - t0
        if dt >= seconds:
            break
    return dt / n


def cpu_baseline(torch, seconds=12.0, sample_rows=1024):
    """TOPS of the CPU path on a bounded sample of the same workload (first `sample_rows` rows)."""
    a, w, w_scale, bias = _make_problem(torch, sample_rows, "cpu", 1234 + 1)
    threads = _host_threads()
    ops_ = 2.0 * sample_rows * K_DIM * N_DIM
    try:
        t = _cpu_onednn(torch, a, w, w_scale, bias, seconds, threads)
        engine = "oneDNN int8 matmul via torch.ops.onednn.qlinear_pointwise, prepacked weight"
    except Exception as e:  # op missing on this build of torch: time the C restatement instead
        t = _cpu_oracle_port(a, w, w_scale, bias, seconds)
        engine = f"oracle/qpath_oracle.c (OpenMP); onednn op unavailable: {type(e).__name__}"
    return {"value": ops_ / t / 1e12, "unit": "TOPS", "cores": threads, "kind": "port",
            "sample": f"first {sample_rows} of {M_ROWS} rows x (K={K_DIM}, N={N_DIM}), repeated for {seconds:.0f} s",
            "engine": engine, "ms_per_sample": t * 1e3}


def _host_threads():
    """Threads the CPU arm may use: the cores this process is allowed to run on."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return os.cpu_count() or 1


def _reexec_with_all_threads():
    """A launcher (torch.distributed.run) exports OMP_NUM_THREADS=1 to its workers; the OpenMP runtime
    and oneDNN size their pools from it when they are loaded, before any later call can raise it.  The CPU arm is
    meant to use every host thread it can, so it starts itself again once with the variable set."""
    want = str(_host_threads())
    if os.environ.get("OMP_NUM_THREADS") == want or os.environ.get("DISC_BENCH_CPU_ARM") == "1":
        return
    env = dict(os.environ, OMP_NUM_THREADS=want, MKL_NUM_THREADS=want, DISC_BENCH_CPU_ARM="1")
    os.execve(sys.executable, [sys.executable] + sys.argv, env)


def _workload_config(rows):
    return {"workload": f"cfg1 quantized linear M={rows} K={K_DIM} N={N_DIM}, per-channel w scales, "
                        f"f32 bias, int8 out @ {S_OUT}"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    _reexec_with_all_threads()
    import torch
    sample_rows = 1024
    a, w, w_scale, bias = _make_problem(torch, sample_rows, "cpu", 1234 + 1)
    threads = _host_threads()
    torch.set_num_threads(threads)
    ops_ = 2.0 * sample_rows * K_DIM * N_DIM
    try:
        packed = torch.ops.onednn.qlinear_prepack(w.contiguous(), list(a.shape))
        zp = torch.zeros(N_DIM, dtype=torch.int64)
        step = lambda: torch.ops.onednn.qlinear_pointwise(a, S_X, 0, packed, w_scale, zp, bias, S_OUT, 0,
                                                          torch.int8, "none", [], "")
        engine = "oneDNN int8 matmul via torch.ops.onednn.qlinear_pointwise, prepacked weight"
        step()
    except Exception as e:
        from oracle import c
        an, wn, sn, bn = a.numpy(), w.numpy(), w_scale.numpy(), bias.numpy()
        step = lambda: c.qgemm_ral_i8(an, wn, S_X, sn, S_OUT, bn)
        engine = f"oracle/qpath_oracle.c (OpenMP); onednn op unavailable: {type(e).__name__}"
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    tops = ops_ / dt / 1e12
    cfg = _workload_config(args.rows)
    cfg["sample"] = f"each step times the first {sample_rows} of the {args.rows} rows (TOPS is per operation, so the " \
                    "sample does not change the metric)"
    line = {
        "impl": "reference", "metric": "qgemm_int8_tops", "value": tops, "unit": "TOPS", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "i8", "data": "synthetic",
        "config": cfg,
        "cpu_baseline": {"value": tops, "unit": "TOPS", "cores": threads, "kind": "port", "engine": engine,
                         "threads_used": torch.get_num_threads(),
                         "sample": f"first {sample_rows} of {args.rows} rows per step"},
        "e2e": {"value": tops, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference's own x86 executable cannot be built (oneDNN v2 submodule empty, bazel/TF absent); "
                "this arm runs the same library (oneDNN) on the same int8 operands on all host cores",
    }
    print(json.dumps(line), flush=True)


def _build_boundary_executable(torch, w_h, w_scale_h, bias_h, device):
    """Compiles the stand-in program (bladedisc_b200/standin/qlinear_program.c) with the host compiler, writes
    its constants into a metadata file and opens both the way torch_blade opens an engine."""
    import tempfile
    import numpy as np
    from bladedisc_b200 import metadata as M
    from bladedisc_b200.executable import Executable
    from bladedisc_b200.ral import pack_attrs
    tmp = Path(tempfile.mkdtemp(prefix="disc_b200_bench_"))
    blob = pack_attrs({"activation": "none"})
    (tmp / "attrs_blob.h").write_text("static const unsigned char attrs_blob[] = {" + ",".join(str(b) for b in blob) + "};\n")
    n, k = w_h.shape
    names = {"CONST_W": f"0_i8_{n}x{k}", "CONST_B": f"1_f32_{n}", "CONST_SW": f"3_f32_{n}"}
    so = tmp / "qlinear_program.so"
    cmd = ["gcc", "-shared", "-fPIC", "-O1", "-Wno-main", f"-DATTRS_BLOB_H=\"{tmp / 'attrs_blob.h'}\""]
    cmd += [f"-D{key}=\"{val}\"" for key, val in names.items()]
    cmd += ["-o", str(so), str(ROOT / "bladedisc_b200" / "standin" / "qlinear_program.c")]
    subprocess.run(cmd, check=True, capture_output=True)
    meta = tmp / "meta"
    M.write_metadata(meta, [(names["CONST_W"], False, w_h.numpy()), (names["CONST_B"], False, bias_h.numpy()),
                            ("2_f32_", False, np.float32(S_X)), (names["CONST_SW"], False, w_scale_h.numpy()),
                            ("4_f32_", False, np.float32(S_OUT))])
    return Executable(so, meta, [("i8", "cuda")], device=device)


def _verify_rows(torch, out_d, a_h, w_h, w_scale_h, bias_h, seed):
    """Sampled rows of a step's int8 output against the CPU oracle's statement of the same epilogue
    (divide-based).  The launch uses the reciprocal form, so a value may sit one level off at a rounding
    tie.  Returns (rows checked, largest difference in int8 levels, share of values that differ)."""
    import numpy as np
    from oracle import c
    rows = a_h.shape[0]
    g = torch.Generator().manual_seed(seed)
    pick = torch.unique(torch.cat([torch.tensor([0, rows - 1]), torch.randint(0, rows, (VERIFY_ROWS,), generator=g)]))
    got = out_d[pick.to(out_d.device)].cpu().numpy()
    acc = c.qgemm_acc(a_h[pick].numpy(), w_h.numpy())
    _, want = c.qgemm_epilogue(acc, x_scale=np.float32(S_X), w_scale=w_scale_h.numpy(), out_scale=np.float32(S_OUT),
                               bias=bias_h.numpy(), div_out=True)
    d = np.abs(got.astype(np.int32) - want.astype(np.int32))
    return int(pick.numel()), int(d.max()), float((d > 0).mean())


def run_ours(args):
    import torch
    import torch.distributed as dist
    from bladedisc_b200 import build, ops
    from bladedisc_b200.host_api import HostQLinear

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the quantized path has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if not build.LIB.exists():
        build.build()

    rows = args.rows
    a_h, w_h, ws_h, b_h = _make_problem(torch, rows, "cpu", 1234 + 1 + rank)
    w, w_scale, bias = w_h.to(dev), ws_h.to(dev), b_h.to(dev)
    x_scale = torch.tensor([S_X], device=dev)
    out_scale = torch.tensor([S_OUT], device=dev)
    n_sets = 4  # rotating operand sets keep A and the output out of L2 between steps
    a_sets = [a_h.to(dev).roll(i, 0).contiguous() for i in range(n_sets)]
    o_sets = [torch.empty((rows, N_DIM), dtype=torch.int8, device=dev) for _ in range(n_sets)]

    def step(i):
        ops.qgemm(a_sets[i % n_sets], w, x_scale=x_scale, w_scale=w_scale, out_scale=out_scale, bias=bias,
                  out=o_sets[i % n_sets])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(max(1, args.warmup)):
        step(i)
    barrier()
    # Outside the timed region: sampled rows of the first step's output against the CPU oracle.
    verified_rows, max_lsb_diff, flip_share = _verify_rows(torch, o_sets[0], a_sets[0].cpu(), w_h, ws_h, b_h, 77 + rank)
    if max_lsb_diff > 1 or flip_share > 1e-3:
        raise SystemExit(f"rank {rank}: the timed kernel's output differs from the oracle (max {max_lsb_diff} levels, "
                         f"{flip_share:.2e} of the values): not printing a number for a wrong result")
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    # Untimed: keep the same kernel running for a moment so that clocks settle under load and
    # the sampler (10 ms period) sees the loaded state even when K steps take only milliseconds.
    t_hold = time.perf_counter()
    j = 0
    while not args.profile and time.perf_counter() - t_hold < 0.5:
        for _ in range(20):
            step(j)
            j += 1
        torch.cuda.synchronize()
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    barrier()
    evs[0].record()
    for i in range(args.steps):
        step(i)
        evs[i + 1].record()
    barrier()
    total_ms = evs[0].elapsed_time(evs[-1])
    per_launch_ms = sorted(evs[i].elapsed_time(evs[i + 1]) for i in range(args.steps))
    clocks = sampler.stop() if rank == 0 else None
    status = ops.kernel_status()
    if status != 0:
        raise SystemExit(f"kernel status {status}: a bounded wait ran out; numbers would be meaningless")

    if args.profile:
        print(json.dumps({"profile_run": True, "ms_per_step": total_ms / args.steps, "rows": rows}), flush=True)
        return

    # ---- the library kernel the reference's GPU custom call runs (cuBLASLt int8 -> int32 through
    # torch._int_mm, quantized_gpu_kernel_impl.cc:130-159), same shape and rotating operand sets
    lib_ms = None
    if hasattr(torch, "_int_mm"):
        try:
            acc_sets = [torch.empty((rows, N_DIM), dtype=torch.int32, device=dev) for _ in range(n_sets)]
            wt = w.t()
            # the same treatment as the kernel above: half a second of itself first, so that both are timed
            # in the clock state their own load produces
            t_hold = time.perf_counter()
            j = 0
            while time.perf_counter() - t_hold < 0.5:
                for _ in range(20):
                    torch._int_mm(a_sets[j % n_sets], wt, out=acc_sets[j % n_sets])
                    j += 1
                torch.cuda.synchronize()
            l0, l1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            l0.record()
            for i in range(args.steps):
                torch._int_mm(a_sets[i % n_sets], wt, out=acc_sets[i % n_sets])
            l1.record()
            torch.cuda.synchronize()
            lib_ms = l0.elapsed_time(l1) / args.steps
            del acc_sets
        except Exception:
            lib_ms = None
            torch.cuda.synchronize()

    # ---- end to end through the host-buffer API
    layer = HostQLinear(w, w_scale, x_scale, bias=bias, out_scale=out_scale, chunk_rows=2048)
    a_pin = a_h.pin_memory()
    o_pin = torch.empty((rows, N_DIM), dtype=torch.int8).pin_memory()
    for _ in range(max(3, args.warmup)):
        layer(a_pin, o_pin)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2e_steps = max(3, min(args.steps, 20))
    launches_before = layer.kernel_launches
    barrier()
    e0.record()
    for _ in range(e2e_steps):
        layer(a_pin, o_pin)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    e2e_launches = layer.kernel_launches - launches_before

    # ---- end to end through the boundary itself: a compiled executable (the stand-in program) run by the
    # host mirror of torch_blade's engine, every runtime service through tao_ral_call_impl
    ral_ms, ral_steps, ral_note = None, max(3, min(args.steps, 10)), None
    try:
        exe = _build_boundary_executable(torch, w_h, ws_h, b_h, local)
        a_dev = torch.empty((rows, K_DIM), dtype=torch.int8, device=dev)

        def ral_step():
            a_dev.copy_(a_pin, non_blocking=True)
            q = exe.run([a_dev])[0]
            o_pin.copy_(q, non_blocking=True)
            torch.cuda.current_stream().synchronize()
            return q
        for _ in range(3):
            q = ral_step()
        if not torch.equal(q, o_sets[0]) and not torch.equal(q.cpu(), o_pin):
            raise RuntimeError("the executable's output differs from the direct call's")
        barrier()
        r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        r0.record()
        for _ in range(ral_steps):
            ral_step()
        r1.record()
        barrier()
        ral_ms = r0.elapsed_time(r1)
        exe.close()
        del a_dev
    except Exception as e:   # gcc missing on the box, for instance: the leg is reported as absent, with the reason
        ral_note = f"{type(e).__name__}: {e}"
        ral_ms = None
        if world > 1:
            barrier()
            barrier()

    times = torch.tensor([total_ms, e2e_ms, ral_ms if ral_ms is not None else -1.0], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms, ral_ms_max = times.tolist()
    if ral_ms is not None:
        ral_ms = ral_ms_max

    # ---- second record in the same process group: the W8A8 BERT-base encoder over a fixed global batch
    # split over the ranks (the other half of the headline metric); the linear's operands are released first
    del a_sets, o_sets, layer, a_pin, o_pin
    torch.cuda.empty_cache()
    encoder = None
    if not args.skip_encoder:
        enc_steps = max(5, min(args.steps, 30))
        encoder = _encoder_measure(torch, dist, "bert_base", enc_steps, args.warmup, rank, world, local, dev, False)

    if rank == 0:
        ops_per_step = 2.0 * rows * K_DIM * N_DIM
        value = world * ops_per_step * args.steps / (total_ms * 1e-3) / 1e12
        e2e_value = world * ops_per_step * e2e_steps / (e2e_ms * 1e-3) / 1e12
        peaks = _peaks()
        # The timed region is one kernel launched back to back for a few milliseconds: the burst figure is
        # the denominator.  When the power cap engaged during the half second of the same kernel before it,
        # the fraction of the sustained figure is printed beside it.
        capped = bool(clocks and "sw_power_cap" in clocks.get("reasons", []))
        peak_i8 = 2.0 * peaks["bf16"]
        launch_ms = total_ms / args.steps
        achieved = ops_per_step / (launch_ms * 1e-3) / 1e12
        algo_bytes = rows * K_DIM + N_DIM * K_DIM + rows * N_DIM + 8 * N_DIM
        lib_tops = ops_per_step / (lib_ms * 1e-3) / 1e12 if lib_ms else None
        cfg = _workload_config(rows)
        cfg.update({"rows_per_gpu": rows, "path": ops.qgemm_path(rows, N_DIM, K_DIM),
                    "requantisation": "reciprocal form (at most 1 int8 level from the divide-based formula)",
                    "l2": f"{n_sets} rotating operand sets ({n_sets * (rows * K_DIM + rows * N_DIM) >> 20} MiB) > 126 MB L2"})
        line = {
            "metric": "qgemm_int8_tops", "value": value, "unit": "TOPS", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": launch_ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "i8", "data": "synthetic",
            "config": cfg,
            "verified_rows": verified_rows, "max_lsb_diff": max_lsb_diff, "lsb_flip_share": flip_share,
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak_i8, "unit": "TOPS",
                         "frac": achieved / peak_i8, "traffic": NCU_DRAM_BYTES_PER_LAUNCH,
                         "peak_source": f"2 x {peaks['source']} cuBLAS bf16 burst ({peaks['bf16']} TF/s): int8 issues "
                                        f"at twice the bf16 rate; of {peaks['source']}",
                         "frac_of_sustained_peak": achieved / (2.0 * peaks["bf16_sustained"]),
                         "power_capped_before_timing": capped,
                         "frac_of_nominal_4500": achieved / NOMINAL_INT8_TOPS,
                         "cublaslt_int8_tops": lib_tops,
                         "vs_cublaslt": (achieved / lib_tops) if lib_tops else None,
                         "cublaslt_note": "torch._int_mm, int32 output, no epilogue; ours writes requantized int8",
                         "algorithmic_bytes": algo_bytes, "algorithmic_ops": ops_per_step,
                         "launch_ms_median": per_launch_ms[len(per_launch_ms) // 2]},
            "e2e": {"value": e2e_value, "unit": "TOPS", "h2d_bytes_per_step": rows * K_DIM,
                    "d2h_bytes_per_step": rows * N_DIM, "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps},
            "gpu_launches": args.steps, "e2e_gpu_launches": e2e_launches,
            "clocks": clocks,
        }
        line["e2e_ral"] = ({"value": world * ops_per_step * ral_steps / (ral_ms * 1e-3) / 1e12, "unit": "TOPS",
                            "ms_per_step": ral_ms / ral_steps, "steps": ral_steps,
                            "h2d_bytes_per_step": rows * K_DIM, "d2h_bytes_per_step": rows * N_DIM,
                            "path": "pinned host -> device copy, compiled stand-in executable (ral_recv_input, ral_const, "
                                    "disc_b200_qgemm, ral_send_output through tao_ral_call_impl), device -> pinned host "
                                    "copy; one copy each way, not overlapped with the kernel"}
                           if ral_ms is not None else {"value": None, "unavailable": ral_note})
        if encoder is not None:
            line["encoder"] = encoder
        if world == 1 and not args.skip_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(torch)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def _encoder_measure(torch, dist, workload, steps, warmup, rank, world, local, dev, profile, shard_of=None):
    """Configurations 2 / 3: one step = one forward of the W8A8 encoder over the global batch
    (32 sequences of length U[16,512] for BERT-base, 64 of U[64,512] for BERT-large), the
    sequences split over the ranks by length (no collective; total work fixed: "strong").
    Every rank calls this; rank 0 gets the record (a dict), the others None."""
    from bladedisc_b200 import encoder as E
    from bladedisc_b200 import ops

    if workload == "bert_base":
        cfg, batch, lo = E.EncoderConfig.bert_base(), 32, 16
    else:
        cfg, batch, lo = E.EncoderConfig.bert_large(), 64, 64
    enc, qenc, scales = E.build_quant_encoder(cfg, seed=1234, device=dev, min_len=lo)
    del enc
    ids_h, lens_h = E.synthetic_batch(cfg, batch, lo, 512, seed=4321, device="cpu")
    if shard_of:   # one process standing in for rank 0 of `shard_of` ranks (for profiling one shard)
        my_ids_h, my_lens_h, assign = E.shard_batch(ids_h, lens_h, shard_of, 0)
    else:
        my_ids_h, my_lens_h, assign = E.shard_batch(ids_h, lens_h, world, rank)
    ids_pin, lens_pin = my_ids_h.pin_memory(), my_lens_h.pin_memory()
    have_work = len(assign) > 0
    ids_d = torch.empty_like(ids_pin, device=dev)
    lens_d = torch.empty_like(lens_pin, device=dev)
    cls_pin = torch.empty((max(len(assign), 1), cfg.hidden), dtype=torch.float16).pin_memory()

    # The forward is a fixed sequence of short launches: capture it once per batch shape
    # and replay it, so that launch latency does not dominate small per-GPU batches.
    side = torch.cuda.Stream(dev)
    graph, out_ref = None, [None]
    if have_work:
        ids_d.copy_(ids_pin)
        lens_d.copy_(lens_pin)
        qenc.prepare(ids_d, lens_d)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                out_ref[0] = qenc.forward_packed(ids_d, lens_d)
        torch.cuda.synchronize()
        launches_per_fwd = qenc.kernel_launches // 2
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                out_ref[0] = qenc.forward_packed(ids_d, lens_d)
        except Exception:
            graph = None
            torch.cuda.synchronize()
    else:
        launches_per_fwd = 0

    def device_step():
        if not have_work:
            return
        if graph is not None:
            graph.replay()
        else:
            out_ref[0] = qenc.forward_packed(ids_d, lens_d)

    def e2e_step():
        if not have_work:
            return
        ids_d.copy_(ids_pin, non_blocking=True)
        lens_d.copy_(lens_pin, non_blocking=True)
        device_step()
        cls_pin[:len(assign)].copy_(qenc.first_tokens(out_ref[0]), non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        barrier()
        return e0.elapsed_time(e1)

    for _ in range(max(3, warmup)):
        device_step()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    t_hold = time.perf_counter()
    while not profile and time.perf_counter() - t_hold < 0.5:
        device_step()
        torch.cuda.synchronize()
    dev_ms = timed(device_step, steps)
    clocks = sampler.stop() if rank == 0 else None
    if profile:
        return {"profile_run": True, "ms_per_step": dev_ms / steps, "workload": workload, "sequences": len(assign),
                "tokens": int(my_lens_h.sum()), "launches_per_forward": launches_per_fwd} if rank == 0 else None
    for _ in range(3):
        e2e_step()
    e2e_steps = max(3, min(steps, 20))
    e2e_ms = timed(e2e_step, e2e_steps)
    if ops.kernel_status() != 0:
        raise SystemExit("kernel status non-zero: a bounded wait ran out")
    times = torch.tensor([dev_ms, e2e_ms], dtype=torch.float64, device=dev)
    tokens = torch.tensor([float(qenc.rows_processed if have_work else 0), float(my_lens_h.sum())],
                          dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        dist.all_reduce(tokens, op=dist.ReduceOp.SUM)
    dev_ms, e2e_ms = times.tolist()
    if rank != 0:
        return None
    return {
        "metric": f"quant_{workload}_seqs_per_s", "value": batch * steps / (dev_ms * 1e-3), "unit": "sequences/s",
        "n_gpus": world, "steps": steps, "warmup": max(3, warmup), "ms_per_step": dev_ms / steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "i8", "data": "synthetic",
        "config": {"workload": f"{workload} W8A8 encoder forward, {cfg.layers} layers, hidden {cfg.hidden}, "
                               f"global batch {batch}, lengths U[{lo},512], masked attention",
                   "sharding": "sequences split by length over ranks, no collective",
                   "rows_through_the_linears_all_ranks": int(tokens[0]), "real_tokens": int(tokens[1]),
                   "cuda_graph": graph is not None,
                   "l2": "activations of a forward are rewritten every step",
                   "note": qenc.describe()},
        "e2e": {"value": batch * e2e_steps / (e2e_ms * 1e-3), "unit": "sequences/s",
                "h2d_bytes_per_step": int(ids_pin.numel() * 8 + lens_pin.numel() * 4),
                "d2h_bytes_per_step": int(len(assign) * cfg.hidden * 2), "steps": e2e_steps},
        "gpu_launches": launches_per_fwd * steps, "launches_per_forward": launches_per_fwd,
        "clocks": clocks,
    }


def run_encoder(args):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the quantized path has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    line = _encoder_measure(torch, dist, args.workload, args.steps, args.warmup, rank, world, local, dev, args.profile,
                            args.shard_of)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_decoder(args):
    """Configuration 4: Llama-7B-shaped W8A8 decoder, every linear split by output channels over
    the ranks and followed by an NCCL all-gather.  One step = prefill of 8 x 2048 tokens through
    all layers; decode steps (one token per sequence) are timed beside it.  Total work is fixed
    as ranks are added ("strong")."""
    import torch
    import torch.distributed as dist
    from bladedisc_b200 import ops, tp
    from bladedisc_b200.decoder import DecoderConfig, QuantDecoder

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the quantized path has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    comm = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        comm = tp.Communicator.from_torch_distributed(dev)
    if args.tp_row_blocks is not None:
        tp.MAX_ROW_BLOCKS = args.tp_row_blocks
    cfg = DecoderConfig.llama7b(layers=args.layers)
    dec = QuantDecoder(cfg, comm, seed=1238, device=dev)
    batch, seq = 8, 2048
    gen = torch.Generator().manual_seed(4324)
    ids_pin = torch.randint(0, cfg.vocab, (batch, seq), generator=gen).pin_memory()
    ids_d = ids_pin.to(dev)
    last_pin = torch.empty((batch, cfg.hidden), dtype=torch.float16).pin_memory()
    dec.start(batch, seq + 8)
    out = [None]

    def device_step():
        dec.pos = 0
        out[0] = dec.forward(ids_d)

    def e2e_step():
        ids_d.copy_(ids_pin, non_blocking=True)
        device_step()
        last_pin.copy_(out[0].view(batch, seq, cfg.hidden)[:, -1, :], non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        return e0.elapsed_time(e1)

    steps = min(args.steps, 10)
    for _ in range(3):
        device_step()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    dev_ms = timed(device_step, steps)
    clocks = sampler.stop() if rank == 0 else None
    e2e_step()
    e2e_steps = min(steps, 5)
    e2e_ms = timed(e2e_step, e2e_steps)
    # decode: context of 128 tokens, then one token per sequence and step
    decode = {}
    for b in (1, 8, 64):
        dec.start(b, 128 + 40)
        ctx_ids = torch.randint(0, cfg.vocab, (b, 128), generator=gen).to(dev)
        nxt = torch.randint(0, cfg.vocab, (b, 1), generator=gen).to(dev)
        dec.forward(ctx_ids)
        for _ in range(3):
            dec.forward(nxt)
        # A decode step is ~40 short launches per layer: it is replayed from a CUDA graph (captured at one
        # cache position, so every replay does the work of that position).  With several ranks the graph
        # holds the NCCL collectives too.  Nothing of a capture executes, so a capture that fails on one
        # rank stops nobody; but a replay on some ranks only would leave them waiting in a collective, so
        # the ranks agree (minimum over ranks of "my capture succeeded") before anyone replays, and all run
        # eagerly otherwise.  The capture is thread-local: NCCL's helper threads may call the runtime
        # while this thread captures.
        step, graph = (lambda: dec.forward(nxt)), None
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream())
        try:
            with torch.cuda.stream(side):
                dec.forward(nxt)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side, capture_error_mode="thread_local"):
                dec.forward(nxt)
        except Exception:
            graph = None
        torch.cuda.synchronize()
        if world > 1:
            agreed = torch.tensor([1 if graph is not None else 0], device=dev, dtype=torch.int32)
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
            if int(agreed.item()) == 0:
                graph = None
        if graph is not None:
            step = graph.replay
        decode_graph = graph is not None
        for _ in range(3):
            step()
        ms = timed(step, 32)
        decode[b] = ms / 32
        # the graph goes before the communicator: NCCL does not let go of a communicator while a graph
        # that captured its collectives exists (`step` is a bound method of the graph)
        step = None
        del graph
        torch.cuda.synchronize()
    if ops.kernel_status() != 0:
        raise SystemExit("kernel status non-zero: a bounded wait ran out")
    vals = [dev_ms, e2e_ms] + [decode[b] for b in (1, 8, 64)]
    times = torch.tensor(vals, dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms, d1, d8, d64 = times.tolist()
    if rank == 0:
        tokens = batch * seq
        linear_ops = 2.0 * tokens * cfg.layers * (4 * cfg.hidden * cfg.hidden + 3 * cfg.hidden * cfg.ffn)
        weight_bytes = cfg.layers * (4 * cfg.hidden * cfg.hidden + 3 * cfg.hidden * cfg.ffn)
        line = {
            "metric": "quant_llama7b_prefill_tokens_per_s", "value": tokens * steps / (dev_ms * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": steps, "warmup": 3, "ms_per_step": dev_ms / steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "i8", "data": "synthetic",
            "config": {"workload": f"llama-7b-shaped W8A8 decoder, {cfg.layers} layers, hidden {cfg.hidden}, ffn {cfg.ffn}, "
                                   f"prefill {batch} x {seq} tokens, per-token dynamic int8 activations",
                       "parallelism": f"column-parallel N-split over {world} rank(s), NCCL all-gather after every "
                                      "gathered linear (4 per layer), all-reduce(max) of row scales (2 per layer); "
                                      f"up to {tp.MAX_ROW_BLOCKS} row block(s) per linear, gathers on a side stream",
                       "l2": "activations of a step (hundreds of MB) are rewritten every step",
                       "note": "attention (SDPA) and RoPE run in torch, a library call as the reference's ral_gemm; "
                               "every linear, norm and quantize is this library's kernel",
                       "linear_int8_tops": linear_ops * steps / (dev_ms * 1e-3) / 1e12,
                       "decode_ms_per_step": {"batch1": d1, "batch8": d8, "batch64": d64, "context": 128,
                                              "cuda_graph": decode_graph},
                       "decode_weight_stream_gbs_batch1": weight_bytes / world / (d1 * 1e-3) / 1e9},
            "e2e": {"value": tokens * e2e_steps / (e2e_ms * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": int(ids_pin.numel() * 8), "d2h_bytes_per_step": int(last_pin.numel() * 2),
                    "steps": e2e_steps},
            "gpu_launches": dec.launches_per_layer() * cfg.layers * steps,
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if comm is not None:
        comm.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    args = _args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "llama7b":
        run_decoder(args)
    elif args.workload != "qlinear":
        run_encoder(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
