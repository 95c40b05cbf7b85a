"""Benchmark of the hot path: the tiled GEMM of MoYe's examples/gemm.jl on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one pass of the hot path over one batch of synthetic input.  The default
workload is the dense fp16 x fp16 -> fp32 GEMM with M = N = K = 8192 (K-major A and B,
U[-1,1) entries, alpha = 1, beta = 0).  With N GPUs every rank owns one M-shard of a global
(N*8192) x 8192 x 8192 product with B replicated, so per-GPU work is fixed (weak scaling) and
there is no collective in the timed region.

Rank 0 prints ONE JSON line.  `value` is whole-job TFLOP/s with the operands resident in HBM
(CUDA events on the launching stream, max over ranks); `e2e` is the same product through the
package's public call with pinned HOST buffers, host<->device copies inside the timed region;
`roofline` compares the kernel with the measured cuBLAS bf16 peak (MEASURED_PEAKS.json);
`cpu_baseline` times the CPU restatement of the reference's host path on a bounded sample.

`--impl reference` times only the reference's host implementation (the CPU restatement under
oracle/, all host threads) on bounded samples of the same workload.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# DRAM traffic of one launch of the 8192^3 fp16 GEMM kernel (dram__bytes_read.sum +
# dram__bytes_write.sum from the ncu captures summarised under profiles/), bytes per launch.
NCU_TRAFFIC_BYTES = {"gemm_f16_8192": 0.8291e9 + 0.2346e9,     # profiles/gemm_tcgen05_2cta_wide_f16_8192_dram_traffic.txt
                     "decode_bf16_16x28672x8192": 471.24e6 + 6.1e6,  # profiles/gemm_skinny_bf16_16x28672x8192.txt
                     "gemm_f16_4096x8192x4096": 179.6e6 + 100.5e6}

WORKLOADS = {
    # name: (kind, M, N, K, out)
    "gemm_f16_8192": ("f16", 8192, 8192, 8192, "f32"),
    "gemm_f16_4096": ("f16", 4096, 4096, 4096, "f32"),
    "gemm_bf16_8192": ("bf16", 8192, 8192, 8192, "f32"),
    "gemm_s8_16384x8192x8192": ("s8", 16384, 8192, 8192, "s32"),
    "gemm_e4m3_16384x8192x8192": ("e4m3", 16384, 8192, 8192, "bf16"),
    "decode_bf16_16x28672x8192": ("bf16", 16, 28672, 8192, "bf16"),
    "copy_f16_8192": ("copy", 8192, 8192, 0, "f16"),
    # copyto!(dest, transpose(src)), the reference's transpose_kernel at the copy workload's size (fp16 and fp32)
    "transpose_8192": ("transpose", 8192, 8192, 0, "f16"),
    # the storage of the reference's examples/gemm.jl: A (M,K), B (N,K), C (M,N) all column-major
    "gemm_f16_8192_colmajor": ("f16", 8192, 8192, 8192, "f32"),
    # a smaller case of the same dense kernel (224 MB of operands + output, still larger than L2),
    # sized for multi-pass profiler captures
    "gemm_f16_4096x8192x4096": ("f16", 4096, 8192, 4096, "f32"),
    # the same for the 256 x 512 tile kernel: 37 x 8 = 296 tiles = 4 full waves of the 74 SM pairs, 211 MB
    "gemm_f16_9472x4096x2048": ("f16", 9472, 4096, 2048, "f32"),
    # Float32 storage, column-major like examples/gemm.jl (its literal element type): three tf32 products of the
    # operands' high and low parts (Float32 accuracy), and ONE tf32 product (allow_tf32, about 1e-3 relative)
    "gemm_f32_8192_colmajor": ("f32", 8192, 8192, 8192, "f32"),
    "gemm_f32_8192_colmajor_tf32": ("f32", 8192, 8192, 8192, "f32"),
    # a few hundred rows against a mid-sized weight matrix: 32 output tiles, the case of the split-K cluster kernel
    "gemm_bf16_256x4096x4096": ("bf16", 256, 4096, 4096, "bf16"),
    # 3.46 waves of 256 x 512 tiles: the last wave is cut along K over all CTA pairs (320 MB on the device)
    "gemm_f16_4096x8192x8192": ("f16", 4096, 8192, 8192, "f32"),
    # the elementwise copyto!(dst, src) through two layouts and the layout function itself, 2^24 elements
    "layout_copy_f32_4096": ("layout", 4096, 4096, 0, "f32"),
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return {k: float(d[k]) for k in FALLBACK_PEAKS}, "measured"
    except Exception:
        return dict(FALLBACK_PEAKS), "fallback"


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU while the timed region runs."""

    REASONS = {0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown", 0x8: "hw_slowdown", 0x4: "sw_power_cap",
               0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting", 0x100: "display_clock_setting",
               0x10: "sync_boost"}

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        self._h = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._h = None

    def _run(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                bits = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._h))
                for b, name in self.REASONS.items():
                    if bits & b:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        if self._h is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "samples": len(s),
                "reasons": sorted(self.reasons)}


# ----------------------------------------------------------------------------- helpers
def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


def flops_of(kind, M, N, K):
    return 2.0 * M * N * K


def make_operands(torch, kind, M, N, K, out, dev, seed, colmajor=False):
    g = torch.Generator(device=dev).manual_seed(seed)
    if kind == "f16":
        A = (torch.rand(M, K, device=dev, generator=g) * 2 - 1).half()
        B = (torch.rand(N, K, device=dev, generator=g) * 2 - 1).half()
    elif kind == "f32":
        A = torch.rand(M, K, device=dev, generator=g) * 2 - 1
        B = torch.rand(N, K, device=dev, generator=g) * 2 - 1
    elif kind == "bf16":
        A = (torch.randn(M, K, device=dev, generator=g) * 0.02).bfloat16()
        B = (torch.randn(N, K, device=dev, generator=g) * 0.02).bfloat16()
    elif kind == "s8":
        A = torch.randint(-128, 128, (M, K), device=dev, generator=g, dtype=torch.int8)
        B = torch.randint(-128, 128, (N, K), device=dev, generator=g, dtype=torch.int8)
    else:
        A = torch.randn(M, K, device=dev, generator=g).clamp(-448, 448).to(torch.float8_e4m3fn)
        B = torch.randn(N, K, device=dev, generator=g).clamp(-448, 448).to(torch.float8_e4m3fn)
    odt = {"f32": torch.float32, "s32": torch.int32, "bf16": torch.bfloat16, "f16": torch.float16}[out]
    C = torch.zeros(M, N, device=dev, dtype=odt)
    if colmajor:
        A, B, C = A.t().contiguous().t(), B.t().contiguous().t(), C.t().contiguous().t()
    return A, B, C


def gemm_kw(name):
    kind = WORKLOADS[name][0]
    kw = {"scale_a": 0.05, "scale_b": 0.02} if kind == "e4m3" else {}
    if name.endswith("_tf32"):
        kw["allow_tf32"] = True
    return kw


def is_colmajor(name):
    return "_colmajor" in name


def time_launches(torch, fn, steps, warmup, stream, settle=0.0):
    """Average device time of `fn` in ms: CUDA events on the launching stream, sync on both sides.  `settle` seconds of idle
    before the warm-up let the clocks recover when the previous workload ran into the power cap (the `also` workloads are each
    meant to be timed alone, and a bandwidth-bound kernel timed in the first milliseconds after a 1 kW GEMM measured 5-15 % slow)."""
    if settle > 0:
        torch.cuda.synchronize()
        time.sleep(settle)
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        fn()
    e1.record(stream)
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


# ----------------------------------------------------------------------------- CPU baseline
def cpu_reference_rate(ho, np, M, N, K, seconds, threads):
    """Times the threaded host GEMM of the reference (restated in oracle/moye_host.c after
    test/host/tiling_matmul.jl:20-39) on the first rows of C of an (M,N,K) fp32 problem.
    Returns (TFLOP/s, rows, elapsed seconds, thread layout)."""
    tr = 1
    while tr * tr * 4 <= threads:
        tr *= 2
    tc = max(1, threads // tr)
    A = ho.uniform_pm1(3, (M * K,))
    B = ho.uniform_pm1(4, (N * K,))
    probe_rows = tr
    t0 = time.perf_counter()
    ho.matmul_threads_f32(A, B, M, N, K, thread_layout=(tr, tc), m_limit=probe_rows)
    dt = max(time.perf_counter() - t0, 1e-6)
    rate = 2.0 * probe_rows * N * K / dt
    rows = int(max(tr, min(M, (seconds * rate / (2.0 * N * K)) // tr * tr)))
    t0 = time.perf_counter()
    ho.matmul_threads_f32(A, B, M, N, K, thread_layout=(tr, tc), m_limit=rows)
    dt = time.perf_counter() - t0
    return 2.0 * rows * N * K / dt / 1e12, rows, dt, (tr, tc)


def cpu_other_configs(ho, np, threads):
    """The reference's own CPU-runnable cases, timed on the host cores beside the headline baseline: configuration 1
    (256^3 fp32 through the emulated `matmul_kernel` and the plain host gemm!, one thread, and the threaded host GEMM)
    and the copy kernel of configuration 2 on a 2048 x 2048 fp16 slice."""
    out = {}
    M = N = K = 256
    A, B = ho.uniform_pm1(0, (M * K,)), ho.uniform_pm1(1, (N * K,))
    t0 = time.perf_counter()
    ho.matmul_kernel_f32(A, B, M, N, K)
    out["cfg1_matmul_kernel_emulated_1thread_GFLOP/s"] = 2.0 * M * N * K / (time.perf_counter() - t0) / 1e9
    t0 = time.perf_counter()
    ho.gemm_f32(A, (1, M), B, (1, N), M, N, K)
    out["cfg1_host_gemm_1thread_GFLOP/s"] = 2.0 * M * N * K / (time.perf_counter() - t0) / 1e9
    tr = 1
    while tr * tr * 4 <= threads:
        tr *= 2
    tc = max(1, threads // tr)
    t0 = time.perf_counter()
    ho.matmul_threads_f32(A, B, M, N, K, thread_layout=(tr, tc))
    out[f"cfg1_host_gemm_{tr * tc}threads_GFLOP/s"] = 2.0 * M * N * K / (time.perf_counter() - t0) / 1e9
    m = n = 2048
    src = ho.uniform_pm1_f16_bits(2, (m * n,))
    dst = np.zeros_like(src)
    t0 = time.perf_counter()
    ho.copy_kernel(dst, src, m, n, bm=128, bn=64, tm=16, tn=16)
    out["cfg2_copy_kernel_2048x2048_f16_1thread_GB/s"] = 2.0 * m * n * 2 / (time.perf_counter() - t0) / 1e9
    return out


def run_reference_arm(args):
    rank, _, world = dist_env()
    if rank != 0:
        return 0
    import numpy as np
    import __graft_entry__ as ge
    ho, _ = ge.load_oracle()
    ho.lib()
    kind, M, N, K, out = WORKLOADS[args.workload]
    if kind in ("copy", "transpose"):
        raise SystemExit("the reference arm times the GEMM workloads")
    threads = os.cpu_count() or 1
    total = args.steps + args.warmup
    per_step = min(5.0, max(0.2, 75.0 / max(1, total)))
    tr = 1
    while tr * tr * 4 <= threads:
        tr *= 2
    tc = max(1, threads // tr)
    A = ho.uniform_pm1(3, (M * K,))
    B = ho.uniform_pm1(4, (N * K,))
    t0 = time.perf_counter()
    ho.matmul_threads_f32(A, B, M, N, K, thread_layout=(tr, tc), m_limit=tr)
    rate = 2.0 * tr * N * K / max(time.perf_counter() - t0, 1e-6)
    rows = int(max(tr, min(M, (per_step * rate / (2.0 * N * K)) // tr * tr)))
    for _ in range(args.warmup):
        ho.matmul_threads_f32(A, B, M, N, K, thread_layout=(tr, tc), m_limit=rows)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        ho.matmul_threads_f32(A, B, M, N, K, thread_layout=(tr, tc), m_limit=rows)
    dt = (time.perf_counter() - t0) / args.steps
    val = 2.0 * rows * N * K / dt / 1e12
    sample = f"first {rows} of {M} rows of C per step, N={N}, K={K}, fp32 (inputs widened), thread layout ({tr},{tc})"
    line = {
        "impl": "reference", "metric": "GEMM TFLOP/s", "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.workload, args.gpus),
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": tr * tc, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "MoYe.jl is Julia and cannot run here; this is the C restatement of its threaded host gemm "
                "(oracle/moye_host.c), throughput measured on a row sample, not extrapolated in time",
    }
    print(json.dumps(line), flush=True)
    return 0


def workload_config(name, gpus):
    kind, M, N, K, out = WORKLOADS[name]
    return {"workload": name, "M_per_gpu": M, "N": N, "K": K, "global_M": M * gpus,
            "layout": "A,B,D column-major (MN-major, as examples/gemm.jl)" if is_colmajor(name) else "A,B K-major (TN); D row-major",
            "in": kind, "out": out, "sharding": f"M-sharded x{gpus}, B replicated, no collective",
            "l2": "operands+output exceed the 126 MB L2 (no flush needed)" if M * K + N * K > 64e6
            else "operand/output buffer sets rotated, more than 512 MB in total"}


# ----------------------------------------------------------------------------- our arm
def run_ours(args):
    import numpy as np
    import torch
    import __graft_entry__ as ge

    rank, local_rank, world = dist_env()
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
                   "--master-addr", "127.0.0.1", "--master-port", str(29500 + os.getpid() % 1000), __file__] + sys.argv[1:]
            return subprocess.call(cmd)
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU implementation")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    mb = ge.load_package()
    peaks, peak_src = measured_peaks()
    stream = torch.cuda.current_stream()
    name = args.workload
    kind, M, N, K, out = WORKLOADS[name]

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    if kind in ("copy", "transpose"):
        return run_copy(args, mb, torch, dev, peaks, peak_src, rank, world, dist, barrier, transpose=kind == "transpose")
    if kind == "layout":
        return run_layout(args, mb, torch, dev, peaks, peak_src)

    # operands that would sit in the 126 MB L2 are rotated over enough buffer sets to exceed it several times
    rotate = not (M * K + N * K > 64e6)
    set_bytes = 0
    sets = []
    while True:
        sets.append(make_operands(torch, kind, M, N, K, out, dev, seed=3 + rank + 16 * len(sets),
                                  colmajor=is_colmajor(name)))
        set_bytes += sum(t.numel() * t.element_size() for t in sets[-1])
        if not rotate or set_bytes > 512e6:
            break
    A, B, C = sets[0]
    kw = gemm_kw(name)
    if args.path:
        kw["path"] = args.path
    if args.tail != "auto":
        kw["tail"] = args.tail == "on"
    plans = [mb.plan_gemm(mb.MoYeArray(c), mb.MoYeArray(a), mb.MoYeArray(b), None, **kw) for a, b, c in sets]
    plan = plans[0]                               # the argument marshalling of gemm_ done once per buffer set
    stream_ptr = mb.current_stream_ptr(dev)
    turn = [0]

    def step():
        turn[0] += 1
        plans[turn[0] % len(plans)](stream_ptr)

    for _ in range(max(3, args.warmup)):
        step()
    mb.synchronize_status(dev)
    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        step()
    e1.record(stream)
    barrier()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / args.steps
    mb.synchronize_status(dev)
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max = float(t.item())
    total_flops = flops_of(kind, M, N, K) * world
    value = total_flops / (ms_max * 1e-3) / 1e12
    bytes_bound = kind == "bf16" and M <= 512

    # end to end: pinned host operands -> device -> GEMM -> pinned host result, every step, through the
    # package's host pipeline (copies and kernel on three streams over two device buffer sets).  With several
    # ranks the replicated B crosses PCIe once, on rank 0, and reaches the others over NVLink (NCCL broadcast
    # through the library's communicator); every rank copies its own A shard in and its C shard out.
    comm = mb.Communicator(rank, world, dev) if world > 1 else None
    if args.no_e2e:
        return print_kernel_only(args, rank, world, name, kind, M, N, K, ms, ms_max, value, clocks, peaks, peak_src, comm, dist)
    # pinned host memory is kept to what the step needs: B only where it is copied from (rank 0), one result buffer
    # (the copies out are ordered on one stream)
    hA = A.cpu().pin_memory()
    hB = B.cpu().pin_memory() if rank == 0 else None
    hC = [torch.empty(C.shape, dtype=C.dtype).pin_memory()] * 2
    e2e_steps = max(2, min(args.steps, 48))  # enough steps to amortise filling and draining the three-stream pipeline
    pipe = mb.HostGemmPipeline(M, N, K, A.dtype, C.dtype, dev, depth=2, comm=comm, **kw)
    for i in range(3):
        pipe.submit(hA, hB, hC[i % 2])
    pipe.join()
    barrier()
    e0.record(stream)
    pipe.start_after(e0)
    for i in range(e2e_steps):
        pipe.submit(hA, hB, hC[i % 2])
    pipe.join(stream)
    e1.record(stream)
    barrier()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    t = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item())
    # the same step with its three phases back to back on one stream (no overlap), for reference
    def serial_step():
        A.copy_(hA, non_blocking=True)
        if hB is not None:
            B.copy_(hB, non_blocking=True)
        plan(stream_ptr)
        hC[0].copy_(C, non_blocking=True)

    serial_step()
    barrier()
    e0.record(stream)
    for _ in range(4):
        serial_step()
    e1.record(stream)
    barrier()
    e2e_serial_ms = e0.elapsed_time(e1) / 4
    a_bytes, b_bytes = A.numel() * A.element_size(), B.numel() * B.element_size()
    h2d = a_bytes * world + b_bytes          # whole job: every rank's A shard, B once
    d2h = C.numel() * C.element_size() * world

    if bytes_bound:
        alg_bytes = a_bytes + b_bytes + C.numel() * C.element_size()
        achieved, peak, unit, bound = alg_bytes / (ms * 1e-3) / 1e9, peaks["hbm_gbs"], "GB/s", "hbm"
        metric, munit = "decode GEMM GB/s", "GB/s"
        value = alg_bytes * world / (ms_max * 1e-3) / 1e9
        e2e_val = alg_bytes * world / (e2e_ms * 1e-3) / 1e9
        peak_kind = "hbm copy"
    else:
        long_run = ms * args.steps > 1000.0
        peak_kind = "cuBLAS bf16 sustained" if long_run else "cuBLAS bf16 burst"
        achieved, unit, bound = flops_of(kind, M, N, K) / (ms * 1e-3) / 1e12, "TFLOP/s", "tensor"
        peak = peaks["bf16_tflops_sustained"] if long_run else peaks["bf16_tflops"]
        if kind in ("s8", "e4m3"):
            peak, peak_kind = 2.0 * peak, peak_kind + " x2 (8-bit operands; no measured 8-bit peak)"
        metric, munit = "GEMM TFLOP/s", "TFLOP/s"
        e2e_val = total_flops / (e2e_ms * 1e-3) / 1e12

    line = {
        "metric": metric, "value": value, "unit": munit, "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
        "ms_per_step": ms_max, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": {"f16": "f16 (f32 accumulate)", "bf16": "bf16 (f32 accumulate)", "s8": "s8 (s32 accumulate)",
                  "e4m3": "e4m3 (f32 accumulate)", "f32": "f32 read as tf32 (f32 accumulate)"}[kind],
        "data": "synthetic", "config": workload_config(name, world), "clocks": clocks, "gpu_launches": args.steps,
        "e2e": {"value": e2e_val, "unit": munit, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_ms, "steps": e2e_steps,
                "how": "HostGemmPipeline: H2D, GEMM, D2H on three streams, two device buffer sets; every step copies its own "
                       "operands in and its result out" + ("; B is copied in by rank 0 only and broadcast over NVLink (NCCL)"
                                                            if world > 1 else ""),
                "bytes_are": "summed over all ranks", "h2d_bytes_rank0": a_bytes + b_bytes,
                "h2d_bytes_other_ranks": a_bytes if world > 1 else None, "nvlink_bcast_bytes_per_step": b_bytes if world > 1 else 0,
                "serial_ms_per_step": e2e_serial_ms},
        "roofline": {"bound": bound, "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak,
                     "traffic": NCU_TRAFFIC_BYTES.get(name), "peak_source": f"{peak_kind}, of {peak_src}",
                     "kernel": ("gemm_tcgen05_2cta_wide_kernel" if not bytes_bound else
                                ("gemm_skinny_kernel" if M <= 16 else "gemm_tcgen05_splitk_kernel")),
                     "kernel_ms": ms},
    }
    if dist is not None and world > 1 and not args.no_extras and not bytes_bound:
        try:
            line.update(multi_gpu_extras(mb, torch, dist, comm, dev, rank, world, name, A, B, C, barrier, peaks))
        except Exception as exc:  # reported, never hidden
            line["multi_gpu_extras_error"] = repr(exc)
    if comm is not None:
        comm.destroy()
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        ho, _ = ge.load_oracle()
        threads = os.cpu_count() or 1
        val, rows, dt, tl = cpu_reference_rate(ho, np, M, N, K, seconds=12.0, threads=threads)
        line["cpu_baseline"] = {
            "value": val, "unit": "TFLOP/s", "cores": tl[0] * tl[1], "kind": "port",
            "sample": f"first {rows} of {M} rows of C (N={N}, K={K}), fp32 inputs widened, threaded host gemm with "
                      f"thread layout {tl}, {dt:.1f} s",
            "other_configs": cpu_other_configs(ho, np, threads)}
    if rank == 0 and world == 1 and not args.no_extras:
        line["also"] = extras(mb, torch, dev, peaks)
        if not bytes_bound:
            line["also"]["sustained"] = sustained_rate(mb, torch, dev, plan, stream_ptr, flops_of(kind, M, N, K), peaks)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()
    return 0


def print_kernel_only(args, rank, world, name, kind, M, N, K, ms, ms_max, value, clocks, peaks, peak_src, comm, dist):
    """`--no-e2e`: the device-timed figure alone (what a profiler capture of one kernel needs; not a bench line)."""
    line = {"kernel_only": True, "workload": name, "ms_per_step": ms_max, "TFLOP/s": value, "n_gpus": world,
            "path": args.path, "tail": args.tail, "clocks": clocks, "config": workload_config(name, world)}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if comm is not None:
        comm.destroy()
    if dist is not None:
        dist.destroy_process_group()
    return 0


def run_layout(args, mb, torch, dev, peaks, peak_src):
    """The elementwise `copyto!(dst, src)` through two different layouts (a transposing pair) and the evaluation of
    the layout function, 2^24 elements each: integer index arithmetic per element, reported as GB/s of the bytes
    moved (4 + 4 per element for the copy, 8 written per element for the evaluation)."""
    m = n = 4096
    src = torch.rand(m * n, device=dev)
    dst = torch.zeros_like(src)
    stream = torch.cuda.current_stream()
    a_dst = mb.MoYeArray(dst, mb.make_layout((m, n), (n, 1)))     # row-major destination
    a_src = mb.MoYeArray(src, mb.make_layout(((64, 64), n), ((1, 64 * n), 64)))   # a hierarchical source layout
    steps, warm = args.steps, max(3, args.warmup)
    ms_copy = time_launches(torch, lambda: mb.copyto_(a_dst, a_src, elementwise_ok=True), steps, warm, stream)
    lay = mb.make_layout((8, (4, 2), 16, 16384), (3, (64, 7), 1, 4096))
    ms_eval = time_launches(torch, lambda: mb.layout_eval(lay, device=dev), steps, warm, stream)
    mb.synchronize_status(dev)
    res = {"layout_copy": {"ms": ms_copy, "GB/s": 8.0 * m * n / ms_copy / 1e6},
           "layout_eval": {"ms": ms_eval, "GB/s": 8.0 * m * n / ms_eval / 1e6}}
    line = {"metric": "layout copy GB/s", "value": res["layout_copy"]["GB/s"], "unit": "GB/s", "n_gpus": 1, "steps": steps,
            "warmup": warm, "ms_per_step": ms_copy, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32 (bytes) / int64 indices", "data": "synthetic", "config": {"workload": "layout_copy_f32_4096"},
            "gpu_launches": 2 * steps, "kernels": res,
            "roofline": {"bound": "hbm", "achieved": res["layout_copy"]["GB/s"], "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": res["layout_copy"]["GB/s"] / peaks["hbm_gbs"], "traffic": None,
                         "peak_source": f"hbm copy, of {peak_src}"}}
    print(json.dumps(line), flush=True)
    return 0


def max_ms(torch, dist, dev, ms):
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def multi_gpu_extras(mb, torch, dist, comm, dev, rank, world, name, A, B, C, barrier, peaks):
    """Outside the timed headline, at N > 1 GPUs: the all-gather of the M-sharded C through the library's own entry
    point, the splits the configurations state (one product cut into M / N rows per GPU; the decode weights cut
    along N; the copy cut into row blocks), each timed on the device as the max over ranks, and a parity check of
    this rank's shard against the CPU oracle."""
    import numpy as np
    import __graft_entry__ as ge
    out = {}
    stream = torch.cuda.current_stream()
    sp = mb.current_stream_ptr(dev)
    kind, M, N, K, o = WORKLOADS[name]

    def timed(fn, n=10, w=3):
        for _ in range(w):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(n):
            fn()
        e1.record(stream)
        barrier()
        return max_ms(torch, dist, dev, e0.elapsed_time(e1) / n)

    # (1) all-gather of C: every rank's (M, N) row-major shard into a preallocated (world*M, N) matrix, NCCL behind
    # moye_b200_allgather; checked against the shards themselves
    full = torch.empty(M * world, N, dtype=C.dtype, device=dev)
    ms = timed(lambda: comm.allgather(C, full, mode=0), n=5, w=2)
    shard_bytes = C.numel() * C.element_size()
    mine_ok = bool(torch.equal(full[rank * M:(rank + 1) * M], C))
    sums = torch.stack([full[r * M:(r + 1) * M].double().abs().sum() for r in range(world)])
    own = torch.zeros(world, dtype=torch.float64, device=dev)
    own[rank] = C.double().abs().sum()
    dist.all_reduce(own)
    ok = torch.tensor([1.0 if (mine_ok and bool(torch.equal(sums, own))) else 0.0], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    full[rank * M:(rank + 1) * M].copy_(C)
    ms_in_place = timed(lambda: comm.allgather(full[rank * M:(rank + 1) * M], full, mode=0), n=5, w=2)
    out["allgather_c"] = {"ms": ms, "shard_bytes": shard_bytes, "busbw_GB/s": shard_bytes * (world - 1) / ms / 1e6,
                          "in_place_ms": ms_in_place, "in_place_busbw_GB/s": shard_bytes * (world - 1) / ms_in_place / 1e6,
                          "assembled_equals_shards": bool(ok.item() == 1.0),
                          "how": "moye_b200_allgather (ncclAllGather into a preallocated matrix), not in `value`"}
    del full

    # (2) parity of this rank's shard of the headline product: 8 of its rows against the CPU oracle
    ho, _ = ge.load_oracle()
    ho.lib()
    rows = np.linspace(0, M - 1, 8).astype(np.int32)
    if kind in ("f16", "bf16"):
        bits = lambda t: t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16).ravel()
        ref = ho.gemm_samples(bits(A), bits(B), ho.F16 if kind == "f16" else ho.BF16, M, N, K, rows, by_rows=True,
                              threads=min(16, os.cpu_count() or 1))
        err = ho.max_rel_err(C[torch.from_numpy(rows).to(dev).long()].float().cpu().numpy(), ref)
        good = torch.tensor([1.0 if err <= 1e-2 else 0.0], device=dev)
        dist.all_reduce(good, op=dist.ReduceOp.MIN)
        out["shard_parity"] = bool(good.item() == 1.0)
        out["shard_parity_how"] = "8 rows of every rank's C shard against the CPU oracle (max relative error <= 1e-2)"

    # (3) strong scaling as the configurations state it: ONE product, M / world rows per GPU, B replicated
    strong = {}
    for wl in ("gemm_f16_8192", "gemm_f16_4096"):
        k2, M2, N2, K2, o2 = WORKLOADS[wl]
        lo, hi = mb.shard_range(M2, world, rank, 256)
        a2, b2, c2 = make_operands(torch, k2, M2, N2, K2, o2, dev, seed=40)   # same seed: every rank holds the same problem
        plan_full = mb.plan_gemm(c2, a2, b2, None)
        plan_shard = mb.plan_gemm(c2[lo:hi], a2[lo:hi], b2, None)
        t_shard = timed(lambda: plan_shard(sp), n=20, w=5)
        t_full = timed(lambda: plan_full(sp), n=10, w=3)     # the whole product on every GPU at once: the N = 1 time
        # this rank's shard against the same rows of the whole product (the split of K over CTA pairs may differ
        # between the two launches, so fp32 sums agree to rounding, not bit for bit)
        plan_full(sp)
        whole = c2.clone()
        c2.zero_()
        plan_shard(sp)
        diff = ((c2[lo:hi] - whole[lo:hi]).abs().max() / whole.abs().max()).item()
        same = torch.tensor([1.0 if diff <= 1e-5 else 0.0], device=dev)
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        fl = 2.0 * M2 * N2 * K2
        strong[wl] = {"rows_per_gpu": hi - lo, "ms": t_shard, "TFLOP/s": fl / t_shard / 1e9, "n1_ms": t_full,
                      "n1_TFLOP/s": fl / t_full / 1e9, "efficiency": t_full / (world * t_shard),
                      "shards_match_whole_product": bool(same.item() == 1.0)}
        del a2, b2, c2, whole, plan_full, plan_shard
        torch.cuda.empty_cache()
    out["strong"] = strong

    # (4) decode: W cut into N / world rows per GPU, X replicated; Y column-major so that a rank's columns are one
    # contiguous block; the all-gather of Y timed on its own
    k5, M5, N5, K5, o5 = WORKLOADS["decode_bf16_16x28672x8192"]
    lo, hi = mb.shard_range(N5, world, rank, 128)
    sets = [make_operands(torch, k5, M5, hi - lo, K5, o5, dev, seed=50 + i) for i in range(3)]   # rotate W: HBM, not L2
    ys = [torch.zeros(hi - lo, M5, dtype=torch.bfloat16, device=dev).t() for _ in sets]
    plans = [mb.plan_gemm(y, x, w, None) for (x, w, _), y in zip(sets, ys)]
    turn = [0]

    def decode_step():
        turn[0] += 1
        plans[turn[0] % len(plans)](sp)

    t_dec = timed(decode_step, n=20, w=5)
    nbytes = (M5 * K5 + N5 * K5 + M5 * N5) * 2
    yfull = torch.zeros(N5, M5, dtype=torch.bfloat16, device=dev).t()
    t_gather = timed(lambda: comm.allgather(ys[0], yfull, mode=1, align=128), n=10, w=3)
    out["decode_nshard"] = {"rows_of_W_per_gpu": hi - lo, "ms": t_dec, "GB/s": nbytes / t_dec / 1e6,
                            "frac_of_hbm_peak_per_gpu": nbytes / world / t_dec / 1e6 / peaks["hbm_gbs"],
                            "allgather_y_ms": t_gather, "allgather_y_bytes": M5 * N5 * 2,
                            "y_block_matches": bool(torch.equal(yfull[:, lo:hi], ys[0]))}
    del sets, ys, plans, yfull
    torch.cuda.empty_cache()

    # (5) copy: the 8192 x 8192 fp16 column-major matrix cut into blocks of 8192 / world rows (pitched sub-matrices)
    m = n = 8192
    lo, hi = mb.shard_range(m, world, rank, 128)
    srcs = [(torch.rand(n, m, device=dev) * 2 - 1).half() for _ in range(4)]
    dsts = [torch.zeros_like(x) for x in srcs]
    lay = mb.make_layout((hi - lo, n), (1, m))
    tc = mb.make_tma_tiled_copy(mb._lib.F16, (128, 64))
    cps = [mb.plan_copy(tc, mb.MoYeArray(d[:, lo:hi], lay), mb.MoYeArray(x[:, lo:hi], lay)) for d, x in zip(dsts, srcs)]

    def copy_step():
        turn[0] += 1
        cps[turn[0] % 4](sp)

    t_cp = timed(copy_step, n=20, w=5)
    good = torch.tensor([1.0 if torch.equal(dsts[1][:, lo:hi], srcs[1][:, lo:hi]) else 0.0], device=dev)
    dist.all_reduce(good, op=dist.ReduceOp.MIN)
    out["copy_rowblock"] = {"rows_per_gpu": hi - lo, "ms": t_cp, "GB/s": 2.0 * m * n * 2 / t_cp / 1e6,
                            "frac_of_hbm_peak_per_gpu": 2.0 * m * n * 2 / world / t_cp / 1e6 / peaks["hbm_gbs"],
                            "bit_exact": bool(good.item() == 1.0)}
    mb.synchronize_status(dev)
    return out


def sustained_rate(mb, torch, dev, plan, stream_ptr, flops, peaks, seconds=2.0):
    """The headline GEMM back to back for `seconds`: what the part delivers under its power limit, with the SM
    clock it settles at."""
    stream = torch.cuda.current_stream()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(20):
        plan(stream_ptr)
    e1.record(stream)
    torch.cuda.synchronize()
    n = max(50, int(seconds * 1e3 / (e0.elapsed_time(e1) / 20)))
    sampler = ClockSampler(dev.index)
    sampler.start()
    e0.record(stream)
    for _ in range(n):
        plan(stream_ptr)
    e1.record(stream)
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / n
    tf = flops / ms / 1e9
    return {"launches": n, "ms": ms, "TFLOP/s": tf, "frac_of_sustained_peak": tf / peaks["bf16_tflops_sustained"],
            "sm_mhz_median": clocks["sm_mhz"], "ms_x_mhz": ms * clocks["sm_mhz"] if clocks["sm_mhz"] else None,
            "reasons": clocks["reasons"]}


def extras(mb, torch, dev, peaks):
    """The other configurations, each timed alone for a few launches (reported beside the headline)."""
    out = {}
    stream = torch.cuda.current_stream()
    for name in ("gemm_f16_4096", "gemm_f16_8192_colmajor", "gemm_bf16_8192", "gemm_f32_8192_colmajor",
                 "gemm_f32_8192_colmajor_tf32", "gemm_s8_16384x8192x8192", "gemm_e4m3_16384x8192x8192",
                 "decode_bf16_16x28672x8192", "gemm_bf16_256x4096x4096"):
        kind, M, N, K, o = WORKLOADS[name]
        nset = 3 if M <= 32 else (12 if M <= 512 else 1)  # rotate weight buffers for the HBM-bound shapes
        sets = [make_operands(torch, kind, M, N, K, o, dev, seed=20 + i, colmajor=is_colmajor(name))
                for i in range(nset)]
        plans = [mb.plan_gemm(c, a, b, None, **gemm_kw(name)) for a, b, c in sets]
        sp = mb.current_stream_ptr(dev)
        i = [0]

        def fn():
            i[0] += 1
            plans[i[0] % nset](sp)

        ms = time_launches(torch, fn, 20, 5, stream, settle=0.5)
        if M <= 512:
            nbytes = (M * K + N * K + M * N) * 2
            out[name] = {"ms": ms, "GB/s": nbytes / ms / 1e6, "frac_of_hbm_peak": nbytes / ms / 1e6 / peaks["hbm_gbs"],
                         "TFLOP/s": 2.0 * M * N * K / ms / 1e9}
        else:
            out[name] = {"ms": ms, "TFLOP/s": 2.0 * M * N * K / ms / 1e9}
        del sets, plans
        torch.cuda.empty_cache()
    out["library_same_box"] = library_rates(torch, dev, out)
    out["copy_f16_8192"] = copy_rates(mb, torch, dev, peaks, 20, 5)
    out["transpose_8192"] = transpose_rates(mb, torch, dev, peaks, 20, 5)
    mb.synchronize_status(dev)
    return out


def library_rates(torch, dev, ours):
    """The vendor library (cuBLAS / cuBLASLt through torch) on the same box, same shapes and same data distributions, timed the
    same way: a yardstick for the kinds that have no driver-measured peak (8-bit), never part of `value`.  `ratio` = ours / library."""
    res = {}
    stream = torch.cuda.current_stream()

    def run(name, fn, flops):
        try:
            ms = time_launches(torch, fn, 10, 3, stream, settle=0.5)
        except Exception as e:  # a kind this torch build has no library kernel for
            res[name] = {"unavailable": str(e).splitlines()[0][:120]}
            return
        res[name] = {"ms": ms, "TFLOP/s": flops / ms / 1e9}
        if name in ours and "ms" in ours[name]:
            res[name]["ratio"] = ms / ours[name]["ms"]

    for name in ("gemm_f16_4096", "gemm_bf16_8192", "gemm_s8_16384x8192x8192", "gemm_e4m3_16384x8192x8192", "decode_bf16_16x28672x8192",
                 "gemm_bf16_256x4096x4096"):
        kind, M, N, K, o = WORKLOADS[name]
        nset = 3 if M <= 32 else (12 if M <= 512 else 1)
        sets = [make_operands(torch, kind, M, N, K, o, dev, seed=40 + i) for i in range(nset)]
        i = [0]
        if kind in ("f16", "bf16"):
            outs = [torch.empty(M, N, device=dev, dtype=a.dtype) for a, _, _ in sets]

            def fn():
                i[0] += 1
                a, b, _ = sets[i[0] % nset]
                torch.matmul(a, b.t(), out=outs[i[0] % nset])
        elif kind == "s8":
            def fn():
                i[0] += 1
                a, b, _ = sets[i[0] % nset]
                torch._int_mm(a, b.t())
        else:
            sa = torch.tensor(0.05, device=dev)
            sb = torch.tensor(0.02, device=dev)

            def fn():
                i[0] += 1
                a, b, _ = sets[i[0] % nset]
                torch._scaled_mm(a, b.t(), scale_a=sa, scale_b=sb, out_dtype=torch.bfloat16)
        run(name, fn, 2.0 * M * N * K)
        del sets
        torch.cuda.empty_cache()
    # Float32 operands, the element type of examples/gemm.jl (which checks itself against CUBLAS, :96): the library's fp32 GEMM
    # (no tensor cores) beside our Float32-accurate three-product form, and its tf32 mode beside our single tf32 product
    kind, M, N, K, o = WORKLOADS["gemm_f32_8192_colmajor"]
    a, b, c = make_operands(torch, kind, M, N, K, o, dev, seed=50, colmajor=True)
    was = torch.backends.cuda.matmul.allow_tf32
    try:
        for name, tf32 in (("gemm_f32_8192_colmajor", False), ("gemm_f32_8192_colmajor_tf32", True)):
            torch.backends.cuda.matmul.allow_tf32 = tf32
            run(name, lambda: torch.matmul(a, b.t(), out=c), 2.0 * M * N * K)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = was
    del a, b, c
    torch.cuda.empty_cache()
    res["note"] = ("torch.matmul / torch._int_mm / torch._scaled_mm; 16-bit library outputs are 16-bit where ours are fp32 for the "
                   "f16 / bf16 dense workloads (less output traffic for the library)")
    return res


def copy_rates(mb, torch, dev, peaks, steps, warmup):
    m = n = 8192
    srcs = [(torch.rand(n, m, device=dev) * 2 - 1).half() for _ in range(4)]  # 4 x 134 MB > L2
    dsts = [torch.zeros_like(s) for s in srcs]
    lay = mb.make_layout((m, n))
    res = {}
    stream = torch.cuda.current_stream()
    vec = mb.make_tiled_copy(mb.CopyAtom(mb.UniversalCopy(128), mb._lib.F16), mb.make_layout((16, 16)),
                             mb.make_layout((8, 1)))
    for label, tc in (("universal128", vec), ("tma", mb.make_tma_tiled_copy(mb._lib.F16, (128, 64)))):
        plans = [mb.plan_copy(tc, mb.MoYeArray(d, lay), mb.MoYeArray(s, lay)) for d, s in zip(dsts, srcs)]
        sp = mb.current_stream_ptr(dev)
        i = [0]

        def fn():
            i[0] += 1
            plans[i[0] % 4](sp)

        ms = time_launches(torch, fn, steps, warmup, stream, settle=0.5)
        gbs = 2.0 * m * n * 2 / ms / 1e6
        res[label] = {"ms": ms, "GB/s": gbs, "frac_of_hbm_peak": gbs / peaks["hbm_gbs"]}
    return res


def transpose_rates(mb, torch, dev, peaks, steps, warmup):
    """`copyto!(dest, transpose(src))` of an 8192 x 8192 matrix (the reference's transpose_kernel, test/host/copy_async.jl:51-95,
    at the copy workload's size), rotating 4 buffer pairs so that the traffic is HBM's."""
    m = n = 8192
    res = {}
    stream = torch.cuda.current_stream()
    for label, dt in (("f16", torch.float16), ("f32", torch.float32)):
        nset = 4 if dt == torch.float16 else 2  # each set exceeds the 126 MB L2 together with its destination
        srcs = [(torch.rand(n * m, device=dev) * 2 - 1).to(dt) for _ in range(nset)]
        dsts = [torch.zeros_like(s) for s in srcs]
        plans = [mb.plan_copy(mb.MoYeArray(d, mb.make_layout((m, n))), mb.transpose(mb.MoYeArray(s, mb.make_layout((n, m)))))
                 for d, s in zip(dsts, srcs)]
        sp = mb.current_stream_ptr(dev)
        i = [0]

        def fn():
            i[0] += 1
            plans[i[0] % nset](sp)

        ms = time_launches(torch, fn, steps, warmup, stream, settle=0.5)
        gbs = 2.0 * m * n * srcs[0].element_size() / ms / 1e6
        res[label] = {"ms": ms, "GB/s": gbs, "frac_of_hbm_peak": gbs / peaks["hbm_gbs"]}
        del srcs, dsts, plans
        torch.cuda.empty_cache()
    return res


def run_copy(args, mb, torch, dev, peaks, peak_src, rank, world, dist, barrier, transpose=False):
    sampler = ClockSampler(dev.index)
    barrier()
    sampler.start()
    res = (transpose_rates if transpose else copy_rates)(mb, torch, dev, peaks, args.steps, max(3, args.warmup))
    barrier()
    clocks = sampler.stop()
    best = max(res.values(), key=lambda r: r["GB/s"])
    t = torch.tensor([best["ms"]], device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    nbytes = best["GB/s"] * best["ms"] * 1e6
    line = {"metric": "transposing copy GB/s" if transpose else "copy GB/s", "value": nbytes * world / ms / 1e6, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16 (bytes)", "data": "synthetic",
            "config": {"workload": "transpose_8192" if transpose else "copy_f16_8192",
                       "tile": "TMA stages of 16 KB" if transpose else "128x64", "atoms": "128-bit",
                       "sharding": f"row blocks x{world}", "l2": "rotating buffer pairs, 134 MB or more each"},
            "clocks": clocks, "gpu_launches": args.steps * len(res), "kernels": res,
            "roofline": {"bound": "hbm", "achieved": best["GB/s"], "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": best["GB/s"] / peaks["hbm_gbs"], "traffic": None, "peak_source": f"hbm copy, of {peak_src}"}}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="gemm_f16_8192")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="device-timed kernel only (for profiler captures)")
    ap.add_argument("--path", type=int, default=0, help="force a GEMM kernel (moye_gemm_params_t.path); 0 = the library's choice")
    ap.add_argument("--tail", choices=["auto", "on", "off"], default="auto", help="K-split tail of the 256 x 512 kernel")
    args = ap.parse_args()
    if args.steps < 1:
        raise SystemExit("--steps must be >= 1")
    if args.impl == "reference":
        return run_reference_arm(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
