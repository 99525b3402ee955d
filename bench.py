"""Benchmark of the data-format hot path: fused tilize + Bfp8_b pack.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (per GPU): a batch of 64 fp32 activation tensors [1,1,4096,4096], values N(0,1) with 1 %
of the elements scaled x1e3 and 0.5 % exact zeros, packed to Bfp8_b tiles (17,825,792 bytes per
tensor).  One step = one pass over the batch.  With N GPUs every rank packs its own batch of 64
(weak scaling, no collective on the data path).

  value : whole-job GB/s of algorithmic bytes (5.0625 B per element: 4 read + 1.0625 written),
          inputs resident in HBM, one batched launch per step, timed with CUDA events.
  e2e   : the same metric through the host-buffer entry point (pinned host tensors in, host
          images out; copies inside the timed region).
  roofline : algorithmic bytes per launch / mean CUDA-event launch time, against the measured copy bandwidth of
          this pool's B200s; traffic = DRAM bytes of one launch from a profiler capture.
  cpu_baseline : the CPU port of the same path on the box's host cores, on a bounded sample of the batch.

--impl reference times the CPU implementation of the same path (the oracle port, OpenMP over all
host cores) on the same workload and prints the same line with "impl": "reference".
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tt-buda_b200"))

N_TENSORS = 64
SHAPE = (1, 1, 4096, 4096)
ELEMS = 4096 * 4096
BYTES_PER_ELEM = 4 + 1.0625
IMAGE_BYTES = 17825792
WORKLOAD = "64 x fp32 [1,1,4096,4096] N(0,1), 1% x1e3 outliers, 0.5% zeros -> Bfp8_b tiles"


def tensor_peak_tflops(sustained=False):
    """Measured dense bf16 peak of this pool's B200s (burst, or the seconds-long sustained figure), else the stated fallback."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
            return float(d.get("bf16_tflops_sustained", 1400.0) if sustained else d.get("bf16_tflops", 1590.0))
    return 1400.0 if sustained else 1590.0


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons (NVML, read-only queries) while the timed region runs."""

    def __init__(self, index, period_s=0.01):
        self.index = index
        self.period = period_s
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._nvml = None
        self._h = None
        try:
            import pynvml

            pynvml.nvmlInit()
            # NVML indexes physical devices; honour CUDA_VISIBLE_DEVICES when it lists ordinals
            vis = os.environ.get("CUDA_VISIBLE_DEVICES", "")
            phys = index
            if vis and all(v.strip().isdigit() for v in vis.split(",")):
                phys = int(vis.split(",")[index])
            self._h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
            self._nvml = pynvml
        except Exception:
            self._nvml = None

    def _sample_nvml(self):
        n = self._nvml
        self.samples.append(float(n.nvmlDeviceGetClockInfo(self._h, n.NVML_CLOCK_SM)))
        r = n.nvmlDeviceGetCurrentClocksEventReasons(self._h) if hasattr(n, "nvmlDeviceGetCurrentClocksEventReasons") \
            else n.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
        for name, bit in (("hw_slowdown", 0x8), ("sw_power_cap", 0x4), ("sw_thermal_slowdown", 0x20),
                          ("hw_thermal_slowdown", 0x40), ("hw_power_brake_slowdown", 0x80)):
            if r & bit:
                self.reasons.add(name)

    def _sample_smi(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        out = subprocess.run(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + q, "--format=csv,noheader,nounits"],
                             capture_output=True, text=True, timeout=5).stdout
        f = [x.strip() for x in out.strip().split(",")]
        if len(f) >= 6:
            self.samples.append(float(f[0]))
            self.max_mhz = float(f[1])
            for nme, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    self.reasons.add(nme)

    def _run(self):
        while not self._stop.is_set():
            try:
                if self._nvml is not None:
                    self._sample_nvml()
                else:
                    self._sample_smi()
            except Exception:
                pass
            self._stop.wait(self.period if self._nvml is not None else 0.2)

    def __enter__(self):
        self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s), "source": "nvml" if self._nvml is not None else "nvidia-smi"}


_PROBE = None


def probe_lib():
    global _PROBE
    if _PROBE is None:
        _PROBE = ctypes.CDLL(os.path.join(ROOT, "tt-buda_b200", "lib", "libbuda_probe.so"))
        _PROBE.buda_probe_stream.restype = ctypes.c_int
        _PROBE.buda_probe_stream.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_uint64, ctypes.c_int,
                                             ctypes.POINTER(ctypes.c_float), ctypes.c_void_p]
        _PROBE.buda_probe_peer_stores.restype = ctypes.c_int
        _PROBE.buda_probe_peer_stores.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.c_uint32,
                                                  ctypes.c_uint32, ctypes.c_uint64, ctypes.c_void_p]
    return _PROBE


def stream_probe(torch, mix, schedule, elements=1 << 29, reps=10):
    """GB/s of a bare streaming kernel with the conversion kernels' access shape and none of their arithmetic
    (tt-buda_b200/csrc/bench/stream_probe.cu, built into libbuda_probe.so, which only this benchmark loads).
    mix 0 = 4 bytes read per byte written, 1 = the reverse, 2 = reads only, 3 = writes only; schedule 0 = one block
    per band, 1 = resident blocks on a fixed stride, 2 = resident blocks on a device counter."""
    ms = ctypes.c_float(0.0)
    rc = probe_lib().buda_probe_stream(int(mix), int(schedule), int(elements), int(reps), ctypes.byref(ms),
                                  ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    if rc != 0:
        raise RuntimeError("stream probe failed")
    nbytes = elements * (5.0 if mix in (0, 1) else 4.0)
    return nbytes / (ms.value * 1e-3) / 1e9


def host_cores():
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def gpu_numa_node(torch, index):
    """NUMA node the GPU's PCIe slot hangs off (sysfs; None when it cannot be read)."""
    try:
        p = torch.cuda.get_device_properties(index)
        bdf = "%04x:%02x:%02x.0" % (p.pci_domain_id, p.pci_bus_id, p.pci_device_id)
        with open(f"/sys/bus/pci/devices/{bdf}/numa_node") as f:
            return int(f.read().strip())
    except Exception:
        return None


def make_batch(torch, device, seed0, n):
    """Synthetic batch with the value distribution of the config (generated on the device)."""
    xs = []
    g = torch.Generator(device=device)
    for i in range(n):
        g.manual_seed(seed0 + i)
        x = torch.randn(SHAPE, generator=g, device=device)
        x = torch.where(torch.rand(SHAPE, generator=g, device=device) < 0.01, x * 1e3, x)
        x = torch.where(torch.rand(SHAPE, generator=g, device=device) < 0.005, torch.zeros((), device=device), x)
        xs.append(x)
    return xs


_RESULT_OUT = None


def emit(text):
    """Write a result line to the process's original standard output."""
    out = _RESULT_OUT or sys.stdout
    out.write(text + "\n")
    out.flush()


def keep_stdout_for_results():
    """Point file descriptor 1 at standard error for everything else this process (and the libraries it loads: NCCL
    prints a version banner on fd 1 when NCCL_DEBUG is set) may write, so that standard output carries the result
    line and nothing else."""
    global _RESULT_OUT
    if _RESULT_OUT is None:
        sys.stdout.flush()
        _RESULT_OUT = os.fdopen(os.dup(1), "w")
        os.dup2(2, 1)


def profile_one(torch, cuda_ops, dev, name, reps=20, nt=8):
    """One secondary kernel on a case that ends by itself in milliseconds: for ncu captures."""
    if name == "bare_streams":
        # every mix x schedule of the bare streaming kernels, 2^29 elements (2 GiB on the 4-byte side)
        n_el = 1 << 29
        out = {"elements": n_el, "unit": "GB/s"}
        for mix, mname in ((0, "4_read_1_written"), (1, "1_read_4_written"), (2, "read_only"), (3, "write_only")):
            out[mname] = {sname: round(stream_probe(torch, mix, sv, n_el), 1)
                          for sname, sv in (("one_block_per_band", 0), ("resident_fixed_stride", 1), ("resident_device_counter", 2))}
        emit(json.dumps({"kernel": name, **out}))
        return
    if name == "gemm":
        M, K, N = 8192, 4096, 16384
        a = torch.randn(M, K, device=dev).bfloat16()
        wimg = cuda_ops.tilize_pack(torch.randn(1, 1, K, N, device=dev) * 0.02, cuda_ops.DF.Bfp8_b)
        c = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        fn, work, unit = (lambda: cuda_ops.bfp8b_matmul(a, wimg, N, out=c)), 2.0 * M * N * K / 1e12, "TFLOP/s"
    elif name == "i8gemm":
        M, K, N = 8192, 4096, 16384
        a = torch.randint(-128, 128, (M, K), device=dev, dtype=torch.int8)
        wimg = cuda_ops.tilize_pack(torch.randint(-128, 128, (1, 1, K, N), device=dev, dtype=torch.int8), cuda_ops.DF.Int8)
        sc = torch.rand(N, device=dev) * 2e-5
        fn, work, unit = (lambda: cuda_ops.i8_matmul(a, wimg, N, scale=sc, zero_point=0.0, out="int8")), 2.0 * M * N * K / 1e12, "TOP/s"
    elif name in ("pack_bf16", "unpack_bf16"):
        xs = [torch.randn(SHAPE, device=dev).bfloat16() for _ in range(nt)]
        imgs = cuda_ops.tilize_pack_batch(xs, cuda_ops.DF.Bfp8_b)
        if name == "pack_bf16":
            fn = lambda: cuda_ops.tilize_pack_batch(xs, cuda_ops.DF.Bfp8_b, outs=imgs)
        else:
            fn = lambda: cuda_ops.unpack_untilize_batch(imgs, cuda_ops.DF.Bfp8_b, SHAPE, outs=xs)
        work, unit = nt * ELEMS * 3.0625 / 1e9, "GB/s"
    elif name in ("tilize_fp32", "untilize_fp32", "tilize_int8", "untilize_int8"):
        # plain relayout (no format change): 2 x element size per element
        if name.endswith("int8"):
            xs = [torch.randint(-128, 128, SHAPE, device=dev, dtype=torch.int8) for _ in range(nt)]
            df, es = cuda_ops.DF.Int8, 1
        else:
            xs = [torch.randn(SHAPE, device=dev) for _ in range(nt)]
            df, es = cuda_ops.DF.Float32, 4
        imgs = cuda_ops.tilize_pack_batch(xs, df)
        if name.startswith("tilize"):
            fn = lambda: cuda_ops.tilize_pack_batch(xs, df, outs=imgs)
        else:
            fn = lambda: cuda_ops.unpack_untilize_batch(imgs, df, SHAPE, outs=xs)
        work, unit = nt * ELEMS * 2 * es / 1e9, "GB/s"
    elif name in ("pack_lf8", "unpack_lf8"):
        xs = [torch.randn(SHAPE, device=dev) for _ in range(nt)]
        imgs = cuda_ops.tilize_pack_batch(xs, cuda_ops.DF.Lf8)
        if name == "pack_lf8":
            fn = lambda: cuda_ops.tilize_pack_batch(xs, cuda_ops.DF.Lf8, outs=imgs)
        else:
            fn = lambda: cuda_ops.unpack_untilize_batch(imgs, cuda_ops.DF.Lf8, SHAPE, outs=xs)
        work, unit = nt * ELEMS * 5 / 1e9, "GB/s"
    elif name in ("pack_jobs", "unpack_jobs"):
        # the general kernel flavour (job table) on a uniform batch
        xs = [torch.randn(SHAPE, device=dev) for _ in range(nt)]
        tj = cuda_ops.TensorJobs(xs, cuda_ops.DF.Bfp8_b)
        tj.pack()
        fn = tj.pack if name == "pack_jobs" else tj.unpack
        work, unit = nt * ELEMS * BYTES_PER_ELEM / 1e9, "GB/s"
    elif name in ("pack", "unpack", "pack_direct", "unpack_direct"):
        xs = [torch.randn(SHAPE, device=dev) for _ in range(nt)]
        imgs = cuda_ops.tilize_pack_batch(xs, cuda_ops.DF.Bfp8_b)
        path = 1 if name.endswith("_direct") else None      # 1 = the kernels that unaligned tensors and tiny tiles take
        if name in ("pack", "pack_direct"):
            fn = lambda: cuda_ops.tilize_pack_batch(xs, cuda_ops.DF.Bfp8_b, outs=imgs, path=1 if name == "pack_direct" else None)
        else:
            fn = lambda: cuda_ops.unpack_untilize_batch(imgs, cuda_ops.DF.Bfp8_b, SHAPE, outs=xs, path=path)
        work, unit = nt * ELEMS * BYTES_PER_ELEM / 1e9, "GB/s"
    else:
        n = 32 * 1024 * 1024 * 4  # 512 MiB of fp32: larger than L2
        sc = torch.tensor([0.05], device=dev)
        if name == "quantize":
            x = torch.rand(n, device=dev) * 12 - 6
            fn = lambda: cuda_ops.quantize(x, sc, 3)
        elif name == "dequantize":
            q = torch.randint(-128, 128, (n,), device=dev, dtype=torch.int8)
            fn = lambda: cuda_ops.dequantize(q, sc, 3)
        else:
            acc = torch.randint(-2 ** 20, 2 ** 20, (n // 1024, 1024), device=dev, dtype=torch.int32)
            scs = torch.rand(1024, device=dev) * (1e-2 - 1e-4) + 1e-4
            fn = lambda: cuda_ops.buda_requantize(acc, scs, 0)
        work, unit = n * 5 / 1e9, "GB/s"
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a0.record()
    for _ in range(reps):
        fn()
    a1.record()
    torch.cuda.synchronize()
    ms = a0.elapsed_time(a1) / reps
    emit(json.dumps({"kernel": name, "ms": ms, unit: work / (ms * 1e-3)}))


def run_reference(args, rank, world):
    """The reference path on the host cores: tilize + Bfp8_b pack by the CPU port, all threads."""
    if rank != 0:
        return
    import numpy as np
    from oracle import budaref as R

    R.build()
    # torchrun exports OMP_NUM_THREADS=1 to its workers: give the CPU arm the host's cores back
    R.set_threads(host_cores())
    n_sample = 4  # tensors per step: a bounded sample of the 64-tensor batch
    rng = np.random.default_rng(1000)
    xs = []
    for _ in range(n_sample):
        x = rng.standard_normal(SHAPE, dtype=np.float32)
        x[rng.random(SHAPE) < 0.01] *= 1e3
        x[rng.random(SHAPE) < 0.005] = 0.0
        xs.append(x)
    for _ in range(max(1, args.warmup)):
        R.tilize_pack(xs[0], R.Bfp8_b)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        for x in xs:
            R.tilize_pack(x, R.Bfp8_b)
    dt = time.perf_counter() - t0
    gbs = args.steps * n_sample * ELEMS * BYTES_PER_ELEM / dt / 1e9
    line = {
        "impl": "reference", "metric": "bfp8b_tilize_pack_throughput", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": f"{n_sample} of the 64 tensors per step"},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": R.threads(), "kind": "port",
                         "sample": f"{n_sample} tensors x {args.steps} steps"},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(json.dumps(line))


def main():
    keep_stdout_for_results()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--no-extras", action="store_true", help="skip the secondary kernels' figures")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (for profiler captures)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg (for profiler captures)")
    ap.add_argument("--tensors", type=int, default=N_TENSORS,
                    help="tensors per GPU batch; anything but 64 is a reduced case for profiler captures")
    ap.add_argument("--profile-kernel", default=None, choices=["bare_streams", "gemm", "i8gemm", "tilize_fp32", "untilize_fp32", "tilize_int8", "untilize_int8", "pack_lf8", "unpack_lf8", "pack_jobs", "unpack_jobs", "pack", "unpack", "pack_direct", "unpack_direct", "pack_bf16", "unpack_bf16", "quantize", "dequantize", "requantize"],
                    help="run only this secondary kernel a few times and exit (small, self-ending case for profiler captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU fallback")
    from pybuda import _cabi, cuda_ops

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v):
        if dist is None:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    hbm_peak, peak_kind = peaks()
    if args.profile_kernel:
        profile_one(torch, cuda_ops, dev, args.profile_kernel, nt=8 if args.tensors == N_TENSORS else args.tensors)
        return
    NT = args.tensors
    xs = make_batch(torch, dev, 1000 + N_TENSORS * rank, NT)
    outs = [torch.empty(IMAGE_BYTES, dtype=torch.uint8, device=dev) for _ in range(NT)]
    algo_bytes_step = NT * ELEMS * BYTES_PER_ELEM

    def step():
        cuda_ops.tilize_pack_batch(xs, cuda_ops.DF.Bfp8_b, outs=outs)

    # ------------------------------------------------------------------ value: device resident
    for _ in range(args.warmup):
        step()
    barrier()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    launches0 = _cabi.launch_count()
    with ClockSampler(local_rank) as clocks:
        t_begin = torch.cuda.Event(enable_timing=True)
        t_end = torch.cuda.Event(enable_timing=True)
        t_begin.record()
        for a, b in ev:
            a.record()
            step()
            b.record()
        t_end.record()
        barrier()
    launches = _cabi.launch_count() - launches0
    total_ms = max_over_ranks(t_begin.elapsed_time(t_end))
    kernel_ms = sum(a.elapsed_time(b) for a, b in ev) / len(ev)
    rc, st = _cabi.device_status()
    if rc != 0:
        raise SystemExit(f"device status {st}: a kernel gave up waiting")
    value = world * args.steps * algo_bytes_step / (total_ms * 1e-3) / 1e9
    achieved = algo_bytes_step / (kernel_ms * 1e-3) / 1e9

    # ------------------------------------------------------------------ the bytes that were timed, against the oracle
    parity_sample = None
    if rank == 0 and not args.no_cpu:
        try:
            from oracle import budaref as R

            R.build()
            R.set_threads(host_cores())
            parity_sample = bool((outs[0].cpu().numpy() == R.tilize_pack(xs[0].cpu().numpy(), R.Bfp8_b)).all())
        except Exception as exc:
            parity_sample = f"not checked: {exc}"

    # ------------------------------------------------------------------ strong scaling: the config's 64 tensors dealt to the ranks
    # tensor i -> GPU i mod g: a rank packs 64 / g tensors in one launch per step (8 at 8 GPUs, a ~95 us launch)
    strong = None
    try:
        from pybuda.sharding import units_of_rank

        mine = len(units_of_rank(N_TENSORS, rank, world)) if NT == N_TENSORS else max(1, NT // world)
        sx, so = xs[:mine], outs[:mine]
        for _ in range(args.warmup):
            cuda_ops.tilize_pack_batch(sx, cuda_ops.DF.Bfp8_b, outs=so)
        barrier()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(args.steps):
            cuda_ops.tilize_pack_batch(sx, cuda_ops.DF.Bfp8_b, outs=so)
        s1.record()
        barrier()
        s_ms = max_over_ranks(s0.elapsed_time(s1)) / args.steps
        total_tensors = N_TENSORS if NT == N_TENSORS else mine * world
        s_gbs = total_tensors * ELEMS * BYTES_PER_ELEM / (s_ms * 1e-3) / 1e9
        strong = {"value": s_gbs, "unit": "GB/s", "tensors_total": total_tensors, "tensors_per_gpu": mine, "ms_per_step": s_ms,
                  "launches_per_step_per_gpu": 1, "frac_hbm_per_gpu": s_gbs / world / hbm_peak,
                  "note": "the batch of 64 shared out (tensor i -> GPU i mod g); time = slowest rank's launch"}
    except Exception as exc:
        strong = {"value": None, "error": str(exc)}

    # ------------------------------------------------------------------ e2e: host buffers in and out
    e2e = None
    try:
        if args.no_e2e:
            raise RuntimeError("skipped (--no-e2e)")
        hx = [torch.empty(SHAPE, dtype=torch.float32).pin_memory() for _ in range(NT)]
        for h, x in zip(hx, xs):
            h.copy_(x)
        himg = [torch.empty(IMAGE_BYTES, dtype=torch.uint8).pin_memory() for _ in range(NT)]
        geom = _cabi.QueueGeom.for_shape(SHAPE)
        shape_c, strides_c = _cabi.u32x4(SHAPE), _cabi.u64x4(_cabi.dense_strides(list(SHAPE), 4))

        src_tab, dst_tab = _cabi.ptr_array([h.data_ptr() for h in hx]), _cabi.ptr_array([o.data_ptr() for o in himg])

        def e2e_step():
            # one call for the step's batch: the copy-in / kernel / copy-out pipeline runs across the 64 tensors
            _cabi.check(_cabi.lib.buda_tilize_pack_host_batch(NT, src_tab, 0, shape_c, strides_c, ctypes.byref(geom), 6, 0, dst_tab,
                                                              IMAGE_BYTES, None))

        def e2e_step_per_tensor():
            for h, o in zip(hx, himg):
                _cabi.check(_cabi.lib.buda_tilize_pack_host(h.data_ptr(), 0, shape_c, strides_c, ctypes.byref(geom), 6, 0,
                                                            o.data_ptr(), IMAGE_BYTES, None))

        def run_e2e(fn, steps):
            fn()
            barrier()
            t0 = time.perf_counter()
            for _ in range(steps):
                fn()
            barrier()
            return max_over_ranks(time.perf_counter() - t0)

        e2e_s = run_e2e(e2e_step, args.e2e_steps)
        same = bool(torch.equal(himg[-1], outs[-1].cpu())) and bool(torch.equal(himg[0], outs[0].cpu()))
        per_tensor_s = run_e2e(e2e_step_per_tensor, 1)
        e2e = {"value": world * args.e2e_steps * algo_bytes_step / e2e_s / 1e9, "unit": "GB/s",
               "h2d_bytes_per_step": NT * ELEMS * 4, "d2h_bytes_per_step": NT * IMAGE_BYTES,
               "steps": args.e2e_steps, "api": "buda_tilize_pack_host_batch (pinned host tensors, one call per step)",
               "matches_device_path": same,
               "h2d_gbs_per_gpu": NT * ELEMS * 4 * args.e2e_steps / e2e_s / 1e9,
               "d2h_gbs_per_gpu": NT * IMAGE_BYTES * args.e2e_steps / e2e_s / 1e9,
               "gpu_numa_node": gpu_numa_node(torch, local_rank), "host_cores": host_cores(),
               "limiter": "host-to-device copy over PCIe (4 of every 5.06 bytes moved); with several GPUs behind one "
                          "NUMA node the ranks also share that node's memory bandwidth",
               "one_call_per_tensor": {"value": world * algo_bytes_step / per_tensor_s / 1e9, "api": "buda_tilize_pack_host x 64"}}
        del hx, himg
    except Exception as exc:  # report, never hide
        e2e = {"value": None, "unit": "GB/s", "error": str(exc)}

    # ------------------------------------------------------------------ secondary kernels (not the headline)
    extras = {}
    if not args.no_extras:
        def timed(fn, nbytes, reps=10):
            # each secondary figure is a kernel timed by itself: a short rest first, so that it does not inherit the
            # power state of the loop before it (the same kernel measured 0.91 and 1.01 of the copy peak without one)
            torch.cuda.synchronize()
            time.sleep(0.25)
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(reps):
                fn()
            b.record()
            torch.cuda.synchronize()
            ms = a.elapsed_time(b) / reps
            return {"GB/s": round(nbytes / (ms * 1e-3) / 1e9, 1), "frac_hbm": round(nbytes / (ms * 1e-3) / 1e9 / hbm_peak, 3),
                    "ms": round(ms, 4)}

        try:
            for name, df, ib in (("pack_bfp4_b", cuda_ops.DF.Bfp4_b, 9437184), ("pack_bfp2_b", cuda_ops.DF.Bfp2_b, 5242880)):
                o2 = [o[:ib] for o in outs]
                extras[name] = timed(lambda: cuda_ops.tilize_pack_batch(xs, df, outs=o2), NT * (ELEMS * 4 + ib))
            extras["pack_bfp8_b_direct_kernel"] = timed(
                lambda: cuda_ops.tilize_pack_batch(xs, cuda_ops.DF.Bfp8_b, outs=outs, path=1), algo_bytes_step)
            # the general kernel flavour (job table) on the same uniform batch: what the table look-ups cost by themselves
            tj = cuda_ops.TensorJobs(xs, cuda_ops.DF.Bfp8_b, images=outs)
            extras["pack_bfp8_b_job_table_flavour"] = timed(tj.pack, algo_bytes_step)
            # the same flavour under a non-default layout policy (truncation instead of rounding; then every switch flipped)
            try:
                cuda_ops.set_bfp_policy(_cabi.BfpPolicy(rounding=1))
                extras["pack_bfp8_b_truncate_policy"] = timed(tj.pack, algo_bytes_step)
                cuda_ops.set_bfp_policy(_cabi.BfpPolicy(rounding=0, overflow=1, face_order=(1, 0, 3, 2), exponent_order=1, datum_order=1))
                extras["pack_bfp8_b_all_switches_policy"] = timed(tj.pack, algo_bytes_step)
            finally:
                cuda_ops.set_bfp_policy(None)
            tj.pack()                                       # the images in the default layout again
            del tj
            nu = min(16, NT)
            # bfloat16 source (2 + 1.0625 bytes per element) and bfloat16 destination
            xb = [x.bfloat16() for x in xs[:nu]]
            extras["pack_bfp8_b_from_bf16"] = timed(lambda: cuda_ops.tilize_pack_batch(xb, cuda_ops.DF.Bfp8_b, outs=outs[:nu]),
                                                    nu * ELEMS * 3.0625)
            extras["unpack_bfp8_b_to_bf16"] = timed(
                lambda: cuda_ops.unpack_untilize_batch(outs[:nu], cuda_ops.DF.Bfp8_b, SHAPE, outs=xb), nu * ELEMS * 3.0625)
            del xb
            cuda_ops.tilize_pack_batch(xs[:nu], cuda_ops.DF.Bfp8_b, outs=outs[:nu])      # the images of the fp32 tensors again
            ys = [torch.empty(SHAPE, dtype=torch.float32, device=dev) for _ in range(nu)]
            extras["unpack_bfp8_b"] = timed(
                lambda: cuda_ops.unpack_untilize_batch(outs[:nu], cuda_ops.DF.Bfp8_b, SHAPE, outs=ys), nu * ELEMS * BYTES_PER_ELEM)
            extras["unpack_bfp8_b_direct_kernel"] = timed(
                lambda: cuda_ops.unpack_untilize_batch(outs[:nu], cuda_ops.DF.Bfp8_b, SHAPE, outs=ys, path=1),
                nu * ELEMS * BYTES_PER_ELEM)
            del ys
            # plain relayout (tilize / untilize without a format change): 2 x element size per element
            for tname, tdt, tdf, tes in (("fp32", torch.float32, cuda_ops.DF.Float32, 4), ("bf16", torch.bfloat16, cuda_ops.DF.Float16_b, 2),
                                         ("int8", torch.int8, cuda_ops.DF.Int8, 1)):
                xr = [(torch.randint(-128, 128, SHAPE, device=dev, dtype=torch.int8) if tdt == torch.int8 else x.to(tdt))
                      for x in xs[:nu]]
                ir = cuda_ops.tilize_pack_batch(xr, tdf)
                extras[f"relayout_{tname}_tilize"] = timed(lambda: cuda_ops.tilize_pack_batch(xr, tdf, outs=ir), nu * ELEMS * 2 * tes)
                extras[f"relayout_{tname}_untilize"] = timed(
                    lambda: cuda_ops.unpack_untilize_batch(ir, tdf, SHAPE, outs=xr), nu * ELEMS * 2 * tes)
                del xr, ir
            # Lf8 (one 1-5-2 float per element): conversions of the direct kernels, 5 bytes per element
            il = cuda_ops.tilize_pack_batch(xs[:nu], cuda_ops.DF.Lf8)
            extras["pack_lf8_from_fp32"] = timed(lambda: cuda_ops.tilize_pack_batch(xs[:nu], cuda_ops.DF.Lf8, outs=il), nu * ELEMS * 5)
            yl = [torch.empty(SHAPE, dtype=torch.float32, device=dev) for _ in range(nu)]
            extras["unpack_lf8_to_fp32"] = timed(lambda: cuda_ops.unpack_untilize_batch(il, cuda_ops.DF.Lf8, SHAPE, outs=yl), nu * ELEMS * 5)
            del il, yl
            n3 = 32 * 1024 * 1024
            # config-3 tensors are about the size of L2: every call takes the next of four copies of its input, so no
            # call finds its input (or the previous call's output) still in the cache
            rot = [0]

            def nxt(bufs):
                rot[0] += 1
                return bufs[rot[0] % len(bufs)]

            x3s = [torch.rand(32, 1024, 1024, device=dev) * 12 - 6 for _ in range(4)]
            sc = torch.tensor([0.05], device=dev)
            extras["quantize"] = timed(lambda: cuda_ops.quantize(nxt(x3s), sc, 3), n3 * 5)
            q3s = [cuda_ops.quantize(x, sc, 3) for x in x3s]
            extras["dequantize"] = timed(lambda: cuda_ops.dequantize(nxt(q3s), sc, 3), n3 * 5)
            del x3s
            accs = [torch.randint(-2 ** 20, 2 ** 20, (32, 1024, 1024), device=dev, dtype=torch.int32) for _ in range(4)]
            scs = torch.rand(1024, device=dev) * (1e-2 - 1e-4) + 1e-4
            extras["requantize"] = timed(lambda: cuda_ops.buda_requantize(nxt(accs), scs, 0), n3 * 5)
            del q3s, accs
        except Exception as exc:
            extras["error"] = str(exc)
        try:
            M, K, N = 8192, 4096, 16384
            a = torch.randn(M, K, device=dev).bfloat16()
            w = torch.randn(1, 1, K, N, device=dev) * 0.02
            wimg = cuda_ops.tilize_pack(w, cuda_ops.DF.Bfp8_b)
            c = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
            r = timed(lambda: cuda_ops.bfp8b_matmul(a, wimg, N, out=c), 0, reps=5)
            tf = 2.0 * M * N * K / (r["ms"] * 1e-3) / 1e12
            extras["bfp8b_gemm_8192x4096x16384"] = {"TFLOP/s": round(tf, 1), "ms": r["ms"],
                                                    "frac_tensor_burst": round(tf / tensor_peak_tflops(), 3),
                                                    "frac_tensor_sustained": round(tf / tensor_peak_tflops(True), 3)}
            ai = torch.randint(-128, 128, (M, K), device=dev, dtype=torch.int8)
            wi = cuda_ops.tilize_pack(torch.randint(-128, 128, (1, 1, K, N), device=dev, dtype=torch.int8), cuda_ops.DF.Int8)
            sci = torch.rand(N, device=dev) * 2e-5
            r = timed(lambda: cuda_ops.i8_matmul(ai, wi, N, scale=sci, zero_point=0.0, out="int8"), 0, reps=5)
            i8 = {"TOP/s": round(2.0 * M * N * K / (r["ms"] * 1e-3) / 1e12, 1), "ms": r["ms"]}
            try:
                # the denominator: the library's int8 matmul of the same size on this GPU, now (int32 out, no requantisation)
                bi = torch.randint(-128, 128, (K, N), device=dev, dtype=torch.int8)
                rl = timed(lambda: torch._int_mm(ai, bi), 0, reps=5)
                i8["library_int8_matmul_TOP/s"] = round(2.0 * M * N * K / (rl["ms"] * 1e-3) / 1e12, 1)
                i8["frac_of_library_int8_matmul"] = round(rl["ms"] / r["ms"], 3)
                del bi
            except Exception as exc:
                i8["library_int8_matmul_TOP/s"] = None
                i8["library_note"] = str(exc)[:120]
            extras["i8_gemm_requant_8192x4096x16384"] = i8
            del ai, wi
        except Exception as exc:
            extras["bfp8b_gemm_8192x4096x16384"] = {"error": str(exc)}

    # ------------------------------------------------------------------ what the memory system gives a bare stream
    # Kernels with the conversion kernels' access shape and no arithmetic (buda_stream_probe), on this GPU, now: the
    # measured copy peak is a 1:1 stream, a pack reads 4 bytes per byte written and an unpack the reverse.
    bare_pack_mix = None
    if not args.no_extras:
        try:
            n_el = 1 << 28
            sched = (("one_block_per_band", 0), ("resident_fixed_stride", 1), ("resident_device_counter", 2))
            bare = {"elements": n_el, "unit": "GB/s",
                    "pack_mix_4_read_1_written": {k: round(stream_probe(torch, 0, v, n_el), 1) for k, v in sched},
                    "unpack_mix_1_read_4_written": {k: round(stream_probe(torch, 1, v, n_el), 1) for k, v in sched},
                    "read_only": round(stream_probe(torch, 2, 0, n_el), 1),
                    "write_only": round(stream_probe(torch, 3, 0, n_el), 1)}
            bare_pack_mix = max(bare["pack_mix_4_read_1_written"].values())
            extras["bare_streams"] = bare
        except Exception as exc:
            extras["bare_streams"] = {"error": str(exc)}

    # ------------------------------------------------------------------ BERT-large weight set, layers dealt to the ranks
    if not args.no_extras:
        try:
            from pybuda.sharding import units_of_rank

            layers = units_of_rank(24, rank, world)        # layer l -> rank l % world (3 each at 8 GPUs)
            ws = []                                         # Q, K, V, O [1024,1024]; FFN [1024,4096], [4096,1024]
            for l in layers:
                for j, shp in enumerate([(1024, 1024)] * 4 + [(1024, 4096), (4096, 1024)]):
                    g = torch.Generator(device=dev).manual_seed(2000 + 6 * l + j)
                    ws.append(torch.randn((1, 1) + shp, generator=g, device=dev) * 0.02)
            fwd = cuda_ops.TensorJobs(ws, cuda_ops.DF.Bfp8_b)                      # job tables prepared once
            imgs = fwd.pack()
            backs = [torch.empty_like(t) for t in ws]
            bwd = cuda_ops.TensorJobs(backs, cuda_ops.DF.Bfp8_b, images=imgs)
            lc0 = _cabi.launch_count()

            def round_trip():
                # the whole set, whatever its shapes: one pack launch and one unpack launch
                fwd.pack()
                bwd.unpack()

            round_trip()
            launches_rt = _cabi.launch_count() - lc0
            for _ in range(3):
                round_trip()
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(10):
                round_trip()
            e1.record()
            barrier()
            ms = max_over_ranks(e0.elapsed_time(e1) / 10)
            elems = 24 * (4 * 1024 * 1024 + 2 * 1024 * 4096)          # 301,989,888 over all ranks
            extras["bert_large_weights_fp32_bfp8b_fp32"] = {
                "GB/s": round(elems * 2 * BYTES_PER_ELEM / (ms * 1e-3) / 1e9, 1), "ms": round(ms, 4), "layers_per_rank": len(layers),
                "frac_hbm_per_gpu": round(elems * 2 * BYTES_PER_ELEM / (ms * 1e-3) / 1e9 / world / hbm_peak, 3),
                "launches_per_round_trip": int(launches_rt),
                "note": "pack + unpack of this rank's layers through the job-table entry points (all shapes in one launch "
                        "each way); the set is 1.5 GB over all ranks, so at 8 GPUs a rank's share (191 MB) is near the size of L2"}
            del ws, imgs, backs, fwd, bwd
        except Exception as exc:
            extras["bert_large_weights_fp32_bfp8b_fp32"] = {"error": str(exc)}

    # ------------------------------------------------------------------ column-parallel matmul over the ranks (N > 1)
    if world > 1 and not args.no_extras:
        try:
            from pybuda.parallel_matmul import ColumnParallelBfp8Matmul

            M, K, N = 8192, 4096, 16384
            gmm = torch.Generator(device=dev).manual_seed(6)       # the same activations and weight on every rank
            a = torch.randn(M, K, device=dev, generator=gmm).bfloat16()
            w_full = torch.randn(1, 1, K, N, device=dev, generator=gmm) * 0.02
            op = ColumnParallelBfp8Matmul(K, N, bands=8)
            op.load_weight_shard(w_full)
            cfull = torch.empty(M, N, dtype=torch.bfloat16, device=dev)

            def run(gather):
                for _ in range(2):
                    op(a, out=cfull, gather=gather)
                barrier()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(5):
                    op(a, out=cfull, gather=gather)
                e1.record()
                barrier()
                return max_over_ranks(e0.elapsed_time(e1) / 5)

            ms_local, ms_gather = run(False), run(True)

            # the exchange fused into the kernel: the epilogue stores each tile into every rank's output
            # through peer-mapped memory.  Five launches, then a stream-ordered all-reduce: the closing event is
            # recorded when every rank's kernels (and with them their stores into this rank's matrix) are done.
            flag = torch.zeros(1, device=dev)

            def time_fused():
                for _ in range(2):
                    op.fused(a)
                barrier()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(5):
                    op.fused(a, sync=False)
                dist.all_reduce(flag)
                e1.record()
                barrier()
                return max_over_ranks(e0.elapsed_time(e1) / 5)

            # each route by name (one plain store per peer; the switch's multicast where the system has one), then the
            # route the operator picks by itself, which is the figure reported and the output checked
            ms_multicast = None
            try:
                op.enable_fused_scatter(M, multicast=True)
                ms_multicast = time_fused()
            except RuntimeError:
                pass
            op.enable_fused_scatter(M, multicast=False)
            ms_peer = time_fused()
            fused_out = op.enable_fused_scatter(M)
            route = op.exchange
            ms_fused = time_fused()
            # what NVLink gives bare stores of the same shape: every rank copies its block of columns into the peers'
            # matrices with a kernel that does nothing else (libbuda_probe.so), all ranks at once, timed the same way
            ms_bare = None
            try:
                op.enable_fused_scatter(M, multicast=False)
                probe = probe_lib()
                ptrs = op.block_pointers
                arr = (ctypes.c_void_p * (len(ptrs) - 1))(*[ctypes.c_void_p(p) for p in ptrs[1:]])
                stream_h = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

                def bare():
                    if probe.buda_probe_peer_stores(ctypes.c_void_p(ptrs[0]), arr, len(ptrs) - 1, M, (N // world) * 2, N * 2, stream_h):
                        raise RuntimeError("peer-store probe refused its arguments")

                for _ in range(2):
                    bare()
                barrier()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(5):
                    bare()
                dist.all_reduce(flag)
                e1.record()
                barrier()
                ms_bare = max_over_ranks(e0.elapsed_time(e1) / 5)
                fused_out = op.enable_fused_scatter(M)
                op.fused(a)
            except Exception as exc:  # report, never hide
                extras["peer_store_probe_error"] = str(exc)[:200]
                fused_out = op.enable_fused_scatter(M)
                op.fused(a)
            # correctness on every rank, outside the timed loops: fused == all-gather variant == one-GPU product
            op(a, out=cfull, gather=True)
            w_img_full = cuda_ops.tilize_pack(w_full, cuda_ops.DF.Bfp8_b)
            c_single = cuda_ops.bfp8b_matmul(a, w_img_full, N)
            torch.cuda.synchronize()
            ok_local = float(torch.equal(fused_out, c_single) and torch.equal(cfull, c_single))
            ok_t = torch.tensor([ok_local], device=dev)
            dist.all_reduce(ok_t, op=dist.ReduceOp.MIN)
            fused_matches = bool(ok_t.item() == 1.0)
            del w_img_full, c_single, w_full
            op.disable_fused_scatter()
            # what bounds the fused kernel: the tensor cores, or this rank's stores leaving over NVLink
            flops_rank = 2.0 * M * (N / world) * K
            link_bytes = M * (N / world) * 2 * (world - 1)
            t_floor = max(flops_rank / (tensor_peak_tflops() * 1e12), link_bytes / 770e9)
            # What a launch of whole-K tiles can reach with stores that run at the bare rate: nothing can be sent before the
            # first round of tiles is done, and the last round's stores have no compute beside them.
            tiles_rank = ((M + 511) // 512) * ((N // world) // 256)
            pairs_max = max(1, torch.cuda.get_device_properties(dev).multi_processor_count // 2)
            rounds = max(1, -(-tiles_rank // pairs_max))
            pipe_bound = max(ms_local / rounds + ms_bare, ms_local + ms_bare / rounds) if ms_bare else None
            extras["column_parallel_gemm_8192x4096x16384"] = {
                "TFLOP/s_without_gather": round(2.0 * M * N * K / (ms_local * 1e-3) / 1e12, 1), "ms_without_gather": round(ms_local, 4),
                "TFLOP/s_with_all_gather": round(2.0 * M * N * K / (ms_gather * 1e-3) / 1e12, 1), "ms_with_all_gather": round(ms_gather, 4),
                "TFLOP/s_fused_scatter": round(2.0 * M * N * K / (ms_fused * 1e-3) / 1e12, 1), "ms_fused_scatter": round(ms_fused, 4),
                "fused_matches": fused_matches, "fused_route": route,
                "ms_fused_peer_store_route": round(ms_peer, 4),
                "ms_fused_multicast_route": round(ms_multicast, 4) if ms_multicast is not None else None,
                "nvlink_store_gbs_per_gpu": round(link_bytes / (ms_fused * 1e-3) / 1e9, 1),
                "bare_peer_stores_ms": round(ms_bare, 4) if ms_bare else None,
                "bare_peer_stores_gbs_per_gpu": round(link_bytes / (ms_bare * 1e-3) / 1e9, 1) if ms_bare else None,
                "fused_scatter_vs_matmul_plus_bare_stores": round(ms_fused / (ms_local + ms_bare), 3) if ms_bare else None,
                "fused_peer_store_route_bound_ms": round(pipe_bound, 4) if pipe_bound else None,
                "fused_peer_store_route_frac_of_bound": round(pipe_bound / ms_peer, 3) if pipe_bound else None,
                "bound": "max(first round of tiles + bare stores, matmul + last round's bare stores); rounds = %d" % rounds,
                "fused_scatter_floor_ms": round(t_floor * 1e3, 4), "fused_scatter_frac_of_floor": round(t_floor * 1e3 / ms_fused, 3),
                "floor": "max(flops / measured bf16 burst peak, bytes leaving this GPU / 770 GB/s measured peer copy)",
                "bands": 8}
            del a, cfull
        except Exception as exc:
            extras["column_parallel_gemm_8192x4096x16384"] = {"error": str(exc)}

    # ------------------------------------------------------------------ CPU baseline (rank 0, N = 1 only)
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        try:
            from oracle import budaref as R

            R.build()
            n_cpu = min(8, NT)
            hs = [x.cpu().numpy() for x in xs[:n_cpu]]
            R.tilize_pack(hs[0], R.Bfp8_b)
            t0 = time.perf_counter()
            for h in hs:
                R.tilize_pack(h, R.Bfp8_b)
            dt = time.perf_counter() - t0
            cpu = {"value": n_cpu * ELEMS * BYTES_PER_ELEM / dt / 1e9, "unit": "GB/s", "cores": R.threads(), "kind": "port",
                   "sample": f"first {n_cpu} of the 64 tensors, one pass, OpenMP over all host cores"}
            # the same CPU arm for the secondary kernels, each on a bounded sample (seconds in total)
            if not args.no_extras:
                def cpu_timed(fn, work, unit, cores, sample):
                    fn()
                    t0 = time.perf_counter()
                    fn()
                    return {unit: round(work / (time.perf_counter() - t0), 2), "cores": cores, "sample": sample}

                prev = R.set_threads(1)
                cpu_other = {"pack_bfp8_b_single_thread": cpu_timed(lambda: R.tilize_pack(hs[0][:, :, :1024], R.Bfp8_b),
                                                                    ELEMS / 4 * BYTES_PER_ELEM / 1e9, "GB/s", 1,
                                                                    "a quarter of one tensor, CPU port, one thread")}
                R.set_threads(prev)
                img0 = R.tilize_pack(hs[0], R.Bfp8_b)
                cpu_other["unpack_bfp8_b"] = cpu_timed(lambda: R.unpack_untilize(img0, R.Bfp8_b, SHAPE), ELEMS * BYTES_PER_ELEM / 1e9,
                                                       "GB/s", R.threads(), "one tensor, CPU port, OpenMP over all host cores")
                nthr = torch.get_num_threads()
                xq = torch.rand(32, 1024, 1024) * 12 - 6
                scq = torch.tensor([0.05])
                # the golden evaluation's own torch expressions (op/eval/pybuda/quantize.py:56-66, 79-93, 95-110)
                cpu_other["quantize"] = cpu_timed(lambda: torch.clamp(torch.round(xq / scq) + 3, -128, 127).to(torch.int8),
                                                  xq.numel() * 5 / 1e9, "GB/s", nthr, "config-3 tensor, torch CPU")
                qq = torch.clamp(torch.round(xq / scq) + 3, -128, 127).to(torch.int8)
                cpu_other["dequantize"] = cpu_timed(lambda: (qq.float() - 3) * scq, xq.numel() * 5 / 1e9, "GB/s", nthr,
                                                    "config-3 tensor, torch CPU")
                accq = torch.randint(-2 ** 20, 2 ** 20, (32, 1024, 1024), dtype=torch.int32)
                scs_cpu = torch.rand(1024) * (1e-2 - 1e-4) + 1e-4
                cpu_other["requantize"] = cpu_timed(lambda: torch.clamp(torch.round(accq.float() * scs_cpu + 0.0), -128, 127).to(torch.int8),
                                                    xq.numel() * 5 / 1e9, "GB/s", nthr, "config-3 tensor, torch CPU")
                am = torch.randn(256, 4096)
                wm = torch.randn(4096, 16384) * 0.02
                cpu_other["matmul_fp32"] = cpu_timed(lambda: am @ wm, 2.0 * 256 * 4096 * 16384 / 1e12, "TFLOP/s", nthr,
                                                     "256 of the 8192 activation rows, torch CPU matmul (the golden matmul)")
                cpu["other_kernels"] = cpu_other
                del xq, qq, accq, am, wm, img0
        except Exception as exc:
            cpu = {"value": None, "unit": "GB/s", "error": str(exc)}

    if rank == 0:
        line = {
            "metric": "bfp8b_tilize_pack_throughput", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "value_is": "weak scaling: every GPU packs its own batch of 64 tensors; the config's own 64 tensors shared out "
                        "over the GPUs are in `strong`",
            "strong": strong, "parity_sample": parity_sample,
            "vs_baseline": None, "dtype": "u8", "data": "synthetic",
            "config": {"workload": WORKLOAD if NT == N_TENSORS else WORKLOAD + f" (REDUCED to {NT} tensors)", "per_gpu_batch": NT, "l2": "inputs (4 GiB per step) larger than L2",
                       "launches_per_step": 1},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                         # dram read + write per launch: a constant, not read live -- an ncu capture of an 8-tensor
                         # launch measured 82.57 MB per tensor, and traffic grows with the tensor count
                         "traffic": NT * 82.6e6, "traffic_unit": "bytes per launch", "traffic_source": "constant: 82.57 MB per tensor "
                         "from an ncu capture of an 8-tensor launch, scaled by the tensor count",
                         "peak_kind": peak_kind, "peak_note": "the peak is a 1:1 copy; for a stream that is 4/5 reads the memory system "
                         "gives more (bare_kernel_same_mix_gbs), so frac can exceed 1", "kernel": "pack_staged_kernel<7,4>",
                         # the peak is a 1:1 copy; this stream is 4/5 reads: a bare kernel with the same mix and access
                         # shape, timed in this run (7190 GB/s in an earlier run on this pool if the extras are skipped)
                         "bare_kernel_same_mix_gbs": bare_pack_mix if bare_pack_mix else 7190.0,
                         "frac_of_bare_kernel": achieved / (bare_pack_mix if bare_pack_mix else 7190.0),
                         "kernel_ms": kernel_ms},
            "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks.summary(),
            "other_kernels": extras,
        }
        emit(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
