#!/usr/bin/env python3
"""Benchmark of the MX attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (named in the JSON line): MXFP8 causal MHA prefill B=8 H=16 S=4096 d=128, seeded synthetic
N(0,1) Q/K/V quantized to E4M3 + E8M0 block-32 along d, bf16 output.  A "step" is one pass of the whole
prefill path over that batch through the C ABI: scale re-tiling, V re-blocking along the keys and the tiled
attention kernel.  With N > 1 every rank runs its own batch of independent (batch, head) units (weak
scaling, no data-path collective); time is the max over ranks, value the FLOP of all ranks over it; the
same run also shards ONE global batch over the ranks by (batch, KV head) units (`strong_scaling`), with the
optional NCCL gather of O timed apart.
The line also carries the decode leg (batch 64, 32 query heads / 8 KV heads, d=128, KV length 32768), the
other benchmark configurations and the preparation kernels, each with its own roofline (`extras`), and the
tensor-pipe ceiling measured on this device by a GEMM-only loop of the same block-scaled MMAs.

`--impl reference` times the CPU restatement of the reference path (oracle/) on the host cores on a bounded
sample of the same workload: the reference's own attention cannot run here (its Python model imports an
un-vendored module, its kernels need the Muon toolchain and an RTL simulator).
"""
import argparse
import ctypes as C
import datetime
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PREFILL = dict(B=8, H=16, H_kv=16, S=4096, d=128)
DECODE = dict(B=64, H=32, H_kv=8, L=32768, d=128)
WORKLOAD = "MXFP8 causal MHA prefill B=8 H=16 S=4096 d=128 (E4M3 + E8M0 block-32 along d, P requantized, bf16 out)"
METRIC = "MX attention prefill TFLOP/s (all GPUs) [decode HBM GB/s in `decode`]"
NOMINAL_FP8_TFLOPS = 4500.0
NOMINAL_HBM_GBS = 8000.0


def prefill_flops(c):
    return 4.0 * c["B"] * c["H"] * c["S"] * c["S"] * c["d"] * 0.5      # causal: half the tiles counted


def prefill_algorithmic_bytes(c):
    """Q, K, V codes + E8M0 scales read once, bf16 O and fp32 LSE written once."""
    qkv = (c["B"] * c["H"] * c["S"] + 2 * c["B"] * c["H_kv"] * c["S"]) * c["d"] * (1 + 1 / 32)
    return int(qkv + c["B"] * c["H"] * c["S"] * (2 * c["d"] + 4))


# DRAM traffic of one launch from the ncu captures summarised under profiles/ (dram__bytes_read.sum +
# dram__bytes_write.sum), per unit of work; both kernels' traffic is proportional to the unit count.
NCU_PREFILL_DRAM_BYTES_PER_HEAD = (158.141440e6 + 38.027776e6) / 64         # S=4096, d=128, causal
NCU_DECODE_DRAM_BYTES_PER_SEQUENCE = (553.775104e6 + 6.571264e6) / 8        # H_kv=8, L=32768, d=128


def decode_bytes(c):
    return 2.0 * c["B"] * c["H_kv"] * c["L"] * c["d"] * (1 + 1 / 32) + 2 * c["B"] * c["H"] * c["d"] * 2


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return {"hbm": float(p["hbm_gbs"]), "bf16_sustained": float(p["bf16_tflops_sustained"]),
                "bf16_burst": float(p["bf16_tflops"]), "source": "measured"}
    except Exception:
        return {"hbm": 6650.0, "bf16_sustained": 1400.0, "bf16_burst": 1590.0, "source": "fallback"}


class ClockSampler:
    """SM clock, power and throttle reasons, time-stamped, sampled while the benchmark runs: read-only NVML queries
    from a thread every few milliseconds (so that a timed region of some ten milliseconds still holds samples),
    and an `nvidia-smi -lms` poller beside it as the fallback.  `window(t0, t1)` summarises the samples whose
    time stamps fall inside one timed region (host clock, seconds)."""
    Q = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, gpu_index, period_ms=50, nvml_period_ms=2.0, uuid=None):
        self.gpu, self.period_ms, self.nvml_period = gpu_index, period_ms, nvml_period_ms * 1e-3
        self.uuid = uuid
        self.proc = self.path = self.fh = None
        self.samples = []
        self.nvml_samples = []
        self._thread = None
        self._stop_flag = threading.Event()

    def _nvml_loop(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            try:
                h = nv.nvmlDeviceGetHandleByUUID(("GPU-" + self.uuid).encode()) if self.uuid else None
            except Exception:
                h = None
            if h is None:
                h = nv.nvmlDeviceGetHandleByIndex(self.gpu)
            mx = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            bits = (("hw_slowdown", nv.nvmlClocksEventReasonHwSlowdown if hasattr(nv, "nvmlClocksEventReasonHwSlowdown")
                     else nv.nvmlClocksThrottleReasonHwSlowdown),
                    ("hw_thermal_slowdown", nv.nvmlClocksThrottleReasonHwThermalSlowdown),
                    ("sw_thermal_slowdown", nv.nvmlClocksThrottleReasonSwThermalSlowdown),
                    ("sw_power_cap", nv.nvmlClocksThrottleReasonSwPowerCap))
            reasons_fn = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
            while not self._stop_flag.is_set():
                t = time.time()
                mhz = float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                mask = int(reasons_fn(h))
                watts = nv.nvmlDeviceGetPowerUsage(h) / 1000.0
                self.nvml_samples.append((t, mhz, mx, watts, [n for n, b in bits if mask & b]))
                self._stop_flag.wait(self.nvml_period)
        except Exception:
            return                                   # the nvidia-smi poller still runs

    def __enter__(self):
        self._thread = threading.Thread(target=self._nvml_loop, daemon=True)
        self._thread.start()
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            self.fh = os.fdopen(fd, "w")
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", str(self.period_ms)],
                                         stdout=self.fh, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None
        return self

    def __exit__(self, *exc):
        self._stop()
        return False

    def _stop(self):
        self._stop_flag.set()
        if self._thread is not None:
            self._thread.join(timeout=5)
            self._thread = None
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()
            self.proc = None
        if self.fh is not None:
            self.fh.close()
            self.fh = None
        if self.path is not None:
            try:
                for line in open(self.path):
                    f = [x.strip() for x in line.split(",")]
                    if len(f) < 8:
                        continue
                    try:
                        ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                        self.samples.append((ts, float(f[1]), float(f[2]), float(f[3]),
                                             [n for n, v in zip(self.NAMES, f[4:8]) if v.lower().startswith("active")]))
                    except ValueError:
                        continue
                os.unlink(self.path)
            except Exception:
                pass
            self.path = None

    def window(self, t0, t1):
        """Median SM clock and the throttle reasons seen between host times t0 and t1 (call after the `with` block
        has ended: the poller's file is read when it stops).  A region shorter than the sampling period may hold
        no sample: the nearest one on either side is used and `samples` says 0."""
        if self.proc is not None:
            raise RuntimeError("ClockSampler.window() before the sampler was stopped")
        source = "nvml"
        inside = [s for s in self.nvml_samples if t0 <= s[0] <= t1]
        if not inside:
            source = "nvidia-smi"
            inside = [s for s in self.samples if t0 <= s[0] <= t1]
        n = len(inside)
        if not inside and (self.samples or self.nvml_samples):
            source = "nearest"
            inside = sorted(self.samples + self.nvml_samples, key=lambda s: min(abs(s[0] - t0), abs(s[0] - t1)))[:2]
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median([s[1] for s in inside])), "sm_max_mhz": float(max(s[2] for s in inside)),
                "power_w_max": float(max(s[3] for s in inside)),
                "reasons": sorted({r for s in inside for r in s[4]}), "samples": n, "source": source}


def cpu_sample(kind, nthreads, seconds_target=10.0):
    """Times the CPU oracle on a bounded sample of the prefill workload: `n` whole (batch, head) slices of
    the B=8 H=16 S=4096 d=128 causal problem, one slice per task over `nthreads` threads, repeated until
    about `seconds_target` of wall time has been spent."""
    import oracle
    c = PREFILL
    rng = np.random.default_rng(0)
    n = min(c["B"] * c["H"], max(nthreads, 8) * 2)
    S, d = c["S"], c["d"]

    def q4(x):
        cc, ss = oracle.quantize(x.reshape(-1, d), nthreads=nthreads)
        return cc.reshape(x.shape), ss.reshape(x.shape[:-1] + (d // 32,))

    Q = rng.standard_normal((1, n, S, d), dtype=np.float32)
    K = rng.standard_normal((1, n, S, d), dtype=np.float32)
    V = rng.standard_normal((1, n, S, d), dtype=np.float32)
    qc, qs = q4(Q); kc, ks = q4(K); vc, vs = q4(V)
    del Q, K, V
    passes, t0 = 0, time.perf_counter()
    while True:
        oracle.attn_prefill(qc, kc, vc, qs, ks, vs, causal=True, softmax_scale=d ** -0.5, block_n=128, nthreads=nthreads)
        passes += 1
        dt = time.perf_counter() - t0
        if dt >= seconds_target or passes >= 50:
            break
    flops = 4.0 * n * passes * S * S * d * 0.5
    return {"value": flops / dt / 1e12, "unit": "TFLOP/s", "cores": nthreads, "kind": kind,
            "sample": f"{passes} pass(es) over {n} of the workload's {c['B'] * c['H']} (batch, head) slices, {dt:.1f} s wall; "
                      f"the full problem extrapolates to {dt / passes * c['B'] * c['H'] / n:.1f} s"}, dt, flops


def run_reference(args, rank, world):
    if rank != 0:
        return
    import oracle
    nthreads = oracle.hardware_threads()
    vals = []
    info = None
    for _ in range(max(1, min(args.steps, 2))):        # each step is a bounded sample; keep the run within minutes
        info, dt, fl = cpu_sample("port", nthreads)
        vals.append(fl / dt / 1e12)
    v = float(np.median(vals))
    info["value"] = v
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": None, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "mxfp8_e4m3 (fp32 accumulate)", "data": "synthetic",
            "config": {"workload": WORKLOAD, "note": "CPU restatement of the reference path (oracle port), all host threads"},
            "cpu_baseline": info,
            "e2e": {"value": v, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-decode", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the other configurations, the preparation kernels, "
                    "the tensor-pipe ceiling and the long (2 s) loop")
    ap.add_argument("--case", default="full", choices=["full", "small"],
                    help="small: a reduced batch of the same shapes, for profiler captures only (not a bench number)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    if args.case == "small":
        PREFILL.update(B=4)
        DECODE.update(B=8)
        args.no_extras = True
    windows = {}                                       # name -> (t0, t1) host times of the timed regions
    try:
        uuid = str(torch.cuda.get_device_properties(local).uuid)
    except Exception:
        uuid = None
    with ClockSampler(local, uuid=uuid) as sampler:    # the pollers are stopped whatever happens below
        line = run_ours(args, rank, world, local, windows)
    if line is not None:
        line["clocks"] = sampler.window(*windows["steps"])
        if "mma_sustained" in windows and line["roofline"].get("peak_measured_mxfp8"):
            line["roofline"]["peak_measured_mxfp8"]["sustained_clocks"] = sampler.window(*windows["mma_sustained"])
        sus = line["roofline"].get("sustained")
        if sus is not None and "long_loop" in windows:
            sus["clocks"] = sampler.window(*windows["long_loop"])
            mhz = sus["clocks"].get("sm_mhz")
            sus["ms_x_mhz"] = sus["ms_per_step"] * mhz if mhz else None
        print(json.dumps(line), flush=True)


def run_ours(args, rank, world, local, windows):
    import torch
    import torch.distributed as dist
    import radiance_kernels_b200 as rk

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed(fn, steps, warm=3):
        """ms per call: CUDA events on the current stream around `steps` back-to-back calls, after `warm` calls."""
        for _ in range(warm):
            fn()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / steps

    def kernel_ms(fn, steps):
        """ms of the main kernel inside `fn` (the library records events around it), averaged over `steps` calls."""
        e0 = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        e1 = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        for ev in e0 + e1:
            ev.record()                                # materialise the cudaEvent_t handles
        torch.cuda.synchronize()
        for i in range(steps):
            L.rk_profile_set_events(C.c_void_p(e0[i].cuda_event), C.c_void_p(e1[i].cuda_event))
            fn()
        L.rk_profile_set_events(None, None)
        torch.cuda.synchronize()
        return float(np.mean([a.elapsed_time(b) for a, b in zip(e0, e1)]))

    L = rk.lib()
    peaks = measured_peaks()
    c = PREFILL
    B, H, Hkv, S, d = c["B"], c["H"], c["H_kv"], c["S"], c["d"]
    g = torch.Generator(device=dev).manual_seed(1000 + rank)
    Q = torch.randn(B, H, S, d, generator=g, device=dev)
    K = torch.randn(B, Hkv, S, d, generator=g, device=dev)
    V = torch.randn(B, Hkv, S, d, generator=g, device=dev)
    qc, qs = rk.mx_quantize(Q); kc, ks = rk.mx_quantize(K); vc, vs = rk.mx_quantize(V)
    del Q, K, V
    o = torch.empty(B, H, S, d, dtype=torch.bfloat16, device=dev)
    ws = torch.empty(rk.attn_prefill_workspace_bytes(B, H, Hkv, S, S, d, rk.V_SCALES_ALONG_D) + 256, dtype=torch.uint8, device=dev)

    def step():
        rk.attn_prefill(qc, kc, vc, qs, ks, vs, causal=True, v_scale_axis=rk.V_SCALES_ALONG_D, out=o, workspace=ws)

    # ---- device-resident timing: exactly `steps` steps, max over ranks --------------------------------------
    for _ in range(args.warmup):
        step()
    kev0 = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    kev1 = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for ev in kev0 + kev1:
        ev.record()
    barrier()
    t_region0 = time.time()
    e0.record()
    for i in range(args.steps):
        L.rk_profile_set_events(C.c_void_p(kev0[i].cuda_event), C.c_void_p(kev1[i].cuda_event))
        step()
    L.rk_profile_set_events(None, None)
    e1.record()
    barrier()
    t_region1 = time.time()
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    ms_step = ms_total / args.steps
    kern_ms = float(np.mean([a.elapsed_time(b) for a, b in zip(kev0, kev1)]))
    status = rk.last_device_status()
    if status != 0:
        raise SystemExit(f"device status {status}: a kernel gave up on a bounded wait; no number reported")
    flops = prefill_flops(c)
    value = flops * world / (ms_step * 1e-3) / 1e12
    achieved = flops / (kern_ms * 1e-3) / 1e12

    # ---- the tensor-pipe ceiling on this device, and the same kernel in a loop of at least 2 s ---------------
    mma_peak = None
    sustained = None
    if not args.no_extras:
        tiles = torch.randint(0, 0x7E, (2, 128 * 128), dtype=torch.uint8, device=dev)      # valid E4M3 codes
        iters = 8192
        sms = torch.cuda.get_device_properties(dev).multi_processor_count

        def mma_loop():
            rc = L.rk_debug_mxfp8_mma_loop(C.c_void_p(tiles[0].data_ptr()), C.c_void_p(tiles[1].data_ptr()), iters,
                                           C.c_void_p(torch.cuda.current_stream().cuda_stream))
            if rc != 0:
                raise SystemExit(f"rk_debug_mxfp8_mma_loop failed: {rc}")

        mma_flops = sms * iters * 2.0 * 128 ** 3
        torch.cuda.synchronize(); time.sleep(0.5)                    # start the burst figure from an idle, cool part
        burst_ms = min(timed(mma_loop, 1, warm=1) for _ in range(3))
        n_sus = max(1, int(2500.0 / burst_ms))
        t0 = time.time()
        sus_ms = timed(mma_loop, n_sus, warm=0)
        t1 = time.time()
        windows["mma_sustained"] = (t0, t1)
        mma_peak = {"burst_tflops": mma_flops / (burst_ms * 1e-3) / 1e12, "sustained_tflops": mma_flops / (sus_ms * 1e-3) / 1e12,
                    "sustained_seconds": sus_ms * n_sus * 1e-3,
                    "what": "tcgen05.mma kind::mxf8f6f4.block_scale M=128 N=128 K=32, operands and scales resident in shared "
                            "memory / TMEM, one CTA per SM, no TMA and no softmax in the loop"}
        code = rk.last_device_status()                                # reads and clears the device status word
        if code != 0:
            # the measurement aid gave up on a bounded wait: its figures are void, the product kernels are not
            # affected (later launches run normally once the word is cleared); fall back to the 2 x bf16 proxy
            sys.stderr.write(f"tensor-pipe ceiling loop: device status {code}, measured ceiling dropped\n")
            mma_peak = None
        # the attention kernel for at least 2 s: its sustained speed and the clock it ran at
        n_long = max(args.steps, int(2200.0 / ms_step))
        t0 = time.time()
        long_ms = timed(step, n_long, warm=0)
        t1 = time.time()
        windows["long_loop"] = (t0, t1)
        long_kern = kernel_ms(step, 10)
        sustained = {"steps": n_long, "ms_per_step": long_ms, "kernel_ms_after_loop": long_kern,
                     "tflops": flops / (long_ms * 1e-3) / 1e12}
        del tiles

    peak_burst = mma_peak["burst_tflops"] if mma_peak else 2.0 * peaks["bf16_burst"]
    roofline = {"bound": "tensor", "achieved": achieved, "peak": peak_burst, "unit": "TFLOP/s",
                "frac": achieved / peak_burst,
                "traffic": NCU_PREFILL_DRAM_BYTES_PER_HEAD * c["B"] * c["H"] if (c["S"], c["d"]) == (4096, 128) else None,
                "traffic_note": "ncu dram read+write of one launch at B=4 (196.17 MB for 64 (batch, head) units), scaled by "
                                "the unit count; algorithmic bytes per launch: %d" % prefill_algorithmic_bytes(c),
                "kernel": "prefill2c_kernel<false>", "kernel_ms": kern_ms,
                "peak_measured_mxfp8": mma_peak,
                "frac_of_2x_bf16_burst": achieved / (2.0 * peaks["bf16_burst"]),
                "frac_of_nominal": achieved / NOMINAL_FP8_TFLOPS,
                "peak_note": ("peak = the tensor-pipe ceiling measured in this run by a GEMM-only loop of the same block-scaled "
                              "MMAs (burst: the timed region is a few ms at full clock)" if mma_peak else
                              f"peak = 2 x {peaks['source']} burst cuBLAS bf16 ({peaks['bf16_burst']} TF/s) as the dense MXFP8 proxy") +
                             f"; 2 x {peaks['source']} cuBLAS bf16 burst = {2 * peaks['bf16_burst']:.1f}, sustained = "
                             f"{2 * peaks['bf16_sustained']:.1f}; nominal dense FP8 {NOMINAL_FP8_TFLOPS:.0f} TF/s"}

    # ---- end to end through the host-buffer entry point ----------------------------------------------------
    e2e = None
    if not args.no_e2e:
        host = [t.cpu().pin_memory() for t in (qc, kc, vc, qs, ks, vs)]
        runner = rk.PrefillHostRunner(*host, causal=True, v_scale_axis=rk.V_SCALES_ALONG_D, device=dev)
        runner.run()
        n_e2e = max(3, min(args.steps, 10))
        barrier()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record()
        for _ in range(n_e2e):
            runner.run()
        f1.record()
        barrier()
        ms_e2e = max_over_ranks(f0.elapsed_time(f1)) / n_e2e
        e2e = {"value": flops * world / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_e2e,
               "h2d_bytes_per_step": runner.h2d_bytes, "d2h_bytes_per_step": runner.d2h_bytes, "steps": n_e2e}
        # what the bus alone allows: the same bytes, host -> device and device -> host on two streams at once,
        # every rank at the same time (the ranks of one box share the host's memory and root complexes)
        s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        dsts = [torch.empty_like(t, device=dev) for t in host]
        barrier()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0.record()
        s_in.wait_event(c0); s_out.wait_event(c0)
        for _ in range(n_e2e):
            with torch.cuda.stream(s_in):
                for hsrc, ddst in zip(host, dsts):
                    ddst.copy_(hsrc, non_blocking=True)
            with torch.cuda.stream(s_out):
                runner.o.copy_(o, non_blocking=True)
        torch.cuda.current_stream().wait_stream(s_in); torch.cuda.current_stream().wait_stream(s_out)
        c1.record()
        barrier()
        ms_copy = max_over_ranks(c0.elapsed_time(c1)) / n_e2e
        e2e.update(copy_ceiling_ms=ms_copy, frac_of_copy_ceiling=ms_copy / ms_e2e,
                   copy_ceiling_note="pinned cudaMemcpyAsync of the step's input bytes in and output bytes out on two streams, "
                                     "all ranks at once, no compute")
        del runner, host, dsts
    code = rk.last_device_status()
    if code != 0:       # the long loop or the end-to-end leg: reported with the line, the device-resident numbers above stand
        sys.stderr.write(f"device status {code} after the sustained loop / end-to-end leg (a bounded device-side wait gave up)\n")
        if e2e is not None:
            e2e["device_status"] = code
        if sustained is not None:
            sustained["device_status"] = code
    launches = args.steps * 2          # per step: the V re-blocking launch (which also re-tiles the Q and K scales) and the attention kernel

    # ---- one global batch sharded over the ranks by (batch, KV head) units (N > 1) ------------------------------
    strong = None
    if world > 1:
        strong = strong_scaling_leg(args, rk, dist, dev, rank, world, barrier, max_over_ranks)

    # ---- the other configurations and the preparation kernels ------------------------------------------------
    extras = None
    if not args.no_extras and rank == 0:
        extras = run_extras(rk, L, dev, peaks, peak_burst, timed, kernel_ms, qc, qs, vc, vs)
    del qc, kc, vc, qs, ks, vs, o, ws
    torch.cuda.empty_cache()

    # ---- decode leg ---------------------------------------------------------------------------------------
    decode = None
    if not args.no_decode:
        dc = DECODE
        Bd, Hd, Hkd, Ld, dd = dc["B"], dc["H"], dc["H_kv"], dc["L"], dc["d"]
        g2 = torch.Generator(device=dev).manual_seed(2000 + rank)
        qd = torch.randn(Bd, Hd, dd, generator=g2, device=dev).bfloat16()
        kcd = torch.empty(Bd, Hkd, Ld, dd, dtype=torch.uint8, device=dev)
        vcd = torch.empty_like(kcd)
        ksd = torch.empty(Bd, Hkd, Ld, dd // 32, dtype=torch.uint8, device=dev)
        vsd = torch.empty_like(ksd)
        for b in range(Bd):               # quantize N(0,1) K/V one sequence at a time (keeps the fp32 staging small)
            x = torch.randn(Hkd, Ld, dd, generator=g2, device=dev)
            kcd[b], ksd[b] = rk.mx_quantize(x)
            x = torch.randn(Hkd, Ld, dd, generator=g2, device=dev)
            vcd[b], vsd[b] = rk.mx_quantize(x)
        del x
        od = torch.empty(Bd, Hd, dd, dtype=torch.bfloat16, device=dev)
        wsd = torch.empty(rk.attn_decode_workspace_bytes(Bd, Hd, Hkd, Ld, dd) + 16, dtype=torch.uint8, device=dev)

        def dstep():
            rk.attn_decode(qd, kcd, vcd, ksd, vsd, out=od, workspace=wsd)

        for _ in range(args.warmup):
            dstep()
        d0, d1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        d0.record()
        for i in range(args.steps):
            dstep()
        d1.record()
        barrier()
        dms = max_over_ranks(d0.elapsed_time(d1)) / args.steps
        dk = kernel_ms(dstep, min(args.steps, 10))
        by = decode_bytes(dc)
        decode = {"metric": "decode attention HBM GB/s (all GPUs)", "value": by * world / (dms * 1e-3) / 1e9, "unit": "GB/s",
                  "ms_per_step": dms, "workload": "batch 64, 32 query heads / 8 KV heads, d=128, KV length 32768, MXFP8 cache",
                  "num_splits": rk.attn_decode_num_splits(Bd, Hd, Hkd, Ld, dd),
                  "roofline": {"bound": "hbm", "achieved": by / (dk * 1e-3) / 1e9, "peak": peaks["hbm"], "unit": "GB/s",
                               "frac": by / (dk * 1e-3) / 1e9 / peaks["hbm"],
                               "traffic": NCU_DECODE_DRAM_BYTES_PER_SEQUENCE * Bd if (Hkd, Ld, dd) == (8, 32768, 128) else None,
                               "traffic_note": "ncu dram read+write of one launch at B=8 (560.35 MB), scaled by B",
                               "kernel": "decode_tc_kernel", "kernel_ms": dk, "frac_of_nominal": by / (dk * 1e-3) / 1e9 / NOMINAL_HBM_GBS,
                               "peak_note": f"{peaks['source']} HBM copy bandwidth; nominal {NOMINAL_HBM_GBS:.0f} GB/s"}}
        code = rk.last_device_status()
        if code != 0:
            raise SystemExit(f"device status {code} after the decode leg (a bounded device-side wait gave up)")
        launches += args.steps * 2
        del kcd, vcd, ksd, vsd

    windows["steps"] = (t_region0, t_region1)
    if sustained is not None:
        if mma_peak:
            sustained["frac_of_sustained_peak"] = sustained["tflops"] / mma_peak["sustained_tflops"]
        roofline["sustained"] = sustained
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        import oracle
        cpu, _, _ = cpu_sample("port", oracle.hardware_threads())

    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return None
    line = {"metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "mxfp8_e4m3 (e8m0 block scales, fp32 accumulate, bf16 out)", "data": "synthetic",
            "config": {"workload": WORKLOAD if args.case == "full" else "REDUCED BATCH (profiling case, not a bench number): " + WORKLOAD, "per_gpu_batch": "B=8 H=16 (128 independent (batch, head) units per GPU)",
                       "parallelism": f"units sharded over {world} GPU(s), no collective on the data path",
                       "l2": "inputs + output (335 MB) exceed the 126 MB L2; no flush between steps"},
            "roofline": roofline, "e2e": e2e, "gpu_launches": launches, "clocks": None, "decode": decode}
    if strong is not None:
        line["strong_scaling"] = strong
    if extras is not None:
        line["extras"] = extras
    if cpu is not None:
        line["cpu_baseline"] = cpu
    return line


def strong_scaling_leg(args, rk, dist, dev, rank, world, barrier, max_over_ranks):
    """ONE global B=8 H=16 S=4096 d=128 batch, its 128 (batch, KV head) units cut into contiguous blocks (shard_range),
    every rank computing its block with rk_attn_prefill; then the optional gather of O with NCCL, timed apart."""
    import torch
    c = dict(B=8, H=16, H_kv=16, S=4096, d=128)
    grp = c["H"] // c["H_kv"]
    n_units = c["B"] * c["H_kv"]
    lo, hi = rk.shard_range(n_units, rank, world)
    nloc = hi - lo
    S, d = c["S"], c["d"]
    # a unit = one KV head with its `grp` query heads: the slice is a batch of nloc such units
    g = torch.Generator(device=dev).manual_seed(4242)                   # same seed everywhere: one global problem
    out = {"workload": "one global B=8 H=16 S=4096 d=128 causal batch, 128 (batch, KV head) units in contiguous blocks per rank",
           "units_per_rank": [rk.shard_range(n_units, r, world)[1] - rk.shard_range(n_units, r, world)[0] for r in range(world)]}
    if nloc == 0:
        ms = 0.0
        o = torch.empty(0, grp, S, d, dtype=torch.bfloat16, device=dev)
    else:
        # every rank draws the whole problem's random stream unit by unit and keeps its own block
        qc = torch.empty(nloc, grp, S, d, dtype=torch.uint8, device=dev); qs = torch.empty(nloc, grp, S, d // 32, dtype=torch.uint8, device=dev)
        kc = torch.empty(nloc, 1, S, d, dtype=torch.uint8, device=dev); ks = torch.empty(nloc, 1, S, d // 32, dtype=torch.uint8, device=dev)
        vc = torch.empty_like(kc); vs = torch.empty_like(ks)
        for u in range(n_units):
            x = torch.randn(grp + 2, S, d, generator=g, device=dev)
            if lo <= u < hi:
                qc[u - lo], qs[u - lo] = rk.mx_quantize(x[:grp].contiguous())
                kc[u - lo, 0], ks[u - lo, 0] = rk.mx_quantize(x[grp].contiguous())
                vc[u - lo, 0], vs[u - lo, 0] = rk.mx_quantize(x[grp + 1].contiguous())
        o = torch.empty(nloc, grp, S, d, dtype=torch.bfloat16, device=dev)
        ws = torch.empty(rk.attn_prefill_workspace_bytes(nloc, grp, 1, S, S, d, rk.V_SCALES_ALONG_D) + 256, dtype=torch.uint8, device=dev)

        def step():
            rk.attn_prefill(qc, kc, vc, qs, ks, vs, causal=True, v_scale_axis=rk.V_SCALES_ALONG_D, out=o, workspace=ws)

        for _ in range(args.warmup):
            step()
    barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    if nloc:
        for _ in range(args.steps):
            step()
    b.record()
    barrier()
    ms = max_over_ranks(a.elapsed_time(b)) / args.steps
    flops = prefill_flops(c)
    out.update(ms_per_step=ms, value=flops / (ms * 1e-3) / 1e12, unit="TFLOP/s")
    # optional gather of O on every rank (equal blocks only: all_gather_into_tensor wants equal shapes)
    if n_units % world == 0:
        full = torch.empty(n_units, grp, S, d, dtype=torch.bfloat16, device=dev)
        for _ in range(2):
            dist.all_gather_into_tensor(full, o)
        barrier()
        a.record()
        for _ in range(5):
            dist.all_gather_into_tensor(full, o)
        b.record()
        barrier()
        gms = max_over_ranks(a.elapsed_time(b)) / 5
        out.update(gather_ms=gms, gather_bytes_per_rank=int(o.numel() * 2),
                   gather_note="ncclAllGather of the bf16 O blocks (optional: only for callers that need O on one device)")
    return out


def run_extras(rk, L, dev, peaks, peak_burst, timed, kernel_ms, qc, qs, vc, vs):
    """The other benchmark configurations (whole C-ABI call and attention kernel alone) and the preparation kernels,
    each against its own roofline."""
    import torch
    out = {}

    def prefill_case(name, B, H, Hkv, S, d, mul=1.0, softcap=0.0, q_fmt=0, kv_fmt=0, steps=5):
        g = torch.Generator(device=dev).manual_seed(77)
        Q = torch.randn(B, H, S, d, generator=g, device=dev) * mul
        K = torch.randn(B, Hkv, S, d, generator=g, device=dev) * mul
        V = torch.randn(B, Hkv, S, d, generator=g, device=dev) * mul
        q_c, q_s = rk.mx_quantize(Q, q_fmt); k_c, k_s = rk.mx_quantize(K, kv_fmt); v_c, v_s = rk.mx_quantize(V, kv_fmt)
        prepared = None
        if q_fmt >= rk.E2M3 and kv_fmt >= rk.E2M3:
            # the same operands prepared once, as a cache kept in a 6- or 4-bit format holds them: dense codes, V blocked
            # along the keys, scale-factor atoms -- the call is then the attention kernel alone
            _, q_a = rk.mx_quantize_ex(Q, q_fmt, rk.SCALES_SF_ATOMS)
            _, k_a = rk.mx_quantize_ex(K, kv_fmt, rk.SCALES_SF_ATOMS)
            v_k, v_a = rk.mx_quantize_keys_ex(V, kv_fmt, rk.SCALES_SF_ATOMS)
            prepared = (rk.mx_pack_rows(q_c, q_fmt), rk.mx_pack_rows(k_c, kv_fmt), rk.mx_pack_vt(v_k, kv_fmt), q_a, k_a, v_a)
            del v_k
        del Q, K, V
        o = torch.empty(B, H, S, d, dtype=torch.bfloat16, device=dev)
        ws = torch.empty(rk.attn_prefill_workspace_bytes(B, H, Hkv, S, S, d, rk.V_SCALES_ALONG_D, q_fmt, kv_fmt) + 256,
                         dtype=torch.uint8, device=dev)

        def fn():
            rk.attn_prefill(q_c, k_c, v_c, q_s, k_s, v_s, causal=True, softcap=softcap, q_fmt=q_fmt, kv_fmt=kv_fmt,
                            v_scale_axis=rk.V_SCALES_ALONG_D, out=o, workspace=ws)

        ms = timed(fn, steps)
        km = kernel_ms(fn, steps)
        fl = 4.0 * B * H * S * S * d * 0.5
        out[name] = {"ms_per_call": ms, "tflops": fl / (ms * 1e-3) / 1e12,
                     "roofline": {"bound": "tensor", "achieved": fl / (km * 1e-3) / 1e12, "peak": peak_burst, "unit": "TFLOP/s",
                                  "frac": fl / (km * 1e-3) / 1e12 / peak_burst, "kernel_ms": km,
                                  "frac_of_nominal": fl / (km * 1e-3) / 1e12 / NOMINAL_FP8_TFLOPS, "traffic": None}}
        if prepared is not None:
            def fn_prepared():
                rk.attn_prefill_packed(*prepared, S_q=S, S_kv=S, d=d, q_fmt=q_fmt, kv_fmt=kv_fmt, causal=True, softcap=softcap,
                                       q_scale_layout=rk.SCALES_SF_ATOMS, k_scale_layout=rk.SCALES_SF_ATOMS,
                                       v_scale_layout=rk.SCALES_SF_ATOMS, out=o, workspace=ws)
            pms = timed(fn_prepared, steps)
            out[name].update(prepared_ms_per_call=pms, prepared_tflops=fl / (pms * 1e-3) / 1e12,
                             prepared_note="dense codes (rk_mx_pack_rows / rk_mx_pack_vt) and scale-factor atoms handed over: one launch")

    prefill_case("prefill_gqa_B4_H32_kv8_S8192_d128", 4, 32, 8, 8192, 128)
    prefill_case("prefill_gemma_B2_H16_kv8_S8192_d256_cap50", 2, 16, 8, 8192, 256, mul=0.5, softcap=50.0)
    prefill_case("prefill_gemma_mxfp6_e2m3q_e3m2kv", 2, 16, 8, 8192, 256, mul=0.5, softcap=50.0, q_fmt=rk.E2M3, kv_fmt=rk.E3M2)
    prefill_case("prefill_gqa_mxfp4_e2m1_B4_H32_kv8_S8192_d128", 4, 32, 8, 8192, 128, mul=0.5, q_fmt=rk.E2M1, kv_fmt=rk.E2M1)

    # quantizer: fp32 and bf16 input, 67 M elements (one tensor of the headline workload)
    x = torch.randn(8 * 16 * 4096, 128, device=dev)
    for nm, xx, bpe in (("quantizer_fp32_67M", x, 4 + 1 + 1 / 32), ("quantizer_bf16_67M", x.bfloat16(), 2 + 1 + 1 / 32)):
        ms = timed(lambda: rk.mx_quantize(xx), 10)
        gbs = xx.numel() * bpe / (ms * 1e-3) / 1e9
        out[nm] = {"ms_per_call": ms, "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm"], "unit": "GB/s",
                                                   "frac": gbs / peaks["hbm"], "bytes_per_element": bpe, "traffic": None,
                                                   "note": "includes torch.empty of the outputs (allocator cache hit)"}}
    del x
    # V re-blocking along the keys, on the headline workload's V (2 bytes per element algorithmic)
    ms = timed(lambda: rk.mx_rebase_v(vc, vs), 10)
    gbs = vc.numel() * 2 * (1 + 1 / 32) / (ms * 1e-3) / 1e9
    out["rebase_v_67M"] = {"ms_per_call": ms, "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm"], "unit": "GB/s",
                                                           "frac": gbs / peaks["hbm"], "traffic": None}}
    # decode with 8 query heads per KV head
    Bd, Hd, Hkd, Ld = 64, 64, 8, 32768
    g2 = torch.Generator(device=dev).manual_seed(78)
    qd = torch.randn(Bd, Hd, 128, generator=g2, device=dev).bfloat16()
    kcd = torch.randint(0, 0x7E, (Bd, Hkd, Ld, 128), generator=g2, dtype=torch.uint8, device=dev)
    vcd = torch.randint(0, 0x7E, (Bd, Hkd, Ld, 128), generator=g2, dtype=torch.uint8, device=dev)
    ksd = torch.randint(118, 122, (Bd, Hkd, Ld, 4), generator=g2, dtype=torch.uint8, device=dev)
    vsd = torch.randint(118, 122, (Bd, Hkd, Ld, 4), generator=g2, dtype=torch.uint8, device=dev)
    od = torch.empty(Bd, Hd, 128, dtype=torch.bfloat16, device=dev)
    wsd = torch.empty(rk.attn_decode_workspace_bytes(Bd, Hd, Hkd, Ld, 128) + 16, dtype=torch.uint8, device=dev)
    fn = lambda: rk.attn_decode(qd, kcd, vcd, ksd, vsd, out=od, workspace=wsd)
    timed(fn, 3)
    km = kernel_ms(fn, 5)
    by = 2.0 * Bd * Hkd * Ld * 128 * (1 + 1 / 32) + 2 * Bd * Hd * 128 * 2
    out["decode_B64_H64_kv8_L32768"] = {"roofline": {"bound": "hbm", "achieved": by / (km * 1e-3) / 1e9, "peak": peaks["hbm"],
                                                     "unit": "GB/s", "frac": by / (km * 1e-3) / 1e9 / peaks["hbm"], "kernel_ms": km,
                                                     "traffic": None}}
    code = rk.last_device_status()
    if code != 0:
        # reported, not fatal for the headline line: the word is cleared by reading it and later launches run normally
        sys.stderr.write(f"device status {code} after the extra configurations (a bounded device-side wait gave up)\n")
        out["device_status"] = code
    return out


if __name__ == "__main__":
    main()
