#!/usr/bin/env python3
"""Benchmark of the MX attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (named in the JSON line): MXFP8 causal MHA prefill B=8 H=16 S=4096 d=128, seeded synthetic
N(0,1) Q/K/V quantized to E4M3 + E8M0 block-32 along d, bf16 output.  A "step" is one pass of the whole
prefill path over that batch through the C ABI: scale re-tiling, V re-blocking along the keys and the tiled
attention kernel.  With N > 1 every rank runs its own batch of independent (batch, head) units (weak
scaling, no data-path collective); time is the max over ranks, value the FLOP of all ranks over it.
The same line also carries the decode leg (batch 64, 32 query heads / 8 KV heads, d=128, KV length 32768).

`--impl reference` times the CPU restatement of the reference path (oracle/) on the host cores on a bounded
sample of the same workload: the reference's own attention cannot run here (its Python model imports an
un-vendored module, its kernels need the Muon toolchain and an RTL simulator).
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PREFILL = dict(B=8, H=16, H_kv=16, S=4096, d=128)
DECODE = dict(B=64, H=32, H_kv=8, L=32768, d=128)
WORKLOAD = "MXFP8 causal MHA prefill B=8 H=16 S=4096 d=128 (E4M3 + E8M0 block-32 along d, P requantized, bf16 out)"
METRIC = "MX attention prefill TFLOP/s (all GPUs) [decode HBM GB/s in `decode`]"


def prefill_flops(c):
    return 4.0 * c["B"] * c["H"] * c["S"] * c["S"] * c["d"] * 0.5      # causal: half the tiles counted


def prefill_algorithmic_bytes(c):
    """Q, K, V codes + E8M0 scales read once, bf16 O and fp32 LSE written once."""
    qkv = (c["B"] * c["H"] * c["S"] + 2 * c["B"] * c["H_kv"] * c["S"]) * c["d"] * (1 + 1 / 32)
    return int(qkv + c["B"] * c["H"] * c["S"] * (2 * c["d"] + 4))


# DRAM traffic of one launch from the ncu captures summarised under profiles/ (dram__bytes_read.sum +
# dram__bytes_write.sum), per unit of work; both kernels' traffic is proportional to the unit count.
NCU_PREFILL_DRAM_BYTES_PER_HEAD = (103.966976e6 + 34.787584e6) / 64        # S=4096, d=128, causal
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
    """nvidia-smi clocks / throttle reasons sampled while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 8:
                    continue
                try:
                    sm.append(float(f[1])); mx.append(float(f[2]))
                except ValueError:
                    continue
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[4:8]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            top = sorted(sm)[len(sm) // 2:]             # the loaded half of the samples
            out.update(sm_mhz=float(np.median(top)), sm_max_mhz=float(max(mx)), reasons=sorted(reasons), samples=len(sm))
        return out


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
    import torch.distributed as dist
    import radiance_kernels_b200 as rk

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
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

    L = rk.lib()
    peaks = measured_peaks()
    if args.case == "small":
        PREFILL.update(B=4)
        DECODE.update(B=8)
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

    # ---- device-resident timing ----------------------------------------------------------------------
    sampler = ClockSampler(local)
    sampler.start()                                    # runs through warm-up and every timed region below
    for _ in range(args.warmup):
        step()
    kev0 = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    kev1 = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for ev in kev0 + kev1:
        ev.record()                                    # materialise the cudaEvent_t handles
    barrier()
    e0.record()
    for i in range(args.steps):
        L.rk_profile_set_events(C.c_void_p(kev0[i].cuda_event), C.c_void_p(kev1[i].cuda_event))
        step()
    L.rk_profile_set_events(None, None)
    e1.record()
    barrier()
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    ms_step = ms_total / args.steps
    kern_ms = float(np.mean([a.elapsed_time(b) for a, b in zip(kev0, kev1)]))
    status = rk.last_device_status()
    if status != 0:
        raise SystemExit(f"device status {status}: a kernel gave up on a bounded wait; no number reported")
    flops = prefill_flops(c)
    value = flops * world / (ms_step * 1e-3) / 1e12
    fp8_peak = 2.0 * peaks["bf16_sustained"]
    roofline = {"bound": "tensor", "achieved": flops / (kern_ms * 1e-3) / 1e12, "peak": fp8_peak, "unit": "TFLOP/s",
                "frac": flops / (kern_ms * 1e-3) / 1e12 / fp8_peak,
                "traffic": NCU_PREFILL_DRAM_BYTES_PER_HEAD * c["B"] * c["H"] if (c["S"], c["d"]) == (4096, 128) else None,
                "traffic_note": "ncu dram read+write of one launch at B=4 (138.75 MB for 64 (batch, head) units), scaled by "
                                "the unit count; algorithmic bytes per launch: %d" % prefill_algorithmic_bytes(c),
                "kernel": "prefill2q_kernel<false>", "kernel_ms": kern_ms,
                "peak_note": f"2 x {peaks['source']} sustained cuBLAS bf16 ({peaks['bf16_sustained']} TF/s) as the dense "
                             f"MXFP8 proxy; nominal dense FP8 is 4500 TF/s (frac of nominal {flops / (kern_ms * 1e-3) / 1e12 / 4500.0:.4f})"}

    # ---- end to end through the host-buffer entry point ----------------------------------------------------
    e2e = None
    if not args.no_e2e:
        host = [t.cpu().pin_memory() for t in (qc, kc, vc, qs, ks, vs)]
        runner = rk.PrefillHostRunner(*host, causal=True, v_scale_axis=rk.V_SCALES_ALONG_D, device=dev)
        runner.run()
        n_e2e = max(3, min(args.steps, 10))
        barrier()
        t0 = time.perf_counter()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record()
        for _ in range(n_e2e):
            runner.run()
        f1.record()
        barrier()
        ms_e2e = max_over_ranks(f0.elapsed_time(f1)) / n_e2e
        e2e = {"value": flops * world / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_e2e,
               "h2d_bytes_per_step": runner.h2d_bytes, "d2h_bytes_per_step": runner.d2h_bytes, "steps": n_e2e}
        del runner, host
    launches = args.steps * 4          # 2 scale re-tilings, V re-blocking, attention kernel per step
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
        k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        k0.record(); k1.record()
        barrier()
        d0.record()
        for i in range(args.steps):
            if i == args.steps - 1:
                L.rk_profile_set_events(C.c_void_p(k0.cuda_event), C.c_void_p(k1.cuda_event))
            dstep()
        L.rk_profile_set_events(None, None)
        d1.record()
        barrier()
        dms = max_over_ranks(d0.elapsed_time(d1)) / args.steps
        dk = k0.elapsed_time(k1)
        by = decode_bytes(dc)
        decode = {"metric": "decode attention HBM GB/s (all GPUs)", "value": by * world / (dms * 1e-3) / 1e9, "unit": "GB/s",
                  "ms_per_step": dms, "workload": "batch 64, 32 query heads / 8 KV heads, d=128, KV length 32768, MXFP8 cache",
                  "num_splits": rk.attn_decode_num_splits(Bd, Hd, Hkd, Ld, dd),
                  "roofline": {"bound": "hbm", "achieved": by / (dk * 1e-3) / 1e9, "peak": peaks["hbm"], "unit": "GB/s",
                               "frac": by / (dk * 1e-3) / 1e9 / peaks["hbm"],
                               "traffic": NCU_DECODE_DRAM_BYTES_PER_SEQUENCE * Bd if (Hkd, Ld, dd) == (8, 32768, 128) else None,
                               "traffic_note": "ncu dram read+write of one launch at B=8 (560.35 MB), scaled by B",
                               "kernel": "decode_tc_kernel",
                               "kernel_ms": dk, "peak_note": f"{peaks['source']} HBM copy bandwidth; nominal 8000 GB/s"}}
        if rk.last_device_status() != 0:
            raise SystemExit("device status non-zero after the decode leg")
        launches += args.steps * 2
        del kcd, vcd, ksd, vsd

    clocks = sampler.stop()
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        import oracle
        cpu, _, _ = cpu_sample("port", oracle.hardware_threads())

    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return
    line = {"metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "mxfp8_e4m3 (e8m0 block scales, fp32 accumulate, bf16 out)", "data": "synthetic",
            "config": {"workload": WORKLOAD if args.case == "full" else "REDUCED BATCH (profiling case, not a bench number): " + WORKLOAD, "per_gpu_batch": "B=8 H=16 (128 independent (batch, head) units per GPU)",
                       "parallelism": f"units sharded over {world} GPU(s), no collective on the data path",
                       "l2": "inputs + output (335 MB) exceed the 126 MB L2; no flush between steps"},
            "roofline": roofline, "e2e": e2e, "gpu_launches": launches, "clocks": clocks, "decode": decode}
    if cpu is not None:
        line["cpu_baseline"] = cpu
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
