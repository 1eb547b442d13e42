#!/usr/bin/env python
"""Benchmark of the FP8 scaled-GEMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

N = 1 : one step = the four Llama-3.1-8B prefill linears at M = 4096 tokens
        (qkv, o_proj, gate_up, down), per-tensor e4m3 scales, bf16 out.
N > 1 : one step = the Llama-3.1-70B-shape gate_up GEMM (M=8192, N=57344,
        K=8192), weight rows sharded over the N ranks, NCCL all-gather of the
        bf16 output slabs (launched under torchrun, one rank per GPU).
Prints ONE JSON line on rank 0.  `--impl reference` times the reference's own
torch CPU path (dequantise -> fp32 matmul -> bf16; the oracle) on a bounded
row sample of the same workload, on all host cores.
The N = 1 line also carries bounded sweeps of the other benchmark
configurations (`configs`: the 1024-cube GEMM, the decode shapes, the
block-scaled shapes, the 70B GEMM on one GPU); the N > 1 line carries a result
check (`check`) of the gathered output against the NCCL path and the oracle.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

LLAMA8B = [("qkv", 6144, 4096), ("o_proj", 4096, 4096), ("gate_up", 28672, 4096), ("down", 4096, 14336)]
M_PREFILL = 4096
L70B = dict(M=8192, N=57344, K=8192)
NOMINAL_FP8_TFLOPS = 4500.0


def workload_config(gpus: int) -> dict:
    """The `config` object of the JSON line; both arms print exactly this."""
    if gpus == 1:
        touched = sum(M_PREFILL * K + N * K + 2 * M_PREFILL * N for _, N, K in LLAMA8B)
        return {"workload": "llama31_8b_prefill_m4096",
                "gemms": [f"{n}:{M_PREFILL}x{N}x{K}" for n, N, K in LLAMA8B],
                "scaling_mode": "per-tensor e4m3, bf16 out",
                "l2": f"no flush: {touched / 1e6:.0f} MB touched per step > 126 MB L2"}
    return {"workload": "llama31_70b_gate_up_nshard", "M": L70B["M"], "N": L70B["N"], "K": L70B["K"],
            "parallelism": f"column-parallel x{gpus}; all-gather fused into the GEMM epilogue (tile stores to peer "
                           "buffers over NVLink)",
            "l2": "no flush: operands and output exceed 126 MB L2"}


def use_all_host_threads() -> int:
    """torch.distributed.run exports OMP_NUM_THREADS=1; the CPU legs use every core of the box regardless."""
    n = os.cpu_count() or 1
    torch.set_num_threads(n)
    return torch.get_num_threads()


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return d, "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML while a timed region runs."""

    def __init__(self, index: int, period_s: float = 0.02):
        super().__init__(daemon=True)
        self.index, self.period = index, period_s
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop_evt = threading.Event()
        self.ok = False
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop_evt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self):
        self._stop_evt.set()
        if self.is_alive():
            self.join(timeout=2)
        if not self.samples:
            return None
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(s)}


# --------------------------------------------------------------------------- inputs
def make_case(M, N, K, dev, seed):
    """Seeded synthetic operands with the stated distributions, quantised on the GPU:
    activations N(0,1) with 0.1 % of the K channels x20, weights N(0, 0.02)."""
    import tilegym_b200 as tg

    g = torch.Generator(device=dev).manual_seed(seed)
    x = torch.randn(M, K, generator=g, device=dev, dtype=torch.bfloat16)
    n_out = max(1, round(0.001 * K))
    cols = torch.randperm(K, generator=g, device=dev)[:n_out]
    x[:, cols] *= 20.0
    a8, sa = tg.quant_per_tensor(x)
    del x
    w = torch.randn(N, K, generator=g, device=dev, dtype=torch.bfloat16) * 0.02
    b8, sb = tg.quant_per_tensor(w)
    del w
    return a8, b8, sa, sb


def cpu_step_sample(shapes, rows, seed=0):
    """One bounded CPU sample: the oracle GEMM on `rows` activation rows of every shape.
    Returns (flops, callable)."""
    from oracle import torch_ref as R

    cases = []
    flops = 0
    for i, (M, N, K) in enumerate(shapes):
        m = min(rows, M)
        g = torch.Generator().manual_seed(seed + i)
        a8 = (torch.randn(m, K, generator=g)).clamp_(-448, 448).to(torch.float8_e4m3fn)
        b8 = (torch.randn(N, K, generator=g)).clamp_(-448, 448).to(torch.float8_e4m3fn)
        cases.append((a8, b8, torch.tensor([0.03]), torch.tensor([0.0002])))
        flops += 2 * m * N * K

    def step():
        for a8, b8, sa, sb in cases:
            R.ref_fp8_scaled_mm(a8, b8, sa, sb)

    return flops, step


# --------------------------------------------------------------------------- reference arm
def run_reference(args, rank, world):
    if rank != 0:
        return
    threads = use_all_host_threads()
    if args.gpus == 1:
        shapes = [(M_PREFILL, N, K) for _, N, K in LLAMA8B]
    else:
        shapes = [(L70B["M"], L70B["N"], L70B["K"])]
    rows = 256
    flops, step = cpu_step_sample(shapes, rows)
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    tflops = flops * args.steps / dt / 1e12
    sample = f"{rows} of the M activation rows of every GEMM of the step (all N, K), torch CPU dequantise->fp32 matmul->bf16"
    line = {
        "impl": "reference", "metric": "fp8_gemm_tflops", "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None, "dtype": "e4m3_f32acc",
        "data": "synthetic", "config": workload_config(args.gpus),
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "host": {"cpu_count": os.cpu_count(), "torch_threads": threads, "torch": torch.__version__},
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- our arm
def timed(fn, steps, warmup, dev, dist=None):
    """W warm-up steps, then exactly `steps` steps between CUDA events on the current
    stream, barrier + synchronize on both sides; returns seconds (max over ranks)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize(dev)
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize(dev)
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize(dev)
    sec = e0.elapsed_time(e1) / 1e3
    if dist is not None:
        t = torch.tensor([sec], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        sec = float(t.item())
    return sec


def run_ours_single(args):
    import tilegym_b200 as tg
    from tilegym_b200 import _lib

    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    peaks, peak_src = measured_peaks()
    cases = []
    for i, (name, N, K) in enumerate(LLAMA8B):
        a8, b8, sa, sb = make_case(M_PREFILL, N, K, dev, 2000 + i)
        out = torch.empty(M_PREFILL, N, dtype=torch.bfloat16, device=dev)
        cases.append((name, a8, b8, sa, sb, out))
    flops_step = sum(2 * M_PREFILL * N * K for _, N, K in LLAMA8B)
    bytes_resident = sum(c[1].numel() + c[2].numel() + c[5].numel() * 2 for c in cases)

    def step():
        for _, a8, b8, sa, sb, out in cases:
            tg.fp8_scaled_mm(a8, b8, sa, sb, None, torch.bfloat16, out=out)

    # per-shape device time, each GEMM back to back for 20 launches: short bursts taken BEFORE the
    # sustained headline loop (which runs into the power cap), so they read higher than the headline
    per_shape = {}
    for name, a8, b8, sa, sb, out in cases:
        s = timed(lambda: tg.fp8_scaled_mm(a8, b8, sa, sb, None, torch.bfloat16, out=out), 20, 3, dev)
        N, K = b8.shape
        per_shape[name] = {"us": s / 20 * 1e6, "tflops": 2 * M_PREFILL * N * K * 20 / s / 1e12, "regime": "burst"}

    sampler = ClockSampler(0)
    sampler.start()
    sec = timed(step, args.steps, args.warmup, dev)
    clocks = sampler.stop()
    _lib.device_status(0)
    tflops = flops_step * args.steps / sec / 1e12

    # end to end through the public API with HOST buffers: pinned activations in, pinned result out
    host_in = [c[1].cpu().pin_memory() for c in cases]
    host_out = [torch.empty(c[5].shape, dtype=torch.bfloat16).pin_memory() for c in cases]
    h2d = sum(t.numel() * t.element_size() for t in host_in)
    d2h = sum(t.numel() * t.element_size() for t in host_out)

    # Three streams: host->device copies, GEMMs (the current stream) and device->host copies overlap across
    # the four GEMMs of a step and across steps; events keep each device buffer from being overwritten
    # while a GEMM or a copy still uses it.  Every byte counted in h2d / d2h crosses PCIe inside the timed region.
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    ev_in = [torch.cuda.Event() for _ in cases]      # activation copy i has landed
    ev_gemm = [torch.cuda.Event() for _ in cases]    # GEMM i is done (input consumed, output ready)
    ev_out = [torch.cuda.Event() for _ in cases]     # result copy i has left the device buffer
    main = torch.cuda.current_stream(dev)
    for e in ev_gemm + ev_out:
        e.record(main)

    def step_e2e():
        for i, ((name, a8, b8, sa, sb, out), hin, hout) in enumerate(zip(cases, host_in, host_out)):
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_gemm[i])  # the previous step's GEMM has read this activation buffer
                a8.copy_(hin, non_blocking=True)
                ev_in[i].record(s_in)
            main.wait_event(ev_in[i])
            main.wait_event(ev_out[i])       # the previous step's result has been copied out of `out`
            tg.fp8_scaled_mm(a8, b8, sa, sb, None, torch.bfloat16, out=out)
            ev_gemm[i].record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_gemm[i])
                hout.copy_(out, non_blocking=True)
                ev_out[i].record(s_out)
        main.wait_stream(s_out)              # the step's results are on the host when the step ends

    e2e_steps = max(3, min(args.steps, 20))
    sec_e2e = timed(step_e2e, e2e_steps, 3, dev)
    e2e_tflops = flops_step * e2e_steps / sec_e2e / 1e12

    # CPU baseline: the oracle on a bounded sample of the same step
    cpu = None
    if not args.no_cpu_baseline:
        threads = use_all_host_threads()
        rows = 512
        cflops, cstep = cpu_step_sample([(M_PREFILL, N, K) for _, N, K in LLAMA8B], rows)
        cstep()
        t0 = time.perf_counter()
        reps = 3
        for _ in range(reps):
            cstep()
        dt = (time.perf_counter() - t0) / reps
        cpu = {"value": cflops / dt / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
               "sample": f"{rows} of the 4096 activation rows of each of the 4 GEMMs, {reps} passes, torch CPU oracle"}

    launches = 4 * args.steps
    # Which measured peak applies: MEASURED_PEAKS.json holds the cuBLAS bf16 rate as a burst (a kernel timed in a
    # short loop at full clocks) and sustained (seconds under the 1 kW cap).  The timed region here is a burst
    # unless it ran for a second or more or the sampler saw the power cap; kind::f8f6f4 issues at twice the bf16 rate.
    capped = bool(clocks and "sw_power_cap" in clocks.get("reasons", []))
    regime = "sustained" if (sec >= 1.0 or capped) else "burst"
    peak_burst, peak_sust = 2.0 * peaks["bf16_tflops"], 2.0 * peaks["bf16_tflops_sustained"]
    peak = peak_sust if regime == "sustained" else peak_burst
    roofline = {
        "bound": "tensor", "kernel": "tg_fp8_gemm_pertensor_2cta_kernel", "achieved": tflops, "peak": peak,
        "unit": "TFLOP/s", "frac": tflops / peak, "regime": regime,
        "peak_source": f"2 x bf16_tflops{'_sustained' if regime == 'sustained' else ''} of {peak_src} "
                       f"(fp8 issues at twice the bf16 rate; timed region {sec * 1e3:.1f} ms, power cap "
                       f"{'seen' if capped else 'not seen'}); nominal dense fp8 {NOMINAL_FP8_TFLOPS}",
        "frac_of_burst_peak": tflops / peak_burst, "frac_of_sustained_peak": tflops / peak_sust,
        "frac_of_nominal": tflops / NOMINAL_FP8_TFLOPS,
        "avg_launch_us": sec / launches * 1e6, "flops_per_launch": flops_step / 4,
        "bytes_per_launch": bytes_resident / 4, "traffic": TRAFFIC_FRACTION * bytes_resident / 4,
        "traffic_source": "ncu capture of the gate_up launch (335.2 MB = 0.908 x its algorithmic bytes), "
                          "scaled to the average launch of the step by algorithmic bytes",
    }
    line = {
        "metric": "fp8_gemm_tflops", "value": tflops, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "e4m3_f32acc", "data": "synthetic",
        "config": workload_config(1),
        "roofline": roofline, "cpu_baseline": cpu,
        "e2e": {"value": e2e_tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": sec_e2e / e2e_steps * 1e3, "steps": e2e_steps},
        "gpu_launches": launches, "clocks": clocks, "per_shape": per_shape,
    }
    if not args.no_configs or args.extra:
        import bench_extra

        del host_in, host_out
        torch.cuda.empty_cache()
        if not args.no_configs:
            line["configs"] = bench_extra.run_configs(dev, peaks)
        if args.extra:
            line["extra"] = bench_extra.run(dev, peaks)
        _lib.device_status(0)
    if not args.no_configs:
        # The same step for more than a second (N = 1 default run only): the board's 1 kW cap, not the tensor pipe,
        # sets this rate; it is reported beside the headline against the sustained peak, never instead of it.
        # Measured last, so that no other figure of the run is taken on a board it has heated.
        long_steps = 1600
        sec_long = timed(step, long_steps, 0, dev)
        t_long = flops_step * long_steps / sec_long / 1e12
        line["sustained"] = {"steps": long_steps, "seconds": sec_long, "value": t_long, "unit": "TFLOP/s",
                             "frac_of_sustained_peak": t_long / (2.0 * peaks["bf16_tflops_sustained"]),
                             "peak": 2.0 * peaks["bf16_tflops_sustained"],
                             "peak_source": f"2 x bf16_tflops_sustained of {peak_src}"}
    print(json.dumps(line), flush=True)


# ncu (profiles/pertensor_2cta_gate_up_4096x28672x4096.md): dram__bytes_read.sum + dram__bytes_write.sum of
# one gate_up launch of the dominant kernel is 335.2 MB against 369.1 MB of algorithmic bytes.
TRAFFIC_FRACTION = 335.2 / 369.1
# NVLink 5 peer copy per direction per GPU as measured on this pool's B200 boxes (nominal 900 GB/s): the link rate
# of the fused GEMM + all-gather roofline.
NVLINK_PEER_GBS = 770.0


def measure_peer_store_rate(dev, rank, world, dist, slab_bytes=64 << 20, reps=8):
    """Bytes per second one rank can RECEIVE while every rank copies a slab into every peer's symmetric buffer at
    once (plain device-to-device copies into peer-mapped memory, one stream per destination, destinations in
    rotated order): the all-gather's traffic pattern without the GEMM, i.e. the NVLink floor of the fused step."""
    import torch.distributed._symmetric_memory as symm_mem

    n = slab_bytes // 2
    buf = symm_mem.empty((world, n), dtype=torch.bfloat16, device=dev)
    hdl = symm_mem.rendezvous(buf, group=dist.group.WORLD)
    src = torch.randn(n, device=dev, dtype=torch.bfloat16)
    peers = [(rank + i) % world for i in range(1, world)]
    views = [hdl.get_buffer(pr, (world, n), torch.bfloat16)[rank] for pr in peers]  # my slot in peer pr's buffer
    streams = [torch.cuda.Stream(dev) for _ in peers]
    main = torch.cuda.current_stream(dev)

    def once():
        ev = torch.cuda.Event()
        ev.record(main)
        for v, st in zip(views, streams):
            st.wait_event(ev)
            with torch.cuda.stream(st):
                v.copy_(src, non_blocking=True)
        for st in streams:
            main.wait_stream(st)

    sec = timed(once, reps, 2, dev, dist)
    hdl.barrier()
    return (world - 1) * slab_bytes * reps / sec  # by symmetry what each rank sends is what each rank receives


def run_ours_multi(args, rank, world, local_rank):
    import torch.distributed as dist

    import tilegym_b200 as tg
    from tilegym_b200 import _lib, sharded

    dev = torch.device(f"cuda:{local_rank}")
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    peaks, peak_src = measured_peaks()
    M, N, K = L70B["M"], L70B["N"], L70B["K"]
    lo, hi = sharded.shard_bounds(N, world, rank)
    n = hi - lo

    def draw_shard(r):
        """Weight rows of rank r (a rank-independent stream position, so the union over ranks is one fixed matrix)."""
        gw = torch.Generator(device=dev).manual_seed(6000 + r)
        return torch.randn(n, K, generator=gw, device=dev, dtype=torch.bfloat16) * 0.02

    # every rank draws the same activations
    g = torch.Generator(device=dev).manual_seed(5000)
    x = torch.randn(M, K, generator=g, device=dev, dtype=torch.bfloat16)
    cols = torch.randperm(K, generator=g, device=dev)[: max(1, round(0.001 * K))]
    x[:, cols] *= 20.0
    a8, sa = tg.quant_per_tensor(x)
    del x
    w = draw_shard(rank)
    # global per-tensor weight scale: amax over all shards
    amax = w.abs().max().float().reshape(1)
    dist.all_reduce(amax, op=dist.ReduceOp.MAX)
    sb = (amax / 448.0).to(torch.float32)
    b8 = (w.float() / sb).clamp_(-448, 448).to(torch.float8_e4m3fn)
    del w
    # headline path: the GEMM kernel itself stores every finished tile into all ranks' [M, N] buffers
    # (bulk tensor stores to peer memory over NVLink); the NCCL variants are timed beside it
    gemm = sharded.FusedColumnParallelFP8Gemm(b8, sb, M)
    gemm_nccl = sharded.ColumnParallelFP8Gemm(b8, sb, M, chunks=args.chunks)
    gemm_serial = sharded.ColumnParallelFP8Gemm(b8, sb, M, chunks=1)

    # ---- result check, before anything is timed: (a) the fused kernel's gathered [M, N] buffer equals, bit for
    # bit, what the GEMM + NCCL all-gather path assembles, on every rank; (b) rank 0 compares 64 sampled rows
    # (all N columns) with the CPU oracle on the same quantised bits; (c) the verdicts are reduced over the ranks.
    gemm.out.fill_(float("nan"))
    gemm.forward(a8, sa)
    gemm_nccl.forward(a8, sa, gather=True)
    torch.cuda.synchronize(dev)
    same = bool(torch.equal(gemm.out, gemm_nccl.logical().reshape(M, N)))
    oracle_ok, oracle_res = True, None
    n_rows = 64
    if rank == 0:
        from oracle import torch_ref as R

        use_all_host_threads()
        rows = torch.randperm(M, generator=torch.Generator().manual_seed(7))[:n_rows].sort().values
        b_full = torch.empty(N, K, dtype=torch.float8_e4m3fn)
        for r in range(world):
            wr = draw_shard(r)
            b_full[r * n:(r + 1) * n] = (wr.float() / sb).clamp_(-448, 448).to(torch.float8_e4m3fn).cpu()
            del wr
        ref = R.ref_fp8_scaled_mm(a8[rows.to(dev)].cpu(), b_full, sa.cpu(), sb.cpu())
        oracle_res = R.check_tolerance(gemm.out[rows.to(dev)], ref)
        oracle_ok = bool(oracle_res["ok"])
        del b_full, ref
    flags = torch.tensor([int(same), int(oracle_ok)], device=dev)
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    check = {"fused_equals_nccl": bool(flags[0]), "oracle_rows": n_rows, "oracle_ok": bool(flags[1]),
             "ok": bool(flags[0]) and bool(flags[1]),
             "what": "every rank: torch.equal(fused [M, N] buffer, NCCL-gathered slabs re-assembled); rank 0: "
                     f"{n_rows} sampled rows x all {N} columns against the CPU oracle (2 bf16 ulps / 1e-2 rel)"}
    if rank == 0 and oracle_res is not None:
        check["oracle_max_ulps"] = oracle_res.get("max_abs_ulps_of_R")
        check["oracle_max_rel"] = oracle_res.get("max_rel")

    def step():
        gemm.forward(a8, sa)

    def step_nccl_overlapped():
        gemm_nccl.forward(a8, sa, gather=True)

    def step_nogather():
        gemm_serial.forward(a8, sa, gather=False)

    def step_serial():
        gemm_serial.forward(a8, sa, gather=True)

    sampler = ClockSampler(local_rank)
    sampler.start()
    sec = timed(step, args.steps, args.warmup, dev, dist)
    clocks = sampler.stop()
    sec_gemm = timed(step_nogather, args.steps, args.warmup, dev, dist)
    sec_serial = timed(step_serial, args.steps, args.warmup, dev, dist)
    sec_nccl = timed(step_nccl_overlapped, args.steps, args.warmup, dev, dist)
    _lib.device_status(local_rank)
    flops = 2.0 * M * N * K
    tflops = flops * args.steps / sec / 1e12
    peer_rate = measure_peer_store_rate(dev, rank, world, dist)
    rate_t = torch.tensor([peer_rate], device=dev, dtype=torch.float64)
    dist.all_reduce(rate_t, op=dist.ReduceOp.MIN)
    peer_rate = float(rate_t.item())

    # end to end: every rank copies the (replicated) activations in from pinned host memory, and the gathered
    # result goes to the host ONCE: rank r copies out rows [r M/G, (r+1) M/G) of its gathered [M, N] buffer, so
    # all G PCIe links share the one output instead of each shipping a full copy
    hin = a8.cpu().pin_memory()
    r0, r1 = rank * M // world, (rank + 1) * M // world
    hout = torch.empty((r1 - r0, N), dtype=torch.bfloat16).pin_memory()

    def step_e2e():
        a8.copy_(hin, non_blocking=True)
        gemm.forward(a8, sa)
        hout.copy_(gemm.out[r0:r1], non_blocking=True)

    e2e_steps = max(3, min(args.steps, 10))
    sec_e2e = timed(step_e2e, e2e_steps, 2, dev, dist)
    if rank == 0:
        # Fused GEMM + all-gather: the target time is the slower of the rank's FLOPs at the measured GEMM peak
        # (burst figure: each phase is a short loop) and the bytes it must receive at the link rate; frac = target
        # / achieved time of the fused step.  Link rate: the peer copy measured on this pool, 770 GB/s per direction
        # per GPU (nominal 900).  The all-to-all copy probe of this run is reported beside it, not used as the
        # bound: with 7 destinations its copy-engine copies reach less than the fused kernel's own stores do.
        peak = 2.0 * peaks["bf16_tflops"] * world
        t_gemm = flops / (peak * 1e12)
        recv_bytes = M * N * 2 * (world - 1) // world
        link_rate = NVLINK_PEER_GBS * 1e9
        t_link = recv_bytes / link_rate
        t_target = max(t_gemm, t_link)
        t_fused = sec / args.steps
        line = {
            "metric": "fp8_gemm_tflops", "value": tflops, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": sec / args.steps * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "e4m3_f32acc", "data": "synthetic",
            "config": workload_config(world),
            "check": check,
            "roofline": {"bound": "tensor" if t_gemm >= t_link else "nvlink",
                         "kernel": "tg_fp8_gemm_pertensor_2cta_kernel (fused all-gather epilogue)",
                         "achieved": flops / t_fused / 1e12, "peak": flops / t_target / 1e12, "unit": "TFLOP/s",
                         "frac": t_target / t_fused,
                         "peak_source": f"slower of FLOPs / ({world} x 2 x bf16_tflops of {peak_src}) = {t_gemm * 1e3:.3f} ms and "
                                        f"{recv_bytes / 1e6:.0f} MB received per rank / {NVLINK_PEER_GBS:.0f} GB/s (peer copy per "
                                        f"direction measured on this pool; nominal 900) = {t_link * 1e3:.3f} ms",
                         "link_gbs": NVLINK_PEER_GBS,
                         "received_gbs_achieved": recv_bytes / t_fused / 1e9,
                         "peer_copy_probe_gbs": peer_rate / 1e9,
                         "peer_copy_probe": "all ranks copying 64 MB slabs into all peers at once (device-to-device copies, "
                                            "one stream per destination), slowest rank",
                         "gemm_only_tflops": flops * args.steps / sec_gemm / 1e12,
                         "gemm_only_frac_of_peak": flops * args.steps / sec_gemm / 1e12 / peak,
                         "traffic": None},
            "cpu_baseline": None,
            "e2e": {"value": flops * e2e_steps / sec_e2e / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": hin.numel() * world, "d2h_bytes_per_step": M * N * 2,
                    "ms_per_step": sec_e2e / e2e_steps * 1e3,
                    "note": "bytes are totals over the ranks: activations to every rank, the gathered result to the "
                            "host once (each rank ships M / G of its rows)"},
            "gpu_launches": args.steps, "clocks": clocks,
            "phases": {"gemm_only_ms": sec_gemm / args.steps * 1e3,
                       "gemm_then_nccl_allgather_serial_ms": sec_serial / args.steps * 1e3,
                       f"gemm_nccl_allgather_overlapped_{args.chunks}_slabs_ms": sec_nccl / args.steps * 1e3,
                       "fused_gemm_allgather_ms": sec / args.steps * 1e3,
                       "nvlink_bytes_received_per_rank": (world - 1) * M * (N // world) * 2},
        }
        print(json.dumps(line), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    if not check["ok"]:
        raise SystemExit(3)


def run_one(args):
    """A single kernel on a single problem, for `ncu` captures of a small case."""
    import tilegym_b200 as tg

    kind, dims = args.one.split(":")
    M, N, K = (int(v) for v in dims.split(","))
    dev = torch.device("cuda:0")
    if kind in ("actquant", "groupquant", "quantpt", "dequant"):
        # quantisers: M x N elements; K is the group size (groupquant) and ignored otherwise
        x = torch.randn(M, N, device=dev, dtype=torch.bfloat16)
        if kind == "actquant":
            fn, nbytes = (lambda: tg.act_quant(x)), 3 * M * N + 4 * M * N // 128
        elif kind == "groupquant":
            fn, nbytes = (lambda: tg.per_token_group_quant_8bit(x, K)), 3 * M * N + 4 * M * N // K
        elif kind == "quantpt":
            fn, nbytes = (lambda: tg.quant_per_tensor(x)), 5 * M * N
        else:
            q = x.to(torch.float8_e4m3fn)
            s = torch.rand((M + 127) // 128, (N + 127) // 128, device=dev) + 0.5
            fn, nbytes = (lambda: tg.weight_dequant(q, s)), 3 * M * N
        sec = timed(fn, args.steps, args.warmup, dev)
        print(json.dumps({"one": args.one, "us_per_launch": sec / args.steps * 1e6,
                          "gbs": nbytes * args.steps / sec / 1e9}), flush=True)
        return
    if kind == "grouped":
        # M rows in 8 equal groups (M a multiple of 8), each with its own [N, K] weight
        G = 8
        a8 = torch.randn(M, K, device=dev).to(torch.float8_e4m3fn)
        b8 = torch.randn(G, N, K, device=dev, dtype=torch.bfloat16).mul_(0.02).to(torch.float8_e4m3fn)
        As = torch.rand(M, (K + 127) // 128, device=dev) + 0.5
        Bs = torch.rand(G, (N + 127) // 128, (K + 127) // 128, device=dev) + 0.5
        ind = (torch.arange(G + 1, device=dev) * (M // G)).to(torch.int32)
        fn = lambda: tg.ragged_block_scaled_bmm(a8, b8, As, Bs, ind, M // G)  # noqa: E731
        sec = timed(fn, args.steps, args.warmup, dev)
        print(json.dumps({"one": args.one, "us_per_launch": sec / args.steps * 1e6,
                          "tflops": 2.0 * M * N * K * args.steps / sec / 1e12}), flush=True)
        return
    if kind == "moe":
        # one FP8 mixture-of-experts layer: M tokens, hidden N, intermediate K, 64 experts, top-6
        from tilegym_b200 import moe

        E, topk = 64, 6
        x = torch.randn(M, N, device=dev, dtype=torch.bfloat16)
        w1 = torch.randn(E, 2 * K, N, device=dev, dtype=torch.bfloat16).mul_(0.05).to(torch.float8_e4m3fn)
        w2 = torch.randn(E, N, K, device=dev, dtype=torch.bfloat16).mul_(0.05).to(torch.float8_e4m3fn)
        w1s = torch.rand(E, 2 * K // 128, N // 128, device=dev) + 0.5
        w2s = torch.rand(E, N // 128, K // 128, device=dev) + 0.5
        ids = torch.randint(0, E, (M, topk), device=dev)
        wts = torch.softmax(torch.randn(M, topk, device=dev), dim=-1)
        w1i, w1si = moe.interleave_gate_up_blocks(w1, w1s)
        fn = lambda: moe.fused_experts_impl(x, w1i, w2, wts, ids, use_fp8_w8a8=True, w1_scale=w1si, w2_scale=w2s,  # noqa: E731
                                            a2_quant="block", w1_interleaved=True, fuse_silu_epilogue=True)
        sec = timed(fn, args.steps, args.warmup, dev)
        print(json.dumps({"one": args.one, "us_per_call": sec / args.steps * 1e6,
                          "tflops": 2.0 * M * topk * 3 * K * N * args.steps / sec / 1e12}), flush=True)
        return
    a8, b8, sa, sb = make_case(M, N, K, dev, 1)
    if kind == "swiglu":
        out = torch.empty(M, N // 2, dtype=torch.bfloat16, device=dev)
        fn = lambda: tg.fp8_scaled_mm_swiglu(a8, b8, sa, sb, None, torch.bfloat16, out=out)  # noqa: E731
    elif kind == "pertensor":
        out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        fn = lambda: tg.fp8_scaled_mm(a8, b8, sa, sb, None, torch.bfloat16, out=out)  # noqa: E731
    elif kind == "blockscaled":
        As = torch.rand(M, (K + 127) // 128, device=dev) + 0.5
        Bs = torch.rand((N + 127) // 128, (K + 127) // 128, device=dev) + 0.5
        fn = lambda: tg.w8a8_block_fp8_matmul(a8, b8, As, Bs, [128, 128], torch.bfloat16)  # noqa: E731
    else:
        raise SystemExit("--one KIND must be pertensor, swiglu, blockscaled, grouped, moe, actquant, groupquant, quantpt or dequant")
    sec = timed(fn, args.steps, args.warmup, dev)
    print(json.dumps({"one": args.one, "us_per_launch": sec / args.steps * 1e6,
                      "tflops": 2.0 * M * N * K * args.steps / sec / 1e12,
                      "gbs": (M * K + N * K + 2 * M * N) * args.steps / sec / 1e9}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--extra", action="store_true",
                    help="also run the grouped GEMM, quantiser, SwiGLU and MLP-block sweeps")
    ap.add_argument("--no-configs", action="store_true",
                    help="N = 1: skip the bounded sweeps of the other benchmark configurations (1024 cube, decode, "
                         "block-scaled, 70B on one GPU)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--chunks", type=int, default=8, help="N>1: M-slabs whose all-gather overlaps the next slab's GEMM")
    ap.add_argument("--one", default=None, metavar="KIND:M,N,K",
                    help="profiling aid: run one kernel steps+warmup times. GEMMs pertensor / swiglu / blockscaled / "
                         "grouped (M rows in 8 groups); moe (M tokens, hidden N, intermediate K, 64 experts, top-6); "
                         "quantisers actquant / groupquant (K = group size) / quantpt / dequant on an M x N tensor")
    args = ap.parse_args()
    if args.one:
        run_one(args)
        return
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if world == 1 and args.gpus == 1:
        run_ours_single(args)
    elif world == 1 and args.gpus > 1:
        raise SystemExit("launch with torchrun: python -m torch.distributed.run --nproc-per-node N bench.py --gpus N")
    else:
        run_ours_multi(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
