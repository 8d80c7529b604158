#!/usr/bin/env python
"""Benchmark of the FNO spectral-convolution path on B200.

    python bench.py --gpus N --steps K --warmup W            (N>1: launched under torchrun)
    python bench.py --impl reference ...                      CPU arm (the reference ships no CPU
                                                              path: the oracle port is timed)

Workload (BASELINE config 3): 1D, bs=8192, dimX=1, DY=256, K=N=64, 64 retained modes, complex64,
batch-sharded over the ranks (strong scaling: the whole job is one bs=8192 layer per step, each
rank owns a contiguous bs/world slice with replicated weights; no collective on the data path).
One step = one fused FFT+CGEMM+iFFT launch per rank.  Prints ONE JSON line on rank 0.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOAD = dict(rank=1, bs=8192, dimX=1, DY=256, K=64, N=64)
WORKLOAD_NAME = "1D spectral conv, bs=8192 dimX=1 DY=256 K=64 N=64, 64 modes (BASELINE config 3)"
METRIC, UNIT = "spectral_conv_layers_per_s", "layers/s"
FALLBACK_HBM_GBS = 6650.0


def shard(bs, world, rank):
    """Contiguous batch slice [lo, hi) of rank `rank` out of `world` (sizes differ by at most 1)."""
    base, rem = divmod(bs, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def algorithmic_bytes(bs, dimX, DY, K, N):
    """Input read once + output written once, complex64 (weights excluded: <= 64 KB)."""
    return 8 * bs * dimX * DY * (K + N)


def hbm_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback (6.65 TB/s, earlier measurement on this pool)"


def traffic_per_row():
    """DRAM bytes READ per signal row of the fused kernel, from the committed ncu capture
    (profiles/traffic.json); read traffic grows in proportion to the rows a launch processes.  The
    capture cannot count the write side: a launch ends with up to an L2's worth (126 MB) of freshly
    written output lines still on chip."""
    p = os.path.join(ROOT, "profiles", "traffic.json")
    try:
        with open(p) as f:
            return json.load(f).get("fused_1d_dy256_k64_n64_dram_read_bytes_per_row")
    except Exception:
        return None


class ClockSampler:
    """Samples SM clock and clock-event (throttle) reasons of one GPU while the timed region runs:
    through NVML every few milliseconds, or, if NVML cannot be loaded, by calling nvidia-smi."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index):
        self.index, self.samples, self._stop = index, [], threading.Event()
        self._t = threading.Thread(target=self._run, daemon=True)
        self._nvml = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nvml = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index(index))
            self._max = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nvml = None

    @staticmethod
    def _physical_index(index):
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [v.strip() for v in vis.split(",") if v.strip()]
            if index < len(ids) and ids[index].isdigit():
                return int(ids[index])
        return index

    def _sample_nvml(self):
        n = self._nvml
        mhz = n.nvmlDeviceGetClockInfo(self._h, n.NVML_CLOCK_SM)
        try:
            bits = n.nvmlDeviceGetCurrentClocksEventReasons(self._h)
        except Exception:
            bits = n.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
        flags = [bool(bits & 0x8), bool(bits & 0x40), bool(bits & 0x20), bool(bits & 0x4)]   # hw_slowdown, hw_thermal, sw_thermal, sw_power_cap
        self.samples.append([str(mhz), str(self._max)] + ["Active" if f else "Not Active" for f in flags])

    def _run(self):
        while not self._stop.is_set():
            try:
                if self._nvml is not None:
                    self._sample_nvml()
                else:
                    out = subprocess.check_output(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.QUERY,
                                                   "--format=csv,noheader,nounits"], text=True, timeout=5)
                    self.samples.append([x.strip() for x in out.strip().split(",")])
            except Exception:
                pass
            self._stop.wait(0.002 if self._nvml is not None else 0.2)

    def __enter__(self):
        self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._t.join(timeout=6)

    def summary(self):
        sm = sorted(int(x[0]) for x in self.samples if x and x[0].isdigit())
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        reasons = [n for i, n in enumerate(self.NAMES) if any(len(x) > 2 + i and x[2 + i].lower().startswith("active") for x in self.samples)]
        smax = [int(x[1]) for x in self.samples if len(x) > 1 and x[1].isdigit()]
        return {"sm_mhz": sm[len(sm) // 2], "sm_min_mhz": sm[0], "sm_max_mhz": max(smax) if smax else None, "reasons": reasons,
                "samples": len(sm), "source": "nvml" if self._nvml is not None else "nvidia-smi"}


# ------------------------------------------------------------------------------------------------
# CPU arm: the oracle port, all host threads, bounded sample of the same workload
# ------------------------------------------------------------------------------------------------
def _cpu_threads():
    # all host threads this process may use (torchrun exports OMP_NUM_THREADS=1, which would
    # otherwise turn the CPU arm into a single-thread run)
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def _cpu_layer_scipy(x, ws, threads):
    """The same layer with scipy's pocketfft (all threads) and numpy's BLAS matmul."""
    import numpy as np
    import scipy.fft

    X = scipy.fft.fft(x, axis=-1, workers=threads)[..., :64]                       # [rows, K, 64]
    Y = np.matmul(np.swapaxes(X, 1, 2), ws)                                        # [rows, 64, N]
    Yp = np.zeros((x.shape[0], ws.shape[1], x.shape[2]), dtype=np.complex64)
    Yp[..., :64] = np.swapaxes(Y, 1, 2)
    return scipy.fft.ifft(Yp, axis=-1, workers=threads)


def time_cpu_port(steps, warmup, budget_s=20.0):
    """CPU arm: a bounded sample of the workload on all host threads.  Two implementations of the
    same math are tried on a probe -- the float C port of the path (oracle/spectral_oracle.c,
    OpenMP) and scipy.fft + numpy.matmul -- and the faster one is timed.  A measurement is `steps`
    passes; measurements repeat until two in a row agree within 10 % (at most six) and the best is
    reported, because host timings on a shared box wander."""
    import numpy as np
    from oracle import oracle_c

    w = WORKLOAD
    threads = _cpu_threads()
    rng = np.random.default_rng(1234)
    probe = 128
    xs = (rng.uniform(-1, 1, (probe, w["K"], w["DY"])) + 1j * rng.uniform(-1, 1, (probe, w["K"], w["DY"]))).astype(np.complex64)
    ws = ((rng.standard_normal((w["K"], w["N"])) + 1j * rng.standard_normal((w["K"], w["N"]))) / np.sqrt(w["K"])).astype(np.complex64)
    impls = {"port": lambda x: oracle_c.spectral_conv_1d(x, ws, double=False, threads=threads)}
    try:
        import scipy.fft  # noqa: F401

        impls["scipy"] = lambda x: _cpu_layer_scipy(x, ws, threads)
    except Exception:
        pass
    per_row = {}
    for name, fn in impls.items():
        fn(xs)                                                  # load + first touch
        best = float("inf")
        for _ in range(3):                                      # best of three: one slow probe must not pick the wrong arm
            t0 = time.perf_counter()
            fn(xs)
            best = min(best, time.perf_counter() - t0)
        per_row[name] = best / probe
    kind = min(per_row, key=per_row.get)
    fn = impls[kind]
    total_iters = max(1, 3 * steps + warmup)                    # room for three measurements in the budget
    rows = int(max(probe, min(w["bs"], budget_s / total_iters / max(per_row[kind], 1e-9))))
    rows -= rows % 64 if rows >= 64 else 0
    x = (rng.uniform(-1, 1, (rows, w["K"], w["DY"])) + 1j * rng.uniform(-1, 1, (rows, w["K"], w["DY"]))).astype(np.complex64)
    for _ in range(warmup):
        fn(x)
    times = []
    for rep in range(6):
        t0 = time.perf_counter()
        for _ in range(steps):
            fn(x)
        times.append((time.perf_counter() - t0) / max(steps, 1))
        if len(times) >= 2 and abs(times[-1] - times[-2]) <= 0.1 * min(times[-1], times[-2]):
            break
    dt = min(times)
    layers_per_s = (rows / w["bs"]) / dt
    what = "float32 C port of the path, OpenMP" if kind == "port" else "scipy.fft (pocketfft) + numpy.matmul"
    sample = "%d of %d signal rows per step (%s), scaled linearly to the full batch; best of %d measurements, probe s/row: %s" % (
        rows, w["bs"], what, len(times), ", ".join("%s %.2e" % kv for kv in sorted(per_row.items())))
    return layers_per_s, dt * 1e3, threads, sample


def run_reference_arm(args, rank, world):
    if rank != 0:
        return
    value, ms, threads, sample = time_cpu_port(args.steps, args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "complex64 (f32 arithmetic)", "data": "synthetic",
        "config": {"workload": WORKLOAD_NAME, **WORKLOAD},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference has no CPU implementation of this path; this times the faster of the CPU port (oracle/spectral_oracle.c) and scipy.fft + numpy.matmul (cpu_baseline.sample says which)",
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
def time_reference_gpu_variant_e(w):
    """The reference's own variant-E program (cuFFT+cuBLAS, as shipped) on this GPU, if it was
    built into oracle/_ref/; returns its printed time in ms or None."""
    exe = os.path.join(ROOT, "oracle", "_ref", "TurboFNO_1D_E_reference")
    if not os.path.exists(exe):
        return None
    try:
        out = subprocess.check_output([exe, str(w["bs"]), str(w["dimX"]), str(w["DY"]), str(w["N"]), str(w["K"])], text=True,
                                      timeout=600, stderr=subprocess.STDOUT)
        for line in out.splitlines():
            if "TIME=" in line:
                return float(line.split("TIME=")[1].replace("ms", "").strip())
    except Exception:
        return None
    return None


def time_2d_config(t, dev, name, bs, K, N, D, layers, variants=("D", "E"), reps=3):
    """One 2D parity configuration of BASELINE.json timed for context (not the bench line):
    variant D = image FFT, CGEMM, image iFFT; variant E = cuFFT + cuBLAS.  `layers` chained layers
    ping-pong two buffers.  Returns ms per layer of this process's `bs` batch items."""
    import torch

    g = torch.Generator(device=dev).manual_seed(7)
    a = torch.empty((K, bs, D, D), dtype=torch.complex64, device=dev)
    for k in range(K):
        a[k] = torch.view_as_complex(torch.rand((bs, D, D, 2), device=dev, generator=g) * 2 - 1)
    b = torch.empty((N, bs, D, D), dtype=torch.complex64, device=dev)
    ws = [torch.view_as_complex(torch.randn((N, K, 2), device=dev, generator=g) / (K ** 0.5)) for _ in range(layers)]
    res = {}
    for variant in variants:
        plan = t.SpectralConv(2, bs, D, K, N, DX=D, variant=variant)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for it in range(reps + 1):
            if it == 1:
                e0.record()
            src, dst = a, b
            for l in range(layers):
                plan(src, ws[l], y=dst)
                if K == N:
                    src, dst = dst, src
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / reps / layers
        res[variant] = {"ms_per_layer": ms, "algorithmic_GBps": 8 * bs * D * D * (K + N) / ms * 1e-6, "kernels": plan.kernels()}
        plan.close()
        del plan
    del a, b
    torch.cuda.empty_cache()
    return res


def time_2d_configs(t, dev):
    out = {}
    for name, bs, K, N, D, layers in (("config2_2d_bs16_k32_n64_256x256", 16, 32, 64, 256, 1),
                                      ("config4_2d_bs256_k64_n64_256x256_4_layers", 256, 64, 64, 256, 4)):
        try:
            res = time_2d_config(t, dev, name, bs, K, N, D, layers)
            peak, _ = hbm_peak()
            res["D_frac_of_hbm_peak"] = res["D"]["algorithmic_GBps"] / peak
            out[name] = res
        except Exception as e:      # context only: never fail the bench line over it
            out[name] = {"error": str(e)[:200]}
    return out


def run_gpu_arm(args, rank, world, local_rank):
    import torch

    import turbofno_b200 as t

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product path has no CPU fallback")
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
        tt = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return float(tt.item())

    w = WORKLOAD
    lo, hi = shard(w["bs"], world, rank)
    bs_local = hi - lo
    K, N, DY = w["K"], w["N"], w["DY"]
    rows_local = bs_local * w["dimX"]
    plan = t.SpectralConv(1, bs_local, DY, K, N, dimX=w["dimX"], variant="D")
    step_bytes = algorithmic_bytes(bs_local, w["dimX"], DY, K, N)
    # ring of buffer pairs so that consecutive steps never find their input in the 126 MB L2
    ring = max(2, -(-(1 << 30) // step_bytes))
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    xs = [torch.view_as_complex(torch.rand((K, rows_local, DY, 2), device=dev, generator=g) * 2 - 1) for _ in range(ring)]
    ys = [torch.empty((N, rows_local, DY), dtype=torch.complex64, device=dev) for _ in range(ring)]
    gw = torch.Generator(device=dev).manual_seed(4321)
    wt = torch.view_as_complex(torch.randn((N, K, 2), device=dev, generator=gw) / (K ** 0.5))

    for i in range(max(args.warmup, 3)):
        plan(xs[i % ring], wt, y=ys[i % ring])
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        barrier()
        ev0.record()
        for i in range(args.steps):
            plan(xs[i % ring], wt, y=ys[i % ring])
        ev1.record()
        torch.cuda.synchronize()
        ms_local = ev0.elapsed_time(ev1)
        barrier()
    ms_total = max_over_ranks(ms_local)
    ms_per_step = ms_total / args.steps
    layers_per_s = 1000.0 / ms_per_step                     # whole job: one bs=8192 layer per step

    # end to end through the host-buffer entry point: pinned host tensors, H2D + layer + D2H per step
    e2e_steps = max(1, min(args.steps, 5))
    xh = torch.empty((K, rows_local, DY), dtype=torch.complex64).pin_memory()
    xh.copy_(xs[0].cpu())
    wh = wt.cpu().pin_memory()
    yh = torch.empty((N, rows_local, DY), dtype=torch.complex64).pin_memory()
    plan.exec_host(xh, wh, yh)                              # allocates staging, warms up
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        plan.exec_host(xh, wh, yh)
    e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3) / e2e_steps
    # the whole host-path output against the device path on the same input (every chunk, the tail included)
    plan(xs[0], wt, y=ys[0])
    torch.cuda.synchronize()
    e2e_check = 0.0
    for n0 in range(0, N, 8):
        e2e_check = max(e2e_check, float((yh[n0:n0 + 8].to(dev) - ys[0][n0:n0 + 8]).abs().max()))
    # no kernel-side wait may have run out anywhere above (read once, outside every timed region)
    status_word = t.Handle.get(local_rank).device_status
    if status_word != 0:
        raise SystemExit("bench.py: device status word is %d: a kernel-side wait ran out, results are incomplete" % status_word)

    # For context at N > 1: the same kernel with the per-GPU work of the N = 1 run (every rank a
    # whole bs = 8192 batch, "weak" scaling).  The headline stays the sharded run above, which is
    # how the workload is defined; its per-GPU launches get short (1024 rows at N = 8) and pay
    # pipeline fill and drain once per launch.
    weak = None
    if world > 1:
        del xs, ys
        torch.cuda.empty_cache()
        rows_full = w["bs"] * w["dimX"]
        plan_full = t.SpectralConv(1, w["bs"], DY, K, N, dimX=w["dimX"], variant="D")
        xf = [torch.view_as_complex(torch.rand((K, rows_full, DY, 2), device=dev, generator=g) * 2 - 1) for _ in range(2)]
        yf = [torch.empty((N, rows_full, DY), dtype=torch.complex64, device=dev) for _ in range(2)]
        for i in range(3):
            plan_full(xf[i % 2], wt, y=yf[i % 2])
        barrier()
        ev0.record()
        for i in range(args.steps):
            plan_full(xf[i % 2], wt, y=yf[i % 2])
        ev1.record()
        torch.cuda.synchronize()
        ms_weak = max_over_ranks(ev0.elapsed_time(ev1)) / args.steps
        barrier()
        weak = {"value": world * 1000.0 / ms_weak, "unit": UNIT, "ms_per_step": ms_weak, "rows_per_gpu": rows_full,
                "what": "every rank runs a whole bs=%d layer per step (per-GPU work of the N=1 run)" % w["bs"]}
        plan_full.close()
        del xf, yf

    # BASELINE config 4 (2D, bs=256, K=N=64, 256x256, four chained layers), batch-sharded like the
    # headline workload: every rank runs its bs/world slice; context number at every N.
    sharded_2d = None
    if not args.no_extras:
        try:
            if world == 1:
                del xs, ys
                xs = ys = None
                torch.cuda.empty_cache()
            lo4, hi4 = shard(256, world, rank)
            barrier()
            r4 = time_2d_config(t, dev, "config4", hi4 - lo4, 64, 64, 256, 4, variants=("D",))
            ms4 = max_over_ranks(r4["D"]["ms_per_layer"])
            barrier()
            sharded_2d = {"ms_per_layer": ms4, "layers_per_s": 1000.0 / ms4, "bs_per_gpu": hi4 - lo4,
                          "aggregate_algorithmic_GBps": 8 * 256 * 256 * 256 * 128 / ms4 * 1e-6, "kernels": r4["D"]["kernels"],
                          "what": "2D bs=256 K=N=64 256x256, 4 chained layers, contiguous bs/world slice per GPU, max over ranks"}
        except Exception as e:
            sharded_2d = {"error": str(e)[:200]}

    if rank == 0:
        peak, peak_src = hbm_peak()
        achieved = step_bytes / (ms_local / args.steps * 1e-3) / 1e9
        tr = traffic_per_row()
        line = {
            "metric": METRIC, "value": layers_per_s, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "complex64 (f32 arithmetic)", "data": "synthetic",
            "config": {"workload": WORKLOAD_NAME, **w, "rows_per_gpu": rows_local, "variant": "D (one fused kernel)",
                       "l2": "ring of %d input/output buffer pairs (%.0f MB per step per GPU), each larger than L2 in total" % (ring, step_bytes / 1e6)},
            "aggregate_algorithmic_GBps": algorithmic_bytes(w["bs"], w["dimX"], DY, K, N) / (ms_per_step * 1e-3) / 1e9,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": (tr * rows_local) if tr else None,
                         "traffic_kind": "DRAM bytes read per launch (ncu at bs=1024, scaled by rows); the write side cannot be captured: up to an L2 of output is still on chip when a launch ends",
                         "peak_source": peak_src, "kernel": "tfno::tc::spectral_tc_kernel<8,true> (tcgen05 fused FFT+CGEMM+iFFT): " + ";".join(plan.kernels()),
                         "algorithmic_bytes_per_launch": step_bytes, "algorithmic_read_bytes_per_launch": step_bytes * K // (K + N)},
            "e2e": {"value": 1000.0 / e2e_ms, "unit": UNIT, "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": 8 * (w["bs"] * w["dimX"] * DY * K + K * N * world),
                    "d2h_bytes_per_step": 8 * w["bs"] * w["dimX"] * DY * N, "max_abs_diff_vs_device_path": e2e_check},
            "gpu_launches": args.steps,
            "clocks": clocks.summary(),
        }
        if weak is not None:
            line["weak_scaling"] = weak
        if sharded_2d is not None:
            line["config4_2d_sharded"] = sharded_2d
        if world == 1:
            v, ms, threads, sample = time_cpu_port(3, 1, budget_s=15.0)
            line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample}
            ref_ms = time_reference_gpu_variant_e(w)
            line["reference_gpu"] = {"variant_E_as_shipped_ms": ref_ms,
                                     "what": "the reference's own TurboFNO_1D_E (cuFFT+cuBLAS, host sync after every kernel) built from its sources, same GPU"}
            if xs is None:
                xs = [torch.view_as_complex(torch.rand((K, rows_local, DY, 2), device=dev, generator=g) * 2 - 1) for _ in range(ring)]
                ys = [torch.empty((N, rows_local, DY), dtype=torch.complex64, device=dev) for _ in range(ring)]
            pe = t.SpectralConv(1, bs_local, DY, K, N, dimX=w["dimX"], variant="E")
            for i in range(3):
                pe(xs[i % ring], wt, y=ys[i % ring])
            torch.cuda.synchronize()
            ev0.record()
            for i in range(10):
                pe(xs[i % ring], wt, y=ys[i % ring])
            ev1.record()
            torch.cuda.synchronize()
            line["variant_E_stream_ordered_ms"] = ev0.elapsed_time(ev1) / 10
            pe.close()
            del xs, ys
            torch.cuda.empty_cache()
            if not args.no_extras:
                line["extras"] = time_2d_configs(t, dev)
        print(json.dumps(line), flush=True)
    plan.close()
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="own", choices=["own", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="skip the 2D context timings (N=1 only)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return
    run_gpu_arm(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
