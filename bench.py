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
    """DRAM bytes (read + write) per signal row of the fused kernel, from the committed ncu
    capture (profiles/traffic.json); traffic grows in proportion to the rows a launch processes."""
    p = os.path.join(ROOT, "profiles", "traffic.json")
    try:
        with open(p) as f:
            return json.load(f).get("fused_1d_dy256_k64_n64_dram_bytes_per_row")
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
def time_cpu_port(steps, warmup, budget_s=20.0):
    import numpy as np
    from oracle import oracle_c

    w = WORKLOAD
    # all host threads this process may use (torchrun exports OMP_NUM_THREADS=1, which would
    # otherwise turn the CPU arm into a single-thread run)
    try:
        threads = len(os.sched_getaffinity(0))
    except AttributeError:
        threads = os.cpu_count() or 1
    rng = np.random.default_rng(1234)
    probe = 128
    xs = (rng.uniform(-1, 1, (probe, w["K"], w["DY"])) + 1j * rng.uniform(-1, 1, (probe, w["K"], w["DY"]))).astype(np.complex64)
    ws = ((rng.standard_normal((w["K"], w["N"])) + 1j * rng.standard_normal((w["K"], w["N"]))) / np.sqrt(w["K"])).astype(np.complex64)
    oracle_c.spectral_conv_1d(xs, ws, double=False, threads=threads)  # load + first touch
    t0 = time.perf_counter()
    oracle_c.spectral_conv_1d(xs, ws, double=False, threads=threads)
    per_row = (time.perf_counter() - t0) / probe
    total_iters = max(1, steps + warmup)
    rows = int(max(probe, min(w["bs"], budget_s / total_iters / max(per_row, 1e-9))))
    rows -= rows % 64 if rows >= 64 else 0
    x = (rng.uniform(-1, 1, (rows, w["K"], w["DY"])) + 1j * rng.uniform(-1, 1, (rows, w["K"], w["DY"]))).astype(np.complex64)
    for _ in range(warmup):
        oracle_c.spectral_conv_1d(x, ws, double=False, threads=threads)
    t0 = time.perf_counter()
    for _ in range(steps):
        oracle_c.spectral_conv_1d(x, ws, double=False, threads=threads)
    dt = (time.perf_counter() - t0) / max(steps, 1)
    layers_per_s = (rows / w["bs"]) / dt
    sample = "%d of %d signal rows per step (float32 C port of the path, OpenMP), scaled linearly to the full batch" % (rows, w["bs"])
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
        "note": "the reference has no CPU implementation of this path; this times the CPU port (oracle/spectral_oracle.c)",
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


def time_2d_configs(t, dev):
    """Not bench lines: the 2D parity configurations of BASELINE.json timed once for context
    (variant D = image FFT, CGEMM, image iFFT; variant E = cuFFT + cuBLAS)."""
    import torch

    out = {}
    for name, bs, K, N, D, layers in (("config2_2d_bs16_k32_n64_256x256", 16, 32, 64, 256, 1),
                                      ("config4_2d_bs256_k64_n64_256x256_4_layers", 256, 64, 64, 256, 4)):
        try:
            g = torch.Generator(device=dev).manual_seed(7)
            a = torch.empty((K, bs, D, D), dtype=torch.complex64, device=dev)
            for k in range(K):
                a[k] = torch.view_as_complex(torch.rand((bs, D, D, 2), device=dev, generator=g) * 2 - 1)
            b = torch.empty((N, bs, D, D), dtype=torch.complex64, device=dev)
            ws = [torch.view_as_complex(torch.randn((N, K, 2), device=dev, generator=g) / (K ** 0.5)) for _ in range(layers)]
            res = {}
            for variant in ("D", "E"):
                plan = t.SpectralConv(2, bs, D, K, N, DX=D, variant=variant)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                reps = 3
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
                bytes_layer = 8 * bs * D * D * (K + N)
                res[variant] = {"ms_per_layer": ms, "algorithmic_GBps": bytes_layer / ms * 1e-6}
                plan.close()
                del plan
            peak, _ = hbm_peak()
            res["D_frac_of_hbm_peak"] = res["D"]["algorithmic_GBps"] / peak
            out[name] = res
            del a, b
            torch.cuda.empty_cache()
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
    e2e_check = float((yh[:, :4].to(dev) - ys[0][:, :4]).abs().max()) if ring > 0 and args.warmup + args.steps > 0 else None

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
                         "traffic": (tr * rows_local) if tr else None, "peak_source": peak_src,
                         "kernel": "tfno::tc::spectral_tc_kernel<4,true> (tcgen05 fused FFT+CGEMM+iFFT)", "algorithmic_bytes_per_launch": step_bytes},
            "e2e": {"value": 1000.0 / e2e_ms, "unit": UNIT, "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": 8 * (w["bs"] * w["dimX"] * DY * K + K * N * world),
                    "d2h_bytes_per_step": 8 * w["bs"] * w["dimX"] * DY * N, "max_abs_diff_vs_device_path": e2e_check},
            "gpu_launches": args.steps,
            "clocks": clocks.summary(),
        }
        if weak is not None:
            line["weak_scaling"] = weak
        if world == 1:
            v, ms, threads, sample = time_cpu_port(3, 1, budget_s=15.0)
            line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample}
            ref_ms = time_reference_gpu_variant_e(w)
            line["reference_gpu"] = {"variant_E_as_shipped_ms": ref_ms,
                                     "what": "the reference's own TurboFNO_1D_E (cuFFT+cuBLAS, host sync after every kernel) built from its sources, same GPU"}
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
