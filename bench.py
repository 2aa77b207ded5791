#!/usr/bin/env python
"""Benchmark of the oxmera matmul path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c3] [--impl ours|reference]

One "step" is one pass over the workload's products (one GEMM for c1..c4,
the forward + two backward GEMMs for c5) on seeded synthetic inputs that are
already resident in HBM.  At N > 1 (one process per GPU, launched by
torch.distributed.run) every rank multiplies its own slice of the batch dim
or of A's rows; there is no exchange step, so the job is timed as the slowest
rank and `value` is total flops / that time.

Prints ONE JSON line (rank 0).  Keys beyond the base contract:
  roofline      the tcgen05 GEMM against the measured cuBLAS bf16 peak
  cpu_baseline  the CPU oracle (a port of oxmera's naive reference matmul) on
                a bounded slab of the same workload, all host threads
  e2e           the same metric through the host-buffer entry point
                (pinned host -> device, multiply, device -> pinned host)

--impl reference times the CPU reference path alone (rank 0 only).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from oxmera_b200 import B200Backend, DType, Tensor, broadcast_shapes  # noqa: E402
from oxmera_b200.dist import init_from_env  # noqa: E402
from oxmera_b200.workloads import WORKLOADS, device_fill, gemm_views, materialise, shard_flops  # noqa: E402

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the tcgen05 GEMM
# on each workload, from the ncu captures summarised under profiles/.
NCU_TRAFFIC_BYTES = {"c3": 971_092_480, "c3f8": 460_873_216}  # the 256x512 pair kernel on c3 (summary of the capture under profiles/)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML (read only)."""

    def __init__(self, index: int, period_s: float = 0.005):
        super().__init__(daemon=True)
        self.index, self.period = index, period_s
        self.samples = []  # (t, sm_mhz, reasons)
        self.max_mhz = None
        self._halt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = None
            try:
                # NVML numbers every GPU of the host, CUDA only the visible ones: match by PCI address
                import torch
                pr = torch.cuda.get_device_properties(index)
                bus = "%08x:%02x:%02x.0" % (pr.pci_domain_id, pr.pci_bus_id, pr.pci_device_id)
                self.h = pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
                self.matched_by = "pci " + bus
            except Exception:
                self.h = None
            if self.h is None:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
                self.matched_by = "index"
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            try:
                self.power_limit_w = pynvml.nvmlDeviceGetEnforcedPowerLimit(self.h) / 1000.0
            except Exception:
                self.power_limit_w = None
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        while not self._halt.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                try:
                    reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    reasons = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                try:
                    watts = nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0
                except Exception:
                    watts = None
                self.samples.append((time.perf_counter(), mhz, reasons, watts))
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self):
        self._halt.set()

    def summary(self, t0: float, t1: float):
        if not self.ok:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvml unavailable"]}
        window = [s for s in self.samples if t0 <= s[0] <= t1]
        label = "timed region"
        if len(window) < 3:
            window, label = self.samples, "warm-up + timed region"
        names = {0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x10: "sync_boost",
                 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown",
                 0x100: "display_clock_setting"}
        seen = set()
        for smp in window:
            for bit, nm in names.items():
                if smp[2] & bit:
                    seen.add(nm)
        mhz = sorted(s[1] for s in window)
        watts = sorted(s[3] for s in window if s[3] is not None)
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(seen), "samples": len(window), "window": label,
                "power_w": watts[len(watts) // 2] if watts else None, "power_limit_w": getattr(self, "power_limit_w", None),
                "nvml_device": getattr(self, "matched_by", None)}


# ---------------------------------------------------------------------------
# the CPU reference arm (also the cpu_baseline of the main arm)
# ---------------------------------------------------------------------------
def cpu_reference(workload_key: str, steps: int, warmup: int, target_s: float = 6.0):
    """Time the CPU oracle's naive triple loop (oxmera-cpu's matmul as its spec
    describes it) on a row slab of every product of the workload, all host
    threads.  The slab is sized so one step takes about `target_s` seconds."""
    from tests.oracle_lib import ACC_NATIVE, BF16, F16, F32, Oracle
    tag = {DType.F32: F32, DType.BF16: BF16, DType.F16: F16, DType.F8E4M3: 8, DType.F8E5M2: 9}
    w = WORKLOADS[workload_key]
    o = Oracle()
    cores = o.threads
    # a first guess of the slab from a tiny probe of the first product
    slabs = []
    for g in w.gemms:
        a_shape, b_shape, o_shape = w.gemm_shapes(g)
        k, n = a_shape[-1], b_shape[-1]
        # host inputs: one slab of A rows (fresh seeded data of the same distribution), B in full for one batch entry
        sa, sb = w.spec(g.a), w.spec(g.b)
        b_full = o.fill(tuple(b_shape[-2:]) if not g.b_perm else tuple(b_shape[-2:][::-1]), tag[w.dtype], w.seed, sb.stream, sb.dist, sb.scale)
        b_view = b_full.T if g.b_perm else b_full
        slabs.append((g, k, n, sa, b_view))

    def run_slab(rows: int):
        inputs = [o.fill((rows, k), tag[w.dtype], w.seed, sa.stream, sa.dist, sa.scale) for _, k, _, sa, _ in slabs]
        flops, t0 = 0, time.perf_counter()  # data generation stays outside the timed part
        for (g, k, n, sa, b_view), a_rows in zip(slabs, inputs):
            st, _ = o.matmul(a_rows, b_view, tag[w.dtype], acc=ACC_NATIVE, nthreads=cores)
            assert st == 0
            flops += 2 * rows * k * n
        return flops, time.perf_counter() - t0

    rows = max(cores, 8)
    f, t = run_slab(rows)
    rate = f / max(t, 1e-6)
    per_row = sum(2 * k * n for _, k, n, _, _ in slabs)
    rows = int(max(cores, min(4096, target_s * rate / per_row)))
    for _ in range(max(0, warmup)):
        run_slab(max(cores, rows // 8))
    total_f, total_t = 0, 0.0
    for _ in range(max(1, steps)):
        f, t = run_slab(rows)
        total_f += f
        total_t += t
    tflops = total_f / total_t / 1e12
    sample = (f"{rows} output rows x full N x full K of each product ({len(slabs)} per step), naive i-j-k loop, "
              f"{cores} threads; throughput of the slab stands for the full workload (linear in M)")
    return {"value": tflops, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample,
            "ms_per_step": 1e3 * total_t / max(1, steps)}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    w = WORKLOADS[args.workload]
    steps, warmup = min(args.steps, 3), min(args.warmup, 1)
    cb = cpu_reference(args.workload, steps, warmup)
    line = {
        "impl": "reference", "metric": "GEMM TFLOP/s", "value": cb["value"], "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": cb["ms_per_step"], "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": w.dtype.name.lower(), "data": "synthetic",
        "config": {"workload": f"{w.key}: {w.title}", "impl": "CPU port of oxmera-cpu's naive matmul (the reference body is todo!())"},
        "cpu_baseline": {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": cb["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------
# the GPU arm
# ---------------------------------------------------------------------------
def measure_brief(be, grp, w, rank, world, steps=10, warmup=3):
    """Device-timed TFLOP/s of one configuration on this rank's shard (max over
    ranks), with inputs generated on the device and outputs allocated once."""
    tensors = materialise(w, device_fill(be))
    work = []
    for g in w.gemms:
        a, b, _ = gemm_views(w, g, tensors, rank, world)
        oshape = tuple(broadcast_shapes(a.shape[:-2], b.shape[:-2])) + (a.shape[-2], b.shape[-1])
        work.append((a, b, Tensor.empty(oshape, w.result_dtype, be)))
    for _ in range(warmup):
        for a, b, out in work:
            be.matmul_into(a, b, out, batched=True)
    be.synchronize()
    grp.barrier()
    timer = be.timer()
    timer.start()
    for _ in range(steps):
        for a, b, out in work:
            be.matmul_into(a, b, out, batched=True)
    timer.stop()
    ms = grp.max_over_ranks(timer.elapsed_ms())
    grp.barrier()
    return {"workload": w.title, "tflops": w.flops() * steps / (ms * 1e-3) / 1e12, "ms_per_step": ms / steps,
            "steps": steps, "kernel": be.last_kernel(), "dtype": w.dtype.name.lower()}


def run_ours(args):
    grp = init_from_env("nccl")
    rank, world, local = grp.rank, grp.world, grp.local_rank
    w = WORKLOADS[args.workload]
    be = B200Backend(local)
    be.set_option("cta_pair", args.cta_pair)
    be.set_option("tile_n", args.tile_n)
    be.set_option("group_m", args.group_m)
    tensors = materialise(w, device_fill(be))
    work = []
    for g in w.gemms:
        a, b, rg = gemm_views(w, g, tensors, rank, world)
        oshape = tuple(broadcast_shapes(a.shape[:-2], b.shape[:-2])) + (a.shape[-2], b.shape[-1])
        out = Tensor.empty(oshape, w.result_dtype, be)  # pooled: allocated once, outside the timed region
        work.append((g, a, b, out))
    be.synchronize()

    def step():
        for _, a, b, out in work:
            be.matmul_into(a, b, out, batched=True)

    sampler = ClockSampler(local)
    sampler.start()
    for _ in range(max(args.warmup, 3)):
        step()
    be.synchronize()
    grp.barrier()
    counts0 = be.launch_counts()
    timer = be.timer()
    t_wall0 = time.perf_counter()
    timer.start()
    for _ in range(args.steps):
        step()
    timer.stop()
    be.synchronize()
    t_wall1 = time.perf_counter()
    ms_local = timer.elapsed_ms()
    grp.barrier()
    counts1 = be.launch_counts()
    sampler.stop()
    ms = grp.max_over_ranks(ms_local)
    kernel_name = be.last_kernel()

    flops_total = w.flops()
    tflops = flops_total * args.steps / (ms * 1e-3) / 1e12
    peaks, peak_src = load_peaks()
    timed_s = ms * 1e-3
    clocks = sampler.summary(t_wall0, t_wall1)
    # Which cuBLAS figure is the fair denominator depends on the regime the
    # timed region ran in: the burst figure while the SM clock stays near its
    # maximum, the sustained one once the 1 kW power cap has pulled it down.
    # The power cap shows as its throttle reason, as a clock well under the
    # maximum, or (the sampled clock lags on some boxes) as a draw at the limit.
    capped = "sw_power_cap" in clocks.get("reasons", []) or (
        clocks.get("sm_mhz") and clocks.get("sm_max_mhz") and clocks["sm_mhz"] < 0.85 * clocks["sm_max_mhz"]) or (
        clocks.get("power_w") and clocks.get("power_limit_w") and clocks["power_w"] >= 0.9 * clocks["power_limit_w"])
    capped = bool(capped)
    # NVML's clock and power readings lag by up to a second on these hosts, so a
    # region of more than 50 ms of back-to-back launches counts as sustained
    # whatever they say: a 42 ms region still ran at the uncapped rate here,
    # regions of 150 ms at the capped one.
    burst = not capped and timed_s < 0.05
    peak = peaks["bf16_tflops"] if burst else peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"])
    if w.dtype == DType.F32:
        peak = peak / 2.0  # tf32 runs at half the bf16 rate; the 3-term split spends 3 MMA flops per useful one
    if w.dtype in (DType.F8E4M3, DType.F8E5M2):
        peak = peak * 2.0  # no fp8 figure was measured: twice the measured bf16 rate, as the nominal rates relate
    launches = counts1["tcgen05"] - counts0["tcgen05"]
    per_gpu_tflops = shard_flops(w, rank, world) * args.steps / (ms_local * 1e-3) / 1e12
    achieved = grp.min_over_ranks(per_gpu_tflops)  # the slowest GPU's own rate
    roofline = {
        "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
        "traffic": NCU_TRAFFIC_BYTES.get(w.key),
        "kernel": kernel_name,
        "peak_source": f"{peak_src} cuBLAS bf16 8192^3, {'burst' if burst else 'sustained'} figure "
                       f"(timed region {timed_s:.3f} s, power cap {'active' if capped else 'not seen'})"
                       + ("; halved for tf32" if w.dtype == DType.F32 else ""),
        "frac_of_burst": achieved / (peaks["bf16_tflops"] / (2.0 if w.dtype == DType.F32 else 1.0)),
        "avg_launch_ms": ms_local / max(1, launches) if launches else None,
        "frac_of_nominal_2250": achieved / ({DType.F32: 1125.0, DType.F8E4M3: 4500.0, DType.F8E5M2: 4500.0}.get(w.dtype, 2250.0)),
        "note": None if w.dtype != DType.F32 else "f32 runs as three TF32 MMA terms: the tensor pipe executes 3x the algorithmic flops counted here",
    }

    # ---- end to end: host buffers in, host buffer out, every step ----
    e2e = None
    if not args.no_e2e and w.result_dtype == w.dtype:
        npdt = {DType.F32: np.float32, DType.BF16: np.uint16, DType.F16: np.float16, DType.F8E4M3: np.uint8,
                DType.F8E5M2: np.uint8}[w.dtype]
        host = {}
        for name, t in tensors.items():
            buf = be.pinned_empty(t.shape, npdt)
            buf[...] = t.to_host()
            host[name] = buf
        from oxmera_b200.backend import shard_ranges
        hwork, h2d, d2h = [], 0, 0
        for g, a, b, out in work:
            ha, hb = host[g.a], host[g.b]
            if world > 1:
                rg = shard_ranges(ha.shape[g.shard_dim], world)[rank]
                idx = [slice(None)] * ha.ndim
                idx[g.shard_dim] = slice(rg.start, rg.stop)
                ha = ha[tuple(idx)]
            if g.a_perm:
                ha = ha.transpose(g.a_perm)
            if g.b_perm:
                hb = hb.transpose(g.b_perm)
            ho = be.pinned_empty(out.shape, npdt)
            hwork.append((ha, hb, ho))
            h2d += (ha.size + hb.size) * ha.itemsize
            d2h += ho.size * ho.itemsize
        e_steps = max(2, min(args.steps, args.e2e_steps))
        for ha, hb, ho in hwork:  # warm-up: staging buffers get allocated here
            be.matmul_host(ha, hb, w.dtype, out=ho)
        grp.barrier()
        t0 = time.perf_counter()
        for _ in range(e_steps):
            for ha, hb, ho in hwork:
                be.matmul_host(ha, hb, w.dtype, out=ho)  # returns after the result bytes have landed
        e_ms = (time.perf_counter() - t0) * 1e3
        grp.barrier()
        e_ms = grp.max_over_ranks(e_ms)
        e2e = {"value": flops_total * e_steps / (e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h), "steps": e_steps,
               "ms_per_step": e_ms / e_steps,
               "note": "per-rank bytes; pinned host memory; oxm_batched_matmul_host per product"}

    # ---- the other configurations, briefly, so one run shows all five ----
    others = None
    if not args.no_others:
        others = {}
        for opt, val in (("cta_pair", -1), ("tile_n", 0), ("group_m", 0)):
            be.set_option(opt, val)  # the library's own choices, whatever the main run forced
        for key in ("c1", "c2", "c4", "c5"):
            if key == w.key:
                continue
            others[key] = measure_brief(be, grp, WORKLOADS[key], rank, world)

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cb = cpu_reference(args.workload, 1, 0, target_s=12.0)
        cpu_baseline = {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")}

    if rank == 0:
        line = {
            "metric": "GEMM TFLOP/s", "value": tflops, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": w.dtype.name.lower(), "data": "synthetic",
            "config": {
                "workload": f"{w.key}: {w.title}",
                "sharding": "none" if world == 1 else f"{'batch' if len(w.gemm_shapes(w.gemms[0])[2]) > 2 else 'M-row blocks'} over {world} GPUs, no collective",
                "l2": "inputs + output exceed the 126 MB L2" if w.algorithmic_bytes() > 126e6 else "working set fits L2 (latency-bound config)",
                "accumulate": "fp32", "flops_per_step": flops_total, "algorithmic_bytes_per_step": w.algorithmic_bytes(),
            },
            "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e,
            "gpu_launches": counts1["total"] - counts0["total"],
            "clocks": clocks,
            "other_configs": others,
            "percent_of_dense_peak": 100.0 * tflops / world / ({DType.F32: 1125.0, DType.F8E4M3: 4500.0, DType.F8E5M2: 4500.0}.get(w.dtype, 2250.0)),
        }
        print(json.dumps(line), flush=True)
    be.close()
    grp.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c3", choices=sorted(WORKLOADS))
    ap.add_argument("--e2e-steps", type=int, default=10)
    ap.add_argument("--cta-pair", type=int, default=-1, choices=[-1, 0, 1], help="-1 auto, 0 one CTA per tile, 1 CTA pairs")
    ap.add_argument("--tile-n", type=int, default=0, choices=[0, 64, 128, 256, 512])
    ap.add_argument("--group-m", type=int, default=0)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-others", action="store_true", help="skip the brief measurement of the other configurations")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
