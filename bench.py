#!/usr/bin/env python
"""Benchmark of the oxmera matmul path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c3] [--impl ours|reference]

One "step" is one pass over the workload's products (one GEMM for c1..c4,
the forward + two backward GEMMs for c5) on seeded synthetic inputs that are
already resident in HBM.  At N > 1 (one process per GPU, launched by
torch.distributed.run) every rank multiplies its own slice of the batch dim
or of A's rows; there is no exchange step, so the job is timed as the slowest
rank and `value` is total flops / that time.

Before anything is timed every rank checks its own shard's output: two float64
checksums over the whole shard (C.1 against A.(B.1), 1^T.C against (1^T.A).B) on
the host; a failing rank makes the run exit non-zero and `shards_checked` false.

Prints ONE JSON line (rank 0).  Keys beyond the base contract:
  roofline      the tcgen05 GEMM against the measured cuBLAS bf16 peak, for the
                `--steps` region (`value`), plus `repeats` (best and median of
                further repeats of that region), `sustained` (launches back to
                back for two seconds and more: TFLOP/s, median SM clock of that
                leg, cycles per launch = time x clock, fraction of the measured
                sustained cuBLAS figure) and `cold_l2_ms` (one launch after
                the L2 has been overwritten)
  cpu_baseline  the CPU oracle (a port of oxmera's naive reference matmul) on
                a bounded slab of the same workload, all host threads
  e2e           the same metric with operands starting and the result ending
                in page-locked host memory: through the host-buffer entry point
                on one GPU; on several GPUs every rank uploads its rows of A and
                1/N of a replicated B, the replicas are completed by an NCCL
                all-gather into each GPU's own memory, and every rank brings
                its rows of C back

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
from oxmera_b200.workloads import WORKLOADS, device_fill, gemm_views, materialise, mx_scales, shard_flops  # noqa: E402

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the tcgen05 GEMM
# on each workload, from the ncu captures summarised under profiles/.
# Valid for the whole product on one GPU only: a shard reads all of B whatever its
# share of A, so the figure does not scale with the shard and is not reported at N > 1.
NCU_TRAFFIC_BYTES = {
    "c3": 972_272_896,     # the 256 x 512 pair kernel (gemm_tcgen05_pair512_c3_bf16_8192.md)
    "c3f8": 446_797_056,   # gemm_tcgen05_mxf8_c3mx_8192.md (the plain fp8 column)
    "c3mx": 431_382_528,   # gemm_tcgen05_mxf8_c3mx_8192.md
    "c2": 1_324_522_280,   # the tf32x3 GEMM alone; the two pack launches add 161 MB (gemm_tcgen05_tf32x3_c2.md)
    "c5": 2_121_017_088 // 3,  # mean of the three launches of a step (gemm_tcgen05_c5_linear_fwd_bwd.md)
}

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
        self._pause = threading.Event()
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
            if self._pause.is_set():
                time.sleep(0.01)
                continue
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

    def pause(self):
        """Stop sampling for a while: the sampling thread competes with a launch-bound Python loop
        for the interpreter (a 14 us-per-launch loop measured 21 us beside it)."""
        self._pause.set()

    def resume(self):
        self._pause.clear()

    def summary(self, t0: float, t1: float):
        if not self.ok:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvml unavailable"]}
        window = [s for s in self.samples if t0 <= s[0] <= t1]
        label = "timed region"
        if len(window) < 3:
            # too short to be sampled: everything up to its end (and the one reading that follows),
            # never the longer legs that run after it
            window, label = [s for s in self.samples if s[0] <= t1 + 0.1] or self.samples, "warm-up + timed region"
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
    cores = 1 if w.mx else o.threads  # the block-scaled port is a plain single-threaded loop
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
            if w.mx:
                rng = np.random.default_rng(rows)
                st, _ = o.matmul_mx(a_rows, rng.integers(124, 131, size=(rows, k // 32), dtype=np.uint8), b_view,
                                    rng.integers(124, 131, size=(k // 32, n), dtype=np.uint8), tag[w.dtype])
                assert st == 0
                flops += 2 * rows * k * n
                continue
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
def _host_f32(x: np.ndarray, dtype: DType) -> np.ndarray:
    """Host copy of a device tensor as float32 (bf16 arrives as uint16 bits)."""
    if dtype == DType.BF16:
        return (x.astype(np.uint32) << 16).view(np.float32)
    return x.astype(np.float32)


def decode_fp8(bits: np.ndarray, dtype: DType) -> np.ndarray:
    """OCP 8-bit floats to float32 through a 256-entry table: e4m3 (bias 7, no
    infinities, S.1111.111 = NaN) and e5m2 (bias 15, IEEE-like)."""
    e_bits, m_bits, bias = (4, 3, 7) if dtype == DType.F8E4M3 else (5, 2, 15)
    table = np.empty(256, np.float32)
    for v in range(256):
        sign = -1.0 if v & 0x80 else 1.0
        e, m = (v >> m_bits) & ((1 << e_bits) - 1), v & ((1 << m_bits) - 1)
        if e == 0:
            x = m * 2.0 ** (1 - bias - m_bits)
        elif dtype == DType.F8E4M3:
            x = float("nan") if (e == 15 and m == 7) else (1 + m / 8.0) * 2.0 ** (e - bias)
        else:
            x = (float("inf") if m == 0 else float("nan")) if e == 31 else (1 + m / 4.0) * 2.0 ** (e - bias)
        table[v] = sign * x
    return table[np.asarray(bits, np.uint8)]


def verify_shard(w, work, oracle_fp8=None, scales=None) -> dict:
    """Size-independent check of this rank's outputs, in float64 on the host:
    for every product C = A.B of the shard, C.1 against A.(B.1) and 1^T.C against
    (1^T.A).B over the WHOLE shard.  A rank that multiplied the wrong rows, read
    the wrong operand or skipped a tile fails it.  The budget is the rounding of
    the stored result summed like sqrt(n) (bf16 / f16), or the f32 path's
    accumulation bias summed like n."""
    import itertools
    worst = 0.0
    for g, a, b, out in work:
        ha, hb, ho = a.to_host(), b.to_host(), out.to_host()
        if w.dtype in (DType.F8E4M3, DType.F8E5M2):
            ha, hb = oracle_fp8(ha), oracle_fp8(hb)
            if scales is not None:  # block-scaled: every 32 of K carry a power of two
                sa, sb = scales[work.index((g, a, b, out))]
                ha = ha * np.repeat(np.ldexp(np.float32(1), sa.to_host().astype(np.int32) - 127), 32, axis=-1)
                hb = hb * np.repeat(np.ldexp(np.float32(1), sb.to_host().astype(np.int32) - 127), 32, axis=-2)
        else:
            ha, hb = _host_f32(ha, w.dtype), _host_f32(hb, w.dtype)
        ho = _host_f32(ho, w.result_dtype)
        lead = ho.shape[:-2]
        m, n = ho.shape[-2:]
        for bi in (list(itertools.product(*[range(d) for d in lead])) or [()]):
            def pick(full):
                nb = full.ndim - 2
                return tuple(0 if full.shape[j] == 1 else bi[len(lead) - nb + j] for j in range(nb))
            A, B, Cm = ha[pick(ha)], hb[pick(hb)], ho[bi]
            rms = float(np.sqrt(np.mean(np.square(Cm, dtype=np.float64)))) + 1e-30
            if w.result_dtype == DType.F32:
                budget = lambda count: 1e-5 * rms * count + 1e-9
            else:
                budget = lambda count: 6 * 2.0 ** -8 * rms * np.sqrt(count) + 1e-9
            row_ref = A.astype(np.float64) @ B.sum(axis=1, dtype=np.float64)
            col_ref = A.sum(axis=0, dtype=np.float64) @ B.astype(np.float64)
            e_row = float(np.max(np.abs(Cm.sum(axis=1, dtype=np.float64) - row_ref))) / budget(n)
            e_col = float(np.max(np.abs(Cm.sum(axis=0, dtype=np.float64) - col_ref))) / budget(m)
            worst = max(worst, e_row, e_col)
    return {"ok": bool(worst <= 1.0), "worst_over_budget": worst}


class _DeviceBytes:
    """A device buffer of this library, seen by torch as a uint8 tensor
    (zero copy), so that NCCL can gather into it."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


def e2e_sharded(be, grp, w, work, tensors, host, steps):
    """End to end on several GPUs.  Per step and per rank: upload from
    page-locked host memory this rank's rows of every tensor it only needs rows
    of, and ITS 1/N of the bytes of every tensor it needs whole (a replicated
    operand, or one it reads a column window of); complete those with an NCCL
    all-gather (whole buffers, into each GPU's own memory, before any kernel
    reads them); multiply; bring this rank's part of every result back.  Every
    input byte crosses PCIe once per step over the whole job.
    Returns (ms per step, h2d bytes per rank, d2h bytes per rank)."""
    import torch
    import torch.distributed as dist
    from oxmera_b200.backend import shard_ranges
    rank, world = grp.rank, grp.world
    esz = w.dtype.size_in_bytes()
    from oxmera_b200.workloads import shard_extent
    # Per base tensor: ("rows", dim) when this rank only ever reads one contiguous block of it (the
    # sharded dim is the outermost one with extent > 1), "full" when it needs all of it.
    need = {}

    def want(name, dim, sharded):
        shape = tensors[name].shape
        block = sharded and shape[dim] != 1 and all(s == 1 for s in shape[:dim])
        if not block:
            need[name] = "full"
        elif need.get(name) != "full":
            need[name] = ("rows", dim)

    for g, a, b, out in work:
        want(g.a, g.shard_dim, True)
        want(g.b, g.shard_b_dim if g.shard_b_dim is not None else 0, g.shard_b_dim is not None)
    extent = {}
    for g, a, b, out in work:
        n = shard_extent(g, tensors[g.a].shape, tensors[g.b].shape)
        for name in (g.a, g.b):
            if need.get(name) != "full":
                extent[name] = n
    uploads, gathers, h2d = [], [], 0
    for name, t in tensors.items():
        if name not in need:
            continue
        flat = host[name].reshape(-1).view(np.uint8)
        nbytes = flat.size
        if need[name] == "full":
            per = (nbytes + world - 1) // world
            if per * world != nbytes or per % 16:
                raise RuntimeError(f"{name}: {nbytes} bytes do not split into {world} aligned parts")
            lo, hi = rank * per, (rank + 1) * per
            full = torch.as_tensor(_DeviceBytes(t.storage().ptr, nbytes), device=f"cuda:{grp.local_rank}")
            gathers.append((full, lo, hi))
        else:
            dim = need[name][1]
            rg = shard_ranges(extent[name], world)[rank]
            unit = nbytes // t.shape[dim]
            lo, hi = rg.start * unit, rg.stop * unit
        uploads.append((t.storage().ptr + lo, flat[lo:hi]))
        h2d += hi - lo
    outs, d2h = [], 0
    for g, a, b, out in work:
        ho = be.pinned_empty(out.shape, host[g.a].dtype)
        outs.append((a, b, out, ho))
        d2h += ho.size * esz

    def step():
        for dst, src in uploads:
            be._h2d(dst, src.ctypes.data, src.size)
        be.synchronize()  # my parts are in my HBM
        for full, lo, hi in gathers:
            dist.all_gather_into_tensor(full, full[lo:hi])
        torch.cuda.synchronize(grp.local_rank)  # every replica is complete before a kernel reads it
        for a, b, out, _ in outs:
            be.matmul_into(a, b, out, batched=True)
        for _, _, out, ho in outs:
            lo_, _hi = out.layout().extent()
            assert out.layout().is_contiguous()
            be._d2h(ho.ctypes.data, out.storage().ptr + lo_ * esz, ho.size * esz)  # returns when the bytes have landed

    step()  # warm-up (NCCL channels)
    grp.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    ms = (time.perf_counter() - t0) * 1e3
    grp.barrier()
    for a, b, out, ho in outs:  # what came back is what the device-resident run produced
        if not np.array_equal(ho, out.to_host()):
            raise RuntimeError("end-to-end result differs from the device-resident one")
    return grp.max_over_ranks(ms) / steps, h2d, d2h


def measure_brief(be, grp, w, rank, world, steps=10, warmup=3):
    """Device-timed TFLOP/s of one configuration on this rank's shard (max over
    ranks), with inputs generated on the device and outputs allocated once."""
    tensors = materialise(w, device_fill(be))
    work = []
    for g in w.gemms:
        a, b, _ = gemm_views(w, g, tensors, rank, world)
        oshape = tuple(broadcast_shapes(a.shape[:-2], b.shape[:-2])) + (a.shape[-2], b.shape[-1])
        work.append((a, b, Tensor.empty(oshape, w.result_dtype, be)))
    if w.mx:
        sc = mx_scales(w, be)
        calls = [be.prepare_matmul_mx(a, sa, b, sb, out)
                 for (a, b, out), (sa, sb) in zip(work, [gemm_views(w, g, sc, rank, world)[:2] for g in w.gemms])]
    else:
        calls = [be.prepare_matmul(a, b, out, batched=True) for a, b, out in work]  # views marshalled once
    for _ in range(warmup):
        for call in calls:
            call()
    # Three bursts of `steps` steps, each after half a second of idle: the burst regime `value` is
    # measured in.  On a 1 kW part the clock follows the last ~100 ms of load: back to back with
    # other work the same ten steps of c5 read 1250-1340 TFLOP/s, after a short idle 1480-1540 (the
    # sustained regime is reported for the main workload, `roofline.sustained`).
    regions = []
    for _ in range(3):
        be.synchronize()
        time.sleep(0.5)
        for call in calls:  # one step to wake the clocks
            call()
        be.synchronize()
        grp.barrier()
        timer = be.timer()
        timer.start()
        for _ in range(steps):
            for call in calls:
                call()
        timer.stop()
        regions.append(grp.max_over_ranks(timer.elapsed_ms()))
        grp.barrier()
    ms = sorted(regions)[1]
    return {"workload": w.title, "tflops": w.flops() * steps / (ms * 1e-3) / 1e12, "ms_per_step": ms / steps,
            "best_tflops": w.flops() * steps / (min(regions) * 1e-3) / 1e12, "regions": 3,
            "steps": steps, "kernel": be.last_kernel(), "dtype": w.dtype.name.lower()}


def run_ours(args):
    grp = init_from_env("nccl")
    rank, world, local = grp.rank, grp.world, grp.local_rank
    w = WORKLOADS[args.workload]
    # --shard-of N on one GPU: the work rank 0 of an N-GPU run would get, timed alone
    # (a cheap look at one shard's tiling; every figure of the line then counts that shard only)
    srank, sworld = (0, args.shard_of) if (world == 1 and args.shard_of > 1) else (rank, world)
    alone = sworld != world
    be = B200Backend(local)
    be.set_option("cta_pair", args.cta_pair)
    be.set_option("tile_n", args.tile_n)
    be.set_option("group_m", args.group_m)
    tensors = materialise(w, device_fill(be))
    work = []
    for g in w.gemms:
        a, b, rg = gemm_views(w, g, tensors, srank, sworld)
        oshape = tuple(broadcast_shapes(a.shape[:-2], b.shape[:-2])) + (a.shape[-2], b.shape[-1])
        out = Tensor.empty(oshape, w.result_dtype, be)  # pooled: allocated once, outside the timed region
        work.append((g, a, b, out))
    be.synchronize()

    scales = None
    if w.mx:
        sc = mx_scales(w, be)
        scales = [gemm_views(w, g, sc, srank, sworld)[:2] for g in w.gemms]
        calls = [be.prepare_matmul_mx(a, sa, b, sb, out) for (_, a, b, out), (sa, sb) in zip(work, scales)]
    else:
        calls = [be.prepare_matmul(a, b, out, batched=True) for _, a, b, out in work]  # views marshalled once

    def step():
        for call in calls:
            call()

    # ---- every rank checks its own shard before anything is timed ----
    step()
    be.synchronize()
    fp8 = None
    if w.dtype in (DType.F8E4M3, DType.F8E5M2):
        fp8 = lambda bits: decode_fp8(bits, w.dtype)
    check = verify_shard(w, work, fp8, scales)
    all_ok = grp.min_over_ranks(1.0 if check["ok"] else 0.0) > 0.5
    worst_check = grp.max_over_ranks(check["worst_over_budget"])
    if not all_ok:
        sys.stderr.write(f"rank {rank}: shard check {'passed' if check['ok'] else 'FAILED'} "
                         f"(worst checksum error / budget = {check['worst_over_budget']:.3g})\n")
        if rank == 0:
            print(json.dumps({"metric": "GEMM TFLOP/s", "value": None, "n_gpus": world, "shards_checked": False,
                              "error": "a rank's output failed its checksums; nothing was timed"}), flush=True)
        be.close()
        grp.close()
        sys.exit(3)

    def timed(n_steps):
        """n_steps back to back between events, bracketed by barriers and synchronisation.
        Returns (this rank's ms, max over ranks, wall-clock window)."""
        be.synchronize()
        grp.barrier()
        tm = be.timer()
        t0 = time.perf_counter()
        tm.start()
        for _ in range(n_steps):
            step()
        tm.stop()
        be.synchronize()
        t1 = time.perf_counter()
        local_ms = tm.elapsed_ms()
        grp.barrier()
        return local_ms, grp.max_over_ranks(local_ms), (t0, t1)

    job_flops = shard_flops(w, srank, sworld) if alone else w.flops()
    sampler = ClockSampler(local)
    sampler.start()
    for _ in range(max(args.warmup, 3)):
        step()
    counts0 = be.launch_counts()
    ms_local, ms, (t_wall0, t_wall1) = timed(args.steps)   # the contract's region: `value`
    counts1 = be.launch_counts()
    kernel_name = be.last_kernel()
    # further repeats of the same region: best and median
    rep_ms = [ms]
    for _ in range(max(0, args.repeats - 1)):
        rep_ms.append(timed(args.steps)[1])
    # ---- the other configurations, briefly, so one run shows them all ----
    # Bursts of ten steps each (median of three, see measure_brief), before the seconds-long leg below.
    others = None
    if alone:
        args.no_e2e = args.no_cpu = args.no_others = True
    if not args.no_others:
        others = {}
        sampler.pause()
        for opt, val in (("cta_pair", -1), ("tile_n", 0), ("group_m", 0)):
            be.set_option(opt, val)  # the library's own choices, whatever the main run forced
        for key in ("c1", "c2", "c4", "c5", "c3f8", "c3mx"):
            if key == w.key:
                continue
            others[key] = measure_brief(be, grp, WORKLOADS[key], rank, world)
        for opt, val in (("cta_pair", args.cta_pair), ("tile_n", args.tile_n), ("group_m", args.group_m)):
            be.set_option(opt, val)
        sampler.resume()

    # launches back to back for two seconds and more, with the clock samples of this leg only
    n_sus = int(max(args.steps, min(200000, np.ceil(args.sustained_s * 1e3 / max(min(rep_ms) / args.steps, 1e-3))))) if args.sustained_s > 0 else 0
    sustained = None
    if n_sus:
        sus_local, sus_ms, (s0, s1) = timed(n_sus)
        sus_clk = sampler.summary(s0 + 0.25 * (s1 - s0), s1)  # the clock has settled by the second quarter
        sustained = {"launches_per_rank": n_sus * len(work), "seconds": sus_ms * 1e-3, "ms_per_step": sus_ms / n_sus,
                     "tflops": job_flops * n_sus / (sus_ms * 1e-3) / 1e12, "sm_mhz_median": sus_clk.get("sm_mhz"),
                     "power_w": sus_clk.get("power_w"), "reasons": sus_clk.get("reasons"), "samples": sus_clk.get("samples")}
        if sus_clk.get("sm_mhz"):
            # the clock-independent figure to compare from run to run: SM cycles one step takes on the slowest rank
            sustained["cycles_per_step"] = sus_ms / n_sus * 1e-3 * sus_clk["sm_mhz"] * 1e6
            sustained["cycles_per_launch"] = sustained["cycles_per_step"] / len(work)
    # one step on a cold L2: a buffer larger than the L2 is overwritten first
    cold_ms = None
    if args.cold_l2:
        flush = Tensor.empty((256 << 20,), DType.U8, be)
        cold = []
        for _ in range(3):
            be._lib.oxm_memset(be._ctx, flush.storage().ptr, 0, 256 << 20)
            tm = be.timer()
            tm.start()
            step()
            tm.stop()
            cold.append(tm.elapsed_ms())
        cold_ms = grp.max_over_ranks(float(np.median(cold)))
        del flush
    sampler.stop()

    flops_total = job_flops
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
    # NVML's clock and power readings lag by up to a second on these hosts, so the length of the
    # region decides: under 50 ms of back-to-back launches it is held against the burst figure
    # (the higher, i.e. stricter, denominator - also when the samples around it show the cap,
    # which then only says that the GPU was still warm from what ran before); a longer region
    # ran at the capped rate in every run here and is held against the sustained figure.
    burst = timed_s < 0.05
    scale = 0.5 if w.dtype == DType.F32 else 2.0 if w.dtype in (DType.F8E4M3, DType.F8E5M2) else 1.0
    # f32: tf32 runs at half the bf16 rate (and the 3-term split spends 3 MMA flops per useful one);
    # fp8: no figure was measured, twice the measured bf16 rate, as the nominal rates relate
    peak = (peaks["bf16_tflops"] if burst else peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"])) * scale
    launches = counts1["tcgen05"] - counts0["tcgen05"]
    per_gpu_tflops = shard_flops(w, srank, sworld) * args.steps / (ms_local * 1e-3) / 1e12
    achieved = grp.min_over_ranks(per_gpu_tflops)  # the slowest GPU's own rate
    if sustained:
        sus_per_gpu = sustained["tflops"] / world
        sustained["tflops_per_gpu"] = sus_per_gpu
        sustained["frac"] = sus_per_gpu / (peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]) * scale)
        sustained["peak"] = peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]) * scale
    rep_sorted = sorted(rep_ms)
    roofline = {
        "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
        "traffic": NCU_TRAFFIC_BYTES.get(w.key) if sworld == 1 else None,
        "kernel": kernel_name,
        "peak_source": f"{peak_src} cuBLAS bf16 8192^3, {'burst' if burst else 'sustained'} figure "
                       f"(timed region {timed_s:.3f} s, power cap {'active' if capped else 'not seen'})"
                       + ("; halved for tf32" if w.dtype == DType.F32 else ""),
        "frac_of_burst": achieved / (peaks["bf16_tflops"] * scale),
        "avg_launch_ms": ms_local / max(1, launches) if launches else None,
        "frac_of_nominal_2250": achieved / ({DType.F32: 1125.0, DType.F8E4M3: 4500.0, DType.F8E5M2: 4500.0}.get(w.dtype, 2250.0)),
        "repeats": {"n": len(rep_ms), "steps_each": args.steps, "best_ms_per_step": rep_sorted[0] / args.steps,
                    "median_ms_per_step": rep_sorted[len(rep_sorted) // 2] / args.steps,
                    "best_tflops": flops_total * args.steps / (rep_sorted[0] * 1e-3) / 1e12,
                    "median_tflops": flops_total * args.steps / (rep_sorted[len(rep_sorted) // 2] * 1e-3) / 1e12},
        "sustained": sustained,
        "cold_l2_ms": cold_ms,
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
    if not args.no_e2e and w.result_dtype == w.dtype and world > 1:
        e_steps = max(2, min(args.steps, args.e2e_steps))
        e_ms, h2d, d2h = e2e_sharded(be, grp, w, work, tensors, host, e_steps)
        e2e = {"value": flops_total / (e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h), "steps": e_steps, "ms_per_step": e_ms,
               "note": "per-rank bytes; pinned host memory; each rank uploads its rows and 1/N of every operand it needs whole, "
                       "an NCCL all-gather completes those in each GPU's own memory, oxm_batched_matmul, oxm_d2h of the rank's rows"}
    elif not args.no_e2e and w.result_dtype == w.dtype:
        from oxmera_b200.backend import shard_ranges
        hwork, h2d, d2h = [], 0, 0
        for g, a, b, out in work:
            ha, hb = host[g.a], host[g.b]
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
                "sharding": f"rank 0's shard of a {sworld}-GPU run, alone on one GPU" if alone else "none" if world == 1 else f"{'batch' if len(w.gemm_shapes(w.gemms[0])[2]) > 2 else 'M-row blocks'} over {world} GPUs, no collective",
                "l2": "inputs + output exceed the 126 MB L2" if w.algorithmic_bytes() > 126e6 else "working set fits L2 (latency-bound config)",
                "accumulate": "fp32", "flops_per_step": flops_total, "algorithmic_bytes_per_step": w.algorithmic_bytes(),
            },
            "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e,
            "gpu_launches": counts1["total"] - counts0["total"],
            "shards_checked": True, "shard_check": {"ranks": world, "worst_checksum_error_over_budget": worst_check,
                                                    "what": "per rank, over its whole shard, float64 on the host: C.1 vs A.(B.1) and 1^T.C vs (1^T.A).B"},
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
    ap.add_argument("--tile-n", type=int, default=0, help="0 auto, else a multiple of 32 from 64 to 512")
    ap.add_argument("--shard-of", type=int, default=0, help="on one GPU: time only the shard rank 0 of an N-GPU run gets")
    ap.add_argument("--group-m", type=int, default=0)
    ap.add_argument("--repeats", type=int, default=5, help="times the --steps region is measured (the first one is `value`)")
    ap.add_argument("--sustained-s", type=float, default=2.2, help="length of the back-to-back leg in seconds (0: skip)")
    ap.add_argument("--no-cold-l2", dest="cold_l2", action="store_false")
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
