#!/usr/bin/env python
"""Benchmark of the dense-reduction path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2]

One "step" is one pass of the headline reduction over one synthetic matrix that is already
resident in HBM: by default config 2 of the baseline (squared-L2 row norms + sqrt of a
1,000,000 x 128 fp32 matrix, N(0,1)-like values from seed 1). With N > 1 (launched by torchrun,
one rank per GPU) every rank reduces its own 1,000,000-row shard - rows shard with no
communication - so per-GPU work is fixed ("weak" scaling) and `value` is the aggregate.

The single JSON line on stdout carries:
  value / unit        achieved HBM GB/s = algorithmic bytes (input read once + output written once)
                      of all ranks / device time (CUDA events, max over ranks)
  rows_per_s          rows reduced per second, all ranks
  roofline            per-launch achieved GB/s of the dominant kernel against the measured copy peak
  e2e                 the same metric through the public host-buffer call: pinned host input ->
                      device, kernel, result -> host, every step
  cpu_baseline        the OpenMP host implementation (oracle/) on a bounded sample, rank 0, N = 1
  configs             (N = 1) every baseline config measured the same way, with the reference's own
                      kernels (oracle/_ref) beside it when that library is present

`--impl reference` times the reference's own raft::linalg kernels (oracle/_ref/libraft_ref.so,
built from the reference headers for sm_100a) on the same workload with the same protocol; when
that library is absent it times the OpenMP host port of the path instead.
"""
import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

L2_BYTES = 126 * 1024 * 1024

# name -> (rows, cols, description)
WORKLOADS = {
    "c1": (4096, 1024, "row sum (coalesced_reduction, add) fp32 4096x1024 U[-1,1) seed 0"),
    "c2": (1_000_000, 128, "L2 row norm with sqrt (norm L2 ALONG_ROWS, sqrt_op) fp32 1000000x128 N(0,1) seed 1"),
    "c2sq": (1_000_000, 128, "squared L2 row norm (norm L2 ALONG_ROWS) fp32 1000000x128 N(0,1) seed 1"),
    "c3": (16_777_216, 64, "column sum (strided_reduction, add) fp32 16777216x64 U[0,1) seed 2"),
    "c3mean": (16_777_216, 64, "column mean (strided_reduction, div_const n_rows) fp32 16777216x64 U[0,1) seed 2"),
    "c4": (8_388_608, 64, "row argmin KeyValuePair<int,float> fp32 8388608x64 U{0..15} seed 3"),
    "c5": (10_000_000, 128, "reduce_rows_by_key fp32 10000000x128 N(0,1) seed 4, int32 keys U[0,1024) seed 5"),
    # the callers next to the path (not baseline configs; never the default workload)
    "normalize": (100_000, 1024, "row_normalize L2 fp32 100000x1024 U[-10,10) seed 6 (read + write)"),
    "mapsum": (1_048_576, 1024, "mapThenSumReduce identity fp32, 2^30 elements U[-1,1) seed 7"),
    "colsbykey": (2_000, 200_000, "reduce_cols_by_key fp32 2000x200000 U[-1,1) seed 8, int32 keys U[0,128) seed 9"),
    "oddrows": (8_000_000, 31, "row sum of rows off 16-byte boundaries fp32 8000000x31 U[-1,1) seed 10"),
    "normalize100": (2_500_000, 100, "row_normalize L2 fp32 2500000x100 (25 vectors per row) U[-10,10) seed 12 (read + write)"),
    "norm96": (2_500_000, 96, "L2 row norm with sqrt fp32 2500000x96 (24 vectors per row: no power of two) N(0,1) seed 11"),
}
COL_NKEYS = 128
NKEYS = 1024


def algorithmic_bytes(name):
    rows, cols, _ = WORKLOADS[name]
    inp = rows * cols * 4
    if name in ("c1", "c2", "c2sq", "oddrows", "norm96"):
        return inp + rows * 4
    if name in ("c3", "c3mean"):
        return inp + cols * 4
    if name == "c4":
        return inp + rows * 8
    if name == "c5":
        return inp + rows * 4 + NKEYS * cols * 4 + NKEYS * 8
    if name in ("normalize", "normalize100"):
        return 2 * inp
    if name == "mapsum":
        return inp + 4
    if name == "colsbykey":
        return inp + cols * 4 + rows * COL_NKEYS * 4
    raise KeyError(name)


def launches_per_step(name):
    return {"c1": 1, "c2": 1, "c2sq": 1, "c3": 2, "c3mean": 2, "c4": 1, "c5": 6, "normalize": 1, "mapsum": 2, "colsbykey": 3,
            "oddrows": 1, "norm96": 1, "normalize100": 1}[name]


class Workload:
    """Device-resident inputs and outputs of one config, plus `run()` = one step."""

    def __init__(self, name, device, impl, first_row=0, world=1):
        import torch
        self.world = world
        from raft_b200 import _lib as L
        from raft_b200 import linalg
        self.name, self.impl, self.torch, self.linalg, self.L = name, impl, torch, linalg, L
        rows, cols, _ = WORKLOADS[name]
        self.rows, self.cols = rows, cols
        self.data = torch.empty((rows, cols), dtype=torch.float32, device=device)
        base = first_row * cols
        if name == "c1":
            linalg.synth_fill(self.data, 0, "uniform", -1, 1, first_index=base)
        elif name == "oddrows":
            linalg.synth_fill(self.data, 10, "uniform", -1, 1, first_index=base)
        elif name == "norm96":
            linalg.synth_fill(self.data, 11, "normal", first_index=base)
        elif name in ("c2", "c2sq"):
            linalg.synth_fill(self.data, 1, "normal", first_index=base)
        elif name in ("c3", "c3mean"):
            linalg.synth_fill(self.data, 2, "uniform", 0, 1, first_index=base)
        elif name == "c4":
            linalg.synth_fill(self.data, 3, "int", 0, 16, first_index=base)
        elif name == "c5":
            linalg.synth_fill(self.data, 4, "normal", first_index=base)
            self.keys = torch.empty((rows,), dtype=torch.int32, device=device)
            linalg.synth_fill(self.keys, 5, "int", 0, NKEYS, first_index=first_row)
        elif name == "normalize":
            linalg.synth_fill(self.data, 6, "uniform", -10, 10, first_index=base)
        elif name == "normalize100":
            linalg.synth_fill(self.data, 12, "uniform", -10, 10, first_index=base)
        elif name == "mapsum":
            linalg.synth_fill(self.data, 7, "uniform", -1, 1, first_index=base)
        elif name == "colsbykey":
            linalg.synth_fill(self.data, 8, "uniform", -1, 1, first_index=base)
            self.keys = torch.empty((cols,), dtype=torch.int32, device=device)
            linalg.synth_fill(self.keys, 9, "int", 0, COL_NKEYS)  # the columns are not sharded: same keys on every rank
        if name in ("c1", "c2", "c2sq", "oddrows", "norm96"):
            self.out = torch.empty(rows, dtype=torch.float32, device=device)
        elif name in ("c3", "c3mean"):
            self.out = torch.empty(cols, dtype=torch.float32, device=device)
        elif name == "c4":
            self.out = linalg.KeyValueVector(rows, torch.float32, device)
        elif name == "c5":
            self.out = torch.empty((NKEYS, cols), dtype=torch.float32, device=device)
            self.counts = torch.empty(NKEYS, dtype=torch.int64, device=device)
        elif name in ("normalize", "normalize100"):
            self.out = torch.zeros_like(self.data)
        elif name == "mapsum":
            self.out = torch.zeros(1, dtype=torch.float32, device=device)
        elif name == "colsbykey":
            self.out = torch.zeros((rows, COL_NKEYS), dtype=torch.float32, device=device)
        # scratch allocated once, outside the timed region (a caller-provided workspace)
        self.ws = None
        if impl == "ours":
            need = 0
            if name in ("c3", "c3mean"):
                need = linalg.reduce_workspace_bytes(self.data, linalg.ALONG_COLUMNS)
            elif name == "c5":
                need = linalg.reduce_rows_by_key_workspace_bytes(self.data, NKEYS)
            elif name == "mapsum":
                need = linalg.reduce_workspace_bytes(self.data.reshape(1, -1))
            if need:
                self.ws = torch.empty(need, dtype=torch.uint8, device=device)
        else:
            from oracle import ref
            self.ref = ref
            ref.load()
        torch.cuda.synchronize(device)

    def run(self, data=None, keys=None):
        data = self.data if data is None else data
        la, L, n = self.linalg, self.L, self.name
        if self.impl == "ours":
            if n in ("c1", "oddrows"):
                la.coalesced_reduction(data, self.out)
            elif n in ("c2", "norm96"):
                la.norm(data, "L2", la.ALONG_ROWS, self.out, fin_op="sqrt")
            elif n == "c2sq":
                la.norm(data, "L2", la.ALONG_ROWS, self.out)
            elif n in ("c3", "c3mean") and self.world > 1:
                # row-sharded: raw partial per GPU, NCCL all-reduce of 64 floats, then final_op
                import torch.distributed as dist
                la.reduce(data, la.ALONG_COLUMNS, self.out, workspace=self.ws)
                dist.all_reduce(self.out)
                if n == "c3mean":
                    la.apply_final(self.out, "div_const", float(self.rows * self.world))
            elif n == "c3":
                la.reduce(data, la.ALONG_COLUMNS, self.out, workspace=self.ws)
            elif n == "c3mean":
                la.reduce(data, la.ALONG_COLUMNS, self.out, final_op="div_const", final_scalar=float(self.rows),
                          workspace=self.ws)
            elif n == "c4":
                la.reduce(data, la.ALONG_ROWS, self.out, init=float("inf"), main_op="to_kvp", reduce_op="argmin")
            elif n == "c5":
                la.reduce_rows_by_key(data, self.keys if keys is None else keys, NKEYS, d_sums=self.out,
                                      counts=self.counts, workspace=self.ws)
                if self.world > 1:
                    import torch.distributed as dist
                    dist.all_reduce(self.out)     # 1024 x 128 fp32 partial tables
                    dist.all_reduce(self.counts)  # 1024 int64 counts
            elif n in ("normalize", "normalize100"):
                la.row_normalize(data, "L2", out=self.out)
            elif n == "colsbykey":
                la.reduce_cols_by_key(data, self.keys, out=self.out)
            elif n == "mapsum":
                la.map_reduce(data, out=self.out, workspace=self.ws)
                if self.world > 1:
                    import torch.distributed as dist
                    dist.all_reduce(self.out)
        else:
            r = self.ref
            st = 0
            if n in ("c1", "oddrows"):
                st = r.reduce(data, L.ALONG_ROWS, self.out)
            elif n in ("c2", "norm96"):
                st = r.reduce(data, L.ALONG_ROWS, self.out, main_op=L.MAIN_SQ, final_op=L.FINAL_SQRT)
            elif n == "c2sq":
                st = r.reduce(data, L.ALONG_ROWS, self.out, main_op=L.MAIN_SQ)
            elif n == "c3":
                st = r.reduce(data, L.ALONG_COLUMNS, self.out)
            elif n == "c3mean":
                st = r.reduce(data, L.ALONG_COLUMNS, self.out, final_op=L.FINAL_DIV_CONST,
                              final_scalar=float(self.rows))
            elif n == "c4":
                st = r.reduce(data, L.ALONG_ROWS, self.out, main_op=L.MAIN_TO_KVP, reduce_op=L.REDUCE_ARGMIN,
                              init=float("inf"))
            elif n == "c5":
                st = r.rows_by_key(self.out, data, self.keys if keys is None else keys, NKEYS)
            elif n in ("normalize", "normalize100"):
                st = r.row_normalize(self.out, data, "L2")
            elif n == "mapsum":
                st = r.map_then_sum_reduce(self.out, data)
            elif n == "colsbykey":
                st = r.cols_by_key(self.out, data, self.keys, COL_NKEYS)
            if st != 0:
                raise RuntimeError(f"reference wrapper status {st} for {n}")

    def result_tensor(self):
        return self.out.raw if self.name == "c4" else self.out

    def flush_l2(self):
        """Overwrites a buffer larger than L2 so that the next step starts from a cold L2
        (only needed when the input itself is smaller than L2, i.e. c1)."""
        if not hasattr(self, "_flush"):
            self._flush = self.torch.empty(3 * L2_BYTES // 4, dtype=self.torch.float32, device=self.data.device)
        self._flush.fill_(1.0)


def time_steps(w, steps, warmup, flush):
    """Per-step device times in ms (CUDA events on the launching stream)."""
    torch = w.torch
    for _ in range(warmup):
        if flush:
            w.flush_l2()
        w.run()
    torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for a, b in evs:
        if flush:
            w.flush_l2()
        a.record()
        w.run()
        b.record()
    torch.cuda.synchronize()
    return [a.elapsed_time(b) for a, b in evs]


class ClockSampler(threading.Thread):
    """Samples SM clocks and throttle reasons through NVML (read-only queries) every few
    milliseconds while the timed region runs."""

    def __init__(self, index, period_s=0.002):
        super().__init__(daemon=True)
        self.index, self.period, self.samples, self._stop_evt = index, period_s, [], threading.Event()
        self.max_mhz, self.ok = None, False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def _sample(self):
        nv = self.nv
        mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
        try:
            reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
        except Exception:
            reasons = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
        self.samples.append((mhz, reasons))

    def run(self):
        if not self.ok:
            return
        while not self._stop_evt.is_set():
            try:
                self._sample()
            except Exception:
                break
            time.sleep(self.period)

    def stop(self):
        if self.ok:
            try:
                self._sample()  # at least one sample taken before the closing synchronize returns
            except Exception:
                pass
        self._stop_evt.set()
        if self.is_alive():
            self.join(timeout=2)

    def summary(self):
        if not self.ok or not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        nv = self.nv
        bits = {"hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
                "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4)}
        mhz = sorted(m for m, _ in self.samples)
        seen = set()
        for _, r in self.samples:
            for name, bit in bits.items():
                if r & bit:
                    seen.add(name)
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(seen),
                "samples": len(mhz)}


def cpu_baseline(name, budget_rows=None):
    """OpenMP host implementation of the same reduction on a bounded sample of the workload."""
    import numpy as np
    from oracle import oracle as o
    rows, cols, _ = WORKLOADS[name]
    sample_rows = min(rows, budget_rows or {"c1": 4096, "c2": 1_000_000, "c2sq": 1_000_000, "c3": 2_000_000,
                                            "c3mean": 2_000_000, "c4": 2_000_000, "c5": 1_000_000,
                                            "normalize": 100_000, "mapsum": 262_144, "colsbykey": 500,
                                            "oddrows": 4_000_000, "norm96": 1_250_000,
                                            "normalize100": 1_000_000}[name])
    seed, kind, lo, hi = {"c1": (0, "uniform", -1, 1), "c2": (1, "normal", 0, 1), "c2sq": (1, "normal", 0, 1),
                          "c3": (2, "uniform", 0, 1), "c3mean": (2, "uniform", 0, 1), "c4": (3, "int", 0, 16),
                          "c5": (4, "normal", 0, 1), "normalize": (6, "uniform", -10, 10),
                          "mapsum": (7, "uniform", -1, 1), "colsbykey": (8, "uniform", -1, 1),
                          "oddrows": (10, "uniform", -1, 1), "norm96": (11, "normal", 0, 1),
                          "normalize100": (12, "uniform", -10, 10)}[name]
    data = o.synth((sample_rows, cols), np.float32, seed, kind, lo, hi)
    keys = o.synth((sample_rows,), np.int32, 5, "int", 0, NKEYS) if name == "c5" else None
    ckeys = o.synth((cols,), np.int32, 9, "int", 0, COL_NKEYS) if name == "colsbykey" else None

    def once():
        if name in ("c1", "oddrows"):
            o.omp_row_sum(data)
        elif name in ("c2", "norm96"):
            o.omp_row_sum(data, square=True, root=True)
        elif name == "c2sq":
            o.omp_row_sum(data, square=True)
        elif name in ("c3", "c3mean"):
            o.omp_col_sum(data, 1.0 / sample_rows if name == "c3mean" else 1.0)
        elif name == "c4":
            o.omp_row_argmin(data)
        elif name == "c5":
            o.omp_rows_by_key(data, keys, NKEYS)
        elif name in ("normalize", "normalize100"):
            o.row_normalize(data, "L2")
        elif name == "mapsum":
            float(o.omp_row_sum(data).astype(np.float64).sum())  # rows in parallel, then the row sums
        elif name == "colsbykey":
            o.cols_by_key(data, ckeys, COL_NKEYS)

    once()
    reps, t0 = 0, time.perf_counter()
    while True:
        once()
        reps += 1
        dt = time.perf_counter() - t0
        if dt > 3.0 or reps >= 50:
            break
    per = dt / reps
    bytes_sample = algorithmic_bytes(name) * sample_rows / rows
    return {"value": bytes_sample / per / 1e9, "unit": "GB/s", "cores": o.omp_threads(), "kind": "port",
            "sample": f"{sample_rows} of {rows} rows x {cols}, {reps} passes, OpenMP fp32-load/fp64-accumulate "
                      f"(oracle/oracle.c omp_*)", "rows_per_s": sample_rows / per}


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


# dram bytes per launch of the dominant kernel from the committed ncu summaries (profiles/), or None
NCU_TRAFFIC = {}
try:
    NCU_TRAFFIC = json.load(open(os.path.join(ROOT, "profiles", "traffic.json")))
except Exception:
    pass


def e2e_measure(w, steps):
    """Host-buffer path: pinned host input -> device, the reduction, result -> host, per step."""
    torch = w.torch
    dev = w.data.device
    host_in = torch.empty(w.data.shape, dtype=w.data.dtype, pin_memory=True)
    host_in.copy_(w.data)
    dev_in = torch.empty_like(w.data)
    res = w.result_tensor()
    host_out = torch.empty(res.shape, dtype=res.dtype, pin_memory=True)
    keys_h = keys_d = None
    if w.name == "c5":
        keys_h = torch.empty(w.keys.shape, dtype=w.keys.dtype, pin_memory=True)
        keys_h.copy_(w.keys)
        keys_d = torch.empty_like(w.keys)
    h2d = host_in.numel() * 4 + (keys_h.numel() * 4 if keys_h is not None else 0)
    d2h = host_out.numel() * host_out.element_size()

    def step():
        dev_in.copy_(host_in, non_blocking=True)
        if keys_h is not None:
            keys_d.copy_(keys_h, non_blocking=True)
        w.run(dev_in, keys_d)
        host_out.copy_(res, non_blocking=True)

    step()
    torch.cuda.synchronize(dev)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        step()
    b.record()
    torch.cuda.synchronize(dev)
    ms = a.elapsed_time(b) / steps
    return ms, h2d, d2h


_REAL_STDOUT = None


def _claim_stdout():
    """Everything any library prints to stdout from here on (NCCL prints its version line there)
    goes to stderr; the one JSON line is written to the real stdout by emit()."""
    global _REAL_STDOUT
    if _REAL_STDOUT is None:
        sys.stdout.flush()
        _REAL_STDOUT = os.dup(1)
        os.dup2(2, 1)


def emit(line):
    data = (json.dumps(line) + "\n").encode()
    sys.stdout.flush()
    if _REAL_STDOUT is not None:
        os.write(_REAL_STDOUT, data)
    else:
        os.write(1, data)


def main():
    _claim_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=500)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="c2")
    ap.add_argument("--no-configs", action="store_true", help="skip the per-config table (N = 1 only)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg")
    ap.add_argument("--rows", type=int, default=0,
                    help="override the row count of the workload (small cases for profiler captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    name = args.workload
    if args.rows > 0:
        r0, c0, d0 = WORKLOADS[name]
        WORKLOADS[name] = (args.rows, c0, d0 + f" [rows overridden: {args.rows}]")
    rows, cols, desc = WORKLOADS[name]

    # ---- reference arm without its library: the OpenMP host port, rank 0 only ----------------
    ref_lib = os.path.join(ROOT, "oracle", "_ref", "libraft_ref.so")
    if args.impl == "reference" and not os.path.exists(ref_lib):
        if rank != 0:
            return
        cb = cpu_baseline(name)
        line = {"impl": "reference", "metric": "hbm_gb_per_s", "value": cb["value"], "unit": "GB/s",
                "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": None,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": desc, "note": "oracle/_ref not built: OpenMP host port of the path"},
                "cpu_baseline": cb, "rows_per_s": cb["rows_per_s"],
                "e2e": {"value": cb["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        emit(line)
        return

    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if world > 1:
            dist.barrier(device_ids=[local_rank])
        torch.cuda.synchronize(device)

    from raft_b200 import _lib
    _lib.load()  # fail loudly if the extension is missing
    w = Workload(name, device, args.impl, first_row=rank * rows, world=world)
    flush = rows * cols * 4 <= L2_BYTES
    alg = algorithmic_bytes(name)

    sampler = ClockSampler(local_rank) if rank == 0 else None
    # warm-up, then EXACTLY `steps` timed steps between two barriers
    for _ in range(args.warmup):
        if flush:
            w.flush_l2()
        w.run()
    barrier()
    if sampler:
        sampler.start()
        time.sleep(0.01)  # let the sampler take its first reading before the launches start
    t_wall0 = time.perf_counter()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    per = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    start.record()
    for a, b in per:
        if flush:
            w.flush_l2()
        a.record()
        w.run()
        b.record()
    end.record()
    barrier()
    t_wall = time.perf_counter() - t_wall0
    if sampler:
        sampler.stop()
    step_ms = [a.elapsed_time(b) for a, b in per]
    total_ms = sum(step_ms) if flush else start.elapsed_time(end)  # the flush writes are not part of a step
    t = torch.tensor([total_ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms = t.item()
    ms_per_step = total_ms / args.steps
    value = alg * world / (ms_per_step * 1e-3) / 1e9
    rows_per_s = rows * world / (ms_per_step * 1e-3)

    # ---- end to end through host buffers -------------------------------------------------------
    e2e_steps = max(2, min(args.steps, 10))
    e_ms, h2d, d2h = e2e_measure(w, e2e_steps) if not args.no_e2e else (float("nan"), 0, 0)
    te = torch.tensor([e_ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e = {"value": alg * world / (te.item() * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d,
           "d2h_bytes_per_step": d2h, "ms_per_step": te.item(), "steps": e2e_steps}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_kind = measured_peak()
    best_ms = min(step_ms)
    avg_ms = sum(step_ms) / len(step_ms)
    roof = {"bound": "hbm", "achieved": alg / (avg_ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
            "frac": alg / (avg_ms * 1e-3) / 1e9 / peak, "peak_kind": peak_kind + " copy bandwidth",
            "traffic": NCU_TRAFFIC.get(name if args.impl == "ours" else "ref_" + name),
            "algorithmic_bytes": alg, "best_launch_gbs": alg / (best_ms * 1e-3) / 1e9,
            "frac_of_nominal_8000": alg / (avg_ms * 1e-3) / 1e9 / 8000.0}
    line = {"metric": "hbm_gb_per_s", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": desc, "rows_per_gpu": rows, "cols": cols, "sharding": f"rows x{world}, " + ("no collective" if name in ("c1", "c2", "c2sq", "c4", "normalize", "colsbykey", "oddrows", "norm96", "normalize100") or world == 1
                                                        else "per-GPU partials + NCCL all-reduce inside the step"),
                       "l2": "L2 flushed by a 378 MB write before every step" if flush
                       else f"input {rows * cols * 4 >> 20} MB per GPU > 126 MB L2"},
            "rows_per_s": rows_per_s, "roofline": roof, "e2e": e2e,
            "gpu_launches": args.steps * launches_per_step(name) if args.impl == "ours" else 0,
            "clocks": sampler.summary() if sampler else None, "wall_s": t_wall}
    if args.impl == "reference":
        line["impl"] = "reference"
        line["config"]["note"] = "reference raft::linalg kernels compiled for sm_100a (oracle/_ref), same protocol"
        line["cpu_baseline"] = {"value": value, "unit": "GB/s", "cores": 0, "kind": "reference",
                                "sample": "full workload on the GPU: the reference has no CPU implementation of "
                                          "this path, its CUDA kernels are what is timed"}
    elif world == 1 and not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline(name)

    # ---- every baseline config, same protocol (N = 1) -----------------------------------------
    if world == 1 and not args.no_configs:
        table = {}
        del w
        torch.cuda.empty_cache()
        for cn in ("c1", "c2sq", "c2", "c3", "c3mean", "c4", "c5", "normalize", "mapsum", "colsbykey", "oddrows", "norm96", "normalize100"):
            r, c, _ = WORKLOADS[cn]
            ent = {}
            for impl in ("ours", "reference"):
                if impl == "reference" and not os.path.exists(ref_lib):
                    continue
                if impl == args.impl and cn == name:
                    ent[impl] = {"gbs": roof["achieved"], "best_gbs": roof["best_launch_gbs"],
                                 "rows_per_s": r / (avg_ms * 1e-3), "frac_measured": roof["frac"]}
                    continue
                try:
                    ww = Workload(cn, device, impl)
                    ms = time_steps(ww, 20, 3, r * c * 4 <= L2_BYTES)
                    a_ms = sum(ms) / len(ms)
                    g = algorithmic_bytes(cn) / (a_ms * 1e-3) / 1e9
                    ent[impl] = {"gbs": g, "best_gbs": algorithmic_bytes(cn) / (min(ms) * 1e-3) / 1e9,
                                 "rows_per_s": r / (a_ms * 1e-3), "frac_measured": g / peak}
                    del ww
                    torch.cuda.empty_cache()
                except Exception as ex:  # a config failing must not lose the headline line
                    ent[impl] = {"error": str(ex)[:200]}
            table[cn] = ent
        line["configs"] = table
    emit(line)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
