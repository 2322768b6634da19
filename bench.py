#!/usr/bin/env python
"""Benchmark of the SBMM hot path on the Llama-2-7B projection shapes.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (the SBMM microbenchmark configuration): the four delta linears of a
Llama-2-7B decoder layer -- qkv 12288x4096, o 4096x4096, gate_up 22016x4096,
down 4096x11008 -- for all 32 layers, fp16 base ~ N(0, 0.02), 8 resident deltas
(4-bit, 2:4, symmetric, per-channel scale, delta ~ N(0, 1e-3)), a decode batch of
64 tokens whose slot ids are uniform over the 8 deltas (sorted, as the
scheduler delivers them).  One step = one decode pass through all 128 SBMM
calls; the weights of a step (32 GB) are far larger than L2, so every step
streams them from HBM.  Data are seeded and synthetic.

N > 1: tensor parallel over N ranks (column-parallel qkv / gate_up, row-parallel
o / down followed by an NCCL all-reduce), shards cut at whole 128-row tiles and
64-column blocks; the total work is fixed ("strong" scaling).

One JSON line is printed by rank 0.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

HIDDEN, INTER, LAYERS = 4096, 11008, 32
NUM_DELTAS, BITS, TOKENS = 8, 4, 64
METRIC = "sbmm_decode_tokens_per_s"
UNIT = "tok/s"


def projections(tp: int, rank: int):
    """(name, N, K, row_parallel) per rank; shards are whole 128-row tiles / 64-col blocks."""
    def split(total, unit):
        units = total // unit
        lo = units * rank // tp
        hi = units * (rank + 1) // tp
        return (hi - lo) * unit
    qkv = 3 * split(HIDDEN, 128)
    gate_up = 2 * split(INTER, 128)
    return [("qkv_proj", qkv, HIDDEN, False),
            ("o_proj", HIDDEN, split(HIDDEN, 64), True),
            ("gate_up_proj", gate_up, HIDDEN, False),
            ("down_proj", HIDDEN, split(INTER, 64), True)]


def algorithmic_bytes(m, n, k, active, bits):
    """Bytes one SBMM call must move: base fp16 once, each active delta's codes
    (bits/16 B per dense element) + 2:4 metadata (1/8 B) + scales, x and y."""
    cb = bits / 16.0 + 1.0 / 8.0
    return 2.0 * n * k + active * (cb * n * k + 2.0 * n) + 2.0 * m * k + 2.0 * m * n


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows = []
        self.proc = None
        self.gpu_index = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-i", str(self.gpu_index), "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), line.strip()))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, smax, reasons = [], None, set()
        for ts, line in self.rows:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                smax = float(parts[2])
                if t0 <= ts <= t1 + 0.1:
                    sm.append(float(parts[1]))
            except ValueError:
                continue
            if t0 <= ts <= t1 + 0.1:
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                      "sw_power_cap"), parts[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": smax,
                "samples": len(sm), "reasons": sorted(reasons)}


def build_model(tp, rank, device, seed=0, num_layers=LAYERS):
    """Per layer and projection: base weight, slot stacks.  Deltas are generated and
    compressed once per projection shape and replicated (device copies) per layer."""
    import torch
    from deltazip_b200 import synth
    projs = projections(tp, rank)
    gen = torch.Generator(device=device).manual_seed(seed + 17 * rank)
    proto = {}
    for i, (name, n, k, _) in enumerate(projs):
        proto[name] = synth.random_delta_slots(NUM_DELTAS, n, k, BITS, seed=seed + 100 * i + rank,
                                               device=device)
    layers = []
    for layer in range(num_layers):
        entry = {}
        for name, n, k, rowp in projs:
            w = torch.empty((n, k), dtype=torch.float16, device=device)
            w.normal_(0.0, 0.02, generator=gen)
            qs, ms, ss = proto[name]
            if layer > 0:
                qs, ms, ss = qs.clone(), ms.clone(), ss.clone()
            entry[name] = dict(w=w, q=qs, m=ms, s=ss, n=n, k=k, row_parallel=rowp)
        layers.append(entry)
    return projs, layers


def run_ours(args):
    import torch
    import torch.distributed as dist
    from deltazip_b200 import _lib, ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus > 1 and world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks (WORLD_SIZE={world})")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    car = None
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
        if args.allreduce == "custom":
            # the library's peer-memory all-reduce for the row-parallel outputs
            from deltazip_b200 import custom_all_reduce
            car = custom_all_reduce.init_custom_ar(rank, world)
    tp = world
    L = _lib.lib()

    projs, layers = build_model(tp, rank, device, num_layers=args.layers)
    g = torch.Generator(device="cpu").manual_seed(1234)
    idx_host = torch.sort(torch.randint(0, NUM_DELTAS, (TOKENS,), generator=g))[0].to(torch.int64)
    active = len(set(idx_host.tolist()))
    x_host = {k: torch.randn((TOKENS, k), generator=g).half().pin_memory()
              for k in sorted({p[2] for p in projs})}
    idx_pinned = idx_host.pin_memory()
    x_dev = {k: v.to(device) for k, v in x_host.items()}
    y_dev = {n: torch.empty((TOKENS, n), dtype=torch.float16, device=device)
             for n in sorted({p[1] for p in projs})}
    y_host = torch.empty((TOKENS, HIDDEN), dtype=torch.float16).pin_memory()
    idx_dev = idx_host.to(device)
    seg = ops.Segments(TOKENS, NUM_DELTAS, device).build(idx_dev, sorted_hint=True)

    ws_bytes = max(L.dz_sbmm_workspace_bytes(TOKENS, n, k, 1) for _, n, k, _ in projs)
    ws = torch.zeros(ws_bytes, dtype=torch.uint8, device=device)
    stream = torch.cuda.current_stream().cuda_stream

    # one prebuilt argument block per (layer, projection): the timed loop is C-ABI calls only
    calls = []
    step_bytes = 0.0
    for entry in layers:
        for name, n, k, rowp in projs:
            e = entry[name]
            a = _lib.SbmmArgs(
                x=x_dev[k].data_ptr(), w_base=e["w"].data_ptr(), qweight=e["q"].data_ptr(),
                meta=e["m"].data_ptr(), scales=e["s"].data_ptr(),
                qweight_stride=e["q"].stride(0) * 4, meta_stride=e["m"].stride(0) * 2,
                scales_stride=e["s"].stride(0) * 2, segments=seg.buf.data_ptr(),
                y=y_dev[n].data_ptr(), M=TOKENS, N=n, K=k, num_slots=NUM_DELTAS, bits=BITS,
                dtype=_lib.DZ_DTYPE_F16, tokens_sorted=1, workspace=ws.data_ptr(),
                workspace_bytes=ws.numel())
            calls.append((a, rowp, y_dev[n]))
            step_bytes += algorithmic_bytes(TOKENS, n, k, active, BITS)

    stage_ptr, stage_len = ctypes.c_void_p(), ctypes.c_size_t()

    def step_device():
        n_launch = 0
        for a, rowp, y in calls:
            reduce = rowp and tp > 1
            if reduce and car is not None:
                # the SBMM writes its partial output straight into the staging buffer of the
                # all-reduce that follows (buffers alternate from call to call)
                L.dz_allreduce_staging(car._ctx, ctypes.byref(stage_ptr), ctypes.byref(stage_len))
                a.y = stage_ptr.value
            rc = L.dz_sbmm(ctypes.byref(a), stream)
            if rc:
                _lib.check(rc, "dz_sbmm")
            n_launch += 1
            if reduce:
                if car is not None:
                    rc = L.dz_allreduce_run(car._ctx, stage_ptr, y.data_ptr(), y.numel(),
                                            _lib.DZ_DTYPE_F16, stream)
                    if rc:
                        _lib.check(rc, "dz_allreduce_run")
                    n_launch += 1
                else:
                    dist.all_reduce(y)
        return n_launch

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    # ---- device-resident timing (value) ----
    for _ in range(args.warmup):
        step_device()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_wall0 = time.time()
    ev0.record()
    launches = 0
    for _ in range(args.steps):
        launches += step_device()
    ev1.record()
    barrier()
    t_wall1 = time.time()
    ms_total = ev0.elapsed_time(ev1)
    status = ops_read_status(L, ws, stream)

    # ---- kernel-only time for the roofline: same launches, no collectives ----
    kev0, kev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    kev0.record()
    for a, _, y in calls:
        a.y = y.data_ptr()
        L.dz_sbmm(ctypes.byref(a), stream)
    kev1.record()
    torch.cuda.synchronize()
    kernel_ms = kev0.elapsed_time(kev1)

    # ---- end to end through the public API: host buffers in, host result out ----
    def step_e2e():
        xd = {k: v.to(device, non_blocking=True) for k, v in x_host.items()}
        idx = idx_pinned.to(device, non_blocking=True)
        seg.build(idx, sorted_hint=True)
        y = None
        for entry in layers:
            for name, n, k, rowp in projs:
                e = entry[name]
                reduce = rowp and tp > 1
                out = car.staging_like((TOKENS, n), torch.float16) if (reduce and car) else y_dev[n]
                y = ops.sbmm(xd[k], e["q"], e["s"], e["m"], seg, e["w"], out=out, bits=BITS)
                if reduce:
                    if car is not None:
                        y = car.all_reduce(y, out=y_dev[n])
                    else:
                        dist.all_reduce(y)
        y_host.copy_(y, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(max(1, min(args.warmup, 3))):
        step_e2e()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step_e2e()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    clocks = sampler.stop(t_wall0, time.time()) if rank == 0 else None

    # max over ranks
    times = torch.tensor([ms_total, e2e_ms, kernel_ms], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_total, e2e_ms, kernel_ms = times.tolist()

    if rank == 0:
        ms_per_step = ms_total / args.steps
        peaks = measured_peaks()
        achieved = step_bytes / (kernel_ms * 1e-3) / 1e9
        n_calls = len(calls)
        line = {
            "metric": METRIC, "value": TOKENS / (ms_per_step * 1e-3), "unit": UNIT,
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {
                "workload": "configs[1]: SBMM over Llama-2-7B projection shapes (qkv 12288x4096, "
                            "o 4096x4096, gate_up 22016x4096, down 4096x11008) x %d layers, " % args.layers +
                            "8 deltas 4-bit 2:4 sym per-channel, 64-token decode batch, slot ids "
                            "uniform over 8 (sorted)",
                "tokens": TOKENS, "deltas": NUM_DELTAS, "active_deltas": active, "bits": BITS,
                "layers": args.layers, "sbmm_calls_per_step": n_calls,
                "parallelism": f"tp{world}",
                "allreduce": ("peer-memory one-shot (dz_allreduce_run)" if car is not None
                              else ("nccl" if world > 1 else "none")),
                "l2": "inputs larger than L2: each step streams %.1f GB of distinct weights"
                      % (step_bytes * 1e-9),
            },
            "e2e": {"value": TOKENS / (e2e_ms / args.steps * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": int(sum(v.numel() * 2 for v in x_host.values()) + TOKENS * 8),
                    "d2h_bytes_per_step": int(y_host.numel() * 2),
                    "ms_per_step": e2e_ms / args.steps},
            "gpu_launches": launches,
            "roofline": {
                "bound": "hbm", "kernel": "sbmm_tc_kernel<4>",
                "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "peak_source": peaks["source"],
                "algorithmic_bytes_per_launch": step_bytes / n_calls,
                "avg_launch_us": kernel_ms * 1e3 / n_calls,
                "traffic": ncu_traffic_per_launch(step_bytes / n_calls),
            },
            "clocks": clocks,
            "kernel_status": status,
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(budget_s=20.0)
        print(json.dumps(line), flush=True)
    if world > 1:
        if car is not None:
            st = car.status()
            if st:
                raise SystemExit(f"peer-memory all-reduce reported status {st}")
            from deltazip_b200 import custom_all_reduce
            custom_all_reduce.destroy_custom_ar()
        dist.destroy_process_group()


def ops_read_status(L, ws, stream):
    host = ctypes.c_int(0)
    L.dz_read_status(ws.data_ptr(), stream, ctypes.byref(host))
    return host.value


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            return {"hbm_gbs": float(json.load(fh)["hbm_gbs"]), "source": "measured (MEASURED_PEAKS.json)"}
    except (OSError, KeyError, ValueError):
        return {"hbm_gbs": 6650.0, "source": "fallback (6.65 TB/s)"}


def ncu_traffic_per_launch(alg_bytes_per_launch):
    """DRAM bytes per launch from the committed ncu summary (profiles/), scaled to the
    benchmark's average launch by algorithmic bytes; None when no capture is recorded."""
    path = os.path.join(ROOT, "profiles", "sbmm_tc_traffic.json")
    try:
        with open(path) as fh:
            rec = json.load(fh)
        return rec["dram_bytes_per_launch"] / rec["algorithmic_bytes_per_launch"] * alg_bytes_per_launch
    except (OSError, KeyError, ValueError, ZeroDivisionError):
        return None


# ---------------------------------------------------------------------------
# CPU arm: the oracle's torch-CPU port of the reference path, on the host cores
# ---------------------------------------------------------------------------

def cpu_sample(threads):
    """One o_proj-shaped call (4096x4096, 8 deltas, 64 tokens) of the reference's CPU path."""
    import torch
    from oracle import torch_port as T
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(7)
    n = k = HIDDEN
    w = (torch.randn((n, k), generator=g) * 0.02).half()
    x = torch.randn((TOKENS, k), generator=g).half()
    idx = torch.sort(torch.randint(0, NUM_DELTAS, (TOKENS,), generator=g))[0]
    # one packed delta reused for every slot: the CPU time does not depend on the values
    per = 32 // BITS
    qweight = torch.randint(-2 ** 31, 2 ** 31 - 1, (k // per, n), generator=g, dtype=torch.int64).to(torch.int32)
    qzeros = torch.full((1, n // per), 0x77777777, dtype=torch.int32)
    scales = (torch.rand((1, n), generator=g) * 1e-3 + 1e-4).half()
    deltas = [(qweight, qzeros, scales, BITS)] * NUM_DELTAS
    return lambda: T.apply_delta(x, w, deltas, idx, dequant_every_call=True)


def layer_scale_factor():
    """How many 4096x4096 calls one full decode step is worth, by weight count."""
    per_layer = sum(n * k for _, n, k, _ in projections(1, 0))
    return LAYERS * per_layer / float(HIDDEN * HIDDEN)


def cpu_baseline(budget_s=20.0):
    import torch
    threads = os.cpu_count() or 1
    fn = cpu_sample(threads)
    fn()
    t0 = time.perf_counter()
    reps = 0
    while True:
        fn()
        reps += 1
        if time.perf_counter() - t0 > budget_s or reps >= 50:
            break
    per_call = (time.perf_counter() - t0) / reps
    step_s = per_call * layer_scale_factor()
    return {"value": TOKENS / step_s, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": "oracle/torch_port.apply_delta (dequantise every call, as the reference's "
                      "PyTorch path does) on one 4096x4096 layer, 8 deltas, 64 tokens, %d reps, "
                      "%.3f s per call; scaled by weight count (x%.1f) to the 128-call step"
                      % (reps, per_call, layer_scale_factor())}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    fn = cpu_sample(threads)
    for _ in range(min(args.warmup, 2)):
        fn()
    steps = max(1, min(args.steps, 10))
    t0 = time.perf_counter()
    for _ in range(steps):
        fn()
    per_call = (time.perf_counter() - t0) / steps
    step_s = per_call * layer_scale_factor()
    value = TOKENS / step_s
    sample = ("each step = one 4096x4096 SBMM (8 deltas, 64 tokens) through the oracle's torch-CPU "
              "port of the reference path, scaled by weight count (x%.1f) to the full 128-call "
              "decode step; %d timed steps" % (layer_scale_factor(), steps))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT,
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": steps, "warmup": min(args.warmup, 2),
        "ms_per_step": step_s * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": "configs[1]: SBMM over Llama-2-7B projection shapes x 32 layers, "
                               "8 deltas 4-bit 2:4, 64-token decode batch (CPU arm: bounded sample)",
                   "parallelism": "cpu"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=LAYERS,
                    help="decoder layers to instantiate (32 = the benchmark; fewer only for profiling captures)")
    ap.add_argument("--allreduce", default="custom", choices=["custom", "nccl"],
                    help="N>1: all-reduce after the row-parallel layers (library peer-memory kernel or NCCL)")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the timed CPU sample (profiling captures)")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
