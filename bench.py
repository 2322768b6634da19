#!/usr/bin/env python
"""Benchmarks of the SBMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config 2|3|4|5]

--config 2 (default, the headline): the SBMM microbenchmark configuration.  The four delta
linears of a Llama-2-7B decoder layer -- qkv 12288x4096, o 4096x4096, gate_up 22016x4096,
down 4096x11008 -- for all 32 layers, fp16 base ~ N(0, 0.02), 8 resident deltas (4-bit, 2:4,
symmetric, per-channel scale, delta ~ N(0, 1e-3)), a decode batch of 64 tokens whose slot ids
are uniform over the 8 deltas (sorted, as the scheduler delivers them).  One step = one decode
pass through all 128 SBMM calls; the weights of a step (32 GB) are far larger than L2, so every
step streams them from HBM.  Data are seeded and synthetic.

--config 3 / 4: full-model decode through deltazip_b200/engine.py: Llama-2-7B with 32 resident
2-bit deltas and 128 sequences; Llama-2-13B with 64 2-bit deltas, 256 sequences and a Zipf(1.5)
request-to-delta map, tensor parallel.  --config 5: Llama-2-70B, 16 4-bit deltas in pinned host
memory, 4 GPU slots, bursty arrivals, swap-in overlapped with decode (--duration seconds of
arrivals on a virtual clock).

N > 1: tensor parallel over N ranks (column-parallel qkv / gate_up, row-parallel o / down
followed by the library's peer-memory all-reduce), shards cut at whole 128-wide units; the total
work is fixed ("strong" scaling).

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


def projections(tp: int, rank: int, hidden: int = HIDDEN, inter: int = INTER):
    """(name, N, K, row_parallel) per rank.  Column- and row-parallel layers are cut at the same
    128-wide units, so that a producer's shard is its consumer's K range for every rank count."""
    def split(total):
        units = total // 128
        return (units * (rank + 1) // tp - units * rank // tp) * 128
    h, i = split(hidden), split(inter)
    return [("qkv_proj", 3 * h, hidden, False),
            ("o_proj", hidden, h, True),
            ("gate_up_proj", 2 * i, hidden, False),
            ("down_proj", hidden, i, True)]


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


def dist_env():
    return (int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")),
            int(os.environ.get("LOCAL_RANK", "0")))


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


def dense_reference(x, e, idx):
    """float32 y = x W^T + x dequant(delta_slot)^T from the unpacked slots (the unpack is
    pinned bit-exact to the reference's QuantLinear.unpack by the parity tests)."""
    import torch
    from deltazip_b200 import ops
    y = x.float() @ e["w"].float().t()
    for s in torch.unique(idx).tolist():
        if s < 0:
            continue
        rows = (idx == s).nonzero().flatten()
        dense = ops.unpack(e["q"][s], e["m"][s], e["s"][s], e["n"], e["k"], BITS)
        y[rows] += x[rows].float() @ dense.float().t()
    return y


def allreduce_selfcheck(car, rank, world, device):
    """Values of the peer-memory all-reduce against the rank-order float32 sum of the gathered
    inputs, bit for bit: several sizes and dtypes, the produce-in-staging path, and a run of
    back-to-back calls (the two staging buffers alternate).  Returns "ok" or what differed."""
    import torch
    import torch.distributed as dist

    def expected(x):
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x)
        acc = torch.zeros(x.shape, dtype=torch.float32, device=device)
        for p in parts:                      # rank order, fp32, one rounding: the kernel's rule
            acc += p.float()
        return acc.to(x.dtype)

    # every rank runs every call whatever it finds (the calls are collective); the first
    # difference is kept and the outcome is agreed on at the end
    bad = None
    g = torch.Generator(device=device).manual_seed(100 + rank)
    for variant in (1, 2):                   # the one-shot and the two-stage kernel, forced in turn
        car.set_variant(variant)
        for dtype in (torch.float16, torch.bfloat16, torch.float32):
            for numel in (8, 4096, 64 * 4096, 8 * 1237, 256 * 5120, 1 << 20):
                x = torch.randn(numel, generator=g, device=device).to(dtype)
                want = expected(x)
                got = car.all_reduce(x)
                if bad is None and not torch.equal(got, want):
                    bad = f"mismatch variant={variant} dtype={dtype} numel={numel}"
    if car.multicast:                        # in-switch reduction: one rounding of slack, ranks identical
        car.set_variant(3)
        for dtype, eps in ((torch.float16, 2.0 ** -10), (torch.bfloat16, 2.0 ** -7), (torch.float32, 2.0 ** -22)):
            for numel in (8, 64 * 4096, 8 * 1237, 256 * 5120):
                x = torch.randn(numel, generator=g, device=device).to(dtype)
                want = expected(x).float()
                got = car.all_reduce(x)
                outs = [torch.empty_like(got) for _ in range(world)]
                dist.all_gather(outs, got)
                same = all(torch.equal(o, outs[0]) for o in outs)
                close = bool(((got.float() - want).abs() <= eps * want.abs() + 1e-6 * world).all())
                if bad is None and not (same and close):
                    bad = f"in-switch mismatch dtype={dtype} numel={numel} same={same} close={close}"
    car.set_variant(0)                       # from here on: chosen by size and rank count
    for it in range(100):                    # produced directly in the staging buffer
        st = car.staging_like((TOKENS, HIDDEN), torch.float16)
        st.copy_(torch.randn((TOKENS, HIDDEN), generator=g, device=device).half())
        want = expected(st.clone())
        got = car.all_reduce(st)
        if bad is None and not torch.equal(got, want):
            bad = f"staging path mismatch at call {it}"
    torch.cuda.synchronize()
    st = car.status()
    if bad is None and st != 0:
        bad = f"status {st}"
    flag = torch.tensor([0 if bad is None else 1], device=device)
    dist.all_reduce(flag)
    if flag.item() == 0:
        return "ok"
    return bad if bad is not None else "mismatch on another rank"


def pick_allreduce_kernel(car, world, device):
    """Times the candidates for the benchmark's message ([64, 4096] fp16 produced in the staging
    buffer) and returns the variant every rank agrees is fastest: the one-shot kernel (1) or,
    where the regions have a multicast address, the in-switch kernel (3)."""
    import torch
    import torch.distributed as dist
    candidates = [1] + ([3] if car.multicast else [])
    if len(candidates) == 1:
        return 0
    out = torch.empty((TOKENS, HIDDEN), dtype=torch.float16, device=device)
    took = []
    for v in candidates:
        car.set_variant(v)
        for timed in (False, True):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            dist.barrier()
            e0.record()
            for _ in range(50):
                st = car.staging_like((TOKENS, HIDDEN), torch.float16)
                car.all_reduce(st, out=out)
            e1.record()
            torch.cuda.synchronize()
        took.append(e0.elapsed_time(e1))
    t = torch.tensor(took, device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    best = int(torch.argmin(t).item())
    return candidates[best]


def run_ours(args):
    import torch
    import torch.distributed as dist
    from deltazip_b200 import _lib, ops

    world, rank, local_rank = dist_env()
    if args.gpus > 1 and world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks (WORLD_SIZE={world})")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    car = None
    ar_check = None
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
        if args.allreduce == "custom":
            # the library's peer-memory all-reduce for the row-parallel outputs
            from deltazip_b200 import custom_all_reduce
            car = custom_all_reduce.init_custom_ar(rank, world)
            ar_check = allreduce_selfcheck(car, rank, world, device)
            ar_choice = args.ar_variant
            if args.ar_variant == 0 and ar_check == "ok":
                ar_choice = pick_allreduce_kernel(car, world, device)
            car.set_variant(ar_choice)
    tp = world
    L = _lib.lib()

    projs, layers = build_model(tp, rank, device, num_layers=args.layers)
    g = torch.Generator(device="cpu").manual_seed(1234)
    idx_host = torch.sort(torch.randint(0, NUM_DELTAS, (TOKENS,), generator=g))[0].to(torch.int64)
    active = len(set(idx_host.tolist()))
    # one activation per distinct K of this rank (a row-parallel layer sees its own K range)
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
                dtype=_lib.DZ_DTYPE_F16, tokens_sorted=1,
                flags=_lib.DZ_SBMM_INPUTS_STABLE,     # static weights, table built once per step
                workspace=ws.data_ptr(), workspace_bytes=ws.numel())
            calls.append((a, rowp, y_dev[n]))
            step_bytes += algorithmic_bytes(TOKENS, n, k, active, BITS)

    stage_ptr, stage_len = ctypes.c_void_p(), ctypes.c_size_t()
    push = _lib.PushTarget()
    fused = car is not None and args.fused_ar and car.can_push(TOKENS, HIDDEN, torch.float16)

    def launch(a, rowp, y, collectives=True):
        """One projection: the SBMM and, for a row-parallel layer under tensor parallelism, the
        all-reduce of its partial output.  Returns the number of this library's launches."""
        reduce = rowp and tp > 1 and collectives
        if reduce and fused:
            # fused: the SBMM's epilogue pushes finished tiles into every rank's receive slot and
            # flags them; the reduction kernel only sums local memory
            L.dz_allreduce_push_target(car._ctx, TOKENS, a.N, _lib.DZ_DTYPE_F16, ctypes.byref(push))
            a.push = ctypes.pointer(push)
            rc = L.dz_sbmm(ctypes.byref(a), stream)
            a.push = None
            if rc:
                _lib.check(rc, "dz_sbmm")
            rc = L.dz_allreduce_run_pushed(car._ctx, y.data_ptr(), TOKENS, a.N, _lib.DZ_DTYPE_F16, stream)
            if rc:
                _lib.check(rc, "dz_allreduce_run_pushed")
            return 2
        if reduce and car is not None:
            # the SBMM writes its partial output straight into the staging buffer of the
            # all-reduce that follows (buffers alternate from call to call)
            L.dz_allreduce_staging(car._ctx, ctypes.byref(stage_ptr), ctypes.byref(stage_len))
            a.y = stage_ptr.value
        else:
            a.y = y.data_ptr()
        rc = L.dz_sbmm(ctypes.byref(a), stream)
        if rc:
            _lib.check(rc, "dz_sbmm")
        if not reduce:
            return 1
        if car is not None:
            rc = L.dz_allreduce_run(car._ctx, stage_ptr, y.data_ptr(), y.numel(),
                                    _lib.DZ_DTYPE_F16, stream)
            if rc:
                _lib.check(rc, "dz_allreduce_run")
            return 2
        dist.all_reduce(y)
        return 1

    def step_device(collectives=True):
        return sum(launch(a, rowp, y, collectives) for a, rowp, y in calls)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    # ---- parity of the launches that get timed (outside the timed region) ----
    # layer 0, all four shapes, every output: SBMM against dequantise-then-matmul in float32;
    # under tensor parallelism the all-reduced output against the all-reduce (NCCL, float32)
    # of the per-rank dense references.
    parity = {"max_rel_l2": 0.0, "shapes": {}}
    for (a, rowp, y), (name, n, k, _) in zip(calls[:len(projs)], projs):
        launch(a, rowp, y)
        ref = dense_reference(x_dev[k], layers[0][name], idx_dev)
        if rowp and tp > 1:
            dist.all_reduce(ref)
        torch.cuda.synchronize()
        rel = ((y.float() - ref).norm() / ref.norm()).item()
        parity["shapes"][f"{name} {n}x{k}"] = rel
        parity["max_rel_l2"] = max(parity["max_rel_l2"], rel)
    parity["tolerance"] = 1e-2
    parity["ok"] = bool(parity["max_rel_l2"] <= 1e-2)
    if world > 1:
        flag = torch.tensor([parity["max_rel_l2"]], device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MAX)
        parity["max_rel_l2"] = flag.item()
        parity["ok"] = bool(parity["max_rel_l2"] <= 1e-2)

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
    ms_total = ev0.elapsed_time(ev1)
    status = ops_read_status(L, ws, stream)

    # ---- time of the SBMM launches alone, for the roofline ----
    # One GPU: the timed region above holds nothing but the SBMM launches, so the average launch
    # time is that region's.  Several GPUs: the same number of warmed steps without the
    # collectives, timed the same way.
    if world == 1:
        kernel_ms = ms_total
        kernel_src = "the timed steps"
    else:
        step_device(collectives=False)
        barrier()
        kev0, kev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        kev0.record()
        for _ in range(args.steps):
            step_device(collectives=False)
        kev1.record()
        torch.cuda.synchronize()
        kernel_ms = kev0.elapsed_time(kev1)
        kernel_src = "a separate pass of the same steps without the all-reduce"

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
                if reduce and fused:
                    ops.sbmm(xd[k], e["q"], e["s"], e["m"], seg, e["w"], bits=BITS, stable=True,
                             push=car.push_target(TOKENS, n, torch.float16))
                    y = car.all_reduce_pushed(TOKENS, n, torch.float16, out=y_dev[n])
                    continue
                out = car.staging_like((TOKENS, n), torch.float16) if (reduce and car) else y_dev[n]
                y = ops.sbmm(xd[k], e["q"], e["s"], e["m"], seg, e["w"], out=out, bits=BITS, stable=True)
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
        n_calls = len(calls)
        kernel_ms_per_step = kernel_ms / args.steps
        achieved = step_bytes / (kernel_ms_per_step * 1e-3) / 1e9
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
                "allreduce": ("fused: SBMM epilogue pushes tiles to every rank, local sum "
                              "(dz_allreduce_run_pushed)" if fused else
                              "peer-memory (dz_allreduce_run, %s%s)" % (
                                  {0: "one-shot kernel at this size", 1: "one-shot kernel",
                                   2: "two-stage kernel", 3: "in-switch multimem kernel"}[ar_choice],
                                  ", timed against the alternatives at start-up" if args.ar_variant == 0 else ", forced")
                              if car is not None
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
                "bound": "hbm", "kernel": "sbmm_tc_kernel<4,0,FULLK,false> (4-bit, fp16, 64-column token block)",
                "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "peak_source": peaks["source"],
                "algorithmic_bytes_per_launch": step_bytes / n_calls,
                "avg_launch_us": kernel_ms_per_step * 1e3 / n_calls,
                "timed_over": kernel_src,
                "traffic": ncu_traffic_per_launch(step_bytes / n_calls),
            },
            "parity_check": parity,
            "clocks": clocks,
            "kernel_status": status,
        }
        if ar_check is not None:
            line["allreduce_check"] = ar_check
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
    if not parity["ok"]:
        raise SystemExit(f"parity check failed: {parity}")
    if ar_check not in (None, "ok"):
        raise SystemExit(f"all-reduce check failed: {ar_check}")


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
# CPU arm: the reference's own PyTorch path on the host cores
# ---------------------------------------------------------------------------

class CpuLayerSample:
    """One decoder layer of the benchmark (its four SBMM calls) on the host: fp16 base weights,
    deltas 2:4-pruned and quantised by the quantiser (so the codes are genuinely 2:4), packed in
    the reference's GPTQ layout.  One compressed delta per shape is shared by the 8 slots: the
    CPU path's time does not depend on the values, and generating 8 x 4 full-size deltas on the
    host would take longer than timing them.

    With oracle/_ref present (the reference's own quant.py / qlinear.py staged by
    oracle/make_ref.py) the calls run QuantLinear.forward itself: kind "reference".  Otherwise
    they run the restatement in oracle/torch_port.py: kind "port"."""

    def __init__(self, threads: int):
        import torch
        from deltazip_b200 import synth                      # data preparation only
        from oracle import reference_path as R
        from oracle import torch_port as T
        torch.set_num_threads(threads)
        self.kind = "reference" if R.available() else "port"
        g = torch.Generator().manual_seed(7)
        self.idx = torch.sort(torch.randint(0, NUM_DELTAS, (TOKENS,), generator=g))[0]
        self.calls = []
        gen_dev = "cuda" if torch.cuda.is_available() else "cpu"
        for name, n, k, _ in projections(1, 0):
            w = (torch.randn((n, k), generator=g) * 0.02).half()
            x = torch.randn((TOKENS, k), generator=g).half()
            delta = (torch.randn((n, k), generator=g) * 1e-3).to(gen_dev)
            qw, qz, sc = (t.cpu() for t in synth.compress_delta_gptq(delta, BITS))
            del delta
            if self.kind == "reference":
                layer = R.quant_linear(qw, qz, sc, BITS)
                layers = [layer] * NUM_DELTAS
                self.calls.append((name, n, k, lambda pre=None, x=x, w=w, layers=layers:
                                   R.apply_delta(x, w, layers, self.idx, pre), layer))
            else:
                deltas = [(qw, qz, sc, BITS)] * NUM_DELTAS
                self.calls.append((name, n, k, lambda pre=None, x=x, w=w, deltas=deltas:
                                   T.apply_delta(x, w, deltas, self.idx, dequant_every_call=pre is None,
                                                 cache=pre), None))
        self._pre = None

    def run_layer(self):
        """The reference's behaviour: dequantise every call."""
        for _, _, _, fn, _ in self.calls:
            fn()

    def time_each(self, reps: int):
        """Median seconds per call for each shape, dequantising every call."""
        out = {}
        for name, n, k, fn, _ in self.calls:
            ts = []
            for _ in range(reps):
                t0 = time.perf_counter()
                fn()
                ts.append(time.perf_counter() - t0)
            out[f"{name} {n}x{k}"] = sorted(ts)[len(ts) // 2]
        return out

    def time_pre_unpacked(self, reps: int):
        """Same calls with the dense deltas unpacked beforehand (pure matmul cost)."""
        import torch
        from oracle import reference_path as R
        from oracle import torch_port as T
        out = {}
        for name, n, k, fn, layer in self.calls:
            if self.kind == "reference":
                pre = [R.unpack_dense_t(layer)] * NUM_DELTAS
            else:
                pre = {}
                fn(pre)                                     # fills the cache
            ts = []
            for _ in range(reps):
                t0 = time.perf_counter()
                fn(pre)
                ts.append(time.perf_counter() - t0)
            out[f"{name} {n}x{k}"] = sorted(ts)[len(ts) // 2]
            del pre
        return out


def cpu_baseline(budget_s=20.0):
    threads = os.cpu_count() or 1
    sample = CpuLayerSample(threads)
    sample.run_layer()                                      # warm-up
    t0 = time.perf_counter()
    per_call = sample.time_each(reps=1)
    layer_s = sum(per_call.values())
    reps = int(max(1, min(5, budget_s / max(layer_s, 1e-3) - 1)))
    if reps > 1:
        per_call = sample.time_each(reps=reps)
        layer_s = sum(per_call.values())
    pre = sample.time_pre_unpacked(reps=max(1, min(3, reps)))
    step_s = layer_s * LAYERS
    return {"value": TOKENS / step_s, "unit": UNIT, "cores": threads, "kind": sample.kind,
            "sample": "one decoder layer = one call of each of the four shapes (8 deltas, 64 tokens, "
                      "quantiser-made 2:4 codes) through %s, dequantising on every call as the "
                      "reference does; median of %d; x32 layers for the step"
                      % ("the reference's QuantLinear.forward + F.linear (oracle/_ref)"
                         if sample.kind == "reference" else "oracle/torch_port.apply_delta", reps),
            "seconds_per_call": per_call,
            "pre_unpacked": {"value": TOKENS / (sum(pre.values()) * LAYERS), "unit": UNIT,
                             "seconds_per_call": pre},
            "wall_s": time.perf_counter() - t0}


def run_reference(args):
    world, rank, _ = dist_env()
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    sample = CpuLayerSample(threads)
    warm = max(1, min(args.warmup, 2))
    for _ in range(warm):
        sample.run_layer()
    steps = max(1, min(args.steps, 20))
    t0 = time.perf_counter()
    for _ in range(steps):
        sample.run_layer()
    layer_s = (time.perf_counter() - t0) / steps
    step_s = layer_s * LAYERS
    value = TOKENS / step_s
    text = ("each timed step = one decoder layer (one call of each of the four shapes, 8 deltas, 64 "
            "tokens, quantiser-made 2:4 codes, dequantised on every call) = 1/32 of the benchmark's "
            "decode step; value = 64 tokens / (32 x the mean step); %d timed steps; code: %s"
            % (steps, "the reference's QuantLinear.forward + F.linear (oracle/_ref)"
               if sample.kind == "reference" else "oracle/torch_port.apply_delta"))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT,
        "n_gpus": world, "steps": steps, "warmup": warm,
        "ms_per_step": step_s * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": "configs[1]: SBMM over Llama-2-7B projection shapes (qkv 12288x4096, "
                               "o 4096x4096, gate_up 22016x4096, down 4096x11008) x 32 layers, "
                               "8 deltas 4-bit 2:4 sym per-channel, 64-token decode batch, slot ids "
                               "uniform over 8 (sorted)",
                   "sampled": "one of the 32 identical layers per timed step",
                   "tokens": TOKENS, "deltas": NUM_DELTAS, "bits": BITS, "layers": LAYERS,
                   "parallelism": "cpu"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": sample.kind,
                         "sample": text},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------
# Full-model decode configurations (3: 7B / 32 deltas, 4: 13B / 64 deltas Zipf, tensor parallel)
# ---------------------------------------------------------------------------

DECODE_CONFIGS = {
    3: dict(model="llama-2-7b", deltas=32, bits=2, seqs=128, prompt=512, decode=128, zipf=None,
            text="configs[2]: Llama-2-7B architecture (32 layers, hidden 4096, 32 heads, inter 11008, "
                 "vocab 32000), random-init fp16 base, 32 resident 2-bit 2:4 deltas, 128 concurrent "
                 "sequences, prompt 512, request-to-delta uniform, paged KV cache"),
    4: dict(model="llama-2-13b", deltas=64, bits=2, seqs=256, prompt=256, decode=256, zipf=1.5,
            text="configs[3]: Llama-2-13B architecture (40 layers, hidden 5120, 40 heads, inter 13824), "
                 "random-init fp16 base, 64 deltas 2-bit 2:4, 256 sequences, request-to-delta Zipf "
                 "alpha=1.5, prompt 256, tensor parallel"),
}


def request_deltas(num_seqs, num_deltas, zipf, seed=0):
    """Delta id (1-based) of every sequence: uniform, or Zipf(alpha) over the delta ranks."""
    import torch
    g = torch.Generator().manual_seed(seed)
    if zipf is None:
        return (torch.randint(0, num_deltas, (num_seqs,), generator=g) + 1).tolist()
    p = 1.0 / torch.arange(1, num_deltas + 1, dtype=torch.float64) ** zipf
    return (torch.multinomial(p / p.sum(), num_seqs, replacement=True, generator=g) + 1).tolist()


def fill_resident_deltas(engine, resident, bits, seed=0):
    """Writes seeded synthetic deltas (N(0, 1e-3), 2:4-pruned, quantised, packed and converted on
    the device) straight into the GPU slots: distinct data per slot and projection shape for the
    first layer, copied to the other layers (every byte the kernel streams is still distinct
    memory; only the generation time is saved)."""
    import torch
    from deltazip_b200 import ops, synth
    mgr = engine.manager
    first = {}
    for name, module in mgr.modules.items():
        leaf = name.rsplit(".", 1)[1]
        if leaf not in first:
            n, k = module.weight.shape
            gen = torch.Generator(device=engine.device).manual_seed(seed + len(first))
            for slot in range(len(resident)):
                delta = torch.randn((n, k), generator=gen, device=engine.device) * 1e-3
                qw, qz, sc = synth.compress_delta_gptq(delta, bits)
                del delta
                ops.convert_from_gptq(qw, qz, sc, bits, check_status=(slot == 0),
                                      out=(module.qweight_stacked[slot], module.meta_stacked[slot],
                                           module.scales_stacked[slot]))
            first[leaf] = module
        else:
            src = first[leaf]
            module.qweight_stacked.copy_(src.qweight_stacked)
            module.meta_stacked.copy_(src.meta_stacked)
            module.scales_stacked.copy_(src.scales_stacked)
    for slot, delta_id in enumerate(resident):
        mgr.adopt_resident(delta_id, slot)


def run_decode(args):
    import torch
    import torch.distributed as dist
    from deltazip_b200 import _lib, ops, parallel_state
    from deltazip_b200.config import DeltaConfig
    from deltazip_b200.engine import DecodeEngine, Sequence
    from deltazip_b200.llama import LLAMA2_7B, LLAMA2_13B, LlamaConfig

    spec = DECODE_CONFIGS[args.config]
    world, rank, local_rank = dist_env()
    if args.gpus > 1 and world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks (WORLD_SIZE={world})")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
        parallel_state.initialize_model_parallel(world, disable_custom_all_reduce=(args.allreduce == "nccl"))
    base = LLAMA2_7B if spec["model"] == "llama-2-7b" else LLAMA2_13B
    layers = args.layers or base.num_hidden_layers
    cfg = LlamaConfig(base.hidden_size, base.intermediate_size, layers, base.num_attention_heads,
                      base.num_key_value_heads, base.vocab_size)
    bits, seqs_total, prompt = spec["bits"], spec["seqs"], spec["prompt"]
    steps, warmup = args.steps, args.warmup
    max_new = warmup + 2 * steps + 3 + 8                    # timed steps, end-to-end steps, margin

    # ---- which deltas the batch needs, and how many of them fit ----
    seq_delta = request_deltas(seqs_total, spec["deltas"], spec["zipf"])
    demand = {}
    for d in seq_delta:
        demand[d] = demand.get(d, 0) + 1
    needed = sorted(demand, key=lambda d: (-demand[d], d))
    projs = projections(world, rank, cfg.hidden_size, cfg.intermediate_size)
    slot_bytes = sum(n * k * (bits / 16 + 1 / 8) + 2 * n for _, n, k, _ in projs) * layers
    base_bytes = sum(2 * n * k for _, n, k, _ in projs) * layers + 2 * 2 * cfg.vocab_size * cfg.hidden_size
    kv_heads_local = max(1, cfg.kv_heads // world)
    block = 16
    blocks_per_seq = (prompt + max_new + block - 1) // block
    kv_bytes = seqs_total * blocks_per_seq * block * kv_heads_local * 128 * 2 * 2 * layers
    free, _total = torch.cuda.mem_get_info()
    fit = int((free * 0.90 - base_bytes - kv_bytes) // slot_bytes)
    if world > 1:
        t = torch.tensor([fit], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        fit = int(t.item())
    slots = max(1, min(len(needed), fit))
    resident = needed[:slots]
    admitted = [i for i, d in enumerate(seq_delta) if d in set(resident)]

    engine = DecodeEngine(cfg, DeltaConfig(max_deltas=slots, max_bitwidth=bits, max_cpu_deltas=slots),
                          max_seqs=seqs_total, kv_blocks=len(admitted) * blocks_per_seq, block_size=block,
                          device=device)
    fill_resident_deltas(engine, resident, bits)
    g = torch.Generator().manual_seed(1)
    prefill_info = None
    if args.prefill == "real":
        # the prompts run through the model (chunks of whole prompts, at most 2048 tokens each:
        # the manager's mapping buffers hold that many rows); timed once, outside the steps
        per = max(1, 2048 // prompt)
        seqs = []
        for i in admitted:
            s = Sequence(seq_id=i, delta_id=seq_delta[i], length=prompt, max_new=max_new,
                         prompt=torch.randint(0, cfg.vocab_size, (prompt,), generator=g))
            s.blocks = engine.cache.allocate(blocks_per_seq)
            seqs.append(s)
        seqs.sort(key=lambda s: (engine._slot_of(s.delta_id), s.seq_id))
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        engine.running.extend(seqs[:per])
        engine.prefill(seqs[:per])                         # first chunk untimed (library warm-up)
        torch.cuda.synchronize()
        p0.record()
        for c in range(per, len(seqs), per):
            engine.running.extend(seqs[c:c + per])
            engine.prefill(seqs[c:c + per])
        p1.record()
        torch.cuda.synchronize()
        timed_tokens = prompt * max(0, len(seqs) - per)
        pms = p0.elapsed_time(p1)
        prefill_info = {"tokens": timed_tokens, "ms": pms, "chunk_tokens": per * prompt,
                        "tok_s": (timed_tokens / (pms * 1e-3)) if pms > 0 else None,
                        "note": "dense product of a chunk through the library GEMM; delta products "
                                "of runs of 256 and more rows of one delta through dz_unpack + the "
                                "library GEMM, of shorter runs by the SBMM kernel per block of 128 "
                                "tokens; causal attention through torch's SDPA"}
    else:
        # prefill is replaced by a synthetic cache of the prompt length: random keys and values
        for li in range(layers):
            engine.cache.k[li].normal_(0.0, 0.5)
            engine.cache.v[li].normal_(0.0, 0.5)
        first_tokens = torch.randint(0, cfg.vocab_size, (seqs_total,), generator=g).tolist()
        for i in admitted:
            s = Sequence(seq_id=i, delta_id=seq_delta[i], length=prompt, max_new=max_new)
            s.blocks = engine.cache.allocate(blocks_per_seq)
            engine.running.append(s)
        engine._rebuild({i: first_tokens[i] for i in admitted})
    b = len(engine.running)
    active = len({s.delta_id for s in engine.running})

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    # ---- device-resident timing ----
    for _ in range(warmup):
        engine.decode_step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_wall0 = time.time()
    ev0.record()
    for _ in range(steps):
        engine.decode_step()
    ev1.record()
    barrier()
    ms_total = ev0.elapsed_time(ev1)
    status = ops.read_status(device)

    # ---- end to end: each step's inputs come from pinned host memory, its tokens go back ----
    tok_host = engine.tokens.cpu().pin_memory()
    pos_host = engine.positions.cpu().pin_memory()
    out_host = torch.empty_like(tok_host).pin_memory()

    def step_e2e():
        engine.tokens = tok_host.to(device, non_blocking=True)
        engine.positions = pos_host.to(device, non_blocking=True)
        out = engine.decode_step()
        out_host.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        tok_host.copy_(out_host)
        pos_host.add_(1)

    step_e2e()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step_e2e()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    clocks = sampler.stop(t_wall0, time.time()) if rank == 0 else None

    # ---- the SBMM launches of a step alone, for the roofline ----
    mgr = engine.manager
    xs = {k: torch.randn((b, k), device=device).half() for k in sorted({p[2] for p in projs})}
    mods = [(m, xs[m.weight.shape[1]]) for _, m in sorted(mgr.modules.items())]

    def sbmm_only():
        for m, x in mods:
            m.apply_weights(x)
    sbmm_only()
    torch.cuda.synchronize()
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    k0.record()
    for _ in range(steps):
        sbmm_only()
    k1.record()
    torch.cuda.synchronize()
    kernel_ms = k0.elapsed_time(k1) / steps
    step_bytes = sum(algorithmic_bytes(b, n, k, active, bits) for _, n, k, _ in projs) * layers

    times = torch.tensor([ms_total, e2e_ms, kernel_ms], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_total, e2e_ms, kernel_ms = times.tolist()

    if rank == 0:
        ms_per_step = ms_total / steps
        peaks = measured_peaks()
        achieved = step_bytes / (kernel_ms * 1e-3) / 1e9
        n_calls = len(mods)
        launches_per_step = n_calls + layers * (4 + (2 if world > 1 else 0)) + 2
        line = {
            "metric": "decode_tokens_per_s", "value": b / (ms_per_step * 1e-3), "unit": UNIT,
            "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic",
            "config": {
                "workload": spec["text"] + "; measured: decode steps of the whole batch (one token per "
                            "sequence per step); " +
                            ("the prompts were prefilled through the model before the steps (timed "
                             "separately, see prefill)" if prefill_info else
                             "prefill replaced by a synthetic KV cache of the prompt length (random "
                             "keys/values)"),
                "layers": layers, "sequences_requested": seqs_total, "sequences_running": b,
                "deltas": spec["deltas"], "deltas_needed_by_the_batch": len(needed),
                "gpu_slots": slots, "active_deltas": active, "bits": bits, "context": prompt,
                "parallelism": f"tp{world}",
                "admission": ("all sequences run" if b == seqs_total else
                              "GPU memory holds %d of the %d deltas the batch needs: sequences of the "
                              "other deltas wait (delta-aware admission)" % (slots, len(needed))),
                "l2": "inputs larger than L2: each step streams %.1f GB of weights per rank"
                      % (step_bytes * 1e-9),
            },
            "e2e": {"value": b / (e2e_ms / steps * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": int(b * 16), "d2h_bytes_per_step": int(b * 8),
                    "ms_per_step": e2e_ms / steps},
            "gpu_launches": launches_per_step * steps,
            "roofline": {
                "bound": "hbm", "kernel": "sbmm_tc_kernel<%d,0,FULLK,%s>" % (bits, "true" if b > 64 else "false"),
                "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "peak_source": peaks["source"],
                "algorithmic_bytes_per_launch": step_bytes / n_calls,
                "avg_launch_us": kernel_ms * 1e3 / n_calls,
                "timed_over": "a separate pass of the step's %d SBMM launches alone" % n_calls,
                "sbmm_share_of_step": kernel_ms / ms_per_step,
                "traffic": ncu_traffic_per_launch(step_bytes / n_calls),
            },
            "clocks": clocks, "kernel_status": status,
        }
        if prefill_info:
            line["prefill"] = prefill_info
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_decode(cfg, b, active, bits, layers)
        print(json.dumps(line), flush=True)
    if world > 1:
        from deltazip_b200 import custom_all_reduce
        h = custom_all_reduce.get_handle()
        if h is not None and h.status():
            raise SystemExit("peer-memory all-reduce reported a status")
        parallel_state.destroy_model_parallel()
        dist.destroy_process_group()


def cpu_sample_decode(cfg, tokens, active, bits, threads):
    """One o_proj-shaped call ([hidden, hidden]) with the batch's tokens and active deltas through
    the reference's CPU path (dequantise every delta on every call)."""
    import torch
    from deltazip_b200 import synth
    from oracle import reference_path as R
    from oracle import torch_port as T
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(3)
    h = cfg.hidden_size
    w = (torch.randn((h, h), generator=g) * 0.02).half()
    x = torch.randn((tokens, h), generator=g).half()
    idx = torch.sort(torch.arange(tokens) % active)[0]
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    qw, qz, sc = (t.cpu() for t in synth.compress_delta_gptq((torch.randn((h, h), generator=g) * 1e-3).to(dev), bits))
    if R.available():
        layer = R.quant_linear(qw, qz, sc, bits)
        return "reference", lambda: R.apply_delta(x, w, [layer] * active, idx)
    return "port", lambda: T.apply_delta(x, w, [(qw, qz, sc, bits)] * active, idx)


def cpu_baseline_decode(cfg, tokens, active, bits, layers):
    threads = os.cpu_count() or 1
    kind, fn = cpu_sample_decode(cfg, tokens, active, bits, threads)
    t0 = time.perf_counter()
    fn()
    per_call = time.perf_counter() - t0
    reps = int(max(1, min(3, 15.0 / max(per_call, 1e-3))))
    t0 = time.perf_counter()
    for _ in range(reps):
        fn()
    per_call = (time.perf_counter() - t0) / reps
    weights = sum(n * k for _, n, k, _ in projections(1, 0, cfg.hidden_size, cfg.intermediate_size))
    scale = layers * weights / float(cfg.hidden_size ** 2)
    return {"value": tokens / (per_call * scale), "unit": UNIT, "cores": threads, "kind": kind,
            "sample": "extrapolated: one %dx%d SBMM call with the batch's %d tokens and %d active %d-bit "
                      "deltas through the reference's CPU path (dequantise every call), %.2f s per call, "
                      "scaled by weight count (x%.0f) to the linear layers of a decode step; attention and "
                      "the other steps are not included" % (cfg.hidden_size, cfg.hidden_size, tokens, active,
                                                            bits, per_call, scale)}


def run_decode_reference(args):
    from deltazip_b200.llama import LLAMA2_7B, LLAMA2_13B
    world, rank, _ = dist_env()
    if rank != 0:
        return
    spec = DECODE_CONFIGS[args.config]
    cfg = LLAMA2_7B if spec["model"] == "llama-2-7b" else LLAMA2_13B
    seq_delta = request_deltas(spec["seqs"], spec["deltas"], spec["zipf"])
    active = len(set(seq_delta))
    base = cpu_baseline_decode(cfg, spec["seqs"], active, spec["bits"], cfg.num_hidden_layers)
    line = {"impl": "reference", "metric": "decode_tokens_per_s", "value": base["value"], "unit": UNIT,
            "n_gpus": world, "steps": 1, "warmup": 1, "ms_per_step": spec["seqs"] / base["value"] * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic", "config": {"workload": spec["text"], "parallelism": "cpu"},
            "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------
# Config 5: arrivals over time, deltas in pinned host memory, swap-in overlapped with decode
# ---------------------------------------------------------------------------

def run_swap(args):
    """Llama-2-70B geometry, 16 4-bit deltas in pinned host memory, at most 4 resident on the
    GPU, gamma-burst arrivals (mean 8 requests/s, CV 3), prompts U[128, 1024], outputs
    U[64, 512], tensor parallel over all ranks.  The serving loop runs on a virtual clock that
    advances by the measured duration of every iteration (prefill + one decode step), so a run
    does not have to last as long as the arrival window; every rank takes the same decisions
    (durations and upload completions are agreed through one small all-reduce per iteration)."""
    import numpy as np
    import torch
    import torch.distributed as dist
    from deltazip_b200 import ops, parallel_state, synth
    from deltazip_b200.config import DeltaConfig
    from deltazip_b200.engine import DecodeEngine, Sequence
    from deltazip_b200.llama import LLAMA2_70B, LlamaConfig
    from deltazip_b200.models import DeltaModel

    world, rank, local_rank = dist_env()
    if args.gpus > 1 and world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks (WORLD_SIZE={world})")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
        parallel_state.initialize_model_parallel(world, disable_custom_all_reduce=(args.allreduce == "nccl"))
    base = LLAMA2_70B
    layers = args.layers or base.num_hidden_layers
    cfg = LlamaConfig(base.hidden_size, base.intermediate_size, layers, base.num_attention_heads,
                      base.num_key_value_heads, base.vocab_size)
    bits, num_deltas, slots, max_seqs = 4, 16, 4, 64
    duration = args.duration or 300.0
    rate, cv = 8.0, 3.0

    # ---- requests (same on every rank) ----
    rng = np.random.default_rng(0)
    shape = 1.0 / cv ** 2
    gaps = rng.gamma(shape, (1.0 / rate) / shape, size=int(duration * rate * 3) + 16)
    arrivals = np.cumsum(gaps)
    arrivals = arrivals[arrivals < duration]
    reqs = [dict(t=float(t), delta=int(rng.integers(1, num_deltas + 1)), prompt=int(rng.integers(128, 1025)),
                 out=int(rng.integers(64, 513))) for t in arrivals]

    kv_blocks = max_seqs * ((1024 + 512 + 15) // 16)
    engine = DecodeEngine(cfg, DeltaConfig(max_deltas=slots, max_bitwidth=bits, max_cpu_deltas=num_deltas),
                          max_seqs=max_seqs, kv_blocks=kv_blocks, device=device)
    engine.attn_splits = 8 if engine.model.kv_heads * max_seqs < 256 else 1
    mgr = engine.manager
    arena_bytes = mgr.layout.total
    # ---- host memory: how many distinct deltas can be pinned ----
    try:
        import psutil
        avail = psutil.virtual_memory().available
    except Exception:
        avail = 64 << 30
    local_world = max(1, world)
    fit = int(0.35 * avail / local_world // max(arena_bytes, 1))
    host_deltas = max(2, min(num_deltas, fit))           # never pin more than a third of the free RAM
    if world > 1:
        t = torch.tensor([host_deltas], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        host_deltas = int(t.item())
    if host_deltas <= slots:
        raise SystemExit(f"host memory holds only {host_deltas} deltas of {arena_bytes >> 20} MiB per rank: "
                         "nothing would ever be swapped; use fewer layers or more ranks")
    # distinct synthetic data per delta for the first layer, copied to the other layers, written
    # into GPU slot 0 as a staging area and read back into the delta's pinned arena
    first = {}
    for name, module in mgr.modules.items():
        first.setdefault(name.rsplit(".", 1)[1], module)
    for d in range(1, host_deltas + 1):
        gen = torch.Generator(device=device).manual_seed(1000 * d + rank)
        for leaf, module in first.items():
            n, k = module.weight.shape
            qw, qz, sc = synth.compress_delta_gptq(torch.randn((n, k), generator=gen, device=device) * 1e-3, bits)
            ops.convert_from_gptq(qw, qz, sc, bits, check_status=(d == 1),
                                  out=(module.qweight_stacked[0], module.meta_stacked[0], module.scales_stacked[0]))
        for name, module in mgr.modules.items():
            src = first[name.rsplit(".", 1)[1]]
            if module is not src:
                module.qweight_stacked[0].copy_(src.qweight_stacked[0])
                module.meta_stacked[0].copy_(src.meta_stacked[0])
                module.scales_stacked[0].copy_(src.scales_stacked[0])
        dm = DeltaModel(d, bits, {})
        dm.arena = torch.empty(arena_bytes, dtype=torch.uint8).pin_memory()
        dm.arena.copy_(mgr.arena[0])
        dm._arena_layout = mgr.layout
        mgr.add_delta(dm)
    mgr.arena[0].zero_()
    torch.cuda.synchronize()

    pending = [Sequence(i, (r["delta"] - 1) % host_deltas + 1, r["prompt"], r["out"], arrival=r["t"],
                        prompt=torch.randint(0, cfg.vocab_size, (r["prompt"],),
                                             generator=torch.Generator().manual_seed(i)))
               for i, r in enumerate(reqs)]
    waiting, done = [], []
    now, iters, tokens_out, busy_with_upload = 0.0, 0, 0, 0
    agree = torch.zeros(1 + num_deltas + 1, device=device, dtype=torch.float64)

    def ready_all_ranks():
        """For every delta being uploaded: has the upload finished on ALL ranks?"""
        flags = {}
        vec = torch.zeros(num_deltas + 1, dtype=torch.float64)
        for d, idx in mgr._loading.items():
            vec[d] = 0.0 if mgr._slot_ready[idx].query() else 1.0      # 1 = some rank still loading
        if world > 1:
            t = vec.to(device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            vec = t.cpu()
        for d in mgr._loading:
            flags[d] = vec[d].item() == 0.0
        return flags

    uploads0 = mgr.uploads
    t_start = time.perf_counter()
    while pending or waiting or engine.running:
        while pending and pending[0].arrival <= now:
            waiting.append(pending.pop(0))
        if not waiting and not engine.running:
            now = pending[0].arrival
            continue
        t0 = time.perf_counter()
        flags = ready_all_ranks() if mgr._loading else {}
        admitted = engine.admit_overlapped(waiting, ready=lambda d: flags.get(d, False))
        group, group_tokens = [], 0
        for s_ in admitted:                      # prompts run in passes of at most 2048 tokens
            n_tok = int(s_.prompt.numel())
            if group and group_tokens + n_tok > 2048:
                engine.prefill(group)
                group, group_tokens = [], 0
            group.append(s_)
            group_tokens += n_tok
        if group:
            engine.prefill(group)
        if mgr._loading:
            busy_with_upload += 1
        if engine.running:
            engine.decode_step()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        if world > 1:
            agree[0] = dt
            dist.all_reduce(agree[:1], op=dist.ReduceOp.MAX)
            dt = agree[0].item()
        now += dt
        iters += 1
        for s_ in list(engine.running):
            if s_.first_token_time is None:
                s_.first_token_time = now
            if s_.generated >= s_.max_new:
                tokens_out += s_.generated
                done.append((s_.arrival, s_.first_token_time, now, s_.generated))
                engine.retire(s_)
        if not engine.running and not waiting and mgr._loading:
            torch.cuda.synchronize()
        if time.perf_counter() - t_start > (args.wall_limit or 600):
            break
    wall = time.perf_counter() - t_start
    status = ops.read_status(device)
    if rank == 0:
        ttft = sorted(f - a for a, f, _, _ in done) or [0.0]
        lat = sorted(e - a for a, _, e, _ in done) or [0.0]
        line = {
            "metric": "decode_tokens_per_s", "value": tokens_out / max(now, 1e-9), "unit": UNIT,
            "n_gpus": world, "steps": iters, "warmup": 0, "ms_per_step": now / max(iters, 1) * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic",
            "config": {
                "workload": "configs[4]: Llama-2-70B architecture (80 layers, hidden 8192, 64 q / 8 kv heads, "
                            "inter 28672), 16 deltas 4-bit 2:4 in pinned host memory, at most 4 GPU-resident, "
                            "gamma-burst arrivals (8 req/s, CV 3), prompt U[128,1024], output U[64,512], "
                            "swap-in overlapped with decode; virtual clock advanced by measured iteration times",
                "layers": layers, "parallelism": f"tp{world}", "arrival_window_s": duration,
                "requests": len(reqs), "requests_finished": len(done), "max_concurrent_sequences": max_seqs,
                "deltas": num_deltas, "deltas_in_host_memory": host_deltas, "gpu_slots": slots,
                "delta_bytes_per_rank": arena_bytes, "swap_ins": engine.swap_ins,
                "iterations_with_an_upload_in_flight": busy_with_upload,
                "mean_ttft_s": sum(ttft) / len(ttft), "p90_ttft_s": ttft[int(0.9 * (len(ttft) - 1))],
                "mean_latency_s": sum(lat) / len(lat), "makespan_s": now, "wall_s": wall,
            },
            "e2e": {"value": tokens_out / max(now, 1e-9), "unit": UNIT,
                    "h2d_bytes_per_step": int((mgr.uploads - uploads0) * arena_bytes / max(iters, 1)),
                    "d2h_bytes_per_step": 0, "note": "the whole loop is host-driven; value is the same measurement"},
            "gpu_launches": iters * (layers * 10 + 3), "kernel_status": status,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        parallel_state.destroy_model_parallel()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", type=int, default=2, choices=[2, 3, 4, 5],
                    help="2: SBMM microbenchmark (headline); 3/4/5: full-model decode configurations")
    ap.add_argument("--layers", type=int, default=None,
                    help="decoder layers to instantiate (default: the model's; fewer only for "
                         "profiling captures and smoke runs)")
    ap.add_argument("--allreduce", default="custom", choices=["custom", "nccl"],
                    help="N>1: all-reduce after the row-parallel layers (library peer-memory kernel or NCCL)")
    ap.add_argument("--fused-ar", type=int, default=0, choices=[0, 1],
                    help="N>1: 1 = row-parallel SBMM pushes its tiles to all ranks, 0 = separate all-reduce "
                         "kernel fed from the staging buffer (default: measured faster)")
    ap.add_argument("--ar-variant", type=int, default=0, choices=[0, 1, 2, 3],
                    help="peer-memory all-reduce kernel: 0 = the fastest of one-shot / in-switch, timed at "
                         "start-up (default), 1 one-shot, 2 two-stage, 3 in-switch (multimem)")
    ap.add_argument("--prefill", default="synthetic", choices=["synthetic", "real"],
                    help="configs 3/4: fill the KV cache with random values (default) or run the prompts")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the timed CPU sample (profiling captures)")
    ap.add_argument("--duration", type=float, default=None,
                    help="config 5: seconds of simulated arrivals (default 300)")
    ap.add_argument("--wall-limit", type=float, default=None,
                    help="config 5: stop the serving loop after this many wall-clock seconds (default 600)")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.config in DECODE_CONFIGS:
        if args.impl == "reference":
            run_decode_reference(args)
        else:
            run_decode(args)
        return
    if args.config == 5:
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "the reference's serving engine needs ray, "
                              "xformers and cupy, none of which is installed; its CPU path for the SBMM is "
                              "timed by --config 2/3/4"}), flush=True)
        else:
            run_swap(args)
        return
    if args.layers is None:
        args.layers = LAYERS
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
