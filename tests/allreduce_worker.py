"""Worker of tests/test_gpu_allreduce.py: one process per GPU under torch.distributed.run.

Checks the peer-memory all-reduce against a rank-order fp32 sum of the gathered inputs
(bit-exact), across sizes and dtypes, through the staging (zero-copy) path, over many
back-to-back calls, through a tensor-parallel row-parallel delta layer, and finally the bounded
wait: one rank issues a call that its peers never join and must get DZ_ERR_TIMEOUT back, with
its CUDA context still usable.
"""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch
import torch.distributed as dist

from deltazip_b200 import _lib, custom_all_reduce, layers, ops, parallel_state, synth
from deltazip_b200.config import DeltaConfig
from deltazip_b200.models import shard_gptq_tensors


def expected_sum(parts, dtype):
    acc = torch.zeros_like(parts[0], dtype=torch.float32)
    for p in parts:                       # rank order, fp32, one rounding at the end
        acc = acc + p.float()
    return acc.to(dtype)


def layer_sep_call(layer, xs):
    """The layer's output through the separate (non-fused) all-reduce."""
    layers.RowParallelLinearWithDelta.FUSED_ALL_REDUCE = False
    try:
        return layer(xs)[0].clone()
    finally:
        layers.RowParallelLinearWithDelta.FUSED_ALL_REDUCE = True      # the caller is in its fused loop


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    parallel_state.initialize_model_parallel(world)
    h = custom_all_reduce.get_handle()
    assert h is not None, "custom all-reduce handle was not created"

    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    # --- sizes x dtypes, out of place, bit-exact against the rank-order fp32 sum ---
    # (both kernels forced in turn -- one-shot and reduce-scatter + all-gather -- then the
    # size-based choice; ragged sizes exercise uneven parts and sub-slices)
    for variant, dtype in [(v, d) for v in (1, 2, 0) for d in (torch.float16, torch.bfloat16, torch.float32)]:
        h.set_variant(variant)
        for numel in (8, 4096, 64 * 4096, 1000 * 8, 8 * 1237, 2 * 1024 * 1024):
            x = torch.randn(numel, device=dev, dtype=torch.float32, generator=g).to(dtype)
            parts = [torch.empty_like(x) for _ in range(world)]
            dist.all_gather(parts, x)
            want = expected_sum(parts, dtype)
            assert h.should_custom_ar(x)
            got = custom_all_reduce.custom_all_reduce(x)
            assert got is not None and got.data_ptr() != x.data_ptr()
            torch.cuda.synchronize()
            assert torch.equal(got, want), (dtype, numel, (got.float() - want.float()).abs().max())
            outs = [torch.empty_like(got) for _ in range(world)]
            dist.all_gather(outs, got)
            assert all(torch.equal(o, outs[0]) for o in outs), "ranks disagree"
    # --- in-switch reduction (regions in symmetric memory with a multicast address): the switch
    #     adds in its own order, so values are compared to within one rounding of the result
    #     type, and all ranks must hold identical bits ---
    if h.multicast:
        h.set_variant(3)
        for dtype in (torch.float16, torch.bfloat16, torch.float32):
            for numel in (8, 4096, 64 * 4096, 8 * 1237, 2 * 1024 * 1024):
                x = torch.randn(numel, device=dev, dtype=torch.float32, generator=g).to(dtype)
                parts = [torch.empty_like(x) for _ in range(world)]
                dist.all_gather(parts, x)
                want = expected_sum(parts, dtype).float()
                got = h.all_reduce(x)
                torch.cuda.synchronize()
                eps = {torch.float16: 2.0 ** -10, torch.bfloat16: 2.0 ** -7, torch.float32: 2.0 ** -22}[dtype]
                assert ((got.float() - want).abs() <= eps * want.abs() + 1e-6 * world).all(), (dtype, numel)
                outs = [torch.empty_like(got) for _ in range(world)]
                dist.all_gather(outs, got)
                assert all(torch.equal(o, outs[0]) for o in outs), "ranks disagree (in-switch)"
        h.set_variant(0)
    print(f"rank {rank}: symmetric={h._symm is not None} multicast={h.multicast}", flush=True)

    # --- messages that do not qualify fall back (None) ---
    assert custom_all_reduce.custom_all_reduce(torch.zeros(3, device=dev, dtype=torch.float16)) is None
    big = torch.zeros(h.max_size // 2 + 8, device=dev, dtype=torch.float16)
    assert custom_all_reduce.custom_all_reduce(big) is None
    y = parallel_state.tensor_model_parallel_all_reduce(torch.ones(3, device=dev))
    assert torch.equal(y, torch.full((3,), float(world), device=dev))

    # --- staging path + many back-to-back calls with changing data (buffer alternation) ---
    shape = (64, 4096)
    for it in range(200):
        # alternate the kernels every 25 calls (in-switch too where it exists)
        h.set_variant((1, 2, 3)[(it // 25) % 3] if h.multicast else 1 + (it // 25) % 2)
        st = h.staging_like(shape, torch.float16)
        st.copy_(torch.full(shape, float(rank + 1 + (it % 7)), device=dev, dtype=torch.float16))
        out = h.all_reduce(st)
        if it % 50 == 49 or it < 4:
            want = float(sum(r + 1 + (it % 7) for r in range(world)))
            assert torch.equal(out, torch.full(shape, want, device=dev, dtype=torch.float16)), it
    torch.cuda.synchronize()
    assert h.status() == 0
    h.set_variant(0)

    # --- row-parallel delta layer under tensor parallelism vs the unsharded layer ---
    n, k, slots, bits, m = 512, 1024, 4, 4, 48
    gen = torch.Generator(device=dev).manual_seed(7)          # same data on every rank
    w = (torch.randn(n, k, generator=gen, device=dev) * 0.02).half()
    x = torch.randn(m, k, generator=gen, device=dev).half()
    idx = torch.sort(torch.randint(-1, slots, (m,), generator=gen, device=dev))[0]
    full = ops.alloc_slots(slots, n, k, bits, dev)
    lo, hi = parallel_state.shard_range(k, 128, rank, world)
    base = layers.RowParallelLinear(k, n, device=dev)
    base.weight.data.copy_(w[:, lo:hi])
    layer = layers.RowParallelLinearWithDelta(base)
    layer.create_delta_weights(slots, DeltaConfig(max_deltas=slots, max_bitwidth=bits))
    for d in range(slots):
        delta = torch.randn((n, k), generator=gen, device=dev) * 1e-2
        qw, qz, sc = synth.compress_delta_gptq(delta, bits)
        ops.convert_from_gptq(qw, qz, sc, bits, out=(full[0][d], full[1][d], full[2][d]))
        sq, sz, ss = shard_gptq_tensors(qw, qz, sc, bits, "row", rank, world)
        layer.set_delta(d, bits, sq, sz, ss, None, None)
    ref = ops.apply_delta(x, full[0], full[2], full[1], idx, w).float()
    layer.set_mapping(idx, None, None, None, [m])
    y_tp = layer(x[:, lo:hi].contiguous())[0].float()
    torch.cuda.synchronize()
    rel = ((y_tp - ref).norm() / ref.norm()).item()
    assert rel < 1e-2, rel
    assert h.status() == 0

    # --- fused form: the SBMM epilogue pushes its tiles to every rank, the reduction sums local
    #     slots; same rounding as the separate all-reduce, so the outputs are bit-identical ---
    for m2, sort in ((48, True), (300, True), (77, False)):
        x2 = torch.randn(m2, k, generator=gen, device=dev).half()
        idx2 = torch.randint(-1, slots, (m2,), generator=gen, device=dev)
        if sort:
            idx2 = torch.sort(idx2)[0]
        seg = ops.Segments(m2, slots, dev).build(idx2, sorted_hint=sort)
        layer.set_mapping(idx2, None, None, None, [m2], segments=seg)
        xs = x2[:, lo:hi].contiguous()
        layers.RowParallelLinearWithDelta.FUSED_ALL_REDUCE = False
        y_sep = layer(xs)[0].clone()
        layers.RowParallelLinearWithDelta.FUSED_ALL_REDUCE = True
        for rep in range(6):                      # repeated: slots and flags alternate correctly
            y_fused = layer(xs)[0]
            assert torch.equal(y_fused, y_sep), (m2, sort, rep, (y_fused.float() - y_sep.float()).abs().max())
            if rep % 2:                           # interleave with reductions of the other kind
                assert torch.equal(layer_sep_call(layer, xs), y_sep)
        ref2 = ops.apply_delta(x2, full[0], full[2], full[1], idx2, w).float()
        assert ((y_fused.float() - ref2).norm() / ref2.norm()).item() < 1e-2
    layers.RowParallelLinearWithDelta.FUSED_ALL_REDUCE = False
    torch.cuda.synchronize()
    assert h.status() == 0 and ops.read_status(dev) == 0

    # --- bounded wait: rank 0 issues a call nobody joins ---
    dist.barrier()
    torch.cuda.synchronize()
    h.set_variant(1)                        # plain peer loads only while a rank waits alone
    if rank == 0:
        lonely = torch.ones(4096, device=dev, dtype=torch.float16)
        h.all_reduce(lonely)
        torch.cuda.synchronize()            # returns after the kernel's one-second limit
        assert h.status() == _lib.DZ_ERR_TIMEOUT, h.status()
        z = torch.ones(8, device=dev) * 2   # the context is still usable
        assert float(z.sum().item()) == 16.0
    dist.barrier()
    parallel_state.destroy_model_parallel()
    dist.destroy_process_group()
    print(f"ALLREDUCE_WORKER_OK rank {rank}", flush=True)


if __name__ == "__main__":
    main()
