"""Host-side logic of the plugin mirror on CPU: configs, mapping conversion, shard
ranges, and the tensor-parallel collectives on two gloo ranks."""
import os
import sys

import pytest
import torch
import torch.multiprocessing as mp

from deltazip_b200.config import CompressionConfig, DeltaConfig
from deltazip_b200.layers import DeltaMapping
from deltazip_b200.models import convert_mapping
from deltazip_b200.parallel_state import shard_range


def test_delta_config_validation():
    c = DeltaConfig(max_deltas=4, max_bitwidth=2)
    assert c.max_cpu_deltas == 4 and c.pack_factor == 16
    with pytest.raises(ValueError):
        DeltaConfig(max_deltas=4, max_cpu_deltas=2)
    with pytest.raises(ValueError):
        DeltaConfig(max_bitwidth=3)


def test_compression_config_roundtrip(tmp_path):
    c = CompressionConfig(bits=2, prunen=2, prunem=4)
    assert c.servable() and c.pack_factor == 16
    c.save_pretrained(str(tmp_path))
    d = CompressionConfig.from_pretrained(str(tmp_path))
    assert d.bits == 2 and d.prunen == 2 and d.prunem == 4 and d.sym
    assert not CompressionConfig(bits=4).servable()          # dense, not 2:4
    with pytest.raises(ValueError):
        CompressionConfig(bits=5)


def test_convert_mapping_matches_reference_semantics():
    # slots: delta 7 -> slot 0, delta 3 -> slot 2; id 0 = base model
    m = DeltaMapping(index_mapping=(0, 7, 7, 3, 0), prompt_mapping=(7, 3))
    base, sampler, padded, emb, lens = convert_mapping(m, [7, None, 3], 4, 32000, 0, device="cpu")
    assert base.tolist() == [-1, 0, 0, 2, -1]
    assert sampler.tolist() == [0, 2]
    assert padded.tolist() == [0 + 0 * 2, 1 + 2 * 2]
    assert emb.shape == (2, 5) and lens == (5, 2, 2, 5)
    assert emb[1].tolist() == [0, 0, 0, 2 * 32000, 0]
    with pytest.raises(ValueError):
        convert_mapping(DeltaMapping((9,), (9,)), [7, None, 3], 4, 32000, 0, device="cpu")


def test_shard_range_whole_units():
    # 172 tiles of 128 rows over 8 ranks: 21 or 22 tiles each, contiguous, complete
    cuts = [shard_range(22016, 128, r, 8) for r in range(8)]
    assert cuts[0][0] == 0 and cuts[-1][1] == 22016
    assert all(cuts[i][1] == cuts[i + 1][0] for i in range(7))
    assert {(hi - lo) // 128 for lo, hi in cuts} == {21, 22}
    with pytest.raises(ValueError):
        shard_range(100, 64, 0, 2)


def _tp_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      WORLD_SIZE=str(world))
    import torch.distributed as dist
    from deltazip_b200 import parallel_state as ps
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ps.initialize_model_parallel(world)
    assert ps.get_tensor_model_parallel_rank() == rank and ps.get_tensor_model_parallel_world_size() == world
    # row-parallel contract: full = sum of per-rank partial products
    g = torch.Generator().manual_seed(0)
    x = torch.randn(5, 256, generator=g)
    w = torch.randn(128, 256, generator=g)
    lo, hi = ps.shard_range(256, 64, rank, world)
    part = x[:, lo:hi] @ w[:, lo:hi].t()
    full = ps.tensor_model_parallel_all_reduce(part.clone())
    ok_reduce = torch.allclose(full, x @ w.t(), atol=1e-4)
    # column-parallel contract: full = concat of per-rank slices
    lo, hi = ps.shard_range(128, 64, rank, world)
    col = x @ w[lo:hi].t()
    gathered = ps.tensor_model_parallel_all_gather(col)
    ok_gather = torch.allclose(gathered, x @ w.t(), atol=1e-4)
    ret[rank] = bool(ok_reduce and ok_gather)
    dist.destroy_process_group()


def test_tensor_parallel_collectives_gloo_world2():
    ctx = mp.get_context("spawn")
    with ctx.Manager() as man:
        ret = man.dict()
        port = 29500 + os.getpid() % 1000
        procs = [ctx.Process(target=_tp_worker, args=(r, 2, port, ret)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            assert p.exitcode == 0
        assert dict(ret) == {0: True, 1: True}


def test_shard_gptq_tensors_matches_slices_of_the_dense_delta():
    """Unpacking a rank's GPTQ shard gives the matching slice of the unsharded dense delta,
    for column (N) and row (K) parallel cuts and 2/4 bits."""
    import numpy as np
    from oracle import deltazip_oracle as orc
    from deltazip_b200.models import shard_gptq_tensors
    from deltazip_b200.parallel_state import shard_range
    rng = np.random.default_rng(5)
    n, k = 384, 640
    for bits in (2, 4):
        delta = (rng.standard_normal((n, k)) * 1e-2).astype(np.float32)
        wq, scale, zero = orc.compress_delta(delta, bits)
        packed = orc.pack(wq, scale, zero, bits)
        qw, qz, sc = (torch.from_numpy(np.ascontiguousarray(t)) for t in packed[:3])
        dense = orc.unpack(packed[0], packed[1], packed[2], bits)   # [N, K]
        for world in (2, 3):
            for rank in range(world):
                cq, cz, cs = shard_gptq_tensors(qw, qz, sc, bits, "column", rank, world)
                lo, hi = shard_range(n, 128, rank, world)
                got = orc.unpack(cq.numpy(), cz.numpy(), cs.numpy(), bits)
                assert got.shape == (hi - lo, k) and np.array_equal(got, dense[lo:hi])
        for world in (2, 5):
            for rank in range(world):
                rq, rz, rs = shard_gptq_tensors(qw, qz, sc, bits, "row", rank, world)
                lo, hi = shard_range(k, 128, rank, world)
                got = orc.unpack(rq.numpy(), rz.numpy(), rs.numpy(), bits)
                assert got.shape == (n, hi - lo) and np.array_equal(got, dense[:, lo:hi])


def test_tensor_parallel_cuts_pair_producer_and_consumer():
    """For every rank count the shard a column-parallel layer produces is exactly the K range of
    the row-parallel layer that consumes it (qkv -> o_proj over the attention width, gate/up ->
    down_proj over the MLP width), also when the 128-wide unit count does not divide by the
    rank count (Llama-2-7B: 11008 = 86 units)."""
    from deltazip_b200.parallel_state import SHARD_UNIT
    for hidden, inter in ((4096, 11008), (5120, 13824), (8192, 28672)):
        for tp in (1, 2, 4, 8):
            seen_h, seen_i = 0, 0
            for rank in range(tp):
                q = shard_range(hidden, SHARD_UNIT, rank, tp)        # q heads of this rank
                o_k = shard_range(hidden, SHARD_UNIT, rank, tp)      # o_proj input columns
                gate = shard_range(inter, SHARD_UNIT, rank, tp)
                down_k = shard_range(inter, SHARD_UNIT, rank, tp)
                assert q == o_k and gate == down_k
                assert (q[1] - q[0]) % 128 == 0 and (gate[1] - gate[0]) % 128 == 0
                assert q[0] == seen_h and gate[0] == seen_i
                seen_h, seen_i = q[1], gate[1]
            assert seen_h == hidden and seen_i == inter
    # the benchmark's per-rank projection table uses the same cuts
    import bench
    for tp in (2, 4, 8):
        for rank in range(tp):
            pr = {name: (n, k) for name, n, k, _ in bench.projections(tp, rank)}
            assert pr["qkv_proj"][0] == 3 * pr["o_proj"][1]
            assert pr["gate_up_proj"][0] == 2 * pr["down_proj"][1]


def test_convert_mapping_reports_the_runs_of_a_sorted_prefill_sized_batch():
    """More than ops.FUSED_MAX_TOKENS rows in slot order: the run list the dequantise-once path
    uses comes from the host's copy of the ids; smaller or unsorted batches get none."""
    from deltazip_b200 import ops
    from deltazip_b200.layers import DeltaMapping
    from deltazip_b200.models import _convert_mapping
    ids = [0] * 100 + [5] * 300 + [3] * 200          # slots: -1, 0, 1
    out, (is_sorted, runs) = _convert_mapping(DeltaMapping(ids, [0, 5, 3]), [5, 3, None], 4, 1000, 0,
                                              device="cpu")
    assert len(ids) > ops.FUSED_MAX_TOKENS and is_sorted
    assert runs == [(-1, 0, 100), (0, 100, 400), (1, 400, 600)]
    assert out[0].tolist() == [-1] * 100 + [0] * 300 + [1] * 200
    _, (is_sorted, runs) = _convert_mapping(DeltaMapping(ids[:200], [0, 5]), [5, 3, None], 4, 1000, 0,
                                            device="cpu")
    assert is_sorted and runs is None                 # decode-sized: the fused kernel serves it
    mixed = [3] * 300 + [5] * 300
    _, (is_sorted, runs) = _convert_mapping(DeltaMapping(mixed, [3, 5]), [5, 3, None], 4, 1000, 0,
                                            device="cpu")
    assert not is_sorted and runs is None
