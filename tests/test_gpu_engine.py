"""The decode engine (admission by delta, prefill, paged-cache decode steps, LRU swap-in) against
`greedy_generate` on the same model and deltas, and the loader of the reference's checkpoint
format end to end: fixture written by the reference's own QuantLinear.pack
(tests/golden/make_golden.py) -> device conversion -> slots -> layer outputs."""
import os

import numpy as np
import pytest
import torch
import torch.nn as nn

pytestmark = pytest.mark.gpu


def small_engine(slots, bits=4, layers=2):
    from deltazip_b200 import synth
    from deltazip_b200.config import DeltaConfig
    from deltazip_b200.engine import DecodeEngine
    from deltazip_b200.llama import LlamaConfig
    from deltazip_b200.models import DeltaModel
    cfg = LlamaConfig(hidden_size=512, intermediate_size=768, num_hidden_layers=layers,
                      num_attention_heads=4, vocab_size=512)
    torch.manual_seed(0)
    eng = DecodeEngine(cfg, DeltaConfig(max_deltas=slots, max_bitwidth=bits, max_cpu_deltas=4),
                       max_seqs=8, kv_blocks=64)
    gen = torch.Generator(device="cuda").manual_seed(1)
    for did in (1, 2, 3):
        tensors = {}
        for name, mod in eng.manager.modules.items():
            n, k = mod.weight.shape
            tensors[name] = synth.compress_delta_gptq(torch.randn((n, k), generator=gen, device="cuda") * 1e-2, bits)
        eng.manager.add_delta(DeltaModel.from_gptq_tensors(did, bits, tensors))
    return eng


def test_engine_matches_greedy_generate_and_swaps_deltas():
    from deltazip_b200.engine import Sequence
    from deltazip_b200.layers import DeltaMapping
    from deltazip_b200.llama import greedy_generate
    eng = small_engine(slots=2)
    mgr = eng.manager
    g = torch.Generator().manual_seed(3)
    prompts = torch.randint(0, 512, (5, 6), generator=g)
    seq_delta = [0, 1, 1, 2, 3]
    steps = 12
    # reference run: all sequences of deltas {0, 1, 2} at once through greedy_generate
    mgr.activate_delta(1)
    mgr.activate_delta(2)

    def set_mapping(t):
        ids = [d for d in seq_delta[:4] for _ in range(t)]
        mgr.set_delta_mapping(DeltaMapping(ids, seq_delta[:4]))
    want = greedy_generate(eng.model, prompts[:4].cuda(), steps, set_mapping).cpu()
    mgr.deactivate_delta(1)
    mgr.deactivate_delta(2)

    # engine run: five sequences, two GPU slots, three deltas -> the sequence of delta 3 waits
    waiting = [Sequence(i, seq_delta[i], 0, steps, prompt=prompts[i].clone()) for i in range(5)]
    for s in waiting:
        s.length = int(s.prompt.numel())
    admitted = eng.admit(waiting)
    assert [s.seq_id for s in admitted] == [0, 1, 2, 3] and [s.seq_id for s in waiting] == [4]
    eng.prefill(admitted)
    got = {s.seq_id: [] for s in admitted}
    for sid, tok in zip(eng._order, eng.tokens.tolist()):
        got[sid].append(tok)
    for _ in range(steps - 1):
        toks = eng.decode_step().tolist()
        for sid, tok in zip(eng._order, toks):
            got[sid].append(tok)
    for i in range(4):
        assert got[i] == want[i].tolist(), f"sequence {i}"
    # sequences of delta 1 finish: delta 3 takes the freed slot (LRU), its sequence runs
    for s in [s for s in eng.running if s.delta_id == 1]:
        eng.retire(s)
    admitted = eng.admit(waiting)
    assert [s.seq_id for s in admitted] == [4] and not waiting
    assert 3 in mgr.delta_index_to_id and 1 not in mgr.delta_index_to_id
    eng.prefill(admitted)
    out = eng.decode_step()
    assert out.shape[0] == 3 and int(out.min()) >= 0 and int(out.max()) < 512
    from deltazip_b200 import ops
    assert ops.read_status() == 0


class OneLayer(nn.Module):
    supported_delta_modules = ["qkv_proj", "o_proj", "gate_up_proj", "down_proj"]
    packed_modules_mapping = {"qkv_proj": ["q_proj", "k_proj", "v_proj"],
                              "gate_up_proj": ["gate_proj", "up_proj"]}

    def __init__(self):
        super().__init__()
        from deltazip_b200 import layers as Ls

        class Block(nn.Module):
            def __init__(self):
                super().__init__()
                self.qkv_proj = Ls.QKVParallelLinear(256, 128, 2)
                self.o_proj = Ls.RowParallelLinear(256, 256)
                self.gate_up_proj = Ls.MergedColumnParallelLinear(256, [512, 512])
                self.down_proj = Ls.RowParallelLinear(512, 256)
        self.layers = nn.ModuleList([Block()])


@pytest.mark.parametrize("bits", [4, 2])
def test_reference_checkpoint_loads_and_serves(golden_dir, bits):
    from deltazip_b200 import layers as Ls
    from deltazip_b200.config import DeltaConfig
    from deltazip_b200.models import DeltaModel, DeltaModelManager
    from deltazip_b200.worker_manager import DeltaRequest, LRUCacheWorkerDeltaManager
    path = os.path.join(golden_dir, f"ref_ckpt_b{bits}")
    dense = np.load(os.path.join(path, "dense.npz"))
    torch.manual_seed(0)
    model = OneLayer()
    mgr = DeltaModelManager(model, 8, 32, 32000, DeltaConfig(max_deltas=2, max_bitwidth=bits))
    worker = LRUCacheWorkerDeltaManager(mgr)
    mapping = Ls.DeltaMapping((7, 7, 0, 7), (7,))
    worker.set_active_deltas([DeltaRequest("ref", 7, path)], mapping)
    assert mgr.delta_index_to_id[0] == 7 and "disk_to_host_s" in worker.load_times[7]
    want = {"qkv_proj": np.concatenate([dense["self_attn.q_proj"], dense["self_attn.k_proj"], dense["self_attn.v_proj"]]),
            "o_proj": dense["self_attn.o_proj"],
            "gate_up_proj": np.concatenate([dense["mlp.gate_proj"], dense["mlp.up_proj"]]),
            "down_proj": dense["mlp.down_proj"]}
    from deltazip_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(2)
    for name, d in want.items():
        layer = getattr(model.layers[0], name)
        n, k = layer.weight.shape
        # slot contents unpack bit-exactly to what the reference's unpack gave
        got = ops.unpack(layer.qweight_stacked[0], layer.meta_stacked[0], layer.scales_stacked[0], n, k, bits)
        assert np.array_equal(got.cpu().numpy().view(np.uint16), d.view(np.uint16)), name
        x = torch.randn((4, k), generator=g, device="cuda").half()
        y, _ = layer(x)
        ref = x.float() @ layer.weight.float().t()
        dd = torch.from_numpy(d).cuda().float()
        for i in (0, 1, 3):
            ref[i] += x[i].float() @ dd.t()
        assert ((y.float() - ref).norm() / ref.norm()).item() <= 2e-3, name
    # a directory that does not exist is reported as a failed load, nothing is registered
    with pytest.raises(ValueError, match="load failed"):
        worker.add_delta(DeltaRequest("gone", 8, path + "-missing"))
    assert 8 not in mgr.list_deltas()
