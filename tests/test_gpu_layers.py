"""Delta layers and slot manager on the GPU, in the shape of the reference's LoRA layer tests
(serving/tests/lora/test_layers.py): wrap a base layer, fill slots, set a mapping, compare
with base(x) + x @ delta^T per token."""
import numpy as np
import pytest
import torch
import torch.nn as nn

from oracle import deltazip_oracle as O
from tests.gpu_util import dev

pytestmark = pytest.mark.gpu
TOL = 1e-2


class TinyModel(nn.Module):
    supported_delta_modules = ["qkv_proj", "o_proj", "gate_up_proj", "down_proj"]
    packed_modules_mapping = {"qkv_proj": ["q_proj", "k_proj", "v_proj"],
                              "gate_up_proj": ["gate_proj", "up_proj"]}

    def __init__(self, hidden=256, inter=384, heads=4):
        super().__init__()
        from deltazip_b200 import layers as Ls
        self.qkv_proj = Ls.QKVParallelLinear(hidden, hidden // heads, heads)
        self.o_proj = Ls.RowParallelLinear(hidden, hidden)
        self.gate_up_proj = Ls.MergedColumnParallelLinear(hidden, [inter, inter])
        self.down_proj = Ls.RowParallelLinear(inter, hidden)


def make_delta(model, delta_id, bits, seed):
    """GPTQ tensors per module from the oracle, then the slot-layout pinned DeltaModel."""
    from deltazip_b200.models import DeltaModel
    gptq, dense = {}, {}
    for name in TinyModel.supported_delta_modules:
        n, k = getattr(model, name).weight.shape
        _, ds = O.make_layer(n, k, 1, bits, seed=seed + hash(name) % 97)
        qw, qz, sc, _ = ds[0]
        gptq[name] = (torch.from_numpy(qw), torch.from_numpy(qz), torch.from_numpy(sc))
        dense[name] = O.unpack(qw, qz, sc, bits)
    return DeltaModel.from_gptq_tensors(delta_id, bits, gptq), dense


@pytest.mark.parametrize("bits", [4, 2])
def test_manager_layers_end_to_end(bits):
    from deltazip_b200 import layers as Ls
    from deltazip_b200.config import DeltaConfig
    from deltazip_b200.models import LRUCacheDeltaModelManager
    torch.manual_seed(0)
    model = TinyModel()
    cfg = DeltaConfig(max_deltas=2, max_bitwidth=bits, max_cpu_deltas=3)
    mgr = LRUCacheDeltaModelManager(model, 16, 64, 32000, cfg)
    assert isinstance(model.qkv_proj, Ls.MergedQKVParallelLinearWithDelta)
    assert isinstance(model.gate_up_proj, Ls.MergedColumnParallelLinearWithDelta)
    assert isinstance(model.o_proj, Ls.RowParallelLinearWithDelta)
    assert model.qkv_proj.qweight_stacked.shape == (2, 256 * bits // 128, 2 * 768)
    assert model.qkv_proj.meta_stacked.shape == (2, 768, 256 // 16)

    dense = {}
    for did in (11, 12, 13):
        d, dense[did] = make_delta(model, did, bits, seed=did)
        mgr.add_delta(d)
    mgr.activate_delta(11)
    mgr.activate_delta(12)
    assert mgr.delta_index_to_id == [11, 12]

    rng = np.random.default_rng(0)

    def check(mapping_ids):
        mgr.set_delta_mapping(Ls.DeltaMapping(mapping_ids, mapping_ids))
        for name in TinyModel.supported_delta_modules:
            layer = getattr(model, name)
            k = layer.weight.shape[1]
            x = rng.standard_normal((len(mapping_ids), k), dtype=np.float32).astype(np.float16)
            y, _ = layer(dev(x))
            w = layer.weight.detach().cpu().numpy()
            ref = O.base_linear(x, w).astype(np.float32)
            for i, did in enumerate(mapping_ids):
                if did > 0:
                    ref[i] += x[i].astype(np.float32) @ dense[did][name].astype(np.float32).T
            assert O.rel_l2(y.cpu().numpy(), ref) <= TOL, name

    check((0, 11, 11, 12, 12, 12, 0))          # unsorted by slot (base tokens at both ends)
    check((11,) * 5 + (12,) * 4)
    # LRU: activating a third delta evicts the least recently used one (11) and reuses its slot
    mgr.activate_delta(13)
    assert mgr.delta_index_to_id == [13, 12]
    check((13, 13, 12, 0))
    with pytest.raises(ValueError):
        mgr.set_delta_mapping(Ls.DeltaMapping((11,), (11,)))   # 11 is no longer on the GPU
    # registry capacity 3: adding a 4th evicts the oldest registered delta
    d4, dense[14] = make_delta(model, 14, bits, seed=14)
    mgr.add_delta(d4)
    assert 11 not in mgr.list_deltas() and len(mgr) == 3


def test_set_delta_accepts_gptq_tensors_and_reset():
    from deltazip_b200 import layers as Ls
    from deltazip_b200.config import DeltaConfig
    base = Ls.ColumnParallelLinear(128, 256)
    layer = Ls.from_layer(base, 2, DeltaConfig(max_deltas=2, max_bitwidth=4), ["x"])
    assert isinstance(layer, Ls.ColumnParallelLinearWithDelta)
    _, ds = O.make_layer(256, 128, 1, 4, seed=3)
    qw, qz, sc, _ = ds[0]
    layer.set_delta(1, 4, torch.from_numpy(qw), torch.from_numpy(qz), torch.from_numpy(sc))
    idx = torch.tensor([1, 1, -1], device="cuda")
    layer.set_mapping(idx, indices_len=[3])
    x = np.random.default_rng(1).standard_normal((3, 128), dtype=np.float32).astype(np.float16)
    y, _ = layer(dev(x))
    ref = O.apply_delta(x, base.weight.detach().cpu().numpy(), [None, ds[0]], np.array([1, 1, -1]))
    assert O.rel_l2(y.cpu().numpy(), ref) <= TOL
    layer.reset_delta(1)
    y0, _ = layer(dev(x))
    assert O.rel_l2(y0.cpu().numpy(), O.base_linear(x, base.weight.detach().cpu().numpy())) <= 2e-3
    with pytest.raises(ValueError):
        layer.set_delta(0, 2, torch.from_numpy(qw), torch.from_numpy(qz), torch.from_numpy(sc))


def make_delta_on_device(model, delta_id, bits, seed):
    """Like make_delta, with the compression done by the GPU twin of the quantiser (bit-equal to
    the oracle, tests/test_gpu_format.py) so that full-size layers take milliseconds."""
    from deltazip_b200 import ops, synth
    from deltazip_b200.models import DeltaModel
    gen = torch.Generator(device="cuda").manual_seed(seed)
    gptq = {}
    for name in TinyModel.supported_delta_modules:
        n, k = getattr(model, name).weight.shape
        gptq[name] = synth.compress_delta_gptq(torch.randn((n, k), generator=gen, device="cuda") * 1e-3, bits)
    dm = DeltaModel.from_gptq_tensors(delta_id, bits, gptq)
    dense = {name: ops.unpack(w.qweight.cuda(), w.meta.cuda(), w.scales.cuda(),
                              *getattr(model, name).weight.shape, bits).float()
             for name, w in dm.deltas.items()}
    return dm, dense


def test_prefetch_overlaps_decode_and_stays_correct():
    """Swap-in at the size of a Llama-2-7B layer: prefetch_delta uploads the delta's pinned arena
    with ONE copy on the side stream while the compute stream keeps decoding with the resident
    deltas; activate_delta then only waits for the upload's event.  Asserted: one copy per
    swap-in, at least half of the upload's time hidden behind the decode, and correct results
    with the swapped-in delta."""
    from deltazip_b200 import layers as Ls
    from deltazip_b200.config import DeltaConfig
    from deltazip_b200.models import DeltaModelManager
    torch.manual_seed(0)
    model = TinyModel(hidden=4096, inter=11008, heads=32)
    mgr = DeltaModelManager(model, 16, 64, 32000, DeltaConfig(max_deltas=3, max_bitwidth=4, max_cpu_deltas=4))
    dense = {}
    for did in (1, 2, 3):
        d, dense[did] = make_delta_on_device(model, did, 4, seed=did)
        mgr.add_delta(d)
        assert d.arena is not None and d.arena.is_pinned() and d.arena.numel() == mgr.layout.total
    mgr.activate_delta(1)
    mgr.activate_delta(2)
    assert mgr.uploads == 2                      # one host-to-device copy per swap-in
    g = torch.Generator(device="cuda").manual_seed(0)
    xs = {name: torch.randn((8, getattr(model, name).weight.shape[1]), generator=g, device="cuda").half()
          for name in TinyModel.supported_delta_modules}

    def decode(iters):
        for _ in range(iters):
            for name in TinyModel.supported_delta_modules:
                getattr(model, name)(xs[name])

    ids = (1, 1, 1, 1, 2, 2, 2, 2)
    mgr.set_delta_mapping(Ls.DeltaMapping(ids, ids))
    decode(3)
    torch.cuda.synchronize()

    def timed(fn):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    t_decode = min(timed(lambda: decode(40)) for _ in range(3))

    def both():
        assert mgr.prefetch_delta(3)
        decode(40)
        mgr.activate_delta(3)          # compute stream waits for the upload's event here
    t_both = timed(both)
    assert mgr.delta_index_to_id == [1, 2, 3] and mgr.uploads == 3
    mgr.deactivate_delta(3)
    t_upload = timed(lambda: mgr.activate_delta(3))
    print(f"swap-in: decode {t_decode:.3f} ms, upload alone {t_upload:.3f} ms, "
          f"decode with upload in flight {t_both:.3f} ms (serial would be {t_decode + t_upload:.3f})")
    assert t_both < t_decode + 0.5 * t_upload, "the upload did not overlap the decode"

    ids = (3, 3, 1, 2, 0, 3, 2, 1)
    mgr.set_delta_mapping(Ls.DeltaMapping(ids, ids))
    for name in TinyModel.supported_delta_modules:
        layer = getattr(model, name)
        x = xs[name]
        y, _ = layer(x)
        ref = x.float() @ layer.weight.float().t()
        for i, did in enumerate(ids):
            if did > 0:
                ref[i] += x[i].float() @ dense[did][name].t()
        assert ((y.float() - ref).norm() / ref.norm()).item() <= TOL, name


def test_delta_checkpoint_roundtrip(tmp_path):
    """A delta saved with the reference's artefact layout (deltazip-compressed.safetensors with
    keys "{module}.{tp_rank}.{qweight|scales|meta}" plus compress_config.json,
    serving/vllm/delta/models.py:239-258) loads into pinned host memory and serves."""
    from safetensors.torch import save_file
    from deltazip_b200 import layers as Ls
    from deltazip_b200.config import CompressionConfig, DeltaConfig
    from deltazip_b200.models import DeltaModel, DeltaModelManager
    torch.manual_seed(1)
    model = TinyModel()
    mgr = DeltaModelManager(model, 8, 32, 32000, DeltaConfig(max_deltas=1, max_bitwidth=4))
    d, dense = make_delta(model, 5, 4, seed=5)
    tensors = {}
    for name, w in d.deltas.items():
        tensors[f"{name}.0.qweight"] = w.qweight.clone()
        tensors[f"{name}.0.scales"] = w.scales.clone()
        tensors[f"{name}.0.meta"] = w.meta.clone()
    save_file(tensors, str(tmp_path / "deltazip-compressed.safetensors"))
    CompressionConfig(bits=4, prunen=2, prunem=4).save_pretrained(str(tmp_path))
    loaded = DeltaModel.from_checkpoint(str(tmp_path), 5, tp_rank=0)
    assert loaded.bitwidth == 4 and set(loaded.deltas) == set(d.deltas)
    mgr.add_delta(loaded)
    assert loaded.arena.is_pinned()             # registered deltas live in one pinned buffer
    assert all(w.qweight.data_ptr() >= loaded.arena.data_ptr() for w in loaded.deltas.values())
    mgr.activate_delta(5)
    mgr.set_delta_mapping(Ls.DeltaMapping((5, 5, 0), (5,)))
    x = np.random.default_rng(2).standard_normal((3, 256), dtype=np.float32).astype(np.float16)
    y, _ = model.o_proj(dev(x))
    ref = O.base_linear(x, model.o_proj.weight.detach().cpu().numpy()).astype(np.float32)
    ref[:2] += x[:2].astype(np.float32) @ dense["o_proj"].astype(np.float32).T
    assert O.rel_l2(y.cpu().numpy(), ref) <= TOL


def test_per_delta_embedding_and_lm_head():
    """Replacement tables per delta for embedding and lm_head, against the reference's
    semantics (rows of slot d use table d, -1 uses the base table)."""
    from deltazip_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(0)
    vocab, hidden, d = 1024, 256, 3
    base = torch.randn((vocab, hidden), generator=g, device="cuda").half()
    tabs = torch.randn((d, vocab, hidden), generator=g, device="cuda").half()
    tok = torch.randint(0, vocab, (37,), generator=g, device="cuda")
    idx = torch.randint(-1, d, (37,), generator=g, device="cuda")
    y = ops.apply_delta_embed(tok, tabs, idx, base)
    ref = torch.where((idx < 0)[:, None], base[tok], tabs[idx.clamp(min=0), tok])
    assert torch.equal(y, ref)
    x = torch.randn((37, hidden), generator=g, device="cuda").half()
    logits = ops.apply_delta_uncompressed(x, tabs, idx, base)
    ref = torch.empty((37, vocab), device="cuda")
    for i in range(37):
        w = base if idx[i] < 0 else tabs[idx[i]]
        ref[i] = x[i].float() @ w.float().t()
    assert O.rel_l2(logits.float().cpu().numpy(), ref.cpu().numpy()) <= 2e-3


class TablesModel(nn.Module):
    """Embedding, one delta linear and the logits processor: the modules that carry full tables."""
    supported_delta_modules = ["embed_tokens", "o_proj", "logits_processor"]
    packed_modules_mapping = {}

    def __init__(self, vocab=1024, hidden=256):
        super().__init__()
        from deltazip_b200 import layers as Ls
        self.embed_tokens = Ls.VocabParallelEmbedding(vocab, hidden)
        self.o_proj = Ls.RowParallelLinear(hidden, hidden)
        self.lm_head = Ls.ParallelLMHead(vocab, hidden)
        self.logits_processor = Ls.LogitsProcessor(vocab)


def test_embedding_and_logits_layers_with_replacement_tables():
    """VocabParallelEmbeddingWithDelta / LogitsProcessorWithDelta installed by the manager: a
    delta that brings its own embedding and output matrix uses them for its rows, base-model rows
    and deltas without tables use the base ones (reference semantics,
    serving/vllm/delta/deltazip_marlin.py:21-86)."""
    from deltazip_b200 import layers as Ls
    from deltazip_b200.config import DeltaConfig
    from deltazip_b200.models import DeltaLayerWeights, DeltaModel, DeltaModelManager
    torch.manual_seed(3)
    model = TablesModel()
    mgr = DeltaModelManager(model, 16, 64, 1024, DeltaConfig(max_deltas=3, max_bitwidth=4))
    assert isinstance(model.embed_tokens, Ls.VocabParallelEmbeddingWithDelta)
    assert isinstance(model.logits_processor, Ls.LogitsProcessorWithDelta)
    assert model.logits_processor.weight_stacked.shape == (3, 1024, 256)
    g = torch.Generator().manual_seed(4)
    tables = {}
    for did in (1, 2):
        emb = torch.randn((1024, 256), generator=g).half()
        head = torch.randn((1024, 256), generator=g).half()
        tables[did] = (emb.cuda(), head.cuda())
        mgr.add_delta(DeltaModel(did, 4, {"embed_tokens": DeltaLayerWeights("embed_tokens", weight=emb),
                                           "lm_head": DeltaLayerWeights("lm_head", weight=head)}))
        mgr.activate_delta(did)
    mgr.add_delta(DeltaModel(3, 4, {}))                      # a delta without tables
    mgr.activate_delta(3)
    ids = (0, 1, 1, 2, 3, 3, 0, 2)                            # per token == per sequence here
    mgr.set_delta_mapping(Ls.DeltaMapping(ids, ids))
    tok = torch.randint(0, 1024, (8,), generator=g).cuda()
    h = model.embed_tokens(tok)
    base_e, base_h = model.embed_tokens.base_layer.weight, model.lm_head.weight
    for i, did in enumerate(ids):
        want = tables[did][0][tok[i]] if did in tables else base_e[tok[i]]
        assert torch.equal(h[i], want), i
    x = torch.randn((8, 256), generator=g).half().cuda()
    logits = model.logits_processor(model.lm_head.weight, x)
    assert logits.shape == (8, 1024)
    for i, did in enumerate(ids):
        w = tables[did][1] if did in tables else base_h
        ref = x[i].float() @ w.float().t()
        assert ((logits[i].float() - ref).norm() / ref.norm()).item() <= 2e-3, i


def test_grouped_gemm_many_groups_and_two_token_blocks():
    """The grouped launch at output-matrix size: 32000 x 4096, 200 rows over 6 groups (base rows
    included), unsorted rows; absent groups' matrices are never read (poisoned with NaN)."""
    from deltazip_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(9)
    vocab, hidden, d = 32000, 4096, 7
    base = (torch.randn((vocab, hidden), generator=g, device="cuda") * 0.05).half()
    tabs = (torch.randn((d, vocab, hidden), generator=g, device="cuda") * 0.05).half()
    tabs[5] = float("nan")                                   # slot 5 has no rows
    tabs[6] = float("nan")
    idx = torch.randint(-1, 5, (200,), generator=g, device="cuda")
    x = torch.randn((200, hidden), generator=g, device="cuda").half()
    y = ops.apply_delta_uncompressed(x, tabs, idx, base)
    torch.cuda.synchronize()
    assert torch.isfinite(y).all()
    for s in range(-1, 5):
        rows = (idx == s).nonzero().flatten()
        w = base if s < 0 else tabs[s]
        ref = x[rows].float() @ w.float().t()
        assert ((y[rows].float() - ref).norm() / ref.norm()).item() <= 2e-3, s
