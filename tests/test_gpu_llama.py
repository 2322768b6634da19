"""Greedy decoding of a small random-init Llama through the delta layers against the same
model evaluated with the reference's PyTorch path (dequantise the delta, base matmul + delta
matmul per token group; deltazip/nn_modules/qlinear.py:266-341 and
serving/vllm/delta/deltazip.py:24-30), 8 sequences x 4 deltas, 64 steps."""
import numpy as np
import pytest
import torch

from oracle import deltazip_oracle as O

pytestmark = pytest.mark.gpu


def build(bits, seed=0):
    from deltazip_b200 import ops
    from deltazip_b200.config import DeltaConfig
    from deltazip_b200.llama import LlamaConfig, LlamaForCausalLM
    from deltazip_b200.models import DeltaModel, DeltaModelManager
    cfg = LlamaConfig(hidden_size=512, intermediate_size=768, num_hidden_layers=2,
                      num_attention_heads=4, vocab_size=512)
    torch.manual_seed(seed)
    model = LlamaForCausalLM(cfg, seed=seed)
    mgr = DeltaModelManager(model, 8, 8 * 16, cfg.vocab_size, DeltaConfig(max_deltas=4, max_bitwidth=bits))
    dense = {}
    gen = torch.Generator(device="cuda").manual_seed(seed + 1)
    from deltazip_b200 import synth
    for did in (1, 2, 3, 4):
        tensors = {}
        for name, mod in mgr.modules.items():
            n, k = mod.weight.shape
            d = torch.randn((n, k), generator=gen, device="cuda") * 1e-2   # deltas large enough to change the decoded tokens
            tensors[name] = synth.compress_delta_gptq(d, bits)
        dm = DeltaModel.from_gptq_tensors(did, bits, tensors)
        mgr.add_delta(dm)
        mgr.activate_delta(did)
        dense[did] = {name: ops.unpack(w.qweight.cuda(), w.meta.cuda(), w.scales.cuda(),
                                       *mgr.modules[name].weight.shape, bits)
                      for name, w in dm.deltas.items()}
    return model, mgr, dense


def reference_linear(mgr, dense, seq_delta, math):
    """The reference's PyTorch path: base matmul, then per delta the rows of its tokens times
    the dequantised delta.  math = torch.float16 reproduces its two fp16 roundings, float32
    evaluates the same formula without them."""
    def fn(name, module, x):
        base = module.base_layer if hasattr(module, "base_layer") else module
        w = base.weight
        t = x.shape[0] // len(seq_delta)
        ids = torch.tensor(seq_delta, device=x.device).repeat_interleave(t)
        y = (x.to(math) @ w.to(math).t())
        for did in sorted(set(seq_delta)):
            if did <= 0:
                continue
            rows = ids == did
            y[rows] += x[rows].to(math) @ dense[did][name].to(math).t()
        return y.to(torch.float16)
    return fn


@pytest.mark.parametrize("bits", [4, 2])
def test_greedy_tokens_match_reference_path(bits):
    from deltazip_b200.layers import DeltaMapping
    from deltazip_b200.llama import greedy_generate
    model, mgr, dense = build(bits)
    seq_delta = [0, 1, 1, 2, 2, 3, 4, 4]                     # one base-model sequence, sorted by delta
    prompts = torch.randint(0, 512, (8, 8), generator=torch.Generator().manual_seed(5)).cuda()

    def set_mapping(t):
        ids = [d for d in seq_delta for _ in range(t)]
        mgr.set_delta_mapping(DeltaMapping(ids, seq_delta))

    ours = greedy_generate(model, prompts, 64, set_mapping)

    model.linear_override = reference_linear(mgr, dense, seq_delta, torch.float32)
    ref32 = greedy_generate(model, prompts, 64, lambda t: None)
    model.linear_override = reference_linear(mgr, dense, seq_delta, torch.float16)
    ref16 = greedy_generate(model, prompts, 64, lambda t: None)
    model.linear_override = None

    # deltas matter: the base-only evaluation decodes different tokens
    model.linear_override = reference_linear(mgr, dense, [0] * 8, torch.float32)
    base_only = greedy_generate(model, prompts, 64, lambda t: None)
    model.linear_override = None
    assert (base_only[1:] != ref32[1:]).float().mean() > 0.05

    agree32 = (ours == ref32).float().mean().item()
    agree16 = (ours == ref16).float().mean().item()
    print(f"bits={bits}: token agreement with the reference path: fp32 math {agree32:.4f}, "
          f"fp16 math {agree16:.4f}; fp16-vs-fp32 reference {(ref16 == ref32).float().mean().item():.4f}")
    assert agree32 == 1.0, "greedy tokens differ from the reference path (fp32 evaluation)"
    assert agree16 == 1.0, "greedy tokens differ from the reference path (fp16 evaluation)"
