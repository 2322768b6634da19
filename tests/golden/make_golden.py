"""Generate the golden vectors under tests/golden/ from the reference's own code.

Run once, in a container that has the reference checkout (it is not needed at
test time):  python tests/golden/make_golden.py [/path/to/reference]

The reference package cannot be imported as a package (its __init__ pulls in
cupy), so the two files on the path are loaded by file path:
  deltazip/core/quant.py          Quantizer.find_params, quantize
  deltazip/nn_modules/qlinear.py  QuantLinear.pack / unpack / forward
Everything runs on CPU with torch.  The 2:4 mask is the reference's rule
(deltazip/core/sparsegpt.py:123-125: per row and per 4 consecutive columns,
torch.topk(..., 2, largest=False) of w^2 / diag(Hinv)^2 marks the pruned pair)
with Hinv = I.

Each case is stored as one .npz holding inputs and the reference's outputs.
"""
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def reference_case(quant, qlinear, n, k, bits, m, seed, zero_row=False):
    g = torch.Generator().manual_seed(seed)
    delta = torch.randn(n, k, generator=g, dtype=torch.float32) * 1e-3
    if zero_row:
        delta[1, :] = 0.0          # exercises the all-zero-row branch of find_params
        delta[2, :] = delta[2, :].abs()  # a row with no negative entry
    x = torch.randn(m, k, generator=g, dtype=torch.float32).half()
    w_base = (torch.randn(n, k, generator=g, dtype=torch.float32) * 0.02).half()

    quantizer = quant.Quantizer()
    quantizer.configure(bits, perchannel=True, sym=True, mse=False)
    quantizer.find_params(delta, weight=True)
    scale = quantizer.scale.clone()          # [N, 1]
    zero = quantizer.zero.clone()            # [N, 1]

    # 2:4 mask, the reference's rule with Hinv = I
    pruned = torch.zeros_like(delta, dtype=torch.bool)
    for i in range(0, k, 4):
        tmp = delta[:, i:i + 4] ** 2
        pruned.scatter_(1, i + torch.topk(tmp, 2, dim=1, largest=False)[1], True)
    q_in = delta.clone()
    q_in[pruned] = 0
    wq = quant.quantize(q_in, scale, zero, quantizer.maxq)

    layer = qlinear.QuantLinear(bits, k, n, bias=False)
    lin = torch.nn.Linear(k, n, bias=False)
    lin.weight.data = wq.clone()
    layer.pack(lin, scale.clone(), zero.clone(), g_idx=None)
    dense = layer.unpack().weight.data            # [N, K] float32 holding fp16 values
    y_delta = layer.forward(x)                    # fp16 [M, N]
    y_base = torch.nn.functional.linear(x, w_base)  # fp16
    return dict(
        bits=np.int32(bits),
        delta=delta.numpy(), x=x.numpy(), w_base=w_base.numpy(),
        scale=scale.flatten().numpy(), zero=zero.flatten().numpy(),
        keep=(~pruned).numpy(), wq=wq.numpy(),
        qweight=layer.qweight.numpy(), qzeros=layer.qzeros.numpy(),
        scales=layer.scales.numpy(), g_idx=layer.g_idx.numpy(),
        dense=dense.half().numpy(),
        dense_is_fp16_exact=np.bool_(bool((dense.half().float() == dense).all())),
        y_delta=y_delta.numpy(), y_base=y_base.numpy(),
    )


def reference_checkpoint(quant, qlinear, out_dir, bits, seed, hidden=256, inter=512):
    """A one-layer delta in the form the reference's compressor saves it
    (deltazip/modeling/_base.py:597-648 for anything but the 4-bit structured-sparse re-pack,
    which needs an external package): the QuantLinear buffers of every projection under
    HuggingFace module names in deltazip-compressed.safetensors, plus compress_config.json with
    the keys of deltazip/modeling/_base.py's config.  dense.npz holds what the reference's
    unpack gives for each projection."""
    import json
    from safetensors.torch import save_file
    g = torch.Generator().manual_seed(seed)
    shapes = {"self_attn.q_proj": (hidden, hidden), "self_attn.k_proj": (hidden, hidden),
              "self_attn.v_proj": (hidden, hidden), "self_attn.o_proj": (hidden, hidden),
              "mlp.gate_proj": (inter, hidden), "mlp.up_proj": (inter, hidden),
              "mlp.down_proj": (hidden, inter)}
    state, dense = {}, {}
    for name, (n, k) in shapes.items():
        delta = torch.randn(n, k, generator=g, dtype=torch.float32) * 1e-3
        quantizer = quant.Quantizer()
        quantizer.configure(bits, perchannel=True, sym=True, mse=False)
        quantizer.find_params(delta, weight=True)
        scale, zero = quantizer.scale.clone(), quantizer.zero.clone()
        pruned = torch.zeros_like(delta, dtype=torch.bool)
        for i in range(0, k, 4):
            tmp = delta[:, i:i + 4] ** 2
            pruned.scatter_(1, i + torch.topk(tmp, 2, dim=1, largest=False)[1], True)
        q_in = delta.clone()
        q_in[pruned] = 0
        wq = quant.quantize(q_in, scale, zero, quantizer.maxq)
        layer = qlinear.QuantLinear(bits, k, n, bias=False)
        lin = torch.nn.Linear(k, n, bias=False)
        lin.weight.data = wq.clone()
        layer.pack(lin, scale.clone(), zero.clone(), g_idx=None)
        for buf in ("qweight", "qzeros", "scales", "g_idx"):
            state[f"model.layers.0.{name}.{buf}"] = getattr(layer, buf).clone().contiguous()
        dense[name] = layer.unpack().weight.data.half().numpy()
    state["model.norm.weight"] = torch.ones(hidden, dtype=torch.float16)       # an uncompressed module
    os.makedirs(out_dir, exist_ok=True)
    save_file(state, os.path.join(out_dir, "deltazip-compressed.safetensors"))
    with open(os.path.join(out_dir, "compress_config.json"), "w") as fh:
        json.dump({"bits": bits, "group_size": -1, "sparsity": 0.5, "damp_percent": 0.01,
                   "desc_act": False, "sym": True, "true_sequential": True, "lossless": "none",
                   "prunen": 2, "prunem": 4, "block_size": 128}, fh, indent=2)
    np.savez_compressed(os.path.join(out_dir, "dense.npz"), **dense)
    print(out_dir, {k: tuple(v.shape) for k, v in state.items() if k.endswith("qweight")})


def _load_sparsegpt(ref):
    """deltazip/core/sparsegpt.py uses relative imports: give it a stand-in parent package made of
    the two sibling files it needs, all loaded by file path."""
    import types
    pkg = types.ModuleType("dz_ref_core")
    pkg.__path__ = [os.path.join(ref, "deltazip/core")]
    sys.modules["dz_ref_core"] = pkg
    for name in ("quant", "sparsity_utils", "sparsegpt"):
        spec = importlib.util.spec_from_file_location(f"dz_ref_core.{name}",
                                                      os.path.join(ref, f"deltazip/core/{name}.py"))
        mod = importlib.util.module_from_spec(spec)
        sys.modules[f"dz_ref_core.{name}"] = mod
        spec.loader.exec_module(mod)
    return sys.modules["dz_ref_core.sparsegpt"], sys.modules["dz_ref_core.quant"]


def sparsegpt_case(ref, out_path, n, k, bits, seed):
    """SparseGPT.fasterprune (deltazip/core/sparsegpt.py:45-196) of the reference itself, on CPU,
    with a Hessian accumulated by its add_batch from random calibration inputs, prunen:prunem =
    2:4 and the symmetric per-row quantiser.  Stored: the delta, the upper Cholesky factor of the
    damped H^-1 (recomputed here with the same torch calls fasterprune makes, on the same H), and
    fasterprune's outputs.  The only change to the reference's behaviour is that its call of
    torch.cuda.synchronize() is made a no-op (this machine has no GPU)."""
    sparsegpt, quant = _load_sparsegpt(ref)
    torch.cuda.synchronize = lambda *a, **kw: None
    g = torch.Generator().manual_seed(seed)
    delta = torch.randn(n, k, generator=g) * 1e-2
    calib = torch.randn(96, k, generator=g) * (0.5 + torch.rand(k, generator=g))   # uneven column energy
    layer = torch.nn.Linear(k, n, bias=False)
    layer.weight.data = delta.clone()
    sg = sparsegpt.SparseGPT(layer)
    for i in range(0, 96, 32):
        sg.add_batch(calib[i:i + 32], None)
    H = sg.H.clone()
    sg.quantizer = quant.Quantizer()
    sg.quantizer.configure(bits, perchannel=True, sym=True, mse=False)
    scale, zero, g_idx, avg_loss, W = sg.fasterprune(0.5, prunen=2, prunem=4, blocksize=128, percdamp=0.01)
    # the factor fasterprune derived from H (same calls, same machine)
    Hd = H.clone()
    dead = torch.diag(Hd) == 0
    Hd[dead, dead] = 1
    damp = 0.01 * torch.mean(torch.diag(Hd))
    idx = torch.arange(k)
    Hd[idx, idx] += damp
    Hd = torch.linalg.cholesky(Hd)
    Hd = torch.cholesky_inverse(Hd)
    hinv = torch.linalg.cholesky(Hd, upper=True)
    np.savez_compressed(out_path, bits=np.int32(bits), delta=delta.numpy(), H=H.numpy(), hinv=hinv.numpy(),
                        wq=W.float().numpy(), scale=scale.flatten().numpy(), zero=zero.flatten().numpy(),
                        avg_loss=np.float32(avg_loss), nsamples=np.int32(sg.nsamples))
    print(out_path, "avg loss", avg_loss, "zeros", float((W == 0).float().mean()))


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <path of a deltazip checkout>")
    ref = sys.argv[1]
    quant = _load(os.path.join(ref, "deltazip/core/quant.py"), "ref_quant")
    qlinear = _load(os.path.join(ref, "deltazip/nn_modules/qlinear.py"), "ref_qlinear")
    torch.set_num_threads(8)
    cases = [
        # name, N, K, bits, M, seed, zero_row
        ("b4_n128_k256", 128, 256, 4, 8, 0, False),
        ("b2_n128_k256", 128, 256, 2, 8, 1, False),
        ("b4_n256_k192_edge", 256, 192, 4, 5, 2, True),
        ("b2_n256_k320_edge", 256, 320, 2, 3, 3, True),
        ("b8_n64_k128", 64, 128, 8, 4, 4, False),
    ]
    for name, n, k, bits, m, seed, zr in cases:
        out = reference_case(quant, qlinear, n, k, bits, m, seed, zr)
        assert bool(out["dense_is_fp16_exact"])
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
        print(name, {kk: getattr(v, "shape", None) for kk, v in out.items()})
    sparsegpt_case(ref, os.path.join(HERE, "sparsegpt_b4_n32_k256.npz"), 32, 256, 4, seed=20)
    sparsegpt_case(ref, os.path.join(HERE, "sparsegpt_b2_n32_k128.npz"), 32, 128, 2, seed=21)
    reference_checkpoint(quant, qlinear, os.path.join(HERE, "ref_ckpt_b4"), 4, seed=10)
    reference_checkpoint(quant, qlinear, os.path.join(HERE, "ref_ckpt_b2"), 2, seed=11)


if __name__ == "__main__":
    main()
