"""The decode-step kernels around the SBMM (RMSNorm with residual, SiLU*up, rotary + paged-cache
write, paged decode attention) against plain PyTorch float32 evaluations of the same formulas
(the reference's own PyTorch twins: serving/vllm/model_executor/layers/layernorm.py:27-45,
activation.py:28-32, rotary_embedding.py `_forward`, attention as softmax(q k^T / sqrt(d)) v).
Tolerances: results are rounded to fp16 / bf16 once or twice, so 2e-3 (fp16) / 1.6e-2 (bf16)
relative to the row norm."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-9)).item()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m,h", [(1, 256), (64, 4096), (37, 5120), (5, 8192)])
def test_rms_norm_with_and_without_residual(dtype, m, h):
    from deltazip_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(m + h)
    x = torch.randn((m, h), generator=g, device="cuda").to(dtype)
    r = torch.randn((m, h), generator=g, device="cuda").to(dtype)
    w = (1 + 0.1 * torch.randn(h, generator=g, device="cuda")).to(dtype)
    tol = 2e-3 if dtype == torch.float16 else 1.6e-2

    def ref(v):
        vf = v.float()
        n = (vf * torch.rsqrt(vf.pow(2).mean(-1, keepdim=True) + 1e-5)).to(dtype)
        return n * w
    assert rel(ops.rms_norm(x, w, 1e-5), ref(x)) <= tol
    r2 = r.clone()
    out = ops.rms_norm(x, w, 1e-5, residual=r2)
    s = (x.float() + r.float()).to(dtype)
    assert torch.equal(r2, s)                      # residual updated in place, one rounding
    assert rel(out, ref(s)) <= tol


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_silu_and_mul(dtype):
    from deltazip_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn((33, 2 * 11008), generator=g, device="cuda").to(dtype)
    want = torch.nn.functional.silu(x[:, :11008].float()) * x[:, 11008:].float()
    assert rel(ops.silu_and_mul(x), want) <= (2e-3 if dtype == torch.float16 else 1.6e-2)


def rotary_ref(t, positions, theta):
    """neox pairing: (d, d + 64) rotate by pos * theta^(-2d/128); t: [M, H, 128] float32."""
    inv = 1.0 / (theta ** (torch.arange(0, 128, 2, device=t.device, dtype=torch.float32) / 128))
    ang = positions.float()[:, None] * inv
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    a, b = t[..., :64], t[..., 64:]
    return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)


@pytest.mark.parametrize("qh,kvh", [(4, 4), (8, 1), (5, 5)])
def test_rotary_and_cache_write(qh, kvh):
    from deltazip_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(qh)
    m, bs, nblocks = 19, 16, 8
    qkv = torch.randn((m, (qh + 2 * kvh) * 128), generator=g, device="cuda").half()
    pos = torch.randint(0, 3000, (m,), generator=g, device="cuda")
    slots = torch.randperm(nblocks * bs, generator=g, device="cuda")[:m].to(torch.int64)
    slots[3] = -1                                                       # this token is not cached
    kc = torch.zeros((nblocks * bs, kvh, 128), dtype=torch.float16, device="cuda")
    vc = torch.zeros_like(kc)
    orig = qkv.clone()
    ops.rotary_and_cache(qkv, pos, qh, kvh, 10000.0, kc, vc, slots)
    q_ref = rotary_ref(orig[:, :qh * 128].float().reshape(m, qh, 128), pos, 10000.0)
    k_ref = rotary_ref(orig[:, qh * 128:(qh + kvh) * 128].float().reshape(m, kvh, 128), pos, 10000.0)
    assert rel(qkv[:, :qh * 128].reshape(m, qh, 128), q_ref) <= 2e-3
    assert rel(qkv[:, qh * 128:(qh + kvh) * 128].reshape(m, kvh, 128), k_ref) <= 2e-3
    assert torch.equal(qkv[:, (qh + kvh) * 128:], orig[:, (qh + kvh) * 128:])   # v untouched
    keep = slots >= 0
    assert torch.equal(kc[slots[keep]], qkv[keep][:, qh * 128:(qh + kvh) * 128].reshape(-1, kvh, 128))
    assert torch.equal(vc[slots[keep]], orig[keep][:, (qh + kvh) * 128:].reshape(-1, kvh, 128))
    untouched = torch.ones(nblocks * bs, dtype=torch.bool, device="cuda")
    untouched[slots[keep]] = False
    assert not kc[untouched].any() and not vc[untouched].any()


@pytest.mark.parametrize("qh,kvh,splits", [(4, 4, 1), (8, 1, 1), (8, 2, 4), (32, 32, 1), (8, 1, 8), (8, 4, 2), (4, 2, 1)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_paged_decode_attention(qh, kvh, splits, dtype):
    from deltazip_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(qh * 10 + splits)
    b, bs = 6, 16
    lens = torch.tensor([1, 5, 16, 17, 200, 333], dtype=torch.int32, device="cuda")
    maxb = (int(lens.max()) + bs - 1) // bs
    nblocks = b * maxb + 3
    perm = torch.randperm(nblocks, generator=g, device="cuda")[: b * maxb].to(torch.int32)
    tables = perm.reshape(b, maxb).contiguous()
    kc = torch.randn((nblocks * bs, kvh, 128), generator=g, device="cuda").to(dtype)
    vc = torch.randn((nblocks * bs, kvh, 128), generator=g, device="cuda").to(dtype)
    qkv = torch.randn((b, (qh + 2 * kvh) * 128), generator=g, device="cuda").to(dtype)
    scale = 1 / math.sqrt(128)
    for rep in range(2):                           # twice: the split tickets must be back at zero
        out = ops.paged_attention_decode(qkv, kc, vc, tables, lens, qh, kvh, bs, scale, splits=splits)
        torch.cuda.synchronize()
        for i in range(b):
            n = int(lens[i])
            slot = (tables[i].long()[:, None] * bs + torch.arange(bs, device="cuda")[None]).reshape(-1)[:n]
            k = kc[slot].float().repeat_interleave(qh // kvh, dim=1)            # [n, qh, 128]
            v = vc[slot].float().repeat_interleave(qh // kvh, dim=1)
            q = qkv[i, : qh * 128].float().reshape(qh, 128)
            p = torch.softmax(torch.einsum("hd,nhd->hn", q, k) * scale, dim=-1)
            want = torch.einsum("hn,nhd->hd", p, v).reshape(-1)
            assert rel(out[i], want) <= (2e-3 if dtype == torch.float16 else 1.6e-2), (i, rep)
