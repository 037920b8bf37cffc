"""tcgen05 flash attention against an fp32 PyTorch reference."""
import math

import pytest
import torch

from eth_b200 import ops
from eth_b200.ops import native
from eth_b200.ops import functional as Fn
from eth_b200.ops.functional import attention_ref

pytestmark = pytest.mark.gpu


def _rel_err(a, b):
    """max(Frobenius-norm relative error, largest element error relative to the largest reference
    magnitude): the second term catches a single bad row or element that the norm would hide."""
    a, b = a.float(), b.float()
    fro = ((a - b).norm() / (b.norm() + 1e-12)).item()
    worst = ((a - b).abs().max() / (b.abs().max() + 1e-12)).item()
    err = max(fro, worst)
    return err if err == err else float("inf")   # a NaN anywhere must fail every `< tolerance` check


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,S,H,D", [(1, 128, 1, 128), (2, 256, 2, 128), (1, 512, 3, 64), (2, 384, 2, 128),
                                      (1, 200, 2, 64), (2, 2048, 4, 128), (1, 1000, 2, 128)])
@pytest.mark.parametrize("causal", [True, False])
def test_attention_forward(dtype, B, S, H, D, causal):
    torch.manual_seed(0)
    qkv = torch.randn(B, S, H, 3, D, device="cuda", dtype=dtype)
    q, k, v = qkv[:, :, :, 0], qkv[:, :, :, 1], qkv[:, :, :, 2]
    o = ops.flash_attention(q, k, v, causal=causal)
    native.check_status()
    ref = attention_ref(q, k, v, 1.0 / math.sqrt(D), causal)
    assert _rel_err(o, ref) < 1e-2


def test_attention_large_scores_trigger_rescale():
    torch.manual_seed(1)
    B, S, H, D = 1, 512, 2, 128
    q = torch.randn(B, S, H, D, device="cuda", dtype=torch.bfloat16) * 4
    k = torch.randn(B, S, H, D, device="cuda", dtype=torch.bfloat16) * 4
    # make later keys score much higher so the running maximum keeps growing
    k = k * torch.linspace(0.2, 3.0, S, device="cuda").view(1, S, 1, 1).to(torch.bfloat16)
    v = torch.randn(B, S, H, D, device="cuda", dtype=torch.bfloat16)
    o = ops.flash_attention(q, k, v, causal=True)
    native.check_status()
    ref = attention_ref(q, k, v, 1.0 / math.sqrt(D), True)
    assert _rel_err(o, ref) < 2e-2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,S,H,D", [(1, 128, 1, 128), (2, 256, 2, 128), (1, 512, 3, 64), (2, 384, 2, 128),
                                      (1, 200, 2, 64), (1, 2048, 2, 128), (1, 1000, 2, 128)])
@pytest.mark.parametrize("causal", [True, False])
def test_attention_backward(dtype, B, S, H, D, causal):
    torch.manual_seed(0)
    qkv = torch.randn(B, S, H, 3, D, device="cuda", dtype=dtype)
    q, k, v = (qkv[:, :, :, i].detach().requires_grad_(True) for i in range(3))
    o = ops.flash_attention(q, k, v, causal=causal)
    do = torch.randn_like(o)
    gq, gk, gv = torch.autograd.grad(o, (q, k, v), do)
    native.check_status()
    qr, kr, vr = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    ref = attention_ref(qr, kr, vr, 1.0 / math.sqrt(D), causal)
    rq, rk, rv = torch.autograd.grad(ref, (qr, kr, vr), do.float())
    assert _rel_err(gv, rv) < 2e-2
    assert _rel_err(gk, rk) < 2e-2
    assert _rel_err(gq, rq) < 2e-2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("causal", [True, False])
def test_attention_backward_more_tiles_than_sms(dtype, causal):
    """384 key/value tiles and 384 query tiles: the persistent backward kernels take three rounds (the
    second in reversed CTA order, the third partial), so a CTA processes up to three tiles back to back
    with its barrier parities, ring positions and accumulators carried from tile to tile."""
    torch.manual_seed(5)
    B, S, H, D = 4, 1024, 12, 128
    qkv = torch.randn(B, S, H, 3, D, device="cuda", dtype=dtype)
    q, k, v = (qkv[:, :, :, i].detach().requires_grad_(True) for i in range(3))
    o = ops.flash_attention(q, k, v, causal=causal)
    do = torch.randn_like(o)
    gq, gk, gv = torch.autograd.grad(o, (q, k, v), do)
    native.check_status()
    qr, kr, vr = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    ref = attention_ref(qr, kr, vr, 1.0 / math.sqrt(D), causal)
    rq, rk, rv = torch.autograd.grad(ref, (qr, kr, vr), do.float())
    assert _rel_err(o, ref) < 2e-2
    assert _rel_err(gv, rv) < 2e-2
    assert _rel_err(gk, rk) < 2e-2
    assert _rel_err(gq, rq) < 2e-2


def test_unfused_attention_matches_flash():
    """The four-op attention of the older manifest (library batched GEMMs + this library's softmax)
    agrees with the flash kernel, forward and backward."""
    torch.manual_seed(21)
    B, S, H, D = 2, 512, 4, 64
    q, k, v = (torch.randn(B, S, H, D, device="cuda", dtype=torch.bfloat16, requires_grad=True) for _ in range(3))
    out_f = ops.flash_attention(q, k, v)
    out_u = Fn.unfused_attention(q, k, v)
    assert _rel_err(out_u, out_f) < 2e-2
    do = torch.randn_like(out_f)
    gf = torch.autograd.grad(out_f, (q, k, v), do)
    gu = torch.autograd.grad(out_u, (q, k, v), do)
    for a, b in zip(gf, gu):
        assert _rel_err(b, a) < 3e-2
