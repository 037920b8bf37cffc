"""Numerics of the sm_100a kernels against plain PyTorch fp32 references of the same op."""
import math

import pytest
import torch

from eth_b200 import ops
from eth_b200.ops import functional as Fn
from eth_b200.ops import native

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel_err(a, b):
    """max(Frobenius-norm relative error, largest element error relative to the largest reference
    magnitude): the second term catches a single bad row or element that the norm would hide."""
    a, b = a.float(), b.float()
    fro = ((a - b).norm() / (b.norm() + 1e-12)).item()
    worst = ((a - b).abs().max() / (b.abs().max() + 1e-12)).item()
    err = max(fro, worst)
    return err if err == err else float("inf")   # a NaN anywhere must fail every `< tolerance` check


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    native.check_status()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(128, 256, 64), (256, 512, 256), (384, 1024, 512), (100, 136, 72),
                                   (1024, 2048, 1024), (4096, 6144, 2048)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
def test_gemm_layouts(dtype, shape, a_mn, b_mn):
    M, N, K = shape
    if (a_mn and M % 8) or (b_mn and N % 8):
        pytest.skip("MN-major operands need 16-byte aligned rows")
    torch.manual_seed(0)
    a = torch.randn((K, M) if a_mn else (M, K), device=DEV, dtype=dtype)
    b = torch.randn((K, N) if b_mn else (N, K), device=DEV, dtype=dtype)
    out = ops.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    ref = (a.t() if a_mn else a).float() @ (b if b_mn else b.t()).float()
    assert _rel_err(out, ref) < 5e-3
    native.check_status()


@pytest.mark.parametrize("variant", [3, 4])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (True, False), (False, True), (True, True)])
@pytest.mark.parametrize("shape", [(512, 512, 256), (1000, 776, 136), (128, 256, 64), (2304, 1536, 1024)])
def test_gemm_cta_pair_variants(variant, a_mn, b_mn, shape):
    """The two-CTA (256-row) kernels against fp32 matmul, all operand layouts, ragged edges."""
    M, N, K = shape
    torch.manual_seed(5)
    dtype = torch.bfloat16
    a = torch.randn((K, M) if a_mn else (M, K), device=DEV, dtype=dtype)
    b = torch.randn((K, N) if b_mn else (N, K), device=DEV, dtype=dtype)
    bias = torch.randn(N, device=DEV, dtype=dtype)
    native.lib().set_gemm_variant(variant)
    try:
        out = ops.gemm(a, b, a_mn=a_mn, b_mn=b_mn, bias=bias)
        again = ops.gemm(a, b, a_mn=a_mn, b_mn=b_mn, bias=bias)
    finally:
        native.lib().set_gemm_variant(0)
    ref = (a.t() if a_mn else a).float() @ (b if b_mn else b.t()).float() + bias.float()
    assert _rel_err(out, ref) < 5e-3
    assert torch.equal(out, again)
    native.check_status()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_gemm_epilogues(dtype):
    torch.manual_seed(1)
    M, N, K = 512, 768, 256
    a = torch.randn(M, K, device=DEV, dtype=dtype)
    b = torch.randn(N, K, device=DEV, dtype=dtype) * 0.1
    bias = torch.randn(N, device=DEV, dtype=dtype)
    res = torch.randn(M, N, device=DEV, dtype=dtype)
    base = a.float() @ b.float().t()
    # bias + gelu second output
    pre = torch.empty(M, N, device=DEV, dtype=dtype)
    act = torch.empty_like(pre)
    ops.gemm(a, b, out=pre, bias=bias, gelu_out=act)
    assert _rel_err(pre, base + bias.float()) < 5e-3
    assert _rel_err(act, torch.nn.functional.gelu(base + bias.float(), approximate="tanh")) < 1e-2
    # residual add
    out = ops.gemm(a, b, aux=res, aux_mode=Fn.AUX_ADD)
    assert _rel_err(out, base + res.float()) < 5e-3
    # gelu-grad epilogue
    out = ops.gemm(a, b, aux=res, aux_mode=Fn.AUX_GELU_GRAD)
    assert _rel_err(out, base * Fn.gelu_tanh_grad_ref(res.float())) < 1e-2
    # fp32 accumulate output with alpha
    acc = torch.randn(M, N, device=DEV, dtype=torch.float32)
    ref = acc + 0.5 * base
    ops.gemm(a, b, out=acc, accumulate=True, alpha=0.5)
    assert _rel_err(acc, ref) < 2e-3
    # 16-bit accumulate
    acc16 = torch.randn(M, N, device=DEV, dtype=dtype)
    ref = acc16.float() + base
    ops.gemm(a, b, out=acc16, accumulate=True)
    assert _rel_err(acc16, ref) < 1e-2


def test_gemm_strided_views():
    torch.manual_seed(2)
    big = torch.randn(512, 3 * 256, device=DEV, dtype=torch.bfloat16)
    a = big[:, 256:512]  # row stride 768, inner contiguous
    w = torch.randn(384, 256, device=DEV, dtype=torch.bfloat16)
    out = ops.gemm(a, w)
    assert _rel_err(out, a.float() @ w.float().t()) < 5e-3


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("hidden", [64, 2048, 4096, 5120])
def test_layernorm(dtype, hidden):
    torch.manual_seed(3)
    rows = 777
    x = torch.randn(rows, hidden, device=DEV, dtype=dtype, requires_grad=True)
    g = (1 + 0.1 * torch.randn(hidden, device=DEV)).to(dtype).requires_grad_(True)
    b = (0.1 * torch.randn(hidden, device=DEV)).to(dtype).requires_grad_(True)
    y = ops.layer_norm(x, g, b, 1e-5)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr, gr, br = (t.detach().float().requires_grad_(True) for t in (x, g, b))
    yr = torch.nn.functional.layer_norm(xr, (hidden,), gr, br, 1e-5)
    yr.backward(dy.float())
    assert _rel_err(y, yr) < 1e-2
    assert _rel_err(x.grad, xr.grad) < 1e-2
    assert _rel_err(g.grad, gr.grad) < 2e-2
    assert _rel_err(b.grad, br.grad) < 2e-2


def test_layernorm_main_grad_accumulates():
    hidden, rows = 256, 300
    x = torch.randn(rows, hidden, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    g = torch.ones(hidden, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    b = torch.zeros(hidden, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    g.main_grad = torch.full((hidden,), 2.0, device=DEV)
    b.main_grad = torch.full((hidden,), 3.0, device=DEV)
    y = ops.layer_norm(x, g, b, 1e-5)
    dy = torch.randn_like(y)
    y.backward(dy)
    assert g.grad is None and b.grad is None
    assert _rel_err(b.main_grad, 3.0 + dy.float().sum(0)) < 1e-3


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_bias_gelu(dtype):
    x = torch.randn(500, 1024, device=DEV, dtype=dtype, requires_grad=True)
    b = torch.randn(1024, device=DEV, dtype=dtype, requires_grad=True)
    y = ops.bias_gelu(x, b)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr, br = x.detach().float().requires_grad_(True), b.detach().float().requires_grad_(True)
    yr = torch.nn.functional.gelu(xr + br, approximate="tanh")
    yr.backward(dy.float())
    assert _rel_err(y, yr) < 1e-2
    assert _rel_err(x.grad, xr.grad) < 1e-2
    assert _rel_err(b.grad, br.grad) < 2e-2


@pytest.mark.parametrize("p", [0.0, 0.1])
def test_bias_dropout_add(p):
    dtype = torch.bfloat16
    x = torch.randn(300, 512, device=DEV, dtype=dtype, requires_grad=True)
    b = torch.randn(512, device=DEV, dtype=dtype, requires_grad=True)
    r = torch.randn(300, 512, device=DEV, dtype=dtype, requires_grad=True)
    out = ops.bias_dropout_add(x, b, r, p, seed=1234, offset=7)
    keep = Fn._keep_mask_ref(x.shape, p, 1234, 7, "cpu").to(DEV) if p > 0 else torch.ones_like(x, dtype=torch.bool)
    ref = r.float() + torch.where(keep, (x.float() + b.float()) / (1 - p), torch.zeros_like(x.float()))
    assert _rel_err(out, ref) < 1e-2
    if p > 0:
        frac = keep.float().mean().item()
        assert abs(frac - (1 - p)) < 0.01
    dy = torch.randn_like(out)
    out.backward(dy)
    dxr = torch.where(keep, dy.float() / (1 - p), torch.zeros_like(dy.float()))
    assert _rel_err(x.grad, dxr) < 1e-2
    assert _rel_err(r.grad, dy) < 1e-6
    assert _rel_err(b.grad, dxr.sum(0)) < 2e-2


def test_softmax_family():
    dtype = torch.float16
    x = torch.randn(6, 128, 128, device=DEV, dtype=dtype, requires_grad=True)
    y = ops.scaled_upper_triang_masked_softmax(x, 0.5)
    tri = torch.triu(torch.ones(128, 128, dtype=torch.bool, device=DEV), 1)
    xr = x.detach().float().requires_grad_(True)
    yr = torch.softmax((xr * 0.5).masked_fill(tri, float("-inf")), -1)
    assert _rel_err(y, yr) < 5e-3
    dy = torch.randn_like(y)
    y.backward(dy)
    yr.backward(dy.float())
    assert _rel_err(x.grad, xr.grad) < 1e-2
    # explicit mask
    x4 = torch.randn(2, 3, 64, 96, device=DEV, dtype=dtype)
    mask = torch.rand(2, 1, 64, 96, device=DEV) < 0.3
    y4 = ops.scaled_masked_softmax(x4, mask, 2.0)
    ref = torch.softmax((x4.float() * 2.0).masked_fill(mask, -10000.0), -1)
    assert _rel_err(y4, ref) < 5e-3
    y0 = ops.scaled_softmax(x4, 1.5)
    assert _rel_err(y0, torch.softmax(x4.float() * 1.5, -1)) < 5e-3


def test_embedding_fwd_bwd():
    dtype = torch.bfloat16
    V, H, S, B = 1000, 256, 64, 4
    word = torch.randn(500, H, device=DEV, dtype=dtype, requires_grad=True)  # shard [250, 750)
    pos = torch.randn(S, H, device=DEV, dtype=dtype, requires_grad=True)
    tok = torch.randint(0, V, (B, S), device=DEV)
    out = ops.embedding(tok, word, pos, S, vocab_start=250, add_pos=True)
    t = tok.reshape(-1) - 250
    mine = (t >= 0) & (t < 500)
    ref = word.float()[t.clamp(0, 499)] * mine[:, None] + pos.float().repeat(B, 1)
    assert _rel_err(out, ref) < 1e-2
    word.main_grad = torch.zeros(500, H, device=DEV)
    pos.main_grad = torch.zeros(S, H, device=DEV)
    dy = torch.randn_like(out)
    out.backward(dy)
    refw = torch.zeros(500, H, device=DEV).index_add_(0, t[mine], dy.float()[mine])
    assert _rel_err(word.main_grad, refw) < 1e-3
    assert _rel_err(pos.main_grad, dy.float().view(B, S, H).sum(0)) < 1e-3


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_cross_entropy(dtype):
    rows, V = 333, 4096
    logits = (torch.randn(rows, V, device=DEV) * 3).to(dtype)
    tgt = torch.randint(0, V, (rows,), device=DEV)
    lref = logits.detach().float().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(lref, tgt, reduction="none")
    w = torch.rand(rows, device=DEV)
    (ref * w).sum().backward()
    l2 = logits.clone().requires_grad_(True)
    loss = ops.vocab_parallel_cross_entropy(l2, tgt)
    assert _rel_err(loss, ref) < 2e-3
    (loss * w).sum().backward()
    assert _rel_err(l2.grad, lref.grad) < 2e-2
    # two vocab shards combined through the gather hook
    halves = [logits[:, : V // 2].contiguous(), logits[:, V // 2:].contiguous()]
    stats = []
    for i, h in enumerate(halves):
        st = torch.empty(rows, 3, device=DEV)
        native.lib().ce_local_stats(h, tgt, st, i * (V // 2))
        stats.append(st)
    both = torch.stack(stats)
    loss2 = ops.vocab_parallel_cross_entropy(halves[0], tgt, 0, gather_fn=lambda s: both)
    assert _rel_err(loss2, ref) < 2e-3


def test_adam_and_norm():
    n = 100003
    p16 = torch.randn(n, device=DEV).to(torch.bfloat16)
    master = p16.float().clone()
    g = torch.randn(n, device=DEV) * 64.0
    m = torch.zeros(n, device=DEV)
    v = torch.zeros(n, device=DEV)
    ctrl = torch.zeros(2, device=DEV)
    native.lib().grad_norm_sq(g, 1.0, ctrl)
    assert abs(ctrl[0].item() - g.pow(2).sum().item()) / ctrl[0].item() < 1e-4
    ref_p = master.clone().requires_grad_(True)
    opt = torch.optim.AdamW([ref_p], lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.01)
    clip = min(1.0, 1.0 / (ctrl[0].sqrt().item() / 64 + 1e-6))
    for step in (1, 2):
        ref_p.grad = (g / 64) * clip
        opt.step()
        native.lib().fused_adam(p16, master, g, m, v, ctrl, 1e-3, 0.9, 0.95, 1e-8, 0.01, step,
                                1 / 64.0, 1.0, True, False)
    assert _rel_err(master, ref_p.detach()) < 1e-5
    assert _rel_err(p16, ref_p.detach()) < 1e-2
    # overflow flag skips the update
    ctrl[1] = 1.0
    before = master.clone()
    native.lib().fused_adam(p16, master, g, m, v, ctrl, 1e-3, 0.9, 0.95, 1e-8, 0.01, 3, 1 / 64.0, 1.0, True, False)
    assert torch.equal(before, master)


def test_linear_autograd_main_grad():
    torch.manual_seed(5)
    dtype = torch.bfloat16
    x = torch.randn(512, 256, device=DEV, dtype=dtype, requires_grad=True)
    w = (torch.randn(384, 256, device=DEV) * 0.05).to(dtype).requires_grad_(True)
    b = torch.randn(384, device=DEV, dtype=dtype, requires_grad=True)
    w.main_grad = torch.zeros(384, 256, device=DEV)
    b.main_grad = torch.zeros(384, device=DEV)
    for fn, ref_fn in ((ops.linear, lambda z: z), (ops.linear_gelu, lambda z: torch.nn.functional.gelu(z, approximate="tanh"))):
        w.main_grad.zero_(); b.main_grad.zero_(); x.grad = None
        y = fn(x, w, b)
        dy = torch.randn_like(y)
        y.backward(dy)
        xr, wr, br = (t.detach().float().requires_grad_(True) for t in (x, w, b))
        yr = ref_fn(xr @ wr.t() + br)
        yr.backward(dy.float())
        assert _rel_err(y, yr) < 1e-2
        assert _rel_err(x.grad, xr.grad) < 1.5e-2
        assert _rel_err(w.main_grad, wr.grad) < 1.5e-2
        assert _rel_err(b.main_grad, br.grad) < 2e-2
        assert w.grad is None


def test_synthetic_batch_matches_reference_formula():
    ids = torch.tensor([0, 5, 123456], device=DEV)
    S, V = 64, 50257
    tok = torch.empty(3, S, dtype=torch.long, device=DEV)
    lab = torch.empty_like(tok)
    mask = torch.empty(3, S, device=DEV)
    native.lib().synthetic_batch(tok, lab, mask, ids, S, V)
    pos = torch.arange(S, device=DEV)
    ref = (ids[:, None] * 1103515245 + pos[None] * 12345).remainder(V)
    assert torch.equal(tok, ref)
    assert torch.equal(mask, ((ids[:, None] + pos[None]) % 4 != 0).float())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,hidden", [(777, 2048), (130, 4096), (64, 5120), (1000, 256)])
def test_layernorm_bwd_with_residual_gradient(dtype, rows, hidden):
    """Fused LayerNorm backward (dx + residual-branch gradient, dgamma, dbeta) against fp32 autograd."""
    from eth_b200.ops import raw
    torch.manual_seed(11)
    x = torch.randn(rows, hidden, device=DEV, dtype=dtype)
    g = (1 + 0.1 * torch.randn(hidden, device=DEV)).to(dtype)
    b = (0.1 * torch.randn(hidden, device=DEV)).to(dtype)
    g.main_grad = torch.zeros(hidden, device=DEV, dtype=torch.float32)
    b.main_grad = torch.zeros(hidden, device=DEV, dtype=torch.float32)
    y, mean, rstd = raw.ln_fwd(x, g, b, 1e-5)
    dy, res = torch.randn_like(x), torch.randn_like(x)
    dx = raw.ln_bwd(dy, x, g, b, mean, rstd, residual_grad=res)
    xr, gr, br = (t.detach().float().requires_grad_(True) for t in (x, g, b))
    torch.nn.functional.layer_norm(xr, (hidden,), gr, br, 1e-5).backward(dy.float())
    assert _rel_err(dx, xr.grad + res.float()) < 1e-2
    assert _rel_err(g.main_grad, gr.grad) < 5e-3
    assert _rel_err(b.main_grad, br.grad) < 5e-3
    # a second call accumulates into main_grad
    raw.ln_bwd(dy, x, g, b, mean, rstd)
    assert _rel_err(g.main_grad, 2 * gr.grad) < 5e-3


@pytest.mark.parametrize("rows,cols", [(8192, 2048), (333, 4096), (50, 256), (64, 264)])
def test_dropout_bwd_colsum(rows, cols):
    """dx and its column sums from the fused kernel equal the two separate kernels (same Philox mask)."""
    from eth_b200.ops import raw
    torch.manual_seed(12)
    dy = torch.randn(rows, cols, device=DEV, dtype=torch.bfloat16)
    p, seed, off = 0.1, 77, 5
    dx, db = raw.dropout_bwd_colsum(dy, p, seed, off)
    ref = raw.dropout_bwd(dy, p, seed, off)
    assert torch.equal(dx, ref)
    assert db.dtype == torch.float32
    exact = torch.where(ref != 0, dy.float() / (1.0 - p), torch.zeros_like(dy.float())).sum(0)   # unrounded terms
    fused = cols % 256 == 0   # otherwise the two separate kernels run and sum the rounded dx
    assert _rel_err(db, exact) < (1e-5 if fused else 3e-3)
    zeros = (dx == 0).float().mean().item()
    assert abs(zeros - p) < 0.02


@pytest.mark.parametrize("rows,hidden", [(4096, 2048), (777, 1024), (300, 4096)])
def test_deferred_column_sums_equal_per_call_sums(rows, hidden):
    """Three backward calls that leave their partial column sums in the op's slabs and flush with
    the third equal three calls that sum at once: LayerNorm's dgamma / dbeta and the bias gradient
    behind a dropout. A second round shows the flush left the slabs clear."""
    from eth_b200.ops import raw
    torch.manual_seed(21)
    dtype = torch.bfloat16
    g = (1 + 0.1 * torch.randn(hidden, device=DEV)).to(dtype)
    b = (0.1 * torch.randn(hidden, device=DEV)).to(dtype)
    bias = torch.zeros(hidden, device=DEV, dtype=dtype)
    data = []
    for _ in range(3):
        x = torch.randn(rows, hidden, device=DEV, dtype=dtype)
        y, mean, rstd = raw.ln_fwd(x, g, b, 1e-5)
        data.append((x, mean, rstd, torch.randn_like(x)))

    def run(deferred, rounds):
        for t in (g, b, bias):
            t.main_grad = torch.zeros(hidden, device=DEV, dtype=torch.float32)
        ln_slabs, drop_slabs = raw.ColumnSumSlabs(), raw.ColumnSumSlabs()
        outs = []
        for _ in range(rounds):
            for i, (x, mean, rstd, dy) in enumerate(data):
                mode = raw.WS_IMMEDIATE if not deferred else (raw.WS_FLUSH if i == 2 else raw.WS_ACCUMULATE)
                outs.append(raw.ln_bwd(dy, x, g, b, mean, rstd, slabs=ln_slabs, ws_mode=mode))
                if deferred:
                    dx = raw.dropout_bwd_colsum_into(dy, 0.1, 5, i, bias.main_grad, drop_slabs, mode)
                    assert dx is not None
                else:
                    dx, db = raw.dropout_bwd_colsum(dy, 0.1, 5, i)
                    bias.main_grad += db
                outs.append(dx)
        return outs, [t.main_grad.clone() for t in (g, b, bias)]

    for rounds in (1, 2):
        ref_out, ref_grads = run(False, rounds)
        out, grads = run(True, rounds)
        assert all(torch.equal(a, c) for a, c in zip(out, ref_out))
        for got, ref in zip(grads, ref_grads):
            assert _rel_err(got, ref) < 1e-5
    native.check_status()


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True)])
@pytest.mark.parametrize("shape", [(8192, 2048, 256), (8192, 3072, 192), (4864, 4096, 128)])
def test_gemm_tail_split_half_tiles(a_mn, b_mn, shape):
    """Shapes whose last wave of 256 x 256 tiles is sparsely filled run that wave as 256 x 128 half
    tiles; results must equal the unsplit schedule and the fp32 reference, with every epilogue."""
    M, N, K = shape
    torch.manual_seed(8)
    dt = torch.bfloat16
    a = torch.randn((K, M) if a_mn else (M, K), device=DEV, dtype=dt)
    b = torch.randn((K, N) if b_mn else (N, K), device=DEV, dtype=dt) * 0.1
    bias = torch.randn(N, device=DEV, dtype=dt)
    aux = torch.randn(M, N, device=DEV, dtype=dt)
    outs = {}
    for on in (1, 0):
        native.lib().set_gemm_tail_split(on)
        try:
            plain = ops.gemm(a, b, a_mn=a_mn, b_mn=b_mn, bias=bias)
            act = torch.empty_like(plain)
            pre = torch.empty_like(plain)
            ops.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=pre, bias=bias, gelu_out=act)
            res = ops.gemm(a, b, a_mn=a_mn, b_mn=b_mn, aux=aux, aux_mode=Fn.AUX_ADD)
            acc = torch.ones(M, N, device=DEV, dtype=torch.float32)
            ops.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=acc, accumulate=True)
        finally:
            native.lib().set_gemm_tail_split(1)
        outs[on] = (plain, act, res, acc)
    ref = (a.t() if a_mn else a).float() @ (b if b_mn else b.t()).float()
    assert _rel_err(outs[1][0], ref + bias.float()) < 5e-3
    assert _rel_err(outs[1][1], torch.nn.functional.gelu(ref + bias.float(), approximate="tanh")) < 1e-2
    assert _rel_err(outs[1][2], ref + aux.float()) < 5e-3
    assert _rel_err(outs[1][3], ref + 1.0) < 2e-3
    for x, y in zip(outs[1], outs[0]):
        assert torch.equal(x, y)
    native.check_status()


@pytest.mark.parametrize("shape", [(4096, 2048, 512), (1000, 1024, 256), (256, 128, 64)])
@pytest.mark.parametrize("with_residual", [True, False])
def test_gemm_epilogue_dropout_draws_the_mask_of_the_elementwise_kernel(shape, with_residual):
    """bias + dropout (+ residual) in the GEMM epilogue against the GEMM followed by the
    bias-dropout-add kernel with the same (seed, offset): exactly the same elements are dropped, so
    the backward kernels, which regenerate the mask, fit both; kept values agree to rounding."""
    from eth_b200.ops import raw
    m, n, k = shape
    torch.manual_seed(31)
    x = torch.randn(m, k, device=DEV, dtype=torch.bfloat16)
    w = (torch.randn(n, k, device=DEV) * 0.05).to(torch.bfloat16)
    bias = (torch.randn(n, device=DEV) * 0.1).to(torch.bfloat16)
    res = torch.randn(m, n, device=DEV, dtype=torch.bfloat16) if with_residual else None
    p, seed, off = 0.1, 1234, (7 << 24) + 3
    fused = raw.linear_fwd(x, w, bias, residual=res, dropout=(p, seed, off))
    plain = raw.bias_dropout_add_fwd(raw.linear_fwd(x, w), bias, res, p, seed, off)
    # fp32 reference with the mask taken from the kernel itself
    keep = raw.dropout_bwd(torch.ones(m, n, device=DEV, dtype=torch.bfloat16), p, seed, off) != 0
    ref = torch.where(keep, (x.float() @ w.float().t() + bias.float()) / (1 - p), torch.zeros((), device=DEV))
    if with_residual:
        ref = ref + res.float()
        dropped_fused = (fused.float() - res.float()) == 0
    else:
        dropped_fused = fused == 0
    # every element the mask drops is dropped by the fused kernel; a kept element only looks dropped
    # where a small value vanishes in the rounding of (value + residual)
    assert torch.equal(dropped_fused | keep, torch.ones_like(keep))
    assert (dropped_fused & keep).float().mean() < (2e-2 if with_residual else 1e-3)
    assert abs((~keep).float().mean().item() - p) < 0.02
    assert _rel_err(fused, ref) < 1e-2 and _rel_err(plain, ref) < 1.5e-2
    native.check_status()
