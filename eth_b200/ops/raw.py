"""Forward / backward primitives without autograd, used by the explicit stage program.

The training runtime does not build an autograd graph: every op of the stage program has a
hand-written forward and backward that call these primitives, so the host cost per op is one
Python call into the native library and buffers can be reused deterministically. CUDA tensors
run the sm_100a kernels; CPU tensors run a PyTorch restatement (tests, validation).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from . import native
from .functional import (AUX_ADD, AUX_GELU_GRAD, AUX_NONE, _keep_mask_ref, _workspace, attention_ref,  # noqa: F401
                         colsum, gelu_tanh_grad_ref, gemm)


def _grad_of(p):
    mg = getattr(p, "main_grad", None)
    if mg is None:
        raise RuntimeError("parameter has no main_grad buffer")
    return mg


# ---------------------------------------------------------------------------------- LayerNorm
def ln_fwd(x, gamma, beta, eps):
    hidden = x.shape[-1]
    rows = x.numel() // hidden
    if native.use_native(x):
        y = torch.empty_like(x)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        native.lib().layernorm_fwd(x, gamma, beta, y, mean, rstd, eps)
        return y, mean, rstd
    xf = x.float().reshape(rows, hidden)
    mean = xf.mean(1)
    rstd = torch.rsqrt(xf.var(1, unbiased=False) + eps)
    y = ((xf - mean[:, None]) * rstd[:, None] * gamma.float() + beta.float()).to(x.dtype).reshape(x.shape)
    return y, mean, rstd


WS_IMMEDIATE, WS_ACCUMULATE, WS_FLUSH = 0, 1, 2   # what a kernel does with its partial column sums


class ColumnSumSlabs:
    """Partial column sums of one op that live across the micro-batches of a step.

    A backward kernel that also produces a parameter gradient as column sums (LayerNorm's dgamma /
    dbeta, the bias gradient behind a dropout) leaves one partial row per CTA; turning those into
    the gradient takes a second, tiny launch that sits on the critical path of every backward.
    With a slab of its own per op the kernel adds to the partials instead (`WS_ACCUMULATE`) and the
    second launch runs once per step, with the last micro-batch (`WS_FLUSH`), which also clears the
    slab for the next step. The slab is sized for one (rows, cols, dtype) and refuses another."""

    def __init__(self):
        self.buf, self.key = None, None

    def get(self, device, floats: int, key):
        if self.buf is None:
            self.buf, self.key = torch.zeros(floats, dtype=torch.float32, device=device), key
        elif self.key != key:
            raise RuntimeError(f"column-sum slabs were sized for {self.key}, got {key}: deferred column sums "
                               "need equal micro-batch shapes")
        return self.buf


def ln_bwd(dy, x, gamma, beta, mean, rstd, residual_grad=None, slabs=None, ws_mode=WS_IMMEDIATE):
    """Returns dx (+ `residual_grad`, the gradient reaching the input through the residual branch);
    accumulates dgamma / dbeta into the parameters' main_grad: at once, or -- with `slabs` (a
    `ColumnSumSlabs` of the calling op) and `ws_mode` WS_ACCUMULATE / WS_FLUSH -- once per step."""
    hidden = x.shape[-1]
    rows = x.numel() // hidden
    dg, db = _grad_of(gamma).view(-1), _grad_of(beta).view(-1)
    if native.use_native(x):
        dx = torch.empty_like(x)
        fp32 = x.dtype == torch.float32
        parts = native.lib().ln_bwd_parts(rows, hidden, fp32)
        if residual_grad is not None and not residual_grad.is_contiguous():
            residual_grad = residual_grad.contiguous()
        if slabs is not None and ws_mode != WS_IMMEDIATE and native.lib().ln_bwd_fused_ok(hidden, fp32):
            ws = slabs.get(x.device, 2 * parts * hidden, (rows, hidden, x.dtype))
        else:
            ws, ws_mode = _workspace(x.device, 2 * parts * hidden), WS_IMMEDIATE
        native.lib().layernorm_bwd(dy, x, gamma, mean, rstd, dx, dg, db, ws, True, residual_grad, ws_mode)
        return dx
    xf, dyf = x.float().reshape(rows, hidden), dy.float().reshape(rows, hidden)
    xh = (xf - mean[:, None]) * rstd[:, None]
    wdy = dyf * gamma.float()
    m1 = wdy.mean(1, keepdim=True)
    m2 = (wdy * xh).mean(1, keepdim=True)
    dg.add_((dyf * xh).sum(0).to(dg.dtype))
    db.add_(dyf.sum(0).to(db.dtype))
    dx = ((wdy - m1 - xh * m2) * rstd[:, None]).to(x.dtype).reshape(x.shape)
    if residual_grad is not None:
        dx = dx + residual_grad.reshape(x.shape)
    return dx


# ---------------------------------------------------------------------------------- linear
def linear_fwd(x, weight, bias=None, gelu=False, residual=None, dropout=None):
    """x W^T (+bias) (dropout) (+residual). With gelu=True returns (pre_activation, gelu(pre_activation)).
    `dropout` = (p, seed, offset): the bias-dropout-add of a sub-block in the GEMM's epilogue."""
    if gelu:
        pre = torch.empty((x.shape[0], weight.shape[0]), dtype=x.dtype, device=x.device)
        act = torch.empty_like(pre)
        gemm(x, weight, out=pre, bias=bias, gelu_out=act)
        return pre, act
    if dropout is not None and dropout[0] <= 0:
        dropout = None
    if residual is not None:
        return gemm(x, weight, bias=bias, aux=residual, aux_mode=AUX_ADD, dropout=dropout)
    return gemm(x, weight, bias=bias, dropout=dropout)


def linear_dgrad(dy, weight, gelu_pre=None):
    """dx = dy W, optionally multiplied by gelu'(gelu_pre) in the GEMM epilogue."""
    if gelu_pre is not None:
        return gemm(dy, weight, b_mn=True, aux=gelu_pre, aux_mode=AUX_GELU_GRAD)
    return gemm(dy, weight, b_mn=True)


_WGRAD_STREAM = {}   # device index -> side stream for weight gradients (see enable_async_wgrad)


def enable_async_wgrad(device, on: bool = True) -> None:
    """Run weight-gradient GEMMs on a side stream. Nothing on the critical path of backward reads a
    weight gradient, while the data-gradient GEMM of the same layer does lie on it; both are
    persistent kernels of 3-4 waves, so when they may overlap the last, partly filled wave of one
    runs beside the first wave of the other. Accumulation order per weight is kept (one side stream).
    Call `join_async_wgrad` before anything reads `main_grad`."""
    dev = torch.device(device)
    if dev.type != "cuda":
        return
    if on:
        _WGRAD_STREAM.setdefault(dev.index, torch.cuda.Stream(device=dev))
    else:
        _WGRAD_STREAM.pop(dev.index, None)


def join_async_wgrad(device) -> None:
    dev = torch.device(device)
    side = _WGRAD_STREAM.get(dev.index) if dev.type == "cuda" else None
    if side is not None:
        torch.cuda.current_stream(dev).wait_stream(side)


def async_wgrad_event(device):
    """An event recorded now on the weight-gradient side stream (None when weight gradients run on
    the main stream). A consumer of `main_grad` on a third stream waits for it to see every weight
    gradient enqueued so far."""
    dev = torch.device(device)
    side = _WGRAD_STREAM.get(dev.index) if dev.type == "cuda" else None
    if side is None:
        return None
    ev = torch.cuda.Event()
    ev.record(side)
    return ev


def _wgrad_now(dy, x, weight, bias):
    gemm(dy, x, a_mn=True, b_mn=True, out=_grad_of(weight).view(weight.shape), accumulate=True)
    if bias is not None:
        colsum(dy, out=_grad_of(bias).view(-1), accumulate=True)


def linear_wgrad(dy, x, weight, bias=None):
    """main_grad(W) += dy^T x ; main_grad(b) += colsum(dy)."""
    side = _WGRAD_STREAM.get(dy.device.index) if dy.is_cuda else None
    if side is None or getattr(dy, "_ethb_ring", False) or getattr(x, "_ethb_ring", False):
        return _wgrad_now(dy, x, weight, bias)
    ready = torch.cuda.Event()
    ready.record()
    side.wait_event(ready)
    with torch.cuda.stream(side):
        _wgrad_now(dy, x, weight, bias)
    # the caching allocator must not hand these buffers out again before the side stream is done
    dy.record_stream(side)
    x.record_stream(side)


# ---------------------------------------------------------------------------------- GeLU / dropout
def gelu_fwd(x, bias=None):
    if native.use_native(x):
        y = torch.empty_like(x)
        native.lib().bias_gelu_fwd(x, bias, y)
        return y
    return F.gelu(x.float() + (bias.float() if bias is not None else 0.0), approximate="tanh").to(x.dtype)


def gelu_bwd(dy, x, bias=None):
    if native.use_native(x):
        dx = torch.empty_like(x)
        native.lib().bias_gelu_bwd(dy, x, bias, dx)
        return dx
    v = x.float() + (bias.float() if bias is not None else 0.0)
    return (dy.float() * gelu_tanh_grad_ref(v)).to(x.dtype)


def bias_dropout_add_fwd(x, bias, residual, p, seed, offset):
    if native.use_native(x):
        out = torch.empty_like(x)
        native.lib().bias_dropout_add_fwd(x, bias, residual, out, float(p), int(seed), int(offset))
        return out
    v = x.float() + (bias.float() if bias is not None else 0.0)
    if p > 0:
        keep = _keep_mask_ref(x.shape, p, seed, offset, x.device)
        v = torch.where(keep, v / (1.0 - p), torch.zeros_like(v))
    if residual is not None:
        v = v + residual.float()
    return v.to(x.dtype)


def dropout_bwd(dy, p, seed, offset):
    if p <= 0:
        return dy
    if native.use_native(dy):
        dx = torch.empty_like(dy)
        native.lib().dropout_bwd(dy, dx, float(p), int(seed), int(offset))
        return dx
    keep = _keep_mask_ref(dy.shape, p, seed, offset, dy.device)
    return torch.where(keep, dy.float() / (1.0 - p), torch.zeros_like(dy.float())).to(dy.dtype)


def dropout_bwd_colsum_into(dy, p, seed, offset, bias_grad, slabs, ws_mode):
    """dropout_bwd(dy), with its column sums added to `bias_grad` (a parameter's main_grad) through
    the op's own `slabs`: once per step instead of once per micro-batch. Returns None when the fused
    kernel does not take this shape; the caller then uses `dropout_bwd_colsum`."""
    cols = dy.shape[-1]
    if not (p > 0 and ws_mode != WS_IMMEDIATE and native.use_native(dy) and dy.is_contiguous()):
        return None
    rows = dy.numel() // cols
    parts = native.lib().dropout_bwd_colsum_parts(rows, cols, dy.dtype == torch.float32)
    if parts <= 0:
        return None
    dx = torch.empty_like(dy)
    ws = slabs.get(dy.device, parts * cols, (rows, cols, dy.dtype))
    native.lib().dropout_bwd_colsum(dy, dx, bias_grad.view(-1), ws, float(p), int(seed), int(offset), True, ws_mode)
    return dx


def dropout_bwd_colsum(dy, p, seed, offset):
    """(dropout_bwd(dy), fp32 column sums of it): the input gradient of a bias-dropout-add op and the
    gradient of its bias, in one pass where the fused kernel supports the shape."""
    cols = dy.shape[-1]
    if p > 0 and native.use_native(dy) and dy.is_contiguous():
        rows = dy.numel() // cols
        parts = native.lib().dropout_bwd_colsum_parts(rows, cols, dy.dtype == torch.float32)
        if parts > 0:
            dx = torch.empty_like(dy)
            bias_grad = torch.empty(cols, dtype=torch.float32, device=dy.device)
            native.lib().dropout_bwd_colsum(dy, dx, bias_grad, _workspace(dy.device, parts * cols), float(p),
                                            int(seed), int(offset), False)
            return dx, bias_grad
    dx = dropout_bwd(dy, p, seed, offset)
    return dx, colsum(dx, out_dtype=torch.float32)


def add_(a, b):
    """a += b for gradient accumulation of residual branches."""
    return a.add_(b)


# ---------------------------------------------------------------------------------- embedding
def embedding_fwd(tokens, word, pos, seq, vocab_start, add_pos):
    ntok, hidden = tokens.numel(), word.shape[1]
    if native.use_native(word):
        out = torch.empty((ntok, hidden), dtype=word.dtype, device=word.device)
        native.lib().embedding_fwd(tokens.contiguous(), word, pos, out, seq, vocab_start, add_pos)
        return out
    t = tokens.reshape(-1) - vocab_start
    mine = (t >= 0) & (t < word.shape[0])
    out = word[t.clamp(0, word.shape[0] - 1)].float() * mine[:, None]
    if add_pos:
        out = out + pos[torch.arange(ntok, device=tokens.device) % seq].float()
    return out.to(word.dtype)


def embedding_bwd(tokens, dout, word, pos, seq, vocab_start, add_pos):
    dword = _grad_of(word).view(word.shape)
    dpos = _grad_of(pos).view(pos.shape) if add_pos else None
    if native.use_native(dout):
        native.lib().embedding_bwd(tokens.contiguous(), dout, dword, dpos, seq, vocab_start, add_pos)
        return
    t = tokens.reshape(-1) - vocab_start
    mine = (t >= 0) & (t < word.shape[0])
    acc = torch.zeros(word.shape, dtype=torch.float32, device=dout.device)
    acc.index_add_(0, t[mine], dout.float()[mine])
    dword.add_(acc.to(dword.dtype))
    if dpos is not None:
        accp = torch.zeros(pos.shape, dtype=torch.float32, device=dout.device)
        accp.index_add_(0, torch.arange(tokens.numel(), device=tokens.device) % seq, dout.float())
        dpos.add_(accp.to(dpos.dtype))


# ---------------------------------------------------------------------------------- cross entropy
def ce_fwd(logits, targets, vocab_start, gather_fn=None):
    """Per-token loss; returns (loss, gmax, gsum) with the global softmax statistics for backward."""
    rows = logits.shape[0]
    targets = targets.reshape(-1).contiguous()
    if native.use_native(logits):
        stats = torch.empty((rows, 3), dtype=torch.float32, device=logits.device)
        native.lib().ce_local_stats(logits, targets, stats, vocab_start)
        all_stats = gather_fn(stats) if gather_fn is not None else stats.unsqueeze(0)
        loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
        gmax, gsum = torch.empty_like(loss), torch.empty_like(loss)
        native.lib().ce_combine(all_stats.contiguous(), loss, gmax, gsum, all_stats.shape[0])
        return loss, gmax, gsum
    lf = logits.float()
    lmax = lf.max(1).values
    lsum = torch.exp(lf - lmax[:, None]).sum(1)
    t = targets - vocab_start
    mine = (t >= 0) & (t < logits.shape[1])
    tl = lf.gather(1, t.clamp(0, logits.shape[1] - 1)[:, None])[:, 0] * mine
    stats = torch.stack([lmax, lsum, tl], 1)
    all_stats = gather_fn(stats) if gather_fn is not None else stats.unsqueeze(0)
    gmax = all_stats[:, :, 0].max(0).values
    gsum = (all_stats[:, :, 1] * torch.exp(all_stats[:, :, 0] - gmax)).sum(0)
    return torch.log(gsum) + gmax - all_stats[:, :, 2].sum(0), gmax, gsum


def ce_bwd_(logits, targets, gmax, gsum, dloss, vocab_start):
    """Overwrites `logits` with d loss / d logits scaled by dloss[row]; returns it."""
    targets = targets.reshape(-1).contiguous()
    if native.use_native(logits):
        native.lib().ce_bwd(logits, targets, gmax, gsum, dloss.float().contiguous(), vocab_start)
        return logits
    sm = torch.exp(logits.float() - gmax[:, None]) / gsum[:, None]
    t = targets - vocab_start
    mine = (t >= 0) & (t < logits.shape[1])
    onehot = torch.zeros_like(sm)
    onehot[mine, t[mine]] = 1.0
    logits.copy_(((sm - onehot) * dloss.float()[:, None]).to(logits.dtype))
    return logits


# ---------------------------------------------------------------------------------- attention
def attention_fwd(qkv, batch, seq, heads, head_dim, scale=None, causal=True):
    """qkv: [batch*seq, heads*3*head_dim] with per-head [q | k | v] blocks. Returns (out[T, heads*d], lse)."""
    if scale is None:
        scale = 1.0 / math.sqrt(head_dim)
    v5 = qkv.view(batch, seq, heads, 3, head_dim)
    q, k, v = v5[:, :, :, 0], v5[:, :, :, 1], v5[:, :, :, 2]
    if native.use_native(qkv):
        o = torch.empty((batch, seq, heads, head_dim), dtype=qkv.dtype, device=qkv.device)
        lse = torch.empty((batch, heads, seq), dtype=torch.float32, device=qkv.device)
        native.lib().attn_fwd(q, k, v, o, lse, float(scale), bool(causal), native.status(qkv.device))
        return o.view(batch * seq, heads * head_dim), lse
    o = attention_ref(q, k, v, scale, causal).to(qkv.dtype).contiguous()
    return o.view(batch * seq, heads * head_dim), None


def attention_bwd(d_out, qkv, out, lse, batch, seq, heads, head_dim, scale=None, causal=True):
    """Returns dqkv in the same packed layout as qkv."""
    if scale is None:
        scale = 1.0 / math.sqrt(head_dim)
    v5 = qkv.view(batch, seq, heads, 3, head_dim)
    q, k, v = v5[:, :, :, 0], v5[:, :, :, 1], v5[:, :, :, 2]
    if native.use_native(qkv):
        dqkv = torch.empty_like(qkv)
        d5 = dqkv.view(batch, seq, heads, 3, head_dim)
        delta = torch.empty((batch, heads, seq), dtype=torch.float32, device=qkv.device)
        native.lib().attn_bwd(q, k, v, out.view(batch, seq, heads, head_dim),
                              d_out.view(batch, seq, heads, head_dim), lse, d5[:, :, :, 0], d5[:, :, :, 1],
                              d5[:, :, :, 2], delta, delta, float(scale), bool(causal),
                              native.status(qkv.device))
        return dqkv
    with torch.enable_grad():
        qd, kd, vd = (t.detach().float().requires_grad_(True) for t in (q, k, v))
        ref = attention_ref(qd, kd, vd, scale, causal)
        gq, gk, gv = torch.autograd.grad(ref, (qd, kd, vd), d_out.view(batch, seq, heads, head_dim).float())
    return torch.stack([gq, gk, gv], 3).to(qkv.dtype).reshape(qkv.shape)


# ---------------------------------------------------------------------------------- unfused attention (13-op manifest)
def bmm_heads(a, b, out, *, a_mn=False, b_mn=False, alpha=1.0, accumulate=False):
    """out[i, j] = alpha * a[i, j] x b[i, j]^T (+ out[i, j]) over two leading batch dims
    ([batch, heads, rows, cols] views, unit inner stride, any other strides). CUDA: one tcgen05 GEMM
    launch per (batch, head) from a single native call (the reference: torch.baddbmm / torch.bmm on
    cuBLAS, eth/runtime/megatron/model/flex_ops.py:1229-1233, 1502)."""
    if native.use_native(a):
        native.lib().gemm_batched(a, a_mn, b, b_mn, out, float(alpha), bool(accumulate), native.status(a.device))
        return out
    af = (a.transpose(-1, -2) if a_mn else a).float()
    bf = (b if b_mn else b.transpose(-1, -2)).float()
    v = alpha * torch.matmul(af, bf)
    out.copy_((v + out.float() if accumulate else v).to(out.dtype))
    return out


def _qkv_heads(qkv, batch, seq, heads, head_dim):
    """q, k, v as [batch, heads, seq, head_dim] views of the packed [tokens, heads * 3 * head_dim] activation."""
    v5 = qkv.view(batch, seq, heads, 3, head_dim)
    return tuple(v5[:, :, :, j].permute(0, 2, 1, 3) for j in range(3))


def attn_scores_fwd(qkv, batch, seq, heads, head_dim):
    """Raw scores Q K^T per head: [batch, heads, seq, seq] (the scale is applied by the softmax op)."""
    q, k, _ = _qkv_heads(qkv, batch, seq, heads, head_dim)
    scores = torch.empty((batch, heads, seq, seq), dtype=qkv.dtype, device=qkv.device)
    return bmm_heads(q, k, scores)


def attn_scores_bwd(d_scores, qkv, dqkv, batch, seq, heads, head_dim):
    """dQ = dS K and dK = dS^T Q written into the q / k slots of the packed gradient `dqkv`."""
    q, k, _ = _qkv_heads(qkv, batch, seq, heads, head_dim)
    dq, dk, _ = _qkv_heads(dqkv, batch, seq, heads, head_dim)
    bmm_heads(d_scores, k, dq, b_mn=True)
    bmm_heads(d_scores, q, dk, a_mn=True, b_mn=True)


def attn_context_fwd(probs, qkv, batch, seq, heads, head_dim):
    """P V per head, written token-major: [tokens, heads * head_dim]."""
    _, _, v = _qkv_heads(qkv, batch, seq, heads, head_dim)
    out = torch.empty((batch * seq, heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    o4 = out.view(batch, seq, heads, head_dim).permute(0, 2, 1, 3)
    bmm_heads(probs, v, o4, b_mn=True)
    return out


def attn_context_bwd(d_out, probs, qkv, batch, seq, heads, head_dim):
    """(dP, dqkv): dP = dO V^T; dV = P^T dO goes into the v slot of a fresh packed gradient whose
    q / k slots the score op's backward fills."""
    _, _, v = _qkv_heads(qkv, batch, seq, heads, head_dim)
    do4 = d_out.view(batch, seq, heads, head_dim).permute(0, 2, 1, 3)
    d_probs = torch.empty_like(probs)
    bmm_heads(do4, v, d_probs)
    dqkv = torch.empty_like(qkv)
    _, _, dv = _qkv_heads(dqkv, batch, seq, heads, head_dim)
    bmm_heads(probs, do4, dv, a_mn=True, b_mn=True)
    return d_probs, dqkv


def softmax_fwd(x, scale, causal=True):
    """softmax(scale * x) over the last dim with the implicit causal mask (x: [..., sq, sk])."""
    from .functional import SOFTMAX_CAUSAL, SOFTMAX_PLAIN
    mode = SOFTMAX_CAUSAL if causal else SOFTMAX_PLAIN
    if native.use_native(x):
        y = torch.empty_like(x)
        native.lib().softmax_fwd(x.view(-1, x.shape[-2], x.shape[-1]), None, y.view(-1, x.shape[-2], x.shape[-1]),
                                 float(scale), mode)
        return y
    v = x.float() * scale
    if causal:
        sq, sk = x.shape[-2], x.shape[-1]
        v = v.masked_fill(torch.triu(torch.ones(sq, sk, dtype=torch.bool, device=x.device), 1), float("-inf"))
    return torch.softmax(v, -1).to(x.dtype)


def softmax_bwd(dy, y, scale, causal=True):
    from .functional import SOFTMAX_CAUSAL, SOFTMAX_PLAIN
    if native.use_native(y):
        dx = torch.empty_like(y)
        shape = (-1, y.shape[-2], y.shape[-1])
        native.lib().softmax_bwd(dy.contiguous().view(shape), y.view(shape), dx.view(shape), float(scale),
                                 SOFTMAX_CAUSAL if causal else SOFTMAX_PLAIN)
        return dx
    yf, dyf = y.float(), dy.float()
    return ((dyf - (dyf * yf).sum(-1, keepdim=True)) * yf * scale).to(y.dtype)
