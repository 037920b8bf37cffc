"""Functional ops of the GPT stage program.

Each op has two implementations with the same numerics contract:
  * CUDA tensors  -> hand-written sm_100a kernels from `eth_b200._C` (tcgen05 GEMM, fused
    LayerNorm / GeLU / dropout-add / softmax / embedding / cross-entropy kernels);
  * CPU tensors   -> a plain PyTorch reference (used by CPU tests and as the oracle of the GPU tests).

Activations are 2-D token-major matrices `[tokens, features]` (tokens = batch * seq, batch-major),
which keeps every GEMM operand TMA-addressable without transposes.

Parameters may carry a `main_grad` attribute (persistent gradient buffer, the LocalDDP contract of
eth/runtime/megatron/model/distributed.py:68-123). When present, backward kernels accumulate
straight into it (GEMM epilogue `D += ...`, LayerNorm/colsum `accumulate`) and autograd sees no
gradient for that parameter.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F

from . import native



def _workspace(device, numel: int) -> torch.Tensor:
    """Grow-only fp32 scratch per device and stream (partial sums of LayerNorm-backward and column
    sums), kept as named buffers in the process-wide registry of `utils.memory`."""
    from ..utils import memory
    # one scratch per (device, stream): kernels of different streams may run concurrently
    stream = torch.cuda.current_stream(device).cuda_stream if device.type == "cuda" else 0
    name = f"colsum-workspace {device.type}:{device.index} stream {stream}"
    buf = memory._BUFFERS.get(name)
    if buf is None or buf.numel < numel:
        memory.free_mem_buff(name)
        buf = memory.allocate_mem_buff(name, max(numel, 1 << 20), torch.float32, device=device)
    return buf.data


def _main_grad(p) -> Optional[torch.Tensor]:
    return getattr(p, "main_grad", None) if p is not None else None


# ------------------------------------------------------------------------------------------
# GEMM
# ------------------------------------------------------------------------------------------
AUX_NONE, AUX_ADD, AUX_GELU_GRAD = 0, 1, 2


def gemm(a, b, *, a_mn=False, b_mn=False, out=None, out_dtype=None, bias=None, aux=None,
         aux_mode=AUX_NONE, gelu_out=None, accumulate=False, alpha=1.0, dropout=None):
    """D[M,N] = alpha * A x B^T (+bias) (dropout) (aux op) (+D).

    A is [M,K] (a_mn False) or [K,M] (a_mn True); B is [N,K] (b_mn False) or [K,N] (b_mn True).
    `gelu_out`, when given, additionally receives gelu(D). `dropout` = (p, seed, offset) drops
    alpha * A x B^T + bias in the epilogue, before a residual `aux` is added: the mask is the one
    `bias_dropout_add` and `dropout_bwd` draw for the same (seed, offset) on an [M, N] tensor.
    """
    M = a.shape[1] if a_mn else a.shape[0]
    N = b.shape[1] if b_mn else b.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype or a.dtype, device=a.device)
    if native.use_native(a):
        p_drop, seed, offset = dropout if dropout is not None else (0.0, 0, 0)
        native.lib().gemm(a, a_mn, b, b_mn, out, bias, aux, aux_mode, gelu_out, accumulate,
                          float(alpha), native.status(a.device), 0, float(p_drop), int(seed), int(offset))
        return out
    # reference
    af = (a.t() if a_mn else a).float()
    bf = (b if b_mn else b.t()).float()
    v = alpha * (af @ bf)
    if bias is not None:
        v = v + bias.float()
    if dropout is not None and dropout[0] > 0:
        keep = _keep_mask_ref(v.shape, dropout[0], dropout[1], dropout[2], v.device)
        v = torch.where(keep, v / (1.0 - dropout[0]), torch.zeros_like(v))
    if aux is not None and aux_mode == AUX_ADD:
        v = v + aux.float()
    elif aux is not None and aux_mode == AUX_GELU_GRAD:
        v = v * gelu_tanh_grad_ref(aux.float())
    if accumulate:
        v = v + out.float()
    out.copy_(v.to(out.dtype))
    if gelu_out is not None:
        gelu_out.copy_(F.gelu(v, approximate="tanh").to(gelu_out.dtype))
    return out


def gelu_tanh_grad_ref(x):
    k0, k1 = 0.7978845608028654, 0.044715
    t = torch.tanh(k0 * x * (1.0 + k1 * x * x))
    return 0.5 * x * ((1 - t * t) * (k0 + 3 * k0 * k1 * x * x)) + 0.5 * (1 + t)


class _LinearFn(torch.autograd.Function):
    """y = x W^T (+ b); optional fused GeLU second output."""

    @staticmethod
    def forward(ctx, x, weight, bias, with_gelu):
        ctx.has_bias = bias is not None
        ctx.with_gelu = with_gelu
        if with_gelu:
            pre = torch.empty((x.shape[0], weight.shape[0]), dtype=x.dtype, device=x.device)
            act = torch.empty_like(pre)
            gemm(x, weight, out=pre, bias=bias, gelu_out=act)
            ctx.save_for_backward(x, weight, pre)
            ctx.bias_ref = bias
            return act
        out = gemm(x, weight, bias=bias)
        ctx.save_for_backward(x, weight, None)
        ctx.bias_ref = bias
        return out

    @staticmethod
    def backward(ctx, dy):
        x, weight, pre = ctx.saved_tensors
        bias = ctx.bias_ref
        dy = dy.contiguous()
        if ctx.with_gelu:
            if native.use_native(dy):
                du = torch.empty_like(dy)
                native.lib().bias_gelu_bwd(dy, pre, None, du)
            else:
                du = (dy.float() * gelu_tanh_grad_ref(pre.float())).to(dy.dtype)
            dy = du
        dx = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy, weight, b_mn=True)
        dw = _wgrad(dy, x, weight)
        db = _bias_grad(dy, bias) if ctx.has_bias else None
        return dx, dw, db, None


def _wgrad(dy, x, weight):
    """dW[N,K] = dy[M,N]^T x[M,K]; accumulated into weight.main_grad when it exists."""
    if not weight.requires_grad:
        return None
    mg = _main_grad(weight)
    if mg is not None:
        gemm(dy, x, a_mn=True, b_mn=True, out=mg.view(weight.shape), accumulate=True)
        return None
    return gemm(dy, x, a_mn=True, b_mn=True, out_dtype=weight.dtype)


def colsum(x, out=None, accumulate=False, out_dtype=None):
    """Column sums of a 2-D matrix in fp32."""
    cols = x.shape[-1]
    if out is None:
        out = torch.empty(cols, dtype=out_dtype or x.dtype, device=x.device)
        accumulate = False
    if native.use_native(x):
        x2 = x.reshape(-1, cols)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        parts = native.lib().colsum_parts(x2.shape[0])
        native.lib().colsum(x2, out, _workspace(x.device, parts * cols), accumulate)
        return out
    s = x.reshape(-1, cols).float().sum(0)
    if accumulate:
        s = s + out.float()
    out.copy_(s.to(out.dtype))
    return out


def _bias_grad(dy, bias):
    if bias is None or not bias.requires_grad:
        return None
    mg = _main_grad(bias)
    if mg is not None:
        colsum(dy, out=mg.view(-1), accumulate=True)
        return None
    return colsum(dy, out_dtype=bias.dtype)


def linear(x, weight, bias=None):
    return _LinearFn.apply(x, weight, bias, False)


def linear_gelu(x, weight, bias=None):
    """gelu_tanh(x W^T + b) with the activation computed in the GEMM epilogue."""
    return _LinearFn.apply(x, weight, bias, True)


# ------------------------------------------------------------------------------------------
# LayerNorm
# ------------------------------------------------------------------------------------------
class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, eps):
        hidden = x.shape[-1]
        x = x.contiguous()
        rows = x.numel() // hidden
        if native.use_native(x):
            y = torch.empty_like(x)
            mean = torch.empty(rows, dtype=torch.float32, device=x.device)
            rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
            native.lib().layernorm_fwd(x, gamma, beta, y, mean, rstd, eps)
        else:
            xf = x.float().reshape(rows, hidden)
            mean = xf.mean(1)
            var = xf.var(1, unbiased=False)
            rstd = torch.rsqrt(var + eps)
            y = ((xf - mean[:, None]) * rstd[:, None] * gamma.float() + beta.float())
            y = y.to(x.dtype).reshape(x.shape)
        ctx.save_for_backward(x, gamma, mean, rstd)
        ctx.beta_ref = beta
        return y

    @staticmethod
    def backward(ctx, dy):
        x, gamma, mean, rstd = ctx.saved_tensors
        beta = ctx.beta_ref
        hidden = x.shape[-1]
        rows = x.numel() // hidden
        dy = dy.contiguous()
        gmg, bmg = _main_grad(gamma), _main_grad(beta)
        if native.use_native(x):
            dx = torch.empty_like(x)
            fused = gmg is not None and bmg is not None
            if fused:
                dg, db = gmg.view(-1), bmg.view(-1)
            else:
                dg = torch.empty(hidden, dtype=gamma.dtype, device=x.device)
                db = torch.empty(hidden, dtype=gamma.dtype, device=x.device)
            parts = native.lib().ln_bwd_parts(rows, hidden, x.dtype == torch.float32)
            ws = _workspace(x.device, 2 * parts * hidden)
            native.lib().layernorm_bwd(dy, x, gamma, mean, rstd, dx, dg, db, ws, fused)
            if fused:
                return dx, None, None, None
            return dx, dg, db, None
        xf = x.float().reshape(rows, hidden)
        dyf = dy.float().reshape(rows, hidden)
        xh = (xf - mean[:, None]) * rstd[:, None]
        wdy = dyf * gamma.float()
        m1 = wdy.mean(1, keepdim=True)
        m2 = (wdy * xh).mean(1, keepdim=True)
        dx = ((wdy - m1 - xh * m2) * rstd[:, None]).to(x.dtype).reshape(x.shape)
        dg = (dyf * xh).sum(0)
        db = dyf.sum(0)
        if gmg is not None and bmg is not None:
            gmg.view(-1).add_(dg.to(gmg.dtype))
            bmg.view(-1).add_(db.to(bmg.dtype))
            return dx, None, None, None
        return dx, dg.to(gamma.dtype), db.to(gamma.dtype), None


def layer_norm(x, gamma, beta, eps=1e-5):
    return _LayerNormFn.apply(x, gamma, beta, eps)


# ------------------------------------------------------------------------------------------
# bias + GeLU
# ------------------------------------------------------------------------------------------
class _BiasGeluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, bias):
        x = x.contiguous()
        ctx.save_for_backward(x, bias)
        if native.use_native(x):
            y = torch.empty_like(x)
            native.lib().bias_gelu_fwd(x, bias, y)
            return y
        v = x.float() + (bias.float() if bias is not None else 0.0)
        return F.gelu(v, approximate="tanh").to(x.dtype)

    @staticmethod
    def backward(ctx, dy):
        x, bias = ctx.saved_tensors
        dy = dy.contiguous()
        if native.use_native(x):
            dx = torch.empty_like(x)
            native.lib().bias_gelu_bwd(dy, x, bias, dx)
        else:
            v = x.float() + (bias.float() if bias is not None else 0.0)
            dx = (dy.float() * gelu_tanh_grad_ref(v)).to(x.dtype)
        db = _bias_grad(dx, bias) if bias is not None else None
        return dx, db


def bias_gelu(x, bias=None):
    return _BiasGeluFn.apply(x, bias)


# ------------------------------------------------------------------------------------------
# residual + dropout(x + bias)
# ------------------------------------------------------------------------------------------
def _keep_mask_ref(shape, p, seed, offset, device):
    """CPU restatement of the kernel's Philox-4x32-10 keep mask (16 random bits per element)."""
    import numpy as np

    n = int(math.prod(shape))
    nvec = (n + 7) // 8
    ctr = np.arange(nvec, dtype=np.uint64)
    c = [ctr & 0xFFFFFFFF, ctr >> np.uint64(32), np.full(nvec, offset & 0xFFFFFFFF, np.uint64),
         np.full(nvec, (offset >> 32) & 0xFFFFFFFF, np.uint64)]
    k0, k1 = seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF
    M0, M1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
    mask32 = np.uint64(0xFFFFFFFF)
    for _ in range(10):
        p0 = M0 * c[0]
        p1 = M1 * c[2]
        hi0, lo0 = p0 >> np.uint64(32), p0 & mask32
        hi1, lo1 = p1 >> np.uint64(32), p1 & mask32
        c = [hi1 ^ c[1] ^ np.uint64(k0), lo1, hi0 ^ c[3] ^ np.uint64(k1), lo0]
        k0 = (k0 + 0x9E3779B9) & 0xFFFFFFFF
        k1 = (k1 + 0xBB67AE85) & 0xFFFFFFFF
    thr = int(np.float32(p) * np.float32(65536.0))
    bits = np.empty((nvec, 8), dtype=np.uint64)
    for j in range(4):
        bits[:, 2 * j] = c[j] & np.uint64(0xFFFF)
        bits[:, 2 * j + 1] = c[j] >> np.uint64(16)
    keep = (bits >= thr).reshape(-1)[:n]
    return torch.from_numpy(keep).to(device).reshape(shape)


class _BiasDropoutAddFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, bias, residual, p, seed, offset):
        x = x.contiguous()
        ctx.p, ctx.seed, ctx.offset = p, seed, offset
        ctx.bias_ref = bias
        ctx.has_res = residual is not None
        if native.use_native(x):
            out = torch.empty_like(x)
            native.lib().bias_dropout_add_fwd(x, bias, residual.contiguous() if residual is not None
                                              else None, out, p, seed, offset)
            return out
        v = x.float() + (bias.float() if bias is not None else 0.0)
        if p > 0:
            keep = _keep_mask_ref(x.shape, p, seed, offset, x.device)
            v = torch.where(keep, v / (1.0 - p), torch.zeros_like(v))
        if residual is not None:
            v = v + residual.float()
        return v.to(x.dtype)

    @staticmethod
    def backward(ctx, dy):
        dy = dy.contiguous()
        p = ctx.p
        if p > 0:
            if native.use_native(dy):
                dx = torch.empty_like(dy)
                native.lib().dropout_bwd(dy, dx, p, ctx.seed, ctx.offset)
            else:
                keep = _keep_mask_ref(dy.shape, p, ctx.seed, ctx.offset, dy.device)
                dx = torch.where(keep, dy.float() / (1.0 - p), torch.zeros_like(dy.float())).to(dy.dtype)
        else:
            dx = dy
        bias = ctx.bias_ref
        db = _bias_grad(dx, bias) if bias is not None else None
        return dx, db, (dy if ctx.has_res else None), None, None, None


def bias_dropout_add(x, bias, residual, p=0.0, seed=0, offset=0):
    """residual + dropout(x + bias). The keep mask is a function of (seed, offset, element index)."""
    return _BiasDropoutAddFn.apply(x, bias, residual, float(p), int(seed), int(offset))


# ------------------------------------------------------------------------------------------
# softmax family (legacy 13-op attention manifest)
# ------------------------------------------------------------------------------------------
SOFTMAX_PLAIN, SOFTMAX_CAUSAL, SOFTMAX_MASKED = 0, 1, 2


class _SoftmaxFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, mask, scale, mode):
        x = x.contiguous()
        ctx.scale, ctx.mode = scale, mode
        if native.use_native(x):
            y = torch.empty_like(x)
            m = mask.to(torch.uint8).contiguous() if mask is not None else None
            native.lib().softmax_fwd(x, m, y, scale, mode)
        else:
            v = x.float() * scale
            if mode == SOFTMAX_CAUSAL:
                sq, sk = x.shape[-2], x.shape[-1]
                tri = torch.triu(torch.ones(sq, sk, dtype=torch.bool, device=x.device), 1)
                v = v.masked_fill(tri, float("-inf"))
            elif mode == SOFTMAX_MASKED:
                v = v.masked_fill(mask.bool(), -10000.0)
            y = torch.softmax(v, -1).to(x.dtype)
        ctx.save_for_backward(y)
        return y

    @staticmethod
    def backward(ctx, dy):
        (y,) = ctx.saved_tensors
        dy = dy.contiguous()
        if native.use_native(y):
            dx = torch.empty_like(y)
            native.lib().softmax_bwd(dy, y, dx, ctx.scale, ctx.mode)
        else:
            yf, dyf = y.float(), dy.float()
            dx = (ctx.scale * yf * (dyf - (dyf * yf).sum(-1, keepdim=True))).to(y.dtype)
        return dx, None, None, None


def scaled_softmax(x, scale=1.0):
    return _SoftmaxFn.apply(x, None, float(scale), SOFTMAX_PLAIN)


def scaled_upper_triang_masked_softmax(x, scale=1.0):
    """x: [batches, sq, sk] with an implicit causal mask."""
    return _SoftmaxFn.apply(x, None, float(scale), SOFTMAX_CAUSAL)


def scaled_masked_softmax(x, mask, scale=1.0):
    """x: [b, heads, sq, sk]; mask: [b or 1, 1, sq, sk], nonzero == masked (filled with -10000)."""
    return _SoftmaxFn.apply(x, mask, float(scale), SOFTMAX_MASKED)


# ------------------------------------------------------------------------------------------
# embedding
# ------------------------------------------------------------------------------------------
class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tokens, word, pos, seq, vocab_start, add_pos):
        tokens = tokens.contiguous()
        ctx.seq, ctx.vocab_start, ctx.add_pos = seq, vocab_start, add_pos
        ctx.save_for_backward(tokens)
        ctx.word_ref, ctx.pos_ref = word, pos
        ntok, hidden = tokens.numel(), word.shape[1]
        if native.use_native(word):
            out = torch.empty((ntok, hidden), dtype=word.dtype, device=word.device)
            native.lib().embedding_fwd(tokens, word, pos, out, seq, vocab_start, add_pos)
            return out
        t = tokens.reshape(-1) - vocab_start
        mine = (t >= 0) & (t < word.shape[0])
        out = word[t.clamp(0, word.shape[0] - 1)].float() * mine[:, None]
        if add_pos:
            pidx = torch.arange(ntok, device=tokens.device) % seq
            out = out + pos[pidx].float()
        return out.to(word.dtype)

    @staticmethod
    def backward(ctx, dout):
        (tokens,) = ctx.saved_tensors
        word, pos = ctx.word_ref, ctx.pos_ref
        dout = dout.contiguous()
        wmg, pmg = _main_grad(word), _main_grad(pos)
        dword = wmg.view(word.shape) if wmg is not None else torch.zeros_like(word, dtype=torch.float32)
        dpos = None
        if ctx.add_pos and pos.requires_grad:
            dpos = pmg.view(pos.shape) if pmg is not None else torch.zeros_like(pos, dtype=torch.float32)
        if native.use_native(dout):
            native.lib().embedding_bwd(tokens, dout, dword, dpos, ctx.seq, ctx.vocab_start,
                                       ctx.add_pos and dpos is not None)
        else:
            t = tokens.reshape(-1) - ctx.vocab_start
            mine = (t >= 0) & (t < word.shape[0])
            acc = torch.zeros(word.shape, dtype=torch.float32, device=dout.device)
            acc.index_add_(0, t[mine], dout.float()[mine])
            dword.add_(acc.to(dword.dtype))
            if dpos is not None:
                pidx = torch.arange(tokens.numel(), device=tokens.device) % ctx.seq
                accp = torch.zeros(pos.shape, dtype=torch.float32, device=dout.device)
                accp.index_add_(0, pidx, dout.float())
                dpos.add_(accp.to(dpos.dtype))
        gw = None if wmg is not None else dword.to(word.dtype)
        gp = None
        if dpos is not None and pmg is None:
            gp = dpos.to(pos.dtype)
        return None, gw, gp, None, None, None


def embedding(tokens, word, pos, seq, vocab_start=0, add_pos=True):
    """out[t] = word[tokens[t] - vocab_start] (zero when the token lives on another vocab shard)
    + pos[t % seq] (when add_pos). tokens are batch-major [batch, seq]."""
    return _EmbeddingFn.apply(tokens, word, pos, int(seq), int(vocab_start), bool(add_pos))


# ------------------------------------------------------------------------------------------
# vocab-parallel cross entropy
# ------------------------------------------------------------------------------------------
class _VocabParallelCEFn(torch.autograd.Function):
    """Per-token loss from vocab-sharded logits. One exchange of (max, sum-exp, target-logit)
    triples replaces the three all-reduces of eth/runtime/megatron/mpu/cross_entropy.py:33-118.
    Backward overwrites the logits buffer with the gradient."""

    @staticmethod
    def forward(ctx, logits, targets, vocab_start, gather_fn):
        rows = logits.shape[0]
        targets = targets.reshape(-1).contiguous()
        if native.use_native(logits):
            stats = torch.empty((rows, 3), dtype=torch.float32, device=logits.device)
            native.lib().ce_local_stats(logits, targets, stats, vocab_start)
            all_stats = gather_fn(stats) if gather_fn is not None else stats.unsqueeze(0)
            world = all_stats.shape[0]
            loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
            gmax = torch.empty_like(loss)
            gsum = torch.empty_like(loss)
            native.lib().ce_combine(all_stats.contiguous(), loss, gmax, gsum, world)
        else:
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
            loss = torch.log(gsum) + gmax - all_stats[:, :, 2].sum(0)
        ctx.save_for_backward(logits, targets, gmax, gsum)
        ctx.vocab_start = vocab_start
        return loss

    @staticmethod
    def backward(ctx, dloss):
        logits, targets, gmax, gsum = ctx.saved_tensors
        dloss = dloss.float().contiguous()
        if native.use_native(logits):
            native.lib().ce_bwd(logits, targets, gmax, gsum, dloss, ctx.vocab_start)
            return logits, None, None, None
        lf = logits.float()
        sm = torch.exp(lf - gmax[:, None]) / gsum[:, None]
        t = targets - ctx.vocab_start
        mine = (t >= 0) & (t < logits.shape[1])
        onehot = torch.zeros_like(sm)
        onehot[mine, t[mine]] = 1.0
        g = ((sm - onehot) * dloss[:, None]).to(logits.dtype)
        return g, None, None, None


def vocab_parallel_cross_entropy(logits, targets, vocab_start=0, gather_fn=None):
    """logits: [tokens, vocab_local]; targets: [tokens] global ids. `gather_fn(stats[rows,3])`
    returns the `[tp, rows, 3]` stack over the tensor-parallel group (None for TP=1)."""
    return _VocabParallelCEFn.apply(logits, targets, int(vocab_start), gather_fn)


# ------------------------------------------------------------------------------------------
# attention
# ------------------------------------------------------------------------------------------
def attention_ref(q, k, v, scale, causal=True):
    """fp32 reference. q/k/v: [batch, seq, heads, head_dim]."""
    qf, kf, vf = (t.float().permute(0, 2, 1, 3) for t in (q, k, v))
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        sq, sk = s.shape[-2], s.shape[-1]
        tri = torch.triu(torch.ones(sq, sk, dtype=torch.bool, device=s.device), 1 + sk - sq)
        s = s.masked_fill(tri, float("-inf"))
    p = torch.softmax(s, -1)
    return torch.matmul(p, vf).permute(0, 2, 1, 3)


class _FlashAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale, causal):
        ctx.scale, ctx.causal = scale, causal
        if native.use_native(q):
            b, sq, h, d = q.shape
            o = torch.empty((b, sq, h, d), dtype=q.dtype, device=q.device)
            lse = torch.empty((b, h, sq), dtype=torch.float32, device=q.device)
            native.lib().attn_fwd(q, k, v, o, lse, scale, causal, native.status(q.device))
            ctx.save_for_backward(q, k, v, o, lse)
            return o
        o = attention_ref(q, k, v, scale, causal).to(q.dtype).contiguous()
        ctx.save_for_backward(q, k, v, o, None)
        return o

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, o, lse = ctx.saved_tensors
        if native.use_native(q):
            b, sq, h, d = q.shape
            d_o = d_o.contiguous()
            # one packed [b, s, h, 3, d] gradient so that the QKV-GEMM backward reads it in place
            dqkv = torch.empty((b, sq, h, 3, d), dtype=q.dtype, device=q.device)
            dq, dk, dv = dqkv[:, :, :, 0], dqkv[:, :, :, 1], dqkv[:, :, :, 2]
            delta = torch.empty((b, h, sq), dtype=torch.float32, device=q.device)
            native.lib().attn_bwd(q, k, v, o, d_o, lse, dq, dk, dv, delta, delta, ctx.scale,
                                  ctx.causal, native.status(q.device))
            return dq, dk, dv, None, None
        with torch.enable_grad():
            qd, kd, vd = (t.detach().float().requires_grad_(True) for t in (q, k, v))
            out = attention_ref(qd, kd, vd, ctx.scale, ctx.causal)
            gq, gk, gv = torch.autograd.grad(out, (qd, kd, vd), d_o.float())
        return gq.to(q.dtype), gk.to(k.dtype), gv.to(v.dtype), None, None


def flash_attention(q, k, v, scale=None, causal=True):
    """Causal flash attention. q/k/v: [batch, seq, heads, head_dim] views (head_dim contiguous)."""
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    return _FlashAttnFn.apply(q, k, v, float(scale), bool(causal))


def attention_backward_tile_order(num_ctas: int, tiles_per_pair: int, pairs: int, causal: bool = True):
    """Host mirror of the tile assignment of the two persistent backward kernels
    (attn_bwd_dkdv_kernel / attn_bwd_dq_kernel in csrc/attention_sm100.cu): tile id T in
    [0, tiles_per_pair * pairs) means slot T // pairs of (head, batch) pair T % pairs, slot 0 being
    the heaviest tile under the causal mask; round r hands out ids [r * num_ctas, (r + 1) * num_ctas)
    in ascending CTA order when r is even and descending when it is odd. Returns, per CTA, the list
    of (slot, pair, weight) it processes, weight = number of partner tiles the tile meets (key tile j
    meets tiles_per_pair - j query tiles, and the other way round for the dQ kernel)."""
    total = tiles_per_pair * pairs
    out = [[] for _ in range(num_ctas)]
    rnd = 0
    while rnd * num_ctas < total:
        for cta in range(num_ctas):
            tile = rnd * num_ctas + (num_ctas - 1 - cta if rnd & 1 else cta)
            if tile < total:
                slot, pair = divmod(tile, pairs)
                out[cta].append((slot, pair, tiles_per_pair - slot if causal else tiles_per_pair))
        rnd += 1
    return out


def unfused_attention(q, k, v, scale=None, causal=True, dropout_p=0.0, seed=0, offset=0):
    """Attention as the four ops of the 13-op layer manifest: scores (batched GEMM) -> fused
    scale + causal-mask softmax -> dropout -> context (batched GEMM). q, k, v: [b, s, h, d]; returns
    [b, s, h, d]. The softmax is this library's kernel; the two batched GEMMs are torch.baddbmm /
    torch.bmm, as in the reference (eth/runtime/megatron/model/flex_ops.py:1229-1233 scores,
    :1246-1330 softmax, :1332-1374 dropout, :1502 context). The 10-op manifest replaces all four by
    `flash_attention`; this path exists for configs and profiles written against the older manifest."""
    b, s, h, d = q.shape
    scale = float(scale) if scale is not None else d ** -0.5
    qh = q.permute(0, 2, 1, 3).reshape(b * h, s, d)
    kh = k.permute(0, 2, 1, 3).reshape(b * h, s, d)
    vh = v.permute(0, 2, 1, 3).reshape(b * h, s, d)
    scores = torch.bmm(qh, kh.transpose(1, 2))
    if causal:
        probs = scaled_upper_triang_masked_softmax(scores, scale)
    else:
        probs = scaled_softmax(scores.view(b, h, s, s), scale).view(b * h, s, s)
    if dropout_p > 0:
        keep = _keep_mask_ref(probs.shape, dropout_p, seed, offset, probs.device)
        probs = torch.where(keep, probs / (1.0 - dropout_p), torch.zeros_like(probs))
    ctx = torch.bmm(probs, vh)
    return ctx.view(b, h, s, d).permute(0, 2, 1, 3).contiguous()
