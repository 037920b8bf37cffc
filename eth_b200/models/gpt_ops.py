"""The GPT op graph: one class per manifest op, each with an explicit forward and backward.

A GPT model is the flat op list `[encoder-embedding] + 10 ops * L + [final-layernorm,
gpt-post-process]` (reference: eth/runtime/megatron/model/flex_gpt.py:23-43); a pipeline stage owns
a contiguous op range, so a stage cut may fall inside a layer. Ops exchange *named* tensors through
an environment dict (reference: the dict-of-tensors boundary of model/flex_model.py:171-240):

    hidden_states      main stream, [tokens, features] (tokens = batch*seq, batch-major)
    hidden_states_1/2  residual saved by the 1st / 2nd LayerNorm, consumed by the dropout-add op
    qkv                packed per-head [q|k|v], [tokens, 3*hidden/tp]
    output_bias        bias of a row-parallel GEMM, added after the tensor-parallel reduction

Differences from the reference that are deliberate B200 design:
  * no autograd graph: `fwd` stores what `bwd` needs in a per-micro-batch context;
  * biases, GeLU, GeLU-gradient and the gradient accumulation into `main_grad` run in GEMM epilogues;
  * activations stay token-major, so every GEMM / attention operand is TMA-addressable in place.
"""
from __future__ import annotations

import hashlib
import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..contract.config import FIRST_OP, MODEL_IMPLS, TAIL_OPS
from ..ops import raw


# ------------------------------------------------------------------------------------------
# configuration and parameter specs
# ------------------------------------------------------------------------------------------
@dataclass
class GPTModelConfig:
    num_layers: int
    hidden_size: int
    num_attention_heads: int
    seq_length: int
    max_position_embeddings: int
    padded_vocab_size: int
    hidden_dropout: float = 0.0
    layernorm_epsilon: float = 1e-5
    init_method_std: float = 0.02
    params_dtype: torch.dtype = torch.bfloat16
    grad_dtype: torch.dtype = torch.float32
    seed: int = 1234
    canonical_init: bool = False     # U(-0.02, 0.02) seeded by sha256(logical id), CPU generator
    zero_labels: bool = False        # the reference's synthetic labels are all zero
    model_impl: str = "gpt"          # "gpt": 10 ops per layer; "gpt-legacy13": unfused attention, 13 ops
    attention_dropout: float = 0.0   # used by the unfused attention ops only

    @property
    def ffn_hidden_size(self) -> int:
        return 4 * self.hidden_size

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads


@dataclass
class ParamSpec:
    """One parameter of one op: its logical identity and how this rank's piece is cut from it."""
    local_name: str                   # attribute name inside the op
    logical_id: str                   # topology-independent identity, e.g. gpt.layers.3.mlp.dense_h_to_4h.weight
    full_shape: Tuple[int, ...]
    partition_dim: int                # -1: replicated across TP
    partition_stride: int = 1
    init: str = "normal"              # normal | scaled_normal | ones | zeros
    weight_decay: bool = True
    shared_with: Optional[str] = None  # logical id this parameter is tied to (same storage if same stage)

    def local_shape(self, tp: int) -> Tuple[int, ...]:
        if self.partition_dim < 0:
            return tuple(self.full_shape)
        s = list(self.full_shape)
        s[self.partition_dim] //= tp
        return tuple(s)


class TPComm:
    """Tensor-parallel communication of one stage. `size == 1` makes every call a no-op."""

    def __init__(self, size: int = 1, rank: int = 0, group=None, backend=None):
        self.size, self.rank, self.group, self.backend = size, rank, group, backend

    def all_reduce_(self, t: torch.Tensor) -> torch.Tensor:
        if self.size > 1:
            if self.backend is not None:
                return self.backend.all_reduce_(t)
            torch.distributed.all_reduce(t, group=self.group)
        return t

    def linear_all_reduce(self, x, weight, *, b_mn=False, bias=None, residual=None, dropout=None):
        """sum over the TP group of x W^T (b_mn False) or x W (b_mn True): one fused kernel when the
        peer-memory backend is available, else a GEMM followed by an all-reduce. `bias`, `dropout`
        = (p, seed, offset) and `residual` are applied to the sum, once, in the same kernel; see
        `can_fuse_epilogue` for when that is possible."""
        if self.size > 1 and self.backend is not None and x.is_cuda:
            n = weight.shape[1] if b_mn else weight.shape[0]
            if self.backend.supports(x.shape[0], n):
                return self.backend.gemm_all_reduce(x, weight, b_mn=b_mn, bias=bias, residual=residual,
                                                    dropout=dropout)
        if self.size == 1:
            if bias is None and residual is None and dropout is None:
                return raw.gemm(x, weight, b_mn=b_mn)
            return raw.gemm(x, weight, b_mn=b_mn, bias=bias, aux=residual,
                            aux_mode=raw.AUX_ADD if residual is not None else raw.AUX_NONE, dropout=dropout)
        if bias is not None or residual is not None or dropout is not None:
            raise RuntimeError("an epilogue on the reduced sum needs the fused tensor-parallel kernel")
        y = raw.gemm(x, weight, b_mn=b_mn)
        return self.all_reduce_(y)

    def can_fuse_epilogue(self, rows: int, cols: int, on_gpu: bool) -> bool:
        """Whether `linear_all_reduce` can apply bias / dropout / residual to the reduced sum itself:
        always without tensor parallelism, else only inside the fused kernel."""
        if self.size == 1:
            return True
        return self.backend is not None and on_gpu and self.backend.supports(rows, cols)

    def reshard(self, x: torch.Tensor, step) -> torch.Tensor:
        """Run one placement change (`parallel.resharding.ReshardStep`) of a token-major tensor over
        this stage's tensor-parallel group. The placement algebra numbers dims (sequence, batch,
        hidden); here sequence and batch are folded into the rows, so the hidden dim is the last."""
        if self.size == 1 or step.primitive == "identity":
            return x
        from ..parallel.resharding import ReshardStep, apply_reshard
        last = x.dim() - 1
        local = ReshardStep(step.primitive, step.group_size, None if step.src_dim is None else last,
                            None if step.dst_dim is None else last)
        if step.group_size != self.size:
            raise ValueError(f"placement change over {step.group_size} ranks inside a TP group of {self.size}")
        return apply_reshard(x, local, self.group, self.rank)

    def gather_stats(self, stats: torch.Tensor) -> torch.Tensor:
        """[rows, 3] -> [tp, rows, 3] (cross-entropy statistics)."""
        if self.size == 1:
            return stats.unsqueeze(0)
        out = torch.empty((self.size,) + tuple(stats.shape), dtype=stats.dtype, device=stats.device)
        torch.distributed.all_gather_into_tensor(out.view(-1), stats.contiguous().view(-1), group=self.group)
        return out


def _seed_for(logical_id: str, base: int) -> int:
    h = hashlib.sha256(f"{base}:{logical_id}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def init_full_tensor(spec: ParamSpec, cfg: GPTModelConfig, device) -> torch.Tensor:
    """The full logical tensor in fp32; a rank slices its shard from it, so the initial weights do
    not depend on the parallel layout (reference evidence init: grad_sync/evidence.py:12-126)."""
    if spec.init == "ones":
        return torch.ones(spec.full_shape, dtype=torch.float32, device=device)
    if spec.init == "zeros":
        return torch.zeros(spec.full_shape, dtype=torch.float32, device=device)
    if cfg.canonical_init:
        g = torch.Generator(device="cpu")
        g.manual_seed(int.from_bytes(hashlib.sha256(spec.logical_id.encode()).digest()[:8], "little") & ((1 << 63) - 1))
        full = (torch.rand(spec.full_shape, generator=g, dtype=torch.float32) * 2 - 1) * 0.02
        return full.to(device)
    g = torch.Generator(device=device)
    g.manual_seed(_seed_for(spec.shared_with or spec.logical_id, cfg.seed))
    std = cfg.init_method_std
    if spec.init == "scaled_normal":
        std = std / math.sqrt(2.0 * cfg.num_layers)
    return torch.randn(spec.full_shape, generator=g, dtype=torch.float32, device=device) * std


def shard_of(full: torch.Tensor, spec: ParamSpec, tp: int, tp_rank: int) -> torch.Tensor:
    if spec.partition_dim < 0 or tp == 1:
        return full
    n = full.shape[spec.partition_dim]
    chunk = n // (tp * spec.partition_stride)
    parts = [full.narrow(spec.partition_dim, (b * tp + tp_rank) * chunk, chunk) for b in range(spec.partition_stride)]
    return parts[0] if len(parts) == 1 else torch.cat(parts, spec.partition_dim)


# ------------------------------------------------------------------------------------------
# op base
# ------------------------------------------------------------------------------------------
class Op:
    """Base of all stage-program ops. Subclasses define `specs`, `fwd`, `bwd`, `reads`, `writes`."""
    reads: Tuple[str, ...] = ("hidden_states",)
    writes: Tuple[str, ...] = ("hidden_states",)
    consumes: Tuple[str, ...] = ()     # names removed from the environment by this op

    def __init__(self, name: str, op_index: int, layer_index: Optional[int], cfg: GPTModelConfig, tp: TPComm):
        self.name, self.op_index, self.layer_index, self.cfg, self.tp = name, op_index, layer_index, cfg, tp
        self.params: Dict[str, torch.Tensor] = {}
        self.fuse_next = False   # set by the stage builder when the following op is fused into this one
        self.fuse_prev = False
        self.slabs = raw.ColumnSumSlabs()   # used by ops whose backward leaves partial column sums
        self.algo = 0

    def set_algo(self, algo: int) -> None:
        """Sharding choice of a tensor-parallel GEMM op: 0 = its usual column- or row-parallel form,
        1 = the other one (reference: model/flex_ops.py:140-236 `gen_op(..., algo)`). With algo 1 the
        op keeps its placement contract towards its neighbours (what it reads and writes is sharded
        as under algo 0) and converts at its own input and output; the conversions are the ones the
        placement algebra plans between the two algos' specs (`search/model_ops.get_op_spec`,
        `parallel/resharding.plan_reshard`; reference: mpu/mappings.py:381-467 `tensor_adapter`)."""
        from ..parallel.resharding import plan_reshard
        from ..search.model_ops import get_op_spec
        if algo not in (0, 1):
            raise ValueError(f"algo {algo} is not implemented (0 or 1)")
        self.algo = int(algo) if self.tp.size > 1 else 0
        t = self.tp.size
        self.in_step = plan_reshard(get_op_spec(self.name, t, 1, 0, True), get_op_spec(self.name, t, 1, self.algo, True))
        self.out_step = plan_reshard(get_op_spec(self.name, t, 1, self.algo, False), get_op_spec(self.name, t, 1, 0, False))

    def specs(self) -> List[ParamSpec]:
        return []

    def _lid(self, suffix: str) -> str:
        return f"gpt.layers.{self.layer_index}.{suffix}"

    def p(self, name: str) -> torch.Tensor:
        return self.params[name]

    def fwd(self, env: dict, ctx: dict, mb) -> None:
        raise NotImplementedError

    def bwd(self, genv: dict, ctx: dict, mb) -> None:
        raise NotImplementedError

    def dropout_offset(self, mb) -> int:
        """Philox offset: distinct per optimizer step, micro-batch and data-parallel replica, equal
        across the tensor-parallel ranks of a replica (they must draw the same mask)."""
        return ((int(getattr(mb, "global_step", 0)) << 24) + (int(getattr(mb, "index", 0)) << 8)
                + int(getattr(mb, "dp_rank", 0)))

    def __repr__(self):
        return f"{type(self).__name__}({self.op_index}:{self.name})"


def _take(genv: dict, name: str):
    g = genv.pop(name, None)
    if g is None:
        raise RuntimeError(f"missing gradient for {name}")
    return g


def _acc(genv: dict, name: str, g: torch.Tensor) -> None:
    old = genv.get(name)
    if old is None:
        genv[name] = g
    else:
        old.add_(g)


# ------------------------------------------------------------------------------------------
# embedding
# ------------------------------------------------------------------------------------------
class EmbeddingOp(Op):
    """Vocab-parallel word embedding + position embedding (+ dropout). TP ranks hold vocab shards;
    partial rows are summed over the TP group (reference: mpu/layers.py:136-205)."""
    reads = ("enc_input_ids",)
    writes = ("hidden_states",)

    def specs(self):
        c = self.cfg
        return [ParamSpec("word", "gpt.word_embeddings.weight", (c.padded_vocab_size, c.hidden_size), 0),
                ParamSpec("pos", "gpt.position_embeddings.weight", (c.max_position_embeddings, c.hidden_size), -1)]

    def fwd(self, env, ctx, mb):
        tokens = env["enc_input_ids"]
        seq = tokens.shape[-1]
        vstart = self.tp.rank * (self.cfg.padded_vocab_size // self.tp.size)
        out = raw.embedding_fwd(tokens, self.p("word"), self.p("pos"), seq, vstart, self.tp.rank == 0)
        self.tp.all_reduce_(out)
        p = self.cfg.hidden_dropout
        if p > 0:
            ctx["drop"] = (p, self.cfg.seed + self.op_index, self.dropout_offset(mb))
            out = raw.bias_dropout_add_fwd(out, None, None, *ctx["drop"])
        ctx["tokens"], ctx["seq"], ctx["vstart"] = tokens, seq, vstart
        env["hidden_states"] = out

    def bwd(self, genv, ctx, mb):
        d = _take(genv, "hidden_states")
        if "drop" in ctx:
            d = raw.dropout_bwd(d, *ctx["drop"])
        # position embeddings are replicated: every TP rank accumulates the full gradient
        raw.embedding_bwd(ctx["tokens"], d, self.p("word"), self.p("pos"), ctx["seq"], ctx["vstart"], True)


# ------------------------------------------------------------------------------------------
# transformer layer ops
# ------------------------------------------------------------------------------------------
class LayerNormOp(Op):
    """LayerNorm that also publishes its input as the residual of the following sub-block."""

    def __init__(self, *a, residual_name: Optional[str], prefix: str, **k):
        super().__init__(*a, **k)
        self.residual_name, self.prefix = residual_name, prefix
        self.writes = ("hidden_states",) + ((residual_name,) if residual_name else ())

    def specs(self):
        h = self.cfg.hidden_size
        base = self._lid(self.prefix) if self.layer_index is not None else "gpt.final_layernorm"
        return [ParamSpec("weight", base + ".weight", (h,), -1, init="ones", weight_decay=False),
                ParamSpec("bias", base + ".bias", (h,), -1, init="zeros", weight_decay=False)]

    def fwd(self, env, ctx, mb):
        x = env["hidden_states"]
        y, mean, rstd = raw.ln_fwd(x, self.p("weight"), self.p("bias"), self.cfg.layernorm_epsilon)
        ctx["x"], ctx["mean"], ctx["rstd"] = x, mean, rstd
        if self.residual_name:
            env[self.residual_name] = x
        env["hidden_states"] = y

    def bwd(self, genv, ctx, mb):
        dy = _take(genv, "hidden_states")
        res = genv.pop(self.residual_name, None) if self.residual_name else None
        genv["hidden_states"] = raw.ln_bwd(dy, ctx["x"], self.p("weight"), self.p("bias"), ctx["mean"],
                                           ctx["rstd"], residual_grad=res, slabs=self.slabs,
                                           ws_mode=getattr(mb, "colsum_mode", raw.WS_IMMEDIATE))


class ColumnLinearOp(Op):
    """Column-parallel GEMM: weight [out/tp, in]; forward needs no communication, the data gradient
    is summed over the TP group (reference: mpu/layers.py:282-370, mappings.py:84-97)."""

    def __init__(self, *a, in_features: int, out_features: int, suffix: str, out_name: str = "hidden_states", **k):
        super().__init__(*a, **k)
        self.in_features, self.out_features, self.suffix, self.out_name = in_features, out_features, suffix, out_name
        self.writes = (out_name,)
        self.consumes = ("hidden_states",) if out_name != "hidden_states" else ()

    def specs(self):
        # algo 1 runs this GEMM row-parallel: the weight is cut along its input features and the
        # bias, added after the reduction, is replicated
        wdim, bdim = (0, 0) if self.algo == 0 else (1, -1)
        return [ParamSpec("weight", self._lid(self.suffix + ".weight"), (self.out_features, self.in_features), wdim),
                ParamSpec("bias", self._lid(self.suffix + ".bias"), (self.out_features,), bdim, init="zeros",
                          weight_decay=False)]

    def _fwd_row(self, env, ctx):
        x = self.tp.reshard(env.pop("hidden_states"), self.in_step)          # replicated -> my input features
        ctx["x"] = x
        y = self.tp.linear_all_reduce(x, self.p("weight"))                    # [tokens, out], summed over TP
        y = raw.bias_dropout_add_fwd(y, self.p("bias"), None, 0.0, 0, 0)
        env[self.out_name] = self.tp.reshard(y, self.out_step)                # replicated -> my output features

    def _bwd_row(self, genv, ctx):
        dy = self.tp.reshard(_take(genv, self.out_name), self.out_step.dual())
        dx = raw.linear_dgrad(dy, self.p("weight"))                           # my input features only
        raw.linear_wgrad(dy, ctx["x"], self.p("weight"), self.p("bias"))
        genv["hidden_states"] = self.tp.reshard(dx, self.in_step.dual())

    def fwd(self, env, ctx, mb):
        if self.algo == 1:
            return self._fwd_row(env, ctx)
        x = env.pop("hidden_states")
        ctx["x"] = x
        if self.fuse_next:   # GeLU in the GEMM epilogue
            pre, act = raw.linear_fwd(x, self.p("weight"), self.p("bias"), gelu=True)
            env[self.out_name] = pre
            env["_gelu_out"] = act
        else:
            env[self.out_name] = raw.linear_fwd(x, self.p("weight"), self.p("bias"))

    def bwd(self, genv, ctx, mb):
        if self.algo == 1:
            return self._bwd_row(genv, ctx)
        dy = _take(genv, self.out_name)
        dx = self.tp.linear_all_reduce(dy, self.p("weight"), b_mn=True)
        raw.linear_wgrad(dy, ctx["x"], self.p("weight"), self.p("bias"))
        genv["hidden_states"] = dx


class RowLinearOp(Op):
    """Row-parallel GEMM: weight [out, in/tp]; partial outputs are summed over the TP group, the
    bias travels separately (`output_bias`) and is added by the following dropout-add op
    (reference: mpu/layers.py:373-468, model/flex_ops.py:1600-1632)."""
    writes = ("hidden_states", "output_bias")

    def __init__(self, *a, in_features: int, out_features: int, suffix: str, **k):
        super().__init__(*a, **k)
        self.in_features, self.out_features, self.suffix = in_features, out_features, suffix
        self.fused_dropout_add = None   # the following BiasDropoutAddOp when the stage builder fused it in

    def specs(self):
        # algo 1 runs this GEMM column-parallel (weight cut along its output features); the bias stays
        # replicated and still travels to the dropout-add op, which adds it to the gathered output
        return [ParamSpec("weight", self._lid(self.suffix + ".weight"), (self.out_features, self.in_features),
                          1 if self.algo == 0 else 0, init="scaled_normal"),
                ParamSpec("bias", self._lid(self.suffix + ".bias"), (self.out_features,), -1, init="zeros",
                          weight_decay=False)]

    def fwd(self, env, ctx, mb):
        env["output_bias"] = self.p("bias")
        if self.algo == 1:
            x = self.tp.reshard(env["hidden_states"], self.in_step)           # my input features -> all of them
            ctx["x"] = x
            y = raw.linear_fwd(x, self.p("weight"))                            # my output features
            env["hidden_states"] = self.tp.reshard(y, self.out_step)           # -> replicated
            return
        x = env["hidden_states"]
        ctx["x"] = x
        nxt = self.fused_dropout_add
        if nxt is not None and self.tp.can_fuse_epilogue(x.shape[0], self.out_features, x.is_cuda):
            # the following bias-dropout-add runs in this GEMM's epilogue (on the reduced sum under TP);
            # that op then only records what its backward needs
            drop = (self.cfg.hidden_dropout, self.cfg.seed + nxt.op_index, nxt.dropout_offset(mb))
            out = self.tp.linear_all_reduce(x, self.p("weight"), bias=self.p("bias"),
                                            residual=env[nxt.residual_name], dropout=drop)
            if getattr(out, "_ethb_ring", False):
                # the fused tensor-parallel kernel returns a slot of a short ring that peers write into;
                # this tensor is the residual stream, which LayerNorm keeps for its backward: move it out
                out = out.clone()
            env["hidden_states"] = out
            env["_dropout_add_done"] = drop
            return
        env["hidden_states"] = self.tp.linear_all_reduce(x, self.p("weight"))

    def bwd(self, genv, ctx, mb):
        dy = _take(genv, "hidden_states")
        db = genv.pop("output_bias", None)
        if db is not None:
            self.p("bias").main_grad.view(-1).add_(db.to(self.p("bias").main_grad.dtype).view(-1))
        if self.algo == 1:
            dy = self.tp.reshard(dy, self.out_step.dual())
            dx = self.tp.linear_all_reduce(dy, self.p("weight"), b_mn=True)   # all input features, summed over TP
            genv["hidden_states"] = self.tp.reshard(dx, self.in_step.dual())
            raw.linear_wgrad(dy, ctx["x"], self.p("weight"))
            return
        gelu_pre = mb.ctxs[self.op_index - 1]["pre"] if self.fuse_prev else None
        genv["hidden_states"] = raw.linear_dgrad(dy, self.p("weight"), gelu_pre=gelu_pre)
        if gelu_pre is not None:
            genv["_gelu_grad_done"] = True
        raw.linear_wgrad(dy, ctx["x"], self.p("weight"))


class FlashAttentionOp(Op):
    """Causal self-attention over this rank's heads; consumes the packed qkv tensor
    (reference: model/flex_ops.py:1377-1426 + F.scaled_dot_product_attention :66-96)."""
    reads = ("qkv",)
    writes = ("hidden_states",)
    consumes = ("qkv",)

    def fwd(self, env, ctx, mb):
        qkv = env.pop("qkv")
        heads = self.cfg.num_attention_heads // self.tp.size
        out, lse = raw.attention_fwd(qkv, mb.batch, mb.seq, heads, self.cfg.head_dim)
        ctx["qkv"], ctx["out"], ctx["lse"], ctx["shape"] = qkv, out, lse, (mb.batch, mb.seq, heads)
        env["hidden_states"] = out

    def bwd(self, genv, ctx, mb):
        d = _take(genv, "hidden_states")
        b, s, heads = ctx["shape"]
        genv["qkv"] = raw.attention_bwd(d.contiguous(), ctx["qkv"], ctx["out"], ctx["lse"], b, s, heads,
                                        self.cfg.head_dim)


class AttentionScoreOp(Op):
    """Unfused attention, op 1 of 4: raw scores Q K^T per head as batched tcgen05 GEMMs. `qkv` stays
    alive for the context op (reference: ParallelAttentionScoreOp, model/flex_ops.py:1144-1244)."""
    reads = ("qkv",)
    writes = ("attention_scores", "qkv")

    def fwd(self, env, ctx, mb):
        qkv = env["qkv"]
        heads = self.cfg.num_attention_heads // self.tp.size
        ctx["qkv"], ctx["shape"] = qkv, (mb.batch, mb.seq, heads, self.cfg.head_dim)
        env["attention_scores"] = raw.attn_scores_fwd(qkv, *ctx["shape"])

    def bwd(self, genv, ctx, mb):
        d_scores = _take(genv, "attention_scores")
        dqkv = genv.get("qkv")      # created by the context op's backward (v slot already filled)
        if dqkv is None:
            raise RuntimeError("missing gradient for qkv: the context op must run its backward first")
        raw.attn_scores_bwd(d_scores, ctx["qkv"], dqkv, *ctx["shape"])


class AttentionSoftmaxOp(Op):
    """Unfused attention, op 2 of 4: softmax(scores / sqrt(d)) with the implicit causal mask
    (reference: ParallelSoftmaxFusionOp, model/flex_ops.py:1246-1330)."""
    reads = ("attention_scores",)
    writes = ("attention_probs",)
    consumes = ("attention_scores",)

    def fwd(self, env, ctx, mb):
        scale = 1.0 / math.sqrt(self.cfg.head_dim)
        probs = raw.softmax_fwd(env.pop("attention_scores"), scale, causal=True)
        ctx["probs"], ctx["scale"] = probs, scale
        env["attention_probs"] = probs

    def bwd(self, genv, ctx, mb):
        d = _take(genv, "attention_probs")
        genv["attention_scores"] = raw.softmax_bwd(d, ctx["probs"], ctx["scale"], causal=True)


class AttentionDropoutOp(Op):
    """Unfused attention, op 3 of 4: dropout on the attention probabilities
    (reference: ParallelSoftmaxDropoutOp, model/flex_ops.py:1332-1374)."""
    reads = ("attention_probs",)
    writes = ("attention_probs",)

    def fwd(self, env, ctx, mb):
        p = self.cfg.attention_dropout
        if p > 0:
            ctx["drop"] = (p, self.cfg.seed + self.op_index, self.dropout_offset(mb) + self.tp.rank)
            probs = env["attention_probs"]
            env["attention_probs"] = raw.bias_dropout_add_fwd(probs.view(-1, probs.shape[-1]), None, None,
                                                              *ctx["drop"]).view(probs.shape)

    def bwd(self, genv, ctx, mb):
        if "drop" in ctx:
            d = _take(genv, "attention_probs")
            genv["attention_probs"] = raw.dropout_bwd(d.view(-1, d.shape[-1]), *ctx["drop"]).view(d.shape)


class AttentionContextOp(Op):
    """Unfused attention, op 4 of 4: context = P V per head (batched tcgen05 GEMMs), token-major
    (reference: ParallelContextOp, model/flex_ops.py:1431-1519)."""
    reads = ("attention_probs", "qkv")
    writes = ("hidden_states",)
    consumes = ("attention_probs", "qkv")

    def fwd(self, env, ctx, mb):
        probs, qkv = env.pop("attention_probs"), env.pop("qkv")
        heads = self.cfg.num_attention_heads // self.tp.size
        ctx["probs"], ctx["qkv"], ctx["shape"] = probs, qkv, (mb.batch, mb.seq, heads, self.cfg.head_dim)
        env["hidden_states"] = raw.attn_context_fwd(probs, qkv, *ctx["shape"])

    def bwd(self, genv, ctx, mb):
        d = _take(genv, "hidden_states")
        d_probs, dqkv = raw.attn_context_bwd(d.contiguous(), ctx["probs"], ctx["qkv"], *ctx["shape"])
        genv["attention_probs"] = d_probs
        genv["qkv"] = dqkv


class BiasDropoutAddOp(Op):
    """hidden = residual + dropout(hidden + output_bias) (reference: model/flex_ops.py:104-134)."""

    def __init__(self, *a, residual_name: str, **k):
        super().__init__(*a, **k)
        self.residual_name = residual_name
        self.reads = ("hidden_states", "output_bias", residual_name)
        self.consumes = ("output_bias", residual_name)

    def fwd(self, env, ctx, mb):
        x, bias, res = env["hidden_states"], env.pop("output_bias"), env.pop(self.residual_name)
        p = self.cfg.hidden_dropout
        ctx["drop"] = (p, self.cfg.seed + self.op_index, self.dropout_offset(mb))
        ctx["bias"] = bias
        done = env.pop("_dropout_add_done", None)
        if done is not None:      # the producing GEMM already applied bias, this dropout and the residual
            if done != ctx["drop"]:
                raise RuntimeError("fused dropout-add used other dropout parameters than this op")
            return
        env["hidden_states"] = raw.bias_dropout_add_fwd(x, bias, res, *ctx["drop"])

    def bwd(self, genv, ctx, mb):
        dout = _take(genv, "hidden_states")
        genv[self.residual_name] = dout
        mode = getattr(mb, "colsum_mode", raw.WS_IMMEDIATE)
        bias = ctx.get("bias")
        if mode != raw.WS_IMMEDIATE and bias is not None and getattr(bias, "main_grad", None) is not None:
            # the bias is a parameter of this rank: its gradient goes straight to main_grad, through
            # this op's own slabs, once per step
            dx = raw.dropout_bwd_colsum_into(dout, *ctx["drop"], bias.main_grad, self.slabs, mode)
            if dx is not None:
                genv["hidden_states"] = dx
                return
        dx, dbias = raw.dropout_bwd_colsum(dout, *ctx["drop"])
        genv["hidden_states"] = dx
        genv["output_bias"] = dbias


class GeluOp(Op):
    """tanh-GeLU. When the preceding GEMM already produced it in its epilogue, forward is free;
    when the following row-parallel GEMM multiplies by gelu' in its data-gradient epilogue,
    backward is free as well."""

    def fwd(self, env, ctx, mb):
        pre = env["hidden_states"]
        ctx["pre"] = pre
        act = env.pop("_gelu_out", None)
        if act is None:
            act = raw.gelu_fwd(pre)
        env["hidden_states"] = act

    def bwd(self, genv, ctx, mb):
        if genv.pop("_gelu_grad_done", False):
            return
        dy = _take(genv, "hidden_states")
        genv["hidden_states"] = raw.gelu_bwd(dy, ctx["pre"])


class PostProcessOp(Op):
    """Tied LM head (logits = h E^T over this rank's vocab shard) + vocab-parallel cross entropy.
    Output: per-token losses (reference: model/flex_ops.py:1908-1985, mpu/cross_entropy.py:33-118)."""
    writes = ("output",)
    consumes = ("hidden_states",)

    def specs(self):
        c = self.cfg
        return [ParamSpec("word", "gpt.word_embeddings.weight", (c.padded_vocab_size, c.hidden_size), 0,
                          shared_with="gpt.word_embeddings.weight")]

    def fwd(self, env, ctx, mb):
        x = env.pop("hidden_states")
        w = self.p("word")
        logits = raw.linear_fwd(x, w)
        vstart = self.tp.rank * (self.cfg.padded_vocab_size // self.tp.size)
        labels = env["labels"]
        loss, gmax, gsum = raw.ce_fwd(logits, labels, vstart, self.tp.gather_stats if self.tp.size > 1 else None)
        ctx.update(x=x, logits=logits, labels=labels, gmax=gmax, gsum=gsum, vstart=vstart)
        env["output"] = loss

    def bwd(self, genv, ctx, mb):
        dloss = _take(genv, "output")
        dlogits = raw.ce_bwd_(ctx["logits"], ctx["labels"], ctx["gmax"], ctx["gsum"], dloss, ctx["vstart"])
        w = self.p("word")
        dx = self.tp.linear_all_reduce(dlogits, w, b_mn=True)
        raw.linear_wgrad(dlogits, ctx["x"], w)
        ctx.pop("logits")
        genv["hidden_states"] = dx


# ------------------------------------------------------------------------------------------
# manifest -> ops
# ------------------------------------------------------------------------------------------
def build_op_descriptors(num_layers: int, model_impl: str = "gpt") -> List[dict]:
    """Runtime op list in manifest order: [{op_index, name, layer_index, prev_name}]."""
    layer_ops = MODEL_IMPLS[model_impl]["layer_schema"]
    names: List[Tuple[str, Optional[int]]] = [(FIRST_OP, None)]
    for layer in range(num_layers):
        names += [(n, layer) for n in layer_ops]
    names += [(n, None) for n in TAIL_OPS]
    out = []
    for i, (n, layer) in enumerate(names):
        out.append({"op_index": i, "name": n, "layer_index": layer, "prev_name": names[i - 1][0] if i else None})
    return out


def make_op(desc: dict, cfg: GPTModelConfig, tp: TPComm, algo: int = 0) -> Op:
    op = _make_op(desc, cfg, tp)
    if algo:
        if not isinstance(op, (ColumnLinearOp, RowLinearOp)):
            algo = 0      # only the four tensor-parallel GEMMs have a second sharding choice
        else:
            op.set_algo(algo)
    return op


def _make_op(desc: dict, cfg: GPTModelConfig, tp: TPComm) -> Op:
    n, i, layer = desc["name"], desc["op_index"], desc["layer_index"]
    h, f = cfg.hidden_size, cfg.ffn_hidden_size
    a = (n, i, layer, cfg, tp)
    if n == FIRST_OP:
        return EmbeddingOp(*a)
    if n == "enc-1st-layernorm":
        return LayerNormOp(*a, residual_name="hidden_states_1", prefix="input_layernorm")
    if n == "enc-attention-qkv":
        return ColumnLinearOp(*a, in_features=h, out_features=3 * h, suffix="attention.query_key_value", out_name="qkv")
    if n == "enc-flash-attention":
        return FlashAttentionOp(*a)
    if n == "enc-attention-score":
        return AttentionScoreOp(*a)
    if n == "enc-attention-softmax":
        return AttentionSoftmaxOp(*a)
    if n == "enc-attention-dropout":
        return AttentionDropoutOp(*a)
    if n == "enc-attention-context":
        return AttentionContextOp(*a)
    if n == "enc-attention-dense":
        return RowLinearOp(*a, in_features=h, out_features=h, suffix="attention.dense")
    if n == "enc-post-attention-dropout":
        return BiasDropoutAddOp(*a, residual_name="hidden_states_1")
    if n == "enc-2nd-layernorm":
        return LayerNormOp(*a, residual_name="hidden_states_2", prefix="post_attention_layernorm")
    if n == "enc-MLP-GEMM-1":
        return ColumnLinearOp(*a, in_features=h, out_features=f, suffix="mlp.dense_h_to_4h")
    if n == "enc-MLP-gelu":
        return GeluOp(*a)
    if n == "enc-MLP-GEMM-2":
        return RowLinearOp(*a, in_features=f, out_features=h, suffix="mlp.dense_4h_to_h")
    if n == "enc-post-MLP-dropout":
        return BiasDropoutAddOp(*a, residual_name="hidden_states_2")
    if n == "final-layernorm":
        return LayerNormOp(*a, residual_name=None, prefix="final_layernorm")
    if n == "gpt-post-process":
        return PostProcessOp(*a)
    raise ValueError(f"unknown op {n!r}")


# Named tensors alive right after each op, i.e. what crosses a stage boundary placed there:
# name -> (features, tp_sharded, per_token). `features` is a multiple of hidden_size; a TP-sharded
# tensor holds features/tp columns per rank; per_token tensors have one row per token (dim 0 is
# batch-major, so data-parallel ranks own contiguous row blocks), others are [features] vectors.
_H = ("hidden_states", 1, False, True)
_R1 = ("hidden_states_1", 1, False, True)
_R2 = ("hidden_states_2", 1, False, True)
_B = ("output_bias", 1, False, False)
LIVE_AFTER = {
    "encoder-embedding": (_H,),
    "enc-1st-layernorm": (_H, _R1),
    "enc-attention-qkv": (("qkv", 3, True, True), _R1),
    "enc-flash-attention": (("hidden_states", 1, True, True), _R1),
    # the per-head [seq x seq] tensors of the unfused attention block are not token-major: a stage
    # boundary may not fall inside that block
    "enc-attention-score": None,
    "enc-attention-softmax": None,
    "enc-attention-dropout": None,
    "enc-attention-context": (("hidden_states", 1, True, True), _R1),
    "enc-attention-dense": (_H, _B, _R1),
    "enc-post-attention-dropout": (_H,),
    "enc-2nd-layernorm": (_H, _R2),
    "enc-MLP-GEMM-1": (("hidden_states", 4, True, True), _R2),
    "enc-MLP-gelu": (("hidden_states", 4, True, True), _R2),
    "enc-MLP-GEMM-2": (_H, _B, _R2),
    "enc-post-MLP-dropout": (_H,),
    "final-layernorm": (_H,),
    "gpt-post-process": (),
}
