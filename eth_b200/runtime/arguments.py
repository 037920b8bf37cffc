"""Runtime flags of `pretrain_gpt` (reference flag surface: eth/runtime/megatron/arguments.py --
groups network/regularization/training/initialization/learning-rate/checkpointing/mixed-precision/
distributed/data :285-806, grad_sync :712-734, flexpipe :808-821, profiler :823-843).

`parse_args` reads RANK / WORLD_SIZE from the environment, loads and normalizes the HPP config,
builds the canonical topology and derives the per-rank view (pipeline, stage, micro-batch
schedule, nominal loss scale). In profiler mode (`--prof-tp-size`) a single-stage config with
TP = that size is synthesized instead (:161-175).
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from ..contract.config import (apply_normalized_config_to_args, make_config, make_pipe, manifest_size,
                               normalize_flexpipe_config)
from ..parallel.grad_sync.topology import build_canonical_topology


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description="eth_b200 GPT pretraining", allow_abbrev=False)
    g = p.add_argument_group("network size")
    g.add_argument("--num-layers", type=int, default=None, help="Number of transformer layers (taken from the config).")
    g.add_argument("--hidden-size", type=int, default=None, help="Transformer hidden size (taken from the config).")
    g.add_argument("--num-attention-heads", type=int, default=None, help="Number of attention heads (from the config).")
    g.add_argument("--seq-length", type=int, default=None, help="Sequence length (taken from the config).")
    g.add_argument("--max-position-embeddings", type=int, default=None, help="Maximum position embeddings.")
    g.add_argument("--make-vocab-size-divisible-by", type=int, default=128,
                   help="Pad the vocabulary to a multiple of this value times the largest TP degree.")
    g.add_argument("--vocab-size", type=int, default=50257, help="Unpadded vocabulary size.")
    g.add_argument("--layernorm-epsilon", type=float, default=1e-5, help="LayerNorm epsilon.")

    g = p.add_argument_group("regularization")
    g.add_argument("--attention-dropout", type=float, default=0.0,
                   help="Attention dropout probability (the flash-attention path supports 0 only).")
    g.add_argument("--hidden-dropout", type=float, default=0.1, help="Dropout probability of the hidden state.")
    g.add_argument("--weight-decay", type=float, default=0.01, help="Weight decay coefficient.")
    g.add_argument("--clip-grad", type=float, default=1.0, help="Gradient clipping by global L2 norm (0 disables).")
    g.add_argument("--adam-beta1", type=float, default=0.9, help="Adam beta1.")
    g.add_argument("--adam-beta2", type=float, default=0.999, help="Adam beta2.")
    g.add_argument("--adam-eps", type=float, default=1e-8, help="Adam epsilon.")
    g.add_argument("--sgd-momentum", type=float, default=0.9, help="SGD momentum.")

    g = p.add_argument_group("training")
    g.add_argument("--train-iters", type=int, default=3, help="Number of training iterations.")
    g.add_argument("--log-interval", type=int, default=1, help="Iterations between console reports.")
    g.add_argument("--exit-interval", type=int, default=None, help="Save and exit when iteration % this == 0.")
    g.add_argument("--exit-duration-in-mins", type=int, default=None, help="Save and exit after this many minutes.")
    g.add_argument("--tensorboard-dir", type=str, default=None, help="Write tensorboard logs here (last rank).")
    g.add_argument("--optimizer", type=str, default="adam", choices=["adam", "sgd"], help="Optimizer.")
    g.add_argument("--eval-iters", type=int, default=0, help="Evaluation iterations (0 disables evaluation).")
    g.add_argument("--eval-interval", type=int, default=1000, help="Iterations between evaluations.")
    g.add_argument("--async-optimizer", action="store_true",
                   help="Do not read the overflow flag / norm back each step (bf16 runs); the kernels skip on overflow.")
    g.add_argument("--host-data", action="store_true",
                   help="Build every synthetic batch on the host and copy it from pinned memory (the input path "
                        "a dataset takes; ignored with --data-path).")

    g = p.add_argument_group("initialization")
    g.add_argument("--seed", type=int, default=1234, help="Random seed.")
    g.add_argument("--init-method-std", type=float, default=0.02, help="Std of the normal weight initialisation.")

    g = p.add_argument_group("learning rate")
    g.add_argument("--lr", type=float, default=1.5e-4, help="Peak learning rate.")
    g.add_argument("--lr-decay-style", type=str, default="cosine", choices=["constant", "linear", "cosine"],
                   help="Learning-rate decay function.")
    g.add_argument("--lr-decay-iters", type=int, default=320000, help="Iterations over which the rate decays.")
    g.add_argument("--lr-warmup-fraction", type=float, default=0.01, help="Fraction of decay iterations used to warm up.")
    g.add_argument("--lr-warmup-iters", type=int, default=0, help="Warm-up iterations (alternative to the fraction).")
    g.add_argument("--min-lr", type=float, default=1.0e-5, help="Minimum learning rate.")
    g.add_argument("--override-lr-scheduler", action="store_true", help="Ignore scheduler values stored in a checkpoint.")
    g.add_argument("--use-checkpoint-lr-scheduler", action="store_true", help="Use scheduler values from the checkpoint.")

    g = p.add_argument_group("checkpointing")
    g.add_argument("--save", type=str, default=None, help="Directory to save checkpoints to.")
    g.add_argument("--save-interval", type=int, default=None, help="Iterations between checkpoints.")
    g.add_argument("--load", type=str, default=None, help="Directory to load a checkpoint from.")
    g.add_argument("--no-save-optim", action="store_true", help="Do not save the optimizer state.")
    g.add_argument("--no-save-rng", action="store_true", help="Do not save RNG state.")
    g.add_argument("--no-load-optim", action="store_true", help="Do not load the optimizer state.")
    g.add_argument("--no-load-rng", action="store_true", help="Do not load RNG state.")
    g.add_argument("--finetune", action="store_true", help="Load weights only and restart the iteration count.")

    g = p.add_argument_group("mixed precision")
    g.add_argument("--fp16", action="store_true", help="Run the model in fp16 with loss scaling.")
    g.add_argument("--bf16", action="store_true", help="Run the model in bf16 (fp32 gradient accumulation).")
    g.add_argument("--loss-scale", type=float, default=None, help="Static loss scale (dynamic scaling when unset).")
    g.add_argument("--initial-loss-scale", type=float, default=2 ** 32, help="Initial dynamic loss scale.")
    g.add_argument("--min-loss-scale", type=float, default=1.0, help="Minimum dynamic loss scale.")
    g.add_argument("--loss-scale-window", type=float, default=1000, help="Clean steps before the scale grows.")
    g.add_argument("--hysteresis", type=int, default=2, help="Overflows tolerated before the scale shrinks.")
    g.add_argument("--accumulate-allreduce-grads-in-fp32", action="store_true",
                   help="Accumulate and all-reduce gradients in fp32 (forced for bf16).")

    g = p.add_argument_group("distributed")
    g.add_argument("--distributed-backend", default="nccl", choices=["nccl", "gloo"], help="torch.distributed backend.")
    g.add_argument("--DDP-impl", default="local", choices=["local"], help="Gradient buffer implementation.")
    g.add_argument("--local_rank", "--local-rank", type=int, default=None, help="Local rank passed by the launcher.")
    g.add_argument("--tp-comm", default="auto", choices=["auto", "nccl", "fused"],
                   help="Tensor-parallel reductions: NCCL all-reduce, or the fused GEMM + peer all-reduce kernel.")
    g.add_argument("--p2p-backend", default="auto", choices=["auto", "nccl", "peer"],
                   help="Pipeline transfers: NCCL isend/irecv, or copies into ring slots in peer memory with flag "
                        "waits (one node, non-interleaved schedule; auto picks it where it applies).")
    g.add_argument("--device", default=None, help="Device override (cpu for validation runs).")

    g = p.add_argument_group("data")
    g.add_argument("--data-path", nargs="*", default=None,
                   help="One prefix of an indexed token dataset, or weight/prefix pairs to blend. Without it the "
                        "run trains on synthetic tokens.")
    g.add_argument("--split", type=str, default="949,50,1",
                   help="Train/valid/test proportions of the documents of each dataset.")
    g.add_argument("--vocab-file", type=str, default=None,
                   help="GPT-2 vocabulary json; with --merge-file it sets the vocabulary size and the "
                        "end-of-document token.")
    g.add_argument("--merge-file", type=str, default=None, help="GPT-2 BPE merges.")
    g.add_argument("--eod-mask-loss", action="store_true", help="No loss on end-of-document tokens.")
    g.add_argument("--reset-position-ids", action="store_true", help="Not supported (positions run over the sequence).")
    g.add_argument("--reset-attention-mask", action="store_true",
                   help="Not supported (attention is causal over the whole sequence).")
    g.add_argument("--data-impl", type=str, default="mmap", choices=["lazy", "cached", "mmap", "infer"],
                   help="Indexed dataset implementation.")
    g.add_argument("--reference-zero-labels", action="store_true",
                   help="Use all-zero labels like the reference's synthetic post-process op.")

    g = p.add_argument_group("grad_sync")
    g.add_argument("--grad-sync-mode", default="tensor", choices=["tensor", "block"],
                   help="One collective per gradient fragment, or block-wise buckets.")
    g.add_argument("--grad-sync-bucket-size-mb", type=int, default=32, help="Bucket cap in MiB for block mode.")
    g.add_argument("--no-async-wgrad", dest="async_wgrad", action="store_false",
                   help="Run weight-gradient GEMMs on the main stream (default: on a side stream, so that their "
                        "partly filled last wave overlaps the data-gradient GEMM of the same layer).")
    g.add_argument("--no-overlap-grad-sync", dest="overlap_grad_sync", action="store_false",
                   help="Reduce all gradient buckets after backward. By default a bucket served by the peer-memory "
                        "backend is reduced on a side stream as soon as the last micro-batch's backward has passed "
                        "its first op.")
    g.add_argument("--no-deferred-colsums", dest="no_deferred_colsums", action="store_true",
                   help="Sum LayerNorm-weight and bias gradients after every micro-batch (default: partial column "
                        "sums stay in per-op slabs and are summed once per step, with the last micro-batch).")
    g.add_argument("--grad-sync-backend", default="auto", choices=["auto", "collective", "peer"],
                   help="Reduction backend: torch.distributed all-reduce or the peer-memory kernel.")
    g.add_argument("--grad-sync-dump-plan", type=str, default=None, help="Write the gradient sync plan as JSON.")
    g.add_argument("--grad-sync-debug-replicated-check", action="store_true",
                   help="Verify after every sync that replicated gradients agree across their holders.")
    g.add_argument("--grad-sync-metadata-transport", default="auto", choices=["auto", "object", "tensor"],
                   help="How descriptors are gathered at start-up.")
    g.add_argument("--grad-sync-runtime-evidence-dir", type=str, default=None,
                   help="Record per-bucket payload hashes and collective counts here.")
    g.add_argument("--grad-sync-evidence-dir", type=str, default=None, help="Write numerical evidence snapshots here.")
    g.add_argument("--grad-sync-evidence-canonical-init", action="store_true",
                   help="Initialise parameters from their logical ids (layout-independent, CPU generator).")

    g = p.add_argument_group("flexpipe")
    g.add_argument("--flexpipe-config", type=str, default=None, help="Path of the normalized or raw HPP config.")
    g.add_argument("--interleave-factor", type=int, default=1, help="Model chunks per rank (interleaved 1F1B when > 1).")
    g.add_argument("--log-path", type=str, default=None, help="Directory for per-rank CSV summaries.")
    g.add_argument("--mbs-seq", type=str, default=None, help="Literal list of [mbs, seq_len] schedules per pipeline.")
    g.add_argument("--log-detail-compute-time", action="store_true", help="Dump per-interval timer stamps.")

    g = p.add_argument_group("profiler")
    g.add_argument("--prof-tp-size", type=int, default=None, help="Profile ops at this TP degree (profiler mode).")
    g.add_argument("--prof-path", type=str, default=None, help="Output directory of the profiler.")
    g.add_argument("--prof-cache-file", type=str, default=None, help="Pickle cache of measured ops.")
    g.add_argument("--prof-model-name", type=str, default="gpt", help="Model family to profile.")
    g.add_argument("--prof-model-size", type=str, default="all", help="Model size to profile.")
    g.add_argument("--prof-warmup-times", type=int, default=10, help="Warm-up repetitions per op.")
    g.add_argument("--prof-repeat-times", type=int, nargs="+", default=[40], help="Timed repetitions per op.")
    g.add_argument("--prof-repeat-threshold", type=int, default=None, help="Adaptive repeat threshold (us).")
    g.add_argument("--prof-skip-running", action="store_true", help="Write shapes only, skip measurements.")
    g.add_argument("--prof-num-nodes", type=int, default=None, help="Nodes taking part in profiling.")
    g.add_argument("--prof-node-rank", type=int, default=None, help="This node's rank in profiling.")
    g.add_argument("--prof-ref-data", type=str, default=None, help="Reference profile for task distribution.")
    g.add_argument("--prof-mbs-list", type=int, nargs="+", default=None, help="Micro-batch sizes to profile.")
    g.add_argument("--prof-op-time-only", action="store_true", help="Skip the memory probe.")
    return p


def _read_config(path):
    with open(path) as f:
        return json.load(f)


def finalize_args(args, config=None):
    """Derive everything that depends on the environment and the HPP config."""
    args.rank = int(os.getenv("RANK", "0")) if getattr(args, "rank", None) is None else args.rank
    args.world_size = int(os.getenv("WORLD_SIZE", "1")) if getattr(args, "world_size", None) is None else args.world_size
    if args.local_rank is None:
        args.local_rank = int(os.getenv("LOCAL_RANK", "0"))
    if args.fp16 and args.bf16:
        raise ValueError("--fp16 and --bf16 are mutually exclusive")
    args.params_dtype = torch.float16 if args.fp16 else (torch.bfloat16 if args.bf16 else torch.float32)
    if args.bf16:
        args.accumulate_allreduce_grads_in_fp32 = True   # reference: arguments.py:268-277
    args.grad_dtype = torch.float32 if (args.accumulate_allreduce_grads_in_fp32 or not args.fp16) else torch.float16
    if args.interleave_factor < 1:
        raise ValueError("--interleave-factor must be >= 1")

    if args.prof_tp_size is not None:
        config = profiler_config(args)
    elif config is None:
        if not args.flexpipe_config:
            raise ValueError("--flexpipe-config is required")
        config = _read_config(args.flexpipe_config)
    normalized = normalize_flexpipe_config(config, args.world_size)
    apply_normalized_config_to_args(args, normalized)
    args.normalized_config = normalized
    if args.attention_dropout not in (0, 0.0) and normalized["model_impl"] == "gpt":
        raise ValueError("the flash-attention path supports --attention-dropout 0 only "
                         "(the unfused 13-op manifest, model_impl gpt-legacy13, has an attention-dropout op)")
    args.canonical_topology = build_canonical_topology(normalized)
    if args.interleave_factor > 1:
        for i, p in enumerate(normalized["pipe"]):
            n_mb = p["global_batch_size"] // p["micro_batch_size"]
            if p["num_stages"] < 2 or n_mb % p["num_stages"]:
                raise ValueError(f"--interleave-factor > 1 needs at least two stages and a number of micro-batches "
                                 f"divisible by the number of stages (pipeline {i}: {p['num_stages']} stages, "
                                 f"{n_mb} micro-batches)")
    if args.reset_position_ids or args.reset_attention_mask:
        raise ValueError("--reset-position-ids / --reset-attention-mask are not supported: the attention kernels are "
                         "causal over the whole sequence and positions are not restarted at document boundaries")
    args.eod_token = None
    if bool(args.vocab_file) != bool(args.merge_file):
        raise ValueError("--vocab-file and --merge-file go together")
    if args.vocab_file:
        from ..tokenizer.tokenizer import GPT2BPETokenizer
        tokenizer = GPT2BPETokenizer(args.vocab_file, args.merge_file)
        args.vocab_size, args.eod_token = tokenizer.vocab_size, tokenizer.eod
    if args.eod_mask_loss and args.eod_token is None:
        raise ValueError("--eod-mask-loss needs the tokenizer files (--vocab-file, --merge-file) to know the token")
    max_tp = max(s.tp_degree for s in args.canonical_topology.stages)
    multiple = args.make_vocab_size_divisible_by * max_tp
    args.padded_vocab_size = (args.vocab_size + multiple - 1) // multiple * multiple
    args.global_data_cursor = 0
    args.successful_optimizer_steps = 0
    args.consumed_train_samples = 0
    if args.lr_warmup_iters == 0 and args.lr_warmup_fraction:
        args.lr_warmup_samples = int(args.lr_warmup_fraction * args.lr_decay_iters * args.total_gbs)
    else:
        args.lr_warmup_samples = args.lr_warmup_iters * args.total_gbs
    return args


def profiler_config(args):
    """Single stage, TP = --prof-tp-size, DP = 1 over the one-layer op list."""
    tp = args.prof_tp_size
    layers = 1
    return make_config([make_pipe([manifest_size(layers)], [tp], [1], gbs=1, mbs=1)], num_layers=layers,
                       hidden_size=args.hidden_size or 1024, num_attention_heads=args.num_attention_heads or 16,
                       seq_length=args.seq_length or 2048, model_size="profile")


def parse_args(argv=None, config=None, **overrides):
    parser = build_parser()
    args = parser.parse_args(argv)
    for k, v in overrides.items():
        setattr(args, k, v)
    return finalize_args(args, config)
