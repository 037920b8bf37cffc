"""GPT-2 byte-level BPE tokenizer (vocab.json + merges.txt) and vocabulary padding.

The vocabulary is padded to a multiple of `make_vocab_size_divisible_by x (largest TP degree over
all stages of all pipelines)` so that every pipeline shards the same padded embedding
(reference: eth/runtime/megatron/tokenizer/tokenizer.py:45-70 -- 50257 becomes 50304 / 50432 /
50688 for max TP 1 / 2 / 4).
"""
from __future__ import annotations

import json
from functools import lru_cache
from typing import Dict, Iterable, List, Tuple

import regex as re


def vocab_size_with_padding(orig_vocab_size: int, make_divisible_by: int, max_tp: int) -> int:
    multiple = make_divisible_by * max_tp
    return (orig_vocab_size + multiple - 1) // multiple * multiple


def max_tp_of(per_pipeline_tp) -> int:
    """per_pipeline_tp: [pipeline][stage][op] tensor-parallel sizes."""
    return max(t for pipe in per_pipeline_tp for stage in pipe for t in stage)


@lru_cache()
def bytes_to_unicode() -> Dict[int, str]:
    """Reversible map from bytes to printable unicode characters (the GPT-2 byte alphabet)."""
    keep = list(range(ord("!"), ord("~") + 1)) + list(range(ord("¡"), ord("¬") + 1)) + list(range(ord("®"), ord("ÿ") + 1))
    chars = keep[:]
    extra = 0
    for b in range(256):
        if b not in keep:
            keep.append(b)
            chars.append(256 + extra)
            extra += 1
    return dict(zip(keep, (chr(c) for c in chars)))


class GPT2BPETokenizer:
    PATTERN = r"""'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+"""

    def __init__(self, vocab_file: str, merge_file: str):
        with open(vocab_file, encoding="utf-8") as f:
            self.encoder: Dict[str, int] = json.load(f)
        self.decoder = {v: k for k, v in self.encoder.items()}
        with open(merge_file, encoding="utf-8") as f:
            lines = f.read().split("\n")
        merges = [tuple(l.split()) for l in lines[1:] if l and not l.startswith("#") and len(l.split()) == 2]
        self.ranks: Dict[Tuple[str, str], int] = {m: i for i, m in enumerate(merges)}
        self.byte_encoder = bytes_to_unicode()
        self.byte_decoder = {v: k for k, v in self.byte_encoder.items()}
        self.pat = re.compile(self.PATTERN)
        self.cache: Dict[str, str] = {}
        self.eod_id = self.encoder.get("<|endoftext|>", len(self.encoder) - 1)

    @property
    def vocab_size(self) -> int:
        return len(self.encoder)

    @property
    def vocab(self):
        return self.encoder

    @property
    def inv_vocab(self):
        return self.decoder

    @property
    def eod(self) -> int:
        return self.eod_id

    def _bpe(self, token: str) -> str:
        if token in self.cache:
            return self.cache[token]
        word = tuple(token)
        while len(word) > 1:
            pairs = {(a, b) for a, b in zip(word, word[1:])}
            best = min(pairs, key=lambda p: self.ranks.get(p, float("inf")))
            if best not in self.ranks:
                break
            a, b = best
            out, i = [], 0
            while i < len(word):
                if i + 1 < len(word) and word[i] == a and word[i + 1] == b:
                    out.append(a + b)
                    i += 2
                else:
                    out.append(word[i])
                    i += 1
            word = tuple(out)
        res = " ".join(word)
        self.cache[token] = res
        return res

    def tokenize(self, text: str) -> List[int]:
        ids: List[int] = []
        for piece in self.pat.findall(text):
            mapped = "".join(self.byte_encoder[b] for b in piece.encode("utf-8"))
            ids.extend(self.encoder[t] for t in self._bpe(mapped).split(" "))
        return ids

    def detokenize(self, ids: Iterable[int]) -> str:
        text = "".join(self.decoder[i] for i in ids)
        return bytearray(self.byte_decoder[c] for c in text).decode("utf-8", errors="replace")


def build_tokenizer(args):
    """Tokenizer from --vocab-file/--merge-file; also sets args.padded_vocab_size."""
    if not getattr(args, "vocab_file", None) or not getattr(args, "merge_file", None):
        raise ValueError("--vocab-file and --merge-file are required to build the tokenizer")
    tok = GPT2BPETokenizer(args.vocab_file, args.merge_file)
    tps = getattr(args, "model_parallel_size_of_each_op_each_pipe", None) or [getattr(args, "model_parallel_size_of_each_op", [[1]])]
    args.padded_vocab_size = vocab_size_with_padding(tok.vocab_size, args.make_vocab_size_divisible_by, max_tp_of(tps))
    return tok
