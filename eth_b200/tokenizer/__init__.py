"""GPT-2 byte-level BPE tokenizer and vocabulary padding."""
from .tokenizer import GPT2BPETokenizer, build_tokenizer, vocab_size_with_padding  # noqa: F401
