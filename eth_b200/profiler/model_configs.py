"""Profile grid (reference: eth/profiler/model_configs.py:5-23): micro-batch sizes 1/2/4/8, algos
0/1, one transformer layer per size, vocabulary 51200."""
from ..contract.config import GPT_SIZES

model_prof_configs = {"gpt": {"dtype": "bf16", "mbs": [1, 2, 4, 8], "algo": [0, 1]}}
PROFILE_VOCAB = 51200


def gpt_profile_shape(size: str):
    if size == "scale-layer":
        size = "1_3B"
    m = GPT_SIZES[size]
    return dict(num_layers=1, hidden_size=m["hidden_size"], num_attention_heads=m["num_attention_heads"],
                seq_length=m["seq_length"], vocab=PROFILE_VOCAB)
