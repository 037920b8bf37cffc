"""Plain autograd GPT used as the oracle of the explicit stage program (fp32, CPU)."""
import math

import torch
import torch.nn.functional as F


def oracle_loss(params, tokens, labels, mask, cfg, nominal_scale):
    """params: {logical_id: full fp32 tensor requiring grad}. Returns sum(loss*mask)/nominal_scale."""
    B, S = tokens.shape
    h, heads = cfg.hidden_size, cfg.num_attention_heads
    d = h // heads
    x = params["gpt.word_embeddings.weight"][tokens.reshape(-1)] + params["gpt.position_embeddings.weight"][
        torch.arange(B * S) % S]
    for i in range(cfg.num_layers):
        pre = f"gpt.layers.{i}."
        res = x
        y = F.layer_norm(x, (h,), params[pre + "input_layernorm.weight"], params[pre + "input_layernorm.bias"],
                         cfg.layernorm_epsilon)
        qkv = y @ params[pre + "attention.query_key_value.weight"].t() + params[pre + "attention.query_key_value.bias"]
        v5 = qkv.view(B, S, heads, 3, d)
        q, k, v = (v5[:, :, :, j].permute(0, 2, 1, 3) for j in range(3))
        s = q @ k.transpose(-1, -2) / math.sqrt(d)
        s = s.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool), 1), float("-inf"))
        o = (torch.softmax(s, -1) @ v).permute(0, 2, 1, 3).reshape(B * S, h)
        z = o @ params[pre + "attention.dense.weight"].t() + params[pre + "attention.dense.bias"]
        x = res + z
        res = x
        y = F.layer_norm(x, (h,), params[pre + "post_attention_layernorm.weight"],
                         params[pre + "post_attention_layernorm.bias"], cfg.layernorm_epsilon)
        u = F.gelu(y @ params[pre + "mlp.dense_h_to_4h.weight"].t() + params[pre + "mlp.dense_h_to_4h.bias"],
                   approximate="tanh")
        z = u @ params[pre + "mlp.dense_4h_to_h.weight"].t() + params[pre + "mlp.dense_4h_to_h.bias"]
        x = res + z
    x = F.layer_norm(x, (h,), params["gpt.final_layernorm.weight"], params["gpt.final_layernorm.bias"],
                     cfg.layernorm_epsilon)
    logits = x @ params["gpt.word_embeddings.weight"].t()
    loss = F.cross_entropy(logits, labels.reshape(-1), reduction="none")
    return (loss * mask.reshape(-1)).sum() / nominal_scale, loss
