"""TEST INFRASTRUCTURE — CPU fp32 oracle for the encoder path.  Never imported by the product.

`hf_model` instantiates HuggingFace `XLMRobertaModel` (the reference's authority,
models/bge-m3/best_hoid.py:66-76: fp32, TF32 off) from config with the seeded weights;
`encoder_forward` restates transformers/models/xlm_roberta/modeling_xlm_roberta.py
(embeddings with padding_idx + 1 position offset, post-LayerNorm blocks, exact-erf GELU) in
plain torch and is pinned against it in tests/test_oracle.py and tests/golden/encoder_xlmr.npz.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def hf_model(cfg, weights):
    import transformers
    conf = transformers.XLMRobertaConfig(
        vocab_size=cfg.vocab, hidden_size=cfg.hidden, num_hidden_layers=cfg.layers,
        num_attention_heads=cfg.heads, intermediate_size=cfg.inter, hidden_act="gelu",
        max_position_embeddings=cfg.max_pos, type_vocab_size=1, layer_norm_eps=cfg.eps,
        pad_token_id=cfg.pad_id, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
    conf._attn_implementation = "eager"
    model = transformers.XLMRobertaModel(conf, add_pooling_layer=False).float()
    sd = {k: v.float() for k, v in weights.items()}
    missing, unexpected = model.load_state_dict(sd, strict=False)
    missing = [m for m in missing if "position_ids" not in m and "token_type_ids" not in m]
    if missing or unexpected:
        raise RuntimeError(f"weight names do not match HF: {missing} {unexpected}")
    return model.eval()


@torch.no_grad()
def hf_forward(model, ids):
    """ids [B, S] -> (per-layer hidden states, L2-normalised CLS embeddings)."""
    out = model(input_ids=ids.long(), attention_mask=torch.ones_like(ids).long(),
                output_hidden_states=True)
    return list(out.hidden_states), F.normalize(out.last_hidden_state[:, 0], dim=-1)


@torch.no_grad()
def encoder_forward(cfg, w, ids):
    """Plain-torch fp32 restatement; returns (hidden states [L + 1][B, S, H], pooled [B, H])."""
    B, S = ids.shape
    H, nh, hd = cfg.hidden, cfg.heads, cfg.head_dim
    f = lambda n: w[n].float()
    pos = torch.arange(S) + cfg.pad_id + 1
    x = f("embeddings.word_embeddings.weight")[ids.long()] + f("embeddings.position_embeddings.weight")[pos] \
        + f("embeddings.token_type_embeddings.weight")[0]
    x = F.layer_norm(x, (H,), f("embeddings.LayerNorm.weight"), f("embeddings.LayerNorm.bias"), cfg.eps)
    hidden = [x]
    for i in range(cfg.layers):
        p = f"encoder.layer.{i}."
        lin = lambda n, t: t @ f(p + n + ".weight").T + f(p + n + ".bias")
        q = lin("attention.self.query", x).view(B, S, nh, hd).transpose(1, 2)
        k = lin("attention.self.key", x).view(B, S, nh, hd).transpose(1, 2)
        v = lin("attention.self.value", x).view(B, S, nh, hd).transpose(1, 2)
        a = torch.softmax(q @ k.transpose(-1, -2) * hd ** -0.5, -1) @ v
        a = a.transpose(1, 2).reshape(B, S, H)
        x = F.layer_norm(lin("attention.output.dense", a) + x, (H,),
                         f(p + "attention.output.LayerNorm.weight"),
                         f(p + "attention.output.LayerNorm.bias"), cfg.eps)
        m = lin("output.dense", F.gelu(lin("intermediate.dense", x)))
        x = F.layer_norm(m + x, (H,), f(p + "output.LayerNorm.weight"),
                         f(p + "output.LayerNorm.bias"), cfg.eps)
        hidden.append(x)
    return hidden, F.normalize(x[:, 0], dim=-1)
