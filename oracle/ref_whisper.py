"""TEST INFRASTRUCTURE — CPU fp32 oracle for the Whisper path.  Never imported by the product.

`hf_model` instantiates HuggingFace `WhisperForConditionalGeneration` (the reference's
authority, models/whisper-large-v3/common.py:42-47) from config with the seeded weights;
`encoder_forward` / `decoder_forward` restate transformers/models/whisper/modeling_whisper.py
(conv front-end with exact-erf GELU, pre-LayerNorm blocks, q scaled by head_dim^-0.5, k_proj
without bias, tied output projection) in plain torch and are pinned against it in
tests/test_oracle.py and tests/golden/whisper.npz.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def hf_model(cfg, weights):
    import transformers
    conf = transformers.WhisperConfig(
        vocab_size=cfg.vocab, num_mel_bins=cfg.n_mels, d_model=cfg.d_model,
        encoder_layers=cfg.enc_layers, decoder_layers=cfg.dec_layers,
        encoder_attention_heads=cfg.heads, decoder_attention_heads=cfg.heads,
        encoder_ffn_dim=cfg.ffn, decoder_ffn_dim=cfg.ffn, max_source_positions=cfg.n_ctx,
        max_target_positions=cfg.max_target, activation_function="gelu", dropout=0.0,
        attention_dropout=0.0, activation_dropout=0.0, pad_token_id=0, bos_token_id=1,
        eos_token_id=2, decoder_start_token_id=1, suppress_tokens=None, begin_suppress_tokens=None)
    conf._attn_implementation = "eager"
    model = transformers.WhisperForConditionalGeneration(conf).float()
    sd = {k: v.float() for k, v in weights.items()}
    sd["proj_out.weight"] = sd["model.decoder.embed_tokens.weight"]
    missing, unexpected = model.load_state_dict(sd, strict=False)
    if missing or unexpected:
        raise RuntimeError(f"weight names do not match HF: {missing} {unexpected}")
    return model.eval()


@torch.no_grad()
def hf_forward(model, mel, dec_ids):
    """mel [n_mels, frames], dec_ids [T] -> (encoder last hidden [n_ctx, D], logits [T, V])."""
    out = model(input_features=mel[None], decoder_input_ids=dec_ids[None].long())
    return out.encoder_last_hidden_state[0], out.logits[0]


def _ln(x, w, p, eps):
    return F.layer_norm(x, (x.shape[-1],), w[p + ".weight"].float(), w[p + ".bias"].float(), eps)


def _lin(x, w, p, bias=True):
    y = x @ w[p + ".weight"].float().T
    return y + w[p + ".bias"].float() if bias else y


def _mha(cfg, w, p, xq, xkv, causal):
    H, hd = cfg.heads, cfg.head_dim
    q = _lin(xq, w, p + ".q_proj").view(-1, H, hd).transpose(0, 1) * hd ** -0.5
    k = _lin(xkv, w, p + ".k_proj", bias=False).view(-1, H, hd).transpose(0, 1)
    v = _lin(xkv, w, p + ".v_proj").view(-1, H, hd).transpose(0, 1)
    s = q @ k.transpose(-1, -2)
    if causal:
        T = s.shape[-1]
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
    a = torch.softmax(s, -1) @ v
    return _lin(a.transpose(0, 1).reshape(-1, H * hd), w, p + ".out_proj")


@torch.no_grad()
def encoder_forward(cfg, w, mel, keep_hidden=False):
    """mel [n_mels, frames] -> encoder output [n_ctx, D] (and the per-layer residual streams)."""
    e = "model.encoder."
    x = F.gelu(F.conv1d(mel[None], w[e + "conv1.weight"].float(), w[e + "conv1.bias"].float(), padding=1))
    x = F.gelu(F.conv1d(x, w[e + "conv2.weight"].float(), w[e + "conv2.bias"].float(), stride=2, padding=1))
    x = x[0].T + w[e + "embed_positions.weight"].float()
    hidden = []
    for i in range(cfg.enc_layers):
        p = f"{e}layers.{i}."
        x = x + _mha(cfg, w, p + "self_attn", _ln(x, w, p + "self_attn_layer_norm", cfg.eps),
                     _ln(x, w, p + "self_attn_layer_norm", cfg.eps), False)
        h = _ln(x, w, p + "final_layer_norm", cfg.eps)
        x = x + _lin(F.gelu(_lin(h, w, p + "fc1")), w, p + "fc2")
        if keep_hidden:
            hidden.append(x)
    out = _ln(x, w, e + "layer_norm", cfg.eps)
    return (out, hidden) if keep_hidden else out


@torch.no_grad()
def decoder_forward(cfg, w, enc, dec_ids):
    """Teacher-forced decoder over dec_ids [T] with encoder states enc -> logits [T, V]."""
    d = "model.decoder."
    T = dec_ids.numel()
    x = w[d + "embed_tokens.weight"].float()[dec_ids.long()] + w[d + "embed_positions.weight"].float()[:T]
    for i in range(cfg.dec_layers):
        p = f"{d}layers.{i}."
        h = _ln(x, w, p + "self_attn_layer_norm", cfg.eps)
        x = x + _mha(cfg, w, p + "self_attn", h, h, True)
        x = x + _mha(cfg, w, p + "encoder_attn", _ln(x, w, p + "encoder_attn_layer_norm", cfg.eps), enc, False)
        h = _ln(x, w, p + "final_layer_norm", cfg.eps)
        x = x + _lin(F.gelu(_lin(h, w, p + "fc1")), w, p + "fc2")
    x = _ln(x, w, d + "layer_norm", cfg.eps)
    return x @ w[d + "embed_tokens.weight"].float().T
