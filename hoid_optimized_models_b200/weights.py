"""Seeded synthetic checkpoints and RoPE tables.

Tensor names and layouts are the HuggingFace ones the reference loads
(models/llama31-8b/llama31_optimized.py:294-310), so a real safetensors checkpoint
can be dropped in unchanged.  Every matrix is N(0, 0.02^2) drawn from its own
generator seeded by (seed, layer, slot), generated in fp32 and rounded to bf16;
norm weights are 1 + N(0, 0.02^2) so that a kernel that forgets them is caught.
"""
from __future__ import annotations

import math
from typing import Dict

import torch

from .configs import DecoderConfig

STD = 0.02


def _gen(seed: int, layer: int, slot: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed + 1000 * layer + slot)
    return g


def _normal(shape, seed, layer, slot, device, mean=0.0) -> torch.Tensor:
    t = torch.empty(shape, dtype=torch.float32, device=device)
    t.normal_(mean, STD, generator=_gen(seed, layer, slot, device))
    return t.to(torch.bfloat16)


def make_decoder_weights(cfg: DecoderConfig, seed: int = 1234, device="cpu") -> Dict[str, torch.Tensor]:
    """bf16 weights under HuggingFace names.  With device='cpu' the same tensors feed the fp32
    oracle; with device='cuda' generation is fast enough for the full-size benchmark."""
    w: Dict[str, torch.Tensor] = {}
    H, hd = cfg.hidden, cfg.head_dim
    w["model.embed_tokens.weight"] = _normal((cfg.vocab, H), seed, 999, 0, device)
    for i in range(cfg.layers):
        p = f"model.layers.{i}."
        w[p + "input_layernorm.weight"] = _normal((H,), seed, i, 0, device, mean=1.0)
        w[p + "post_attention_layernorm.weight"] = _normal((H,), seed, i, 1, device, mean=1.0)
        w[p + "self_attn.q_proj.weight"] = _normal((cfg.q_size, H), seed, i, 2, device)
        w[p + "self_attn.k_proj.weight"] = _normal((cfg.kv_size, H), seed, i, 3, device)
        w[p + "self_attn.v_proj.weight"] = _normal((cfg.kv_size, H), seed, i, 4, device)
        w[p + "self_attn.o_proj.weight"] = _normal((H, cfg.q_size), seed, i, 5, device)
        if cfg.qk_norm:
            w[p + "self_attn.q_norm.weight"] = _normal((hd,), seed, i, 6, device, mean=1.0)
            w[p + "self_attn.k_norm.weight"] = _normal((hd,), seed, i, 7, device, mean=1.0)
        if cfg.n_experts:
            w[p + "mlp.gate.weight"] = _normal((cfg.n_experts, H), seed, i, 8, device)
            # HuggingFace fused expert layout: gate rows first, then up rows
            w[p + "mlp.experts.gate_up_proj"] = _normal(
                (cfg.n_experts, 2 * cfg.moe_inter, H), seed, i, 9, device)
            w[p + "mlp.experts.down_proj"] = _normal(
                (cfg.n_experts, H, cfg.moe_inter), seed, i, 10, device)
        else:
            w[p + "mlp.gate_proj.weight"] = _normal((cfg.inter, H), seed, i, 8, device)
            w[p + "mlp.up_proj.weight"] = _normal((cfg.inter, H), seed, i, 9, device)
            w[p + "mlp.down_proj.weight"] = _normal((H, cfg.inter), seed, i, 10, device)
    w["model.norm.weight"] = _normal((H,), seed, 998, 0, device, mean=1.0)
    if not cfg.tied:
        w["lm_head.weight"] = _normal((cfg.vocab, H), seed, 997, 0, device)
    return w


def rope_inv_freq(cfg: DecoderConfig) -> torch.Tensor:
    """float64 inverse frequencies; llama3 scaling follows the published rule (wavelengths
    longer than original/low_freq_factor are divided by `factor`, shorter than
    original/high_freq_factor kept, the band between interpolated), computed in f64 like
    models/llama31-8b/llama31_optimized.py:268-291."""
    hd = cfg.head_dim
    j = torch.arange(hd // 2, dtype=torch.float64)
    inv = torch.pow(torch.tensor(cfg.rope_theta, dtype=torch.float64), -2.0 * j / hd)
    sc = cfg.rope_scaling
    if sc is None:
        return inv
    factor, lo, hi = sc["factor"], sc["low_freq_factor"], sc["high_freq_factor"]
    orig = float(sc["original_max_position_embeddings"])
    wavelen = 2.0 * math.pi / inv
    smooth = (orig / wavelen - lo) / (hi - lo)
    mid = (1.0 - smooth) * inv / factor + smooth * inv
    return torch.where(wavelen > orig / lo, inv / factor, torch.where(wavelen < orig / hi, inv, mid))


def rope_tables(cfg: DecoderConfig, max_seq: int, device):
    """fp32 [max_seq, head_dim/2] cos / sin from f64 angles."""
    ang = torch.arange(max_seq, dtype=torch.float64)[:, None] * rope_inv_freq(cfg)[None, :]
    return ang.cos().float().to(device), ang.sin().float().to(device)


def make_encoder_weights(cfg, seed: int = 1234, device="cpu") -> Dict[str, torch.Tensor]:
    """XLM-RoBERTa-architecture encoder weights under HuggingFace `XLMRobertaModel` names
    (models/bge-m3/bge_optimized.py:294-313 reads exactly these).  Matrices N(0, 0.02^2), biases
    N(0, 0.02^2), LayerNorm gamma 1 + N(0, 0.02^2) and beta N(0, 0.02^2), all bf16-rounded."""
    w: Dict[str, torch.Tensor] = {}
    H = cfg.hidden
    w["embeddings.word_embeddings.weight"] = _normal((cfg.vocab, H), seed, 999, 0, device)
    w["embeddings.position_embeddings.weight"] = _normal((cfg.max_pos, H), seed, 999, 1, device)
    w["embeddings.token_type_embeddings.weight"] = _normal((1, H), seed, 999, 2, device)
    w["embeddings.LayerNorm.weight"] = _normal((H,), seed, 999, 3, device, mean=1.0)
    w["embeddings.LayerNorm.bias"] = _normal((H,), seed, 999, 4, device)
    for i in range(cfg.layers):
        p = f"encoder.layer.{i}."
        slot = 0
        for name, shape in (("attention.self.query", (H, H)), ("attention.self.key", (H, H)),
                            ("attention.self.value", (H, H)), ("attention.output.dense", (H, H)),
                            ("intermediate.dense", (cfg.inter, H)), ("output.dense", (H, cfg.inter))):
            w[p + name + ".weight"] = _normal(shape, seed, i, slot, device)
            w[p + name + ".bias"] = _normal((shape[0],), seed, i, slot + 1, device)
            slot += 2
        for name in ("attention.output.LayerNorm", "output.LayerNorm"):
            w[p + name + ".weight"] = _normal((H,), seed, i, slot, device, mean=1.0)
            w[p + name + ".bias"] = _normal((H,), seed, i, slot + 1, device)
            slot += 2
    return w


def make_whisper_weights(cfg, seed: int = 1234, device="cpu") -> Dict[str, torch.Tensor]:
    """Whisper-architecture encoder-decoder weights under HuggingFace
    `WhisperForConditionalGeneration` names (the ones
    models/whisper-large-v3/whisper_decoder_optimized.py:189-228 reads).  Matrices and biases
    N(0, 0.02^2), LayerNorm gamma 1 + N(0, 0.02^2), beta N(0, 0.02^2); k_proj has no bias."""
    w: Dict[str, torch.Tensor] = {}
    D, F = cfg.d_model, cfg.ffn
    slot = [0]

    def nxt():
        slot[0] += 1
        return slot[0]

    def lin(name, n_out, n_in, layer, bias=True):
        w[name + ".weight"] = _normal((n_out, n_in), seed, layer, nxt(), device)
        if bias:
            w[name + ".bias"] = _normal((n_out,), seed, layer, nxt(), device)

    def ln(name, layer):
        w[name + ".weight"] = _normal((D,), seed, layer, nxt(), device, mean=1.0)
        w[name + ".bias"] = _normal((D,), seed, layer, nxt(), device)

    def attn(prefix, layer):
        lin(prefix + ".q_proj", D, D, layer)
        lin(prefix + ".k_proj", D, D, layer, bias=False)
        lin(prefix + ".v_proj", D, D, layer)
        lin(prefix + ".out_proj", D, D, layer)

    e = "model.encoder."
    w[e + "conv1.weight"] = _normal((D, cfg.n_mels, 3), seed, 900, nxt(), device)
    w[e + "conv1.bias"] = _normal((D,), seed, 900, nxt(), device)
    w[e + "conv2.weight"] = _normal((D, D, 3), seed, 900, nxt(), device)
    w[e + "conv2.bias"] = _normal((D,), seed, 900, nxt(), device)
    w[e + "embed_positions.weight"] = _normal((cfg.n_ctx, D), seed, 900, nxt(), device)
    for i in range(cfg.enc_layers):
        slot[0] = 0
        p = f"{e}layers.{i}."
        attn(p + "self_attn", 100 + i)
        ln(p + "self_attn_layer_norm", 100 + i)
        lin(p + "fc1", F, D, 100 + i)
        lin(p + "fc2", D, F, 100 + i)
        ln(p + "final_layer_norm", 100 + i)
    slot[0] = 50
    ln(e + "layer_norm", 900)
    d = "model.decoder."
    w[d + "embed_tokens.weight"] = _normal((cfg.vocab, D), seed, 901, nxt(), device)
    w[d + "embed_positions.weight"] = _normal((cfg.max_target, D), seed, 901, nxt(), device)
    for i in range(cfg.dec_layers):
        slot[0] = 0
        p = f"{d}layers.{i}."
        attn(p + "self_attn", 200 + i)
        ln(p + "self_attn_layer_norm", 200 + i)
        attn(p + "encoder_attn", 200 + i)
        ln(p + "encoder_attn_layer_norm", 200 + i)
        lin(p + "fc1", F, D, 200 + i)
        lin(p + "fc2", D, F, 200 + i)
        ln(p + "final_layer_norm", 200 + i)
    slot[0] = 80
    ln(d + "layer_norm", 901)
    return w
