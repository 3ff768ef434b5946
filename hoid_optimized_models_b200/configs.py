"""Architecture constants of the five benchmarked models, plus reduced shapes for tests.

The full-size values are the ones the reference engines bake in
(models/llama31-8b/llama31_optimized.py:54-72, models/qwen3-4b/qwen3_optimized.py,
models/qwen3-30b-a3b/qwen3_optimized.py, models/bge-m3/bge_optimized.py,
models/whisper-large-v3/whisper_decoder_optimized.py); RoPE bases follow the benchmark
configuration (theta is only an input of the cos/sin tables).
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Optional


@dataclass(frozen=True)
class DecoderConfig:
    name: str
    hidden: int
    layers: int
    n_q: int
    n_kv: int
    head_dim: int
    inter: int
    vocab: int
    eps: float
    rope_theta: float
    rope_scaling: Optional[dict] = None      # llama3: factor / low_freq_factor / high_freq_factor / original
    qk_norm: bool = False
    tied: bool = False
    # mixture of experts (0 experts = dense MLP)
    n_experts: int = 0
    top_k: int = 0
    moe_inter: int = 0

    @property
    def q_size(self) -> int:
        return self.n_q * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.n_kv * self.head_dim

    def decode_bytes_per_token(self, ctx: int) -> int:
        """Algorithmic HBM bytes one decode step must read: every weight once (bf16) plus the
        K and V rows of `ctx` cached positions."""
        attn = self.hidden * (self.q_size + 2 * self.kv_size) + self.q_size * self.hidden
        if self.n_experts:
            mlp = self.hidden * self.n_experts + self.top_k * 3 * self.hidden * self.moe_inter
        else:
            mlp = 3 * self.hidden * self.inter
        norms = 2 * self.hidden + (2 * self.head_dim if self.qk_norm else 0)
        per_layer = attn + mlp + norms
        head = self.vocab * self.hidden
        total = self.layers * per_layer + head + self.hidden
        kv = self.layers * 2 * self.kv_size * ctx
        return 2 * (total + kv)


LLAMA31_8B = DecoderConfig(
    name="llama-3.1-8b", hidden=4096, layers=32, n_q=32, n_kv=8, head_dim=128, inter=14336,
    vocab=128256, eps=1e-5, rope_theta=5e5,
    rope_scaling={"factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                  "original_max_position_embeddings": 8192})

QWEN3_4B = DecoderConfig(
    name="qwen3-4b", hidden=2560, layers=36, n_q=32, n_kv=8, head_dim=128, inter=9728,
    vocab=151936, eps=1e-6, rope_theta=1e6, qk_norm=True, tied=True)

QWEN3_30B_A3B = DecoderConfig(
    name="qwen3-30b-a3b", hidden=2048, layers=48, n_q=32, n_kv=4, head_dim=128, inter=0,
    vocab=151936, eps=1e-6, rope_theta=1e6, qk_norm=True, tied=False,
    n_experts=128, top_k=8, moe_inter=768)


def reduced(cfg: DecoderConfig, layers: int, vocab: int = 0, **kw) -> DecoderConfig:
    """Same widths, fewer layers / smaller vocabulary: the shapes every kernel sees stay real."""
    return replace(cfg, name=f"{cfg.name}-L{layers}", layers=layers, vocab=vocab or cfg.vocab, **kw)


@dataclass(frozen=True)
class EncoderConfig:
    name: str
    hidden: int
    layers: int
    heads: int
    inter: int
    vocab: int
    max_pos: int
    eps: float
    pad_id: int = 1

    @property
    def head_dim(self) -> int:
        return self.hidden // self.heads


XLMR_LARGE = EncoderConfig(name="xlm-roberta-large", hidden=1024, layers=24, heads=16, inter=4096,
                           vocab=250002, max_pos=8194, eps=1e-5)


@dataclass(frozen=True)
class WhisperConfig:
    name: str
    d_model: int
    enc_layers: int
    dec_layers: int
    heads: int
    ffn: int
    n_mels: int
    n_frames: int
    n_ctx: int          # encoder positions after the stride-2 conv
    max_target: int
    vocab: int
    eps: float = 1e-5

    @property
    def head_dim(self) -> int:
        return self.d_model // self.heads


WHISPER_LARGE_V3 = WhisperConfig(name="whisper-large-v3", d_model=1280, enc_layers=32,
                                 dec_layers=32, heads=20, ffn=5120, n_mels=128, n_frames=3000,
                                 n_ctx=1500, max_target=448, vocab=51866)
