"""Host-side partitioning for one 8-GPU box: head-sharded tensor parallelism (dense models) and
expert sharding (MoE).  Pure tensor slicing, device-agnostic, so the same code is exercised by
the gloo CPU tests and by the CUDA engines.  The reference has no distributed code; the
single-GPU call sites these shards feed are models/llama31-8b/llama31_optimized.py:391-414.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from .configs import DecoderConfig


def interleave_rows(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[I, K] gate and up -> [2I, K] with row 2j = gate_j and row 2j + 1 = up_j."""
    I, K = gate.shape
    return torch.stack((gate, up), dim=1).reshape(2 * I, K).contiguous()


def check_divisible(cfg: DecoderConfig, size: int) -> None:
    if cfg.n_experts:
        if cfg.n_experts % size:
            raise ValueError("expert-parallel size must divide the number of experts")
    elif cfg.n_kv % size or cfg.n_q % size or cfg.inter % size or cfg.vocab % size:
        raise ValueError("tensor-parallel size must divide heads, intermediate and vocab")


def shard_attention(cfg: DecoderConfig, w: Dict[str, torch.Tensor], i: int, rank: int,
                    size: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """(packed q|k|v rows of this rank's heads [(nq + 2 nkv) hd / size, H],
        o_proj columns of this rank's heads [H, nq hd / size])."""
    p = f"model.layers.{i}.self_attn."
    qs, ks = cfg.q_size // size, cfg.kv_size // size
    q = w[p + "q_proj.weight"][rank * qs:(rank + 1) * qs]
    k = w[p + "k_proj.weight"][rank * ks:(rank + 1) * ks]
    v = w[p + "v_proj.weight"][rank * ks:(rank + 1) * ks]
    o = w[p + "o_proj.weight"][:, rank * qs:(rank + 1) * qs]
    return torch.cat((q, k, v), dim=0).contiguous(), o.contiguous()


def shard_mlp(cfg: DecoderConfig, w: Dict[str, torch.Tensor], i: int, rank: int,
              size: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """(interleaved gate|up rows [2 I / size, H], down_proj columns [H, I / size])."""
    p = f"model.layers.{i}.mlp."
    n = cfg.inter // size
    g = w[p + "gate_proj.weight"][rank * n:(rank + 1) * n]
    u = w[p + "up_proj.weight"][rank * n:(rank + 1) * n]
    d = w[p + "down_proj.weight"][:, rank * n:(rank + 1) * n]
    return interleave_rows(g, u), d.contiguous()


def shard_experts(cfg: DecoderConfig, w: Dict[str, torch.Tensor], i: int, rank: int,
                  size: int) -> Tuple[torch.Tensor, torch.Tensor, int]:
    """(interleaved gate|up [E / size, 2I, H], down [E / size, H, I], first local expert)."""
    p = f"model.layers.{i}.mlp.experts."
    n = cfg.n_experts // size
    lo = rank * n
    gu = w[p + "gate_up_proj"][lo:lo + n]      # HuggingFace layout: gate rows, then up rows
    I = cfg.moe_inter
    gu = torch.stack((gu[:, :I], gu[:, I:]), dim=2).reshape(n, 2 * I, cfg.hidden).contiguous()
    return gu, w[p + "down_proj"][lo:lo + n].contiguous(), lo


def shard_vocab(head: torch.Tensor, rank: int, size: int) -> torch.Tensor:
    n = head.shape[0] // size
    return head[rank * n:(rank + 1) * n].contiguous()


def merge_candidates(cands: torch.Tensor) -> int:
    """cands [n, 2] = per-rank (max logit, global argmax as float bit pattern of an int32): the
    winner is the highest value, lowest index on ties — what b200_greedy_select computes."""
    vals = cands[:, 0]
    idx = cands.view(torch.int32)[:, 1] if cands.dtype == torch.float32 else cands[:, 1].int()
    best = 0
    for r in range(1, cands.shape[0]):
        if vals[r] > vals[best] or (vals[r] == vals[best] and idx[r] < idx[best]):
            best = r
    return int(idx[best])
