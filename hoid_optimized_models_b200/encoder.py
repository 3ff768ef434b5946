"""XLM-RoBERTa-large-architecture dense-embedding encoder on the b200 ops.

Mirrors the reference's `OptimizedBgeM3` (models/bge-m3/bge_optimized.py:282-393:
`load_inputs`, `forward_static`, `capture`, pooled fp32 output) with a leaner dataflow:

    word / position gather -> add_layernorm (token-type row as bias)
    per layer: gemm[q|k|v packed, + bias] -> flash_prefill (bidirectional, straight from the
               packed projection) -> gemm[out_proj + bias] -> residual + layernorm
               -> gemm[fc1 + bias + exact-erf GELU epilogue] -> gemm[fc2 + bias]
               -> residual + layernorm
    cls_pool_l2 -> fp32 [batch, hidden]

(7 launches per layer against the reference's 10; bias, residual and GELU are GEMM epilogues.)
Data parallel: each rank embeds batch / N sequences, one all-gather of the pooled rows.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from . import ops
from .configs import EncoderConfig


class XlmrEncoder:
    def __init__(self, cfg: EncoderConfig, weights: Dict[str, torch.Tensor], batch: int, seq: int,
                 device="cuda", dp_rank: int = 0, dp_size: int = 1, group=None):
        if batch % dp_size:
            raise ValueError("data-parallel size must divide the batch")
        self.cfg, self.device = cfg, torch.device(device)
        self.dp_rank, self.dp_size, self.group = dp_rank, dp_size, group
        self.batch, self.seq = batch // dp_size, seq
        self.global_batch = batch
        dev, H = self.device, cfg.hidden
        g = lambda n: weights[n].to(dev)
        self.word = g("embeddings.word_embeddings.weight")
        self.pos_emb = g("embeddings.position_embeddings.weight")
        self.tok_type = g("embeddings.token_type_embeddings.weight")[0].contiguous()
        self.emb_ln = (g("embeddings.LayerNorm.weight"), g("embeddings.LayerNorm.bias"))
        self.layers: List[Dict[str, torch.Tensor]] = []
        for i in range(cfg.layers):
            p = f"encoder.layer.{i}."
            a = p + "attention.self."
            self.layers.append({
                "wqkv": torch.cat([g(a + n + ".weight") for n in ("query", "key", "value")], 0).contiguous(),
                "bqkv": torch.cat([g(a + n + ".bias") for n in ("query", "key", "value")], 0).contiguous(),
                "wo": g(p + "attention.output.dense.weight"), "bo": g(p + "attention.output.dense.bias"),
                "ln1": (g(p + "attention.output.LayerNorm.weight"), g(p + "attention.output.LayerNorm.bias")),
                "w1": g(p + "intermediate.dense.weight"), "b1": g(p + "intermediate.dense.bias"),
                "w2": g(p + "output.dense.weight"), "b2": g(p + "output.dense.bias"),
                "ln2": (g(p + "output.LayerNorm.weight"), g(p + "output.LayerNorm.bias")),
            })
        R = self.batch * seq
        bf = lambda *s: torch.empty(*s, dtype=torch.bfloat16, device=dev)
        self.ids = torch.zeros(R, dtype=torch.int32, device=dev)
        # RoBERTa positions: padding_idx + 1 + index (no padding in this workload)
        self.pos_ids = (torch.arange(seq, dtype=torch.int32, device=dev) + cfg.pad_id + 1).repeat(self.batch)
        self.emb_w, self.emb_p = bf(R, H), bf(R, H)
        self.h, self.x = bf(R, H), bf(R, H)
        self.qkv, self.ctx, self.act = bf(R, 3 * H), bf(R, H), bf(R, cfg.inter)
        self.pooled = torch.empty(self.batch, H, dtype=torch.float32, device=dev)
        self.pooled_all = torch.empty(batch, H, dtype=torch.float32, device=dev)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.launches_per_forward = 3 + 7 * cfg.layers + 1

    @classmethod
    def from_checkpoint(cls, cfg: EncoderConfig, weights_dir: str, batch: int, seq: int,
                        device="cuda", strip_prefix: str = "", **kw) -> "XlmrEncoder":
        """Engine on a HuggingFace safetensors checkpoint of an `XLMRobertaModel` (the tensors
        models/bge-m3/bge_optimized.py:294-313 reads from the stock model); `strip_prefix` removes
        a wrapper prefix such as "roberta." from the stored names."""
        from . import checkpoint
        w = checkpoint.load_weights(weights_dir, device=device, keep=lambda n: True,
                                    strip_prefix=strip_prefix)
        return cls(cfg, w, batch, seq, device=device, **kw)

    def load_inputs(self, input_ids: torch.Tensor) -> None:
        """input_ids: this rank's [batch / dp, seq] token ids."""
        self.ids.copy_(input_ids.reshape(-1).to(torch.int32))

    def forward_static(self, collect: Optional[list] = None) -> torch.Tensor:
        cfg = self.cfg
        B, S, H, nh, hd = self.batch, self.seq, cfg.hidden, cfg.heads, cfg.head_dim
        ops.embed_gather(self.emb_w, self.word, self.ids)
        ops.embed_gather(self.emb_p, self.pos_emb, self.pos_ids)
        ops.layernorm(self.h, self.emb_w, self.emb_ln[0], self.emb_ln[1], cfg.eps,
                      bias=self.tok_type, resid=self.emb_p)
        h, x = self.h, self.x
        qkv4 = self.qkv.view(B, S, 3, nh, hd)
        q = qkv4[:, :, 0]                                   # [B, S, nh, hd]
        k = qkv4[:, :, 1].permute(0, 2, 1, 3)               # [B, nh, S, hd] (strided view)
        v = qkv4[:, :, 2].permute(0, 2, 1, 3)
        ctx4 = self.ctx.view(B, S, nh, hd)
        for L in self.layers:
            ops.gemm(self.qkv, h, L["wqkv"], bias=L["bqkv"])
            ops.flash_prefill(ctx4, q, k, v, S, False, hd ** -0.5)
            # the residual add rides in the (memory-bound, coalesced) LayerNorm rather than in
            # the epilogue of these short-K GEMMs, where it could not be hidden
            ops.gemm(x, self.ctx, L["wo"], bias=L["bo"])
            ops.layernorm(h, x, L["ln1"][0], L["ln1"][1], cfg.eps, resid=h)
            ops.gemm(self.act, h, L["w1"], bias=L["b1"], epilogue=ops.EPI_GELU)
            ops.gemm(x, self.act, L["w2"], bias=L["b2"])
            ops.layernorm(h, x, L["ln2"][0], L["ln2"][1], cfg.eps, resid=h)
            if collect is not None:
                collect.append(h.clone())
        ops.cls_pool_l2(self.pooled, h, S)
        return self.pooled

    def capture(self, warmup: int = 2) -> None:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(warmup):
                self.forward_static()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph), torch.no_grad():
            self.forward_static()

    @torch.no_grad()
    def embed(self, input_ids: torch.Tensor) -> torch.Tensor:
        """[batch / dp, seq] ids -> L2-normalised CLS embeddings of the whole batch, fp32."""
        self.load_inputs(input_ids)
        if self.graph is not None:
            self.graph.replay()
        else:
            self.forward_static()
        if self.dp_size > 1:
            torch.distributed.all_gather_into_tensor(self.pooled_all, self.pooled, group=self.group)
        ops.check_status(self.device)        # a bounded wait inside a tensor-core kernel ran out
        return self.pooled_all if self.dp_size > 1 else self.pooled


class OptimizedBgeM3(XlmrEncoder):
    """Name-compatible with the reference engine (models/bge-m3/bge_optimized.py:282)."""
