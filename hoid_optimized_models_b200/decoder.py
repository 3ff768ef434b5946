"""Batch-1 dense decoder engine (Llama-3.1 / Qwen3 families) on the b200 ops.

Mirrors the reference engines' interface — `capture()`, `step(tok, pos)`,
`prefill(ids)`, `generate(ids, n_new)` with all buffers allocated up front
(models/llama31-8b/llama31_optimized.py:317-520, models/qwen3-4b/qwen3_optimized.py:312-517)
— but with a different dataflow:

decode (fp32 activations, one CUDA graph for the whole step)
    per layer: gemv[rmsnorm prologue, packed q|k|v] -> rope_flash_decode (QK-norm + RoPE + cache
    append in the attention prologue, LSE combine fused) -> gemv[o_proj, + residual] ->
    gemv[rmsnorm prologue, gate|up interleaved, SwiGLU epilogue] -> gemv[down_proj, + residual];
    then lm_head gemv (fp32 logits) -> argmax -> greedy_select, which feeds the next step's token
    and position on the device.  Dense models run all layers as ONE persistent launch
    (ops.decode_layers: the same five phases, resident CTAs, weights streaming across the phase
    boundaries, the tensor-parallel exchange inside the kernel): 5 launches per step instead of
    5 per layer.  The launch-per-phase path stays for the MoE model, for the NCCL all-reduce
    variant and for looking at per-layer hidden states (`collect`).

prefill (bf16 activations and residual stream, the reference's own precision; an fp32 stream
was measured to change the distance from an fp32 model by under 10% at the Llama widths, where
the rounding of the GEMM operands dominates)
    add_rmsnorm -> gemm[q|k|v] -> qk_rope_cache -> flash_prefill (reads the cache) ->
    gemm[o_proj + residual] -> add_rmsnorm -> gemm[gate|up, SwiGLU epilogue] ->
    gemm[down + residual]; logits for the last position only.

Tensor parallelism (head-sharded, one process per GPU): q/k/v/gate/up are column-sharded,
o/down row-sharded with an all-reduce after each, lm_head vocabulary-sharded with an
all-gather of per-rank (max logit, argmax) records.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from . import ops
from . import tp as tpart
from .configs import DecoderConfig
from .weights import rope_tables

EPI_SWIGLU = ops.EPI_SWIGLU


class DenseDecoder:
    def __init__(self, cfg: DecoderConfig, weights: Dict[str, torch.Tensor], max_seq: int,
                 device="cuda", tp_rank: int = 0, tp_size: int = 1, group=None,
                 n_splits: Optional[int] = None, max_new_tokens: int = 1024,
                 free_source_weights: bool = False, fused_allreduce: bool = True,
                 fuse_rope: bool = True, fused_layers: bool = False,
                 ep_all_to_all: bool = False):
        self.moe = cfg.n_experts > 0   # expert parallelism: attention replicated, experts sharded
        tpart.check_divisible(cfg, tp_size)
        self.cfg, self.device, self.max_seq = cfg, torch.device(device), max_seq
        self.tp_rank, self.tp_size, self.group = tp_rank, tp_size, group
        H, hd = cfg.hidden, cfg.head_dim
        att_tp = 1 if self.moe else tp_size          # heads are sharded only for dense models
        self.att_tp = att_tp
        self.n_q, self.n_kv = cfg.n_q // att_tp, cfg.n_kv // att_tp
        self.q_size, self.kv_size = self.n_q * hd, self.n_kv * hd
        self.inter = cfg.inter // att_tp
        self.vocab_local = cfg.vocab // att_tp
        self.scale = hd ** -0.5
        r = tp_rank if att_tp > 1 else 0
        self.n_local_experts = cfg.n_experts // tp_size if self.moe else 0
        self.expert_lo = tp_rank * self.n_local_experts
        dev = self.device

        def take(name):
            return weights[name]

        def rows(t, n_local):  # column-parallel: a contiguous block of output rows
            return t[r * n_local:(r + 1) * n_local]

        self.embed = take("model.embed_tokens.weight").to(dev)
        head = self.embed if cfg.tied else take("lm_head.weight").to(dev)
        self.lm_head = rows(head, self.vocab_local).contiguous() if att_tp > 1 else head
        self.final_norm_w = take("model.norm.weight").to(dev)
        self.ln1: List[torch.Tensor] = []
        self.ln2: List[torch.Tensor] = []
        self.wqkv: List[torch.Tensor] = []
        self.wo: List[torch.Tensor] = []
        self.wgu: List[torch.Tensor] = []
        self.wd: List[torch.Tensor] = []
        self.w_router: List[torch.Tensor] = []
        self.qn: List[Optional[torch.Tensor]] = []
        self.kn: List[Optional[torch.Tensor]] = []
        for i in range(cfg.layers):
            p = f"model.layers.{i}."
            self.ln1.append(take(p + "input_layernorm.weight").to(dev))
            self.ln2.append(take(p + "post_attention_layernorm.weight").to(dev))
            wqkv, wo = tpart.shard_attention(cfg, weights, i, r, att_tp)
            self.wqkv.append(wqkv.to(dev))
            self.wo.append(wo.to(dev))
            if self.moe:
                self.w_router.append(weights[p + "mlp.gate.weight"].to(dev))
                gu, dn, _ = tpart.shard_experts(cfg, weights, i, tp_rank, tp_size)
                self.wgu.append(gu.to(dev))
                self.wd.append(dn.to(dev))
            else:
                gu, dn = tpart.shard_mlp(cfg, weights, i, r, att_tp)
                self.wgu.append(gu.to(dev))
                self.wd.append(dn.to(dev))
            if free_source_weights:
                for k in [k for k in weights if k.startswith(p) and "norm" not in k]:
                    del weights[k]
            if cfg.qk_norm:
                self.qn.append(take(p + "self_attn.q_norm.weight").to(dev))
                self.kn.append(take(p + "self_attn.k_norm.weight").to(dev))
            else:
                self.qn.append(None)
                self.kn.append(None)

        self.cos, self.sin = rope_tables(cfg, max_seq, dev)
        # KV cache [layer, k|v, n_kv, max_seq, hd]: the layout cache-write and both attention
        # kernels share (row = (kv_head * max_seq + pos) * hd)
        self.kv = torch.zeros(cfg.layers, 2, self.n_kv, max_seq, hd, dtype=torch.bfloat16, device=dev)

        f32 = lambda *s: torch.zeros(*s, dtype=torch.float32, device=dev)
        # step state on the device: {position, kv_len, generated}; one graph serves every step
        self.state = torch.zeros(4, dtype=torch.int32, device=dev)
        self.pos, self.kv_len = self.state[0:1], self.state[1:2]
        self.tok = torch.zeros(1, dtype=torch.int32, device=dev)
        self.tok_log = torch.zeros(max_new_tokens, dtype=torch.int32, device=dev)
        self.h, self.h2 = f32(H), f32(H)
        self.qkv = f32(self.q_size + 2 * self.kv_size)
        self.q = f32(self.q_size)
        self.attn = f32(self.q_size)
        self.act = f32(cfg.top_k * cfg.moe_inter if self.moe else self.inter)
        if self.moe:
            self.router_logits = f32(cfg.n_experts)
            self.topk_ids = torch.zeros(cfg.top_k, dtype=torch.int32, device=dev)
            self.topk_w = f32(cfg.top_k)
        self.logits = f32(self.vocab_local)
        self.cand = f32(2)
        self.cand_all = f32(tp_size, 2)
        if n_splits is None:
            # about one CTA per SM, at least one 128-key tile per split, and at most 36 splits:
            # beyond that the merge of the splits' records costs more than shorter slices save
            n_splits = max(1, min(148 // self.n_kv, (max_seq + 127) // 128, 36))
        self.n_splits = n_splits
        self.fd_ws = ops.flash_decode_workspace(self.n_q, self.n_kv, hd, n_splits, dev)
        self.am_ws = ops.argmax_workspace(dev)
        # multi-GPU decode: all-reduces fused into the GEMVs over peer memory
        self.link = None
        if tp_size > 1 and fused_allreduce:
            from .comm import PeerLink
            self.link = PeerLink(group, tp_rank, tp_size, H)
        self._pbuf: Dict[int, Dict[str, torch.Tensor]] = {}
        self._prefill_graphs: Dict[int, torch.cuda.CUDAGraph] = {}
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.fuse_rope = fuse_rope
        self.ep_all_to_all = ep_all_to_all
        # all layers of a dense model's step as one persistent launch
        self.plan = None
        if (fused_layers and fuse_rope and not self.moe and (tp_size == 1 or self.link is not None)
                and self._fused_layers_supported()):
            self.plan = ops.decode_layers_plan(
                self.wqkv, self.wo, self.wgu, self.wd, self.ln1, self.ln2, self.kv, self.qn, self.kn,
                self.h, tp_ctx=self.link.ctx if self.link is not None else -1)
        if self.plan is not None:
            self.launches_per_step = 5 + (1 if self.link is not None else 0)
        else:
            self.launches_per_step = (1 + ((8 if self.moe else 6) - int(fuse_rope)) * cfg.layers + 3
                                      + (1 if self.link is not None else 0))   # + sequence advance

    def _fused_layers_supported(self) -> bool:
        """Shapes the persistent kernel takes (include/b200ops.h, b200_decode_layers)."""
        H, sms = self.cfg.hidden, 148
        dims_ok = all(d % 256 == 0 and d <= 16384 for d in (H, self.q_size, self.inter))
        rows = max(-(-(self.q_size + 2 * self.kv_size) // sms), -(-H // sms), -(-2 * self.inter // sms) + 1)
        return (dims_ok and rows <= 256 and self.n_kv * self.n_splits <= sms
                and self.cfg.head_dim in (64, 128) and self.n_q // self.n_kv in (1, 2, 4, 8))

    @classmethod
    def from_checkpoint(cls, cfg: DecoderConfig, weights_dir: str, max_seq: int, device="cuda",
                        **kw) -> "DenseDecoder":
        """Engine on a HuggingFace safetensors checkpoint (the reference's load_weights +
        constructor, models/llama31-8b/llama31_optimized.py:294-346): names and shapes are
        checked against the configuration before anything is packed."""
        from . import checkpoint
        w = checkpoint.load_weights(weights_dir, device=device)
        checkpoint.check_decoder_names(cfg, w)
        kw.setdefault("free_source_weights", True)
        return cls(cfg, w, max_seq, device=device, **kw)

    # ------------------------------------------------------------------ collectives
    def _all_reduce(self, t: torch.Tensor) -> None:
        if self.tp_size > 1:
            torch.distributed.all_reduce(t, group=self.group)

    # ------------------------------------------------------------------ decode
    def _attend(self, i: int) -> None:
        """Layer i's attention for the new position: RoPE, cache append and split-KV attention
        (one launch; two with fuse_rope=False)."""
        cfg = self.cfg
        if self.fuse_rope:
            ops.rope_flash_decode(self.attn, self.kv[i, 0], self.kv[i, 1], self.fd_ws, self.qkv,
                                  self.cos, self.sin, self.kv_len, self.n_q, self.n_kv,
                                  self.n_splits, self.scale, eps=cfg.eps, qn_w=self.qn[i],
                                  kn_w=self.kn[i])
            return
        ops.qk_rope_cache(self.q, self.kv[i, 0], self.kv[i, 1], self.qkv, self.cos, self.sin,
                          self.pos, self.n_q, self.n_kv, eps=cfg.eps, qn_w=self.qn[i],
                          kn_w=self.kn[i])
        ops.flash_decode(self.attn, self.q, self.kv[i, 0], self.kv[i, 1], self.kv_len,
                         self.fd_ws, self.n_q, self.n_kv, self.n_splits, self.scale)

    def step_static(self, collect: Optional[list] = None) -> None:
        """One decode step for the token in self.tok at position self.pos (device state).
        `collect` (eager only) receives a copy of the residual stream after every layer."""
        cfg = self.cfg
        tp = self.att_tp > 1
        ep = self.moe and self.tp_size > 1
        lead = self.tp_rank == 0
        ops.embed_gather(self.h, self.embed, self.tok)
        h, h2 = self.h, self.h2
        if self.plan is not None and collect is None:
            self._step_fused_layers()
            return
        if self.link is not None:
            if self.moe:
                self._step_fused_ep(collect)
            else:
                self._step_fused_tp(collect)
            return
        for i in range(cfg.layers):
            ops.gemv(self.qkv, h, self.wqkv[i], norm_w=self.ln1[i], eps=cfg.eps)
            self._attend(i)
            if tp:
                ops.gemv(h2, self.attn, self.wo[i], resid=h if lead else None)
                self._all_reduce(h2)
                h, h2 = h2, h
            else:
                ops.gemv(h, self.attn, self.wo[i], resid=h)
            if self.moe:
                ops.gemv(self.router_logits, h, self.w_router[i], norm_w=self.ln2[i], eps=cfg.eps)
                ops.moe_router(self.topk_ids, self.topk_w, self.router_logits.view(1, -1))
                ops.moe_decode_gate_up(self.act, h, self.wgu[i], self.topk_ids, self.topk_w,
                                       norm_w=self.ln2[i], eps=cfg.eps,
                                       expert_lo=self.expert_lo)
                if ep:
                    ops.moe_decode_down(h2, self.act, self.wd[i], self.topk_ids,
                                        resid=h if lead else None, expert_lo=self.expert_lo)
                    self._all_reduce(h2)
                    h, h2 = h2, h
                else:
                    ops.moe_decode_down(h, self.act, self.wd[i], self.topk_ids, resid=h)
            else:
                ops.gemv(self.act, h, self.wgu[i], norm_w=self.ln2[i], eps=cfg.eps,
                         epilogue=EPI_SWIGLU)
                if tp:
                    ops.gemv(h2, self.act, self.wd[i], resid=h if lead else None)
                    self._all_reduce(h2)
                    h, h2 = h2, h
                else:
                    ops.gemv(h, self.act, self.wd[i], resid=h)
            if collect is not None:
                collect.append(h.clone())
        if h is not self.h:                      # odd number of buffer swaps (expert parallel)
            self.h.copy_(h)
            h = self.h
        ops.gemv(self.logits, h, self.lm_head, norm_w=self.final_norm_w, eps=cfg.eps)
        ops.argmax(self.cand, self.logits, self.am_ws,
                   idx_base=(self.tp_rank * self.vocab_local) if tp else 0)
        if tp:
            torch.distributed.all_gather_into_tensor(self.cand_all, self.cand.view(1, 2),
                                                     group=self.group)
            ops.greedy_advance(self.tok, self.state, self.tok_log, self.cand_all)
        else:
            ops.greedy_advance(self.tok, self.state, self.tok_log, self.cand)

    def _step_fused_layers(self) -> None:
        """All layers in one persistent launch, then the head.  Under tensor parallelism the
        kernel leaves the last all-reduce (2 * layers - 1) to the lm_head GEMV, which reduces it
        while staging its input, exactly as in _step_fused_tp."""
        cfg, L = self.cfg, self.cfg.layers
        ops.decode_layers(self.plan, self.cos, self.sin, self.kv_len, self.fd_ws, self.n_q,
                          self.n_kv, self.n_splits, self.scale, cfg.eps)
        if self.link is not None:
            ctx = self.link.ctx
            ops.gemv_tp_consume(self.logits, self.lm_head, ctx, 2 * L - 1, x_out=self.h,
                                norm_w=self.final_norm_w, eps=cfg.eps)
            ops.tp_advance(ctx, 2 * L)
            ops.argmax(self.cand, self.logits, self.am_ws, idx_base=self.tp_rank * self.vocab_local)
            torch.distributed.all_gather_into_tensor(self.cand_all, self.cand.view(1, 2),
                                                     group=self.group)
            ops.greedy_advance(self.tok, self.state, self.tok_log, self.cand_all)
        else:
            ops.gemv(self.logits, self.h, self.lm_head, norm_w=self.final_norm_w, eps=cfg.eps)
            ops.argmax(self.cand, self.logits, self.am_ws, idx_base=0)
            ops.greedy_advance(self.tok, self.state, self.tok_log, self.cand)

    def _step_fused_tp(self, collect: Optional[list] = None) -> None:
        """Dense tensor-parallel step with every all-reduce fused into the GEMVs around it: the
        row-parallel GEMVs push their partial sums to all ranks, the next GEMV reduces them while
        staging its input.  2 * layers all-reduces per step, none of them a library call."""
        cfg, ctx, h = self.cfg, self.link.ctx, self.h
        lead = self.tp_rank == 0
        L = cfg.layers
        for i in range(L):
            if i == 0:
                ops.gemv(self.qkv, h, self.wqkv[0], norm_w=self.ln1[0], eps=cfg.eps)
            else:
                ops.gemv_tp_consume(self.qkv, self.wqkv[i], ctx, 2 * i - 1, x_out=h,
                                    norm_w=self.ln1[i], eps=cfg.eps)
                if collect is not None:
                    collect.append(h.clone())
            self._attend(i)
            ops.gemv_tp_publish(self.attn, self.wo[i], ctx, 2 * i, resid=h if lead else None)
            ops.gemv_tp_consume(self.act, self.wgu[i], ctx, 2 * i, x_out=h, norm_w=self.ln2[i],
                                eps=cfg.eps, epilogue=EPI_SWIGLU)
            ops.gemv_tp_publish(self.act, self.wd[i], ctx, 2 * i + 1, resid=h if lead else None)
        ops.gemv_tp_consume(self.logits, self.lm_head, ctx, 2 * L - 1, x_out=h,
                            norm_w=self.final_norm_w, eps=cfg.eps)
        if collect is not None:
            collect.append(h.clone())
        ops.tp_advance(ctx, 2 * L)
        ops.argmax(self.cand, self.logits, self.am_ws, idx_base=self.tp_rank * self.vocab_local)
        torch.distributed.all_gather_into_tensor(self.cand_all, self.cand.view(1, 2), group=self.group)
        ops.greedy_advance(self.tok, self.state, self.tok_log, self.cand_all)

    def _step_fused_ep(self, collect: Optional[list] = None) -> None:
        """Expert-parallel step (attention replicated, experts sharded): the one all-reduce per
        layer, after the routed experts, is pushed by the down projection and reduced by the next
        layer's q|k|v GEMV (the lm_head GEMV after the last layer)."""
        cfg, ctx, h = self.cfg, self.link.ctx, self.h
        lead = self.tp_rank == 0
        L = cfg.layers
        for i in range(L):
            if i == 0:
                ops.gemv(self.qkv, h, self.wqkv[0], norm_w=self.ln1[0], eps=cfg.eps)
            else:
                ops.gemv_tp_consume(self.qkv, self.wqkv[i], ctx, i - 1, x_out=h,
                                    norm_w=self.ln1[i], eps=cfg.eps)
                if collect is not None:
                    collect.append(h.clone())
            self._attend(i)
            ops.gemv(h, self.attn, self.wo[i], resid=h)
            ops.gemv(self.router_logits, h, self.w_router[i], norm_w=self.ln2[i], eps=cfg.eps)
            ops.moe_router(self.topk_ids, self.topk_w, self.router_logits.view(1, -1))
            ops.moe_decode_gate_up(self.act, h, self.wgu[i], self.topk_ids, self.topk_w,
                                   norm_w=self.ln2[i], eps=cfg.eps, expert_lo=self.expert_lo)
            ops.moe_decode_down_tp_publish(self.act, self.wd[i], self.topk_ids, ctx, i,
                                           resid=h if lead else None, expert_lo=self.expert_lo)
        ops.gemv_tp_consume(self.logits, self.lm_head, ctx, L - 1, x_out=h,
                            norm_w=self.final_norm_w, eps=cfg.eps)
        if collect is not None:
            collect.append(h.clone())
        ops.tp_advance(ctx, L)
        ops.argmax(self.cand, self.logits, self.am_ws, idx_base=0)
        ops.greedy_advance(self.tok, self.state, self.tok_log, self.cand)

    def capture(self, warmup: int = 3) -> None:
        """Warm up on a side stream, then record step_static into one CUDA graph.  The step state
        lives on the device, so the same graph replays at every position."""
        saved = (self.state.clone(), self.tok.clone(), self.tok_log.clone(), self.kv[:, :, :, :warmup + 1].clone())
        self.state.zero_()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(warmup):
                self.step_static()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.state.zero_()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph), torch.no_grad():
            self.step_static()
        torch.cuda.synchronize()
        self.state.copy_(saved[0]); self.tok.copy_(saved[1]); self.tok_log.copy_(saved[2])
        self.kv[:, :, :, :warmup + 1].copy_(saved[3])

    def check_status(self) -> None:
        """Raises if a kernel reported through the status word since the last check (a bounded
        wait that ran out, a non-finite router logit).  Synchronises; under tensor / expert
        parallelism the ranks agree on the worst code first, so that all of them stop together
        instead of diverging."""
        word = ops.status_word(self.device)
        if self.tp_size > 1:
            worst = word.clone()
            torch.distributed.all_reduce(worst, op=torch.distributed.ReduceOp.MIN, group=self.group)
            if int(worst.item()) != 0:
                word.copy_(worst)
        try:
            ops.check_status(self.device)
        except Exception:
            if self.plan is not None:
                ops.reset_decode_plan(self.plan)
            raise

    def set_step(self, tok: int, pos: int, generated: int = 0) -> None:
        if pos < 0 or pos + 1 > self.max_seq:
            raise ValueError(f"position {pos} does not fit the cache of {self.max_seq} rows")
        self.tok.fill_(tok)
        self.state.copy_(torch.tensor([pos, pos + 1, generated, 0], dtype=torch.int32),
                         non_blocking=False)

    def step(self, tok: int, pos: int) -> torch.Tensor:
        """Reference-style host-driven step: returns this rank's logits."""
        self.set_step(tok, pos)
        if self.graph is not None:
            self.graph.replay()
        else:
            self.step_static()
        return self.logits

    def step_host(self, tok: int, pos: int) -> int:
        """One host-driven decode step, the way a serving loop that samples on the host uses the
        engine: the token and the step state go up from pinned host memory (20 bytes), the step
        runs (graph replay once captured), the selected token comes back (4 bytes) and the call
        returns it after synchronising."""
        if pos < 0 or pos + 1 > self.max_seq:
            raise ValueError(f"position {pos} does not fit the cache of {self.max_seq} rows")
        if not hasattr(self, "_pin"):
            self._pin = (torch.zeros(1, dtype=torch.int32).pin_memory(),
                         torch.zeros(4, dtype=torch.int32).pin_memory(),
                         torch.zeros(1, dtype=torch.int32).pin_memory())
        tok_h, state_h, out_h = self._pin
        tok_h[0] = tok
        state_h[0], state_h[1], state_h[2], state_h[3] = pos, pos + 1, 0, 0
        self.tok.copy_(tok_h, non_blocking=True)
        self.state.copy_(state_h, non_blocking=True)
        if self.graph is not None:
            self.graph.replay()
        else:
            self.step_static()
        out_h.copy_(self.tok, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return int(out_h[0])

    # ------------------------------------------------------------------ prefill
    def _prefill_buffers(self, P: int) -> Dict[str, torch.Tensor]:
        if P not in self._pbuf:
            bf = lambda *s: torch.empty(*s, dtype=torch.bfloat16, device=self.device)
            H = self.cfg.hidden
            self._pbuf[P] = {
                "ids": torch.zeros(P, dtype=torch.int32, device=self.device),
                "x": bf(P, H), "hn": bf(P, H), "part": bf(P, H),
                "qkv": bf(P, self.q_size + 2 * self.kv_size), "q": bf(P, self.q_size),
                "att": bf(P, self.q_size), "act": bf(P, max(self.inter, 8)),
                "pos0": torch.zeros(1, dtype=torch.int32, device=self.device),
                **self._moe_prefill_buffers(P),
                "last": torch.zeros(H, dtype=torch.float32, device=self.device),
            }
        return self._pbuf[P]

    def _moe_prefill_buffers(self, P: int) -> Dict[str, torch.Tensor]:
        if not self.moe:
            return {}
        cfg, dev = self.cfg, self.device
        pairs = P * cfg.top_k
        i32 = lambda *s: torch.zeros(*s, dtype=torch.int32, device=dev)
        bf = lambda *s: torch.empty(*s, dtype=torch.bfloat16, device=dev)
        b = {
            "rlogits": torch.empty(P, cfg.n_experts, dtype=torch.float32, device=dev),
            "eids": i32(P, cfg.top_k), "ew": torch.empty(P, cfg.top_k, dtype=torch.float32, device=dev),
            "order": i32(pairs), "inv": i32(pairs), "offs": i32(cfg.n_experts + 1),
            "pws": ops.moe_permute_workspace(pairs, cfg.n_experts, dev),
            "xg": bf(pairs, cfg.hidden), "eact": bf(pairs, cfg.moe_inter), "ey": bf(pairs, cfg.hidden),
        }
        if self._ep_dispatch(P):
            # all-to-all dispatch / combine: in the worst case every pair of the prompt is routed
            # to this rank's experts, so the receive side is sized for all P * top_k rows
            n = self.n_local_experts
            b.update({
                "offs_all": i32(self.tp_size, cfg.n_experts + 1),
                "lid": i32(pairs), "lid_recv": i32(pairs), "order2": i32(pairs), "inv2": i32(pairs),
                "offs2": i32(n + 1), "pws2": ops.moe_permute_workspace(pairs, n, dev),
                "x_recv": bf(pairs, cfg.hidden), "y_recv": bf(pairs, cfg.hidden),
                "y_back": bf(pairs, cfg.hidden),
            })
        return b

    def _ep_dispatch(self, P: int) -> bool:
        """Expert-parallel prefill with ep_all_to_all=True moves token rows to the experts' owners
        and back (needs a prompt that splits evenly over the ranks); otherwise - the default,
        because attention is replicated and every rank holds every row anyway - every rank routes
        all tokens, computes its own experts' pairs and the partial layer outputs are all-reduced.
        Measured on two B200s (Qwen3-30B-A3B architecture): time to first token 23.5 ms against
        49.7 ms with the all-to-all at 1024 tokens, 87.0 against 121.2 ms at 8192: the exchange
        moves more bytes than the all-reduce and its split sizes cost a device-to-host copy per
        layer."""
        return self.moe and self.tp_size > 1 and self.ep_all_to_all and P % self.tp_size == 0

    def _moe_prefill(self, e: Dict[str, torch.Tensor], x: torch.Tensor, hn: torch.Tensor, i: int) -> None:
        """x += sum over the routed experts (this rank's share under expert parallelism)."""
        cfg = self.cfg
        if self._ep_dispatch(x.shape[0]):
            self._moe_prefill_all_to_all(e, x, hn, i)
            return
        ops.gemm(e["rlogits"], hn, self.w_router[i])
        ops.moe_router(e["eids"], e["ew"], e["rlogits"])
        ops.moe_permute(e["order"], e["inv"], e["offs"], e["pws"], e["eids"])
        ops.moe_gather_rows(e["xg"], hn, e["order"], cfg.top_k)
        lo, n = self.expert_lo, self.n_local_experts
        offs = e["offs"][lo:lo + n + 1]
        ops.moe_grouped_gemm(e["eact"], e["xg"], self.wgu[i], offs, epilogue=EPI_SWIGLU)
        ops.moe_grouped_gemm(e["ey"], e["eact"], self.wd[i], offs)
        if self.tp_size > 1:
            part = e["part"]
            ops.moe_combine(part, e["ey"], e["inv"], e["ew"], None, e["eids"], lo, n)
            self._all_reduce(part)
        else:
            ops.moe_combine(x, e["ey"], e["inv"], e["ew"], x)

    def _moe_prefill_all_to_all(self, e: Dict[str, torch.Tensor], x: torch.Tensor, hn: torch.Tensor,
                                i: int) -> None:
        """Expert parallelism proper (the chain models/qwen3-30b-a3b/qwen3_optimized.py:573-590
        runs on one GPU, wrapped in a dispatch and a combine).  This rank owns the rows
        [rank * P / N, (rank + 1) * P / N) of the prompt for the MoE half of the layer:
          route own rows -> sort own (token, slot) pairs by expert (= by owner rank, experts are
          numbered rank-major) -> all-to-all: rows + local expert ids to the experts' owners ->
          sort the received rows by local expert -> two grouped GEMMs -> undo the sort ->
          all-to-all back -> weighted sum + residual into the own rows of x -> all-gather x
        (attention is replicated, so every rank needs the whole residual stream again).  The split
        sizes of the exchange come from one all-gather of the per-expert offsets and one small
        device-to-host copy per layer."""
        import torch.distributed as dist
        cfg, N, r = self.cfg, self.tp_size, self.tp_rank
        P, k, n = x.shape[0], cfg.top_k, self.n_local_experts
        per = P // N
        own = slice(r * per, (r + 1) * per)
        pairs = per * k
        # --- route and sort this rank's rows ---
        rl, eids, ew = e["rlogits"][:per], e["eids"][:per], e["ew"][:per]
        order, inv = e["order"][:pairs], e["inv"][:pairs]
        ops.gemm(rl, hn[own], self.w_router[i])
        ops.moe_router(eids, ew, rl)
        ops.moe_permute(order, inv, e["offs"], e["pws"], eids)
        ops.moe_gather_rows(e["xg"][:pairs], hn[own], order, k)
        # local expert id of every sorted row (what the owner sorts by)
        torch.remainder(eids.view(-1)[order.long()], n, out=e["lid"][:pairs])
        # --- split sizes: every rank's expert offsets, once to the host ---
        dist.all_gather_into_tensor(e["offs_all"], e["offs"].view(1, -1), group=self.group)
        offs_all = e["offs_all"].cpu()                                   # [N, E + 1]
        bounds = offs_all[:, ::n]                                        # [N, N + 1]: row ranges by owner
        send = (bounds[r, 1:] - bounds[r, :-1]).tolist()                 # my rows for each owner
        recv = (bounds[:, r + 1] - bounds[:, r]).tolist()                # each rank's rows for my experts
        R = sum(recv)
        # --- dispatch ---
        x_recv, lid_recv = e["x_recv"][:R], e["lid_recv"][:R]
        dist.all_to_all_single(x_recv.view(torch.uint8), e["xg"][:pairs].view(torch.uint8), recv, send,
                               group=self.group)
        dist.all_to_all_single(lid_recv, e["lid"][:pairs], recv, send, group=self.group)
        if R > 0:
            order2, inv2 = e["order2"][:R], e["inv2"][:R]
            ops.moe_permute(order2, inv2, e["offs2"], e["pws2"], lid_recv)
            ops.moe_gather_rows(e["xg"][:R], x_recv, order2, 1)
            ops.moe_grouped_gemm(e["eact"][:R], e["xg"][:R], self.wgu[i], e["offs2"], epilogue=EPI_SWIGLU)
            ops.moe_grouped_gemm(e["ey"][:R], e["eact"][:R], self.wd[i], e["offs2"])
            ops.moe_gather_rows(e["y_recv"][:R], e["ey"][:R], inv2, 1)   # back to arrival order
        # --- combine ---
        dist.all_to_all_single(e["y_back"][:pairs].view(torch.uint8), e["y_recv"][:R].view(torch.uint8),
                               send, recv, group=self.group)
        ops.moe_combine(x[own], e["y_back"][:pairs], inv, ew, x[own])
        dist.all_gather_into_tensor(x, x[own], group=self.group)

    @torch.no_grad()
    def prefill(self, ids: torch.Tensor, collect: Optional[list] = None,
                collect_router: Optional[list] = None, graph: Optional[bool] = None) -> int:
        """Runs the prompt, fills the KV cache and returns the first generated token.
        `collect` receives a copy of the residual stream after every layer, `collect_router`
        the expert ids [P, top_k] every MoE layer chose.
        graph: replay a CUDA graph captured for this prompt length instead of launching the ~9
        kernels per layer from the host, which is what bounds the time to first token of short
        prompts.  Default: on for single-GPU prompts of up to 2048 tokens (multi-rank prefills
        carry collectives and, under expert parallelism, a host-side exchange of split sizes)."""
        P = ids.numel()
        if P + 1 > self.max_seq:
            raise ValueError("prompt too long for this cache")
        e = self._prefill_buffers(P)
        e["ids"].copy_(ids.to(torch.int32))
        if graph is None:
            graph = self.tp_size == 1 and P <= 2048 and self.device.type == "cuda"
        if graph and collect is None and collect_router is None:
            g = self._prefill_graphs.get(P)
            if g is None:
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    self._prefill_launches(e, P, None, None)      # warm-up outside the capture
                torch.cuda.current_stream().wait_stream(side)
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    self._prefill_launches(e, P, None, None)
                self._prefill_graphs[P] = g
            g.replay()
        else:
            self._prefill_launches(e, P, collect, collect_router)
        self.last_prefill_hidden = e["x"]
        first = int(self.tok.item())
        self.check_status()
        return first

    def _prefill_launches(self, e: Dict[str, torch.Tensor], P: int, collect: Optional[list],
                          collect_router: Optional[list]) -> None:
        """Every launch of one prefill over the buffers `e` (no host synchronisation inside)."""
        cfg = self.cfg
        tp = self.att_tp > 1
        ep = self.moe and self.tp_size > 1
        hd = cfg.head_dim
        x, hn, part = e["x"], e["hn"], e["part"]
        ops.embed_gather(x, self.embed, e["ids"])
        ops.rmsnorm(hn, x, self.ln1[0], cfg.eps)
        for i in range(cfg.layers):
            kc, vc = self.kv[i, 0], self.kv[i, 1]
            ops.gemm(e["qkv"], hn, self.wqkv[i])
            ops.qk_rope_cache(e["q"], kc, vc, e["qkv"], self.cos, self.sin, e["pos0"],
                              self.n_q, self.n_kv, eps=cfg.eps, qn_w=self.qn[i], kn_w=self.kn[i])
            ops.flash_prefill(e["att"].view(1, P, self.n_q, hd), e["q"].view(1, P, self.n_q, hd),
                              kc.unsqueeze(0), vc.unsqueeze(0), P, True, self.scale)
            if tp:
                ops.gemm(part, e["att"], self.wo[i])
                self._all_reduce(part)
                ops.add_rmsnorm(hn, x, x, part, self.ln2[i], cfg.eps)
            else:
                ops.gemm(x, e["att"], self.wo[i], resid=x)
                ops.rmsnorm(hn, x, self.ln2[i], cfg.eps)
            nw = self.ln1[i + 1] if i + 1 < cfg.layers else self.final_norm_w
            if self.moe:
                self._moe_prefill(e, x, hn, i)
                if ep and not self._ep_dispatch(P):
                    ops.add_rmsnorm(hn, x, x, part, nw, cfg.eps)
                else:
                    ops.rmsnorm(hn, x, nw, cfg.eps)
            else:
                ops.gemm(e["act"], hn, self.wgu[i], epilogue=EPI_SWIGLU)
                if tp:
                    ops.gemm(part, e["act"], self.wd[i])
                    self._all_reduce(part)
                    ops.add_rmsnorm(hn, x, x, part, nw, cfg.eps)
                else:
                    ops.gemm(x, e["act"], self.wd[i], resid=x)
                    ops.rmsnorm(hn, x, nw, cfg.eps)
            if collect is not None:
                collect.append(x.clone())
            if collect_router is not None and self.moe:
                collect_router.append(e["eids"].clone())
        # hn now holds the final-norm output; project the last position only
        ops.gemv(self.logits, hn[P - 1], self.lm_head)
        ops.argmax(self.cand, self.logits, self.am_ws,
                   idx_base=(self.tp_rank * self.vocab_local) if tp else 0)
        if tp:
            torch.distributed.all_gather_into_tensor(self.cand_all, self.cand.view(1, 2),
                                                     group=self.group)
            ops.greedy_select(self.tok, self.cand_all)
        else:
            ops.greedy_select(self.tok, self.cand)

    # ------------------------------------------------------------------ generation
    @torch.no_grad()
    def generate(self, ids: torch.Tensor, n_new: int, sync_every_step: bool = False) -> List[int]:
        """Greedy generation.  The decode loop replays one graph per token; token selection and
        position bookkeeping stay on the device, so the host reads the tokens once at the end
        (or every step with sync_every_step, the reference's behaviour)."""
        P = ids.numel()
        if n_new > self.tok_log.numel() + 1:
            raise ValueError("n_new exceeds max_new_tokens")
        if P + n_new - 1 > self.max_seq:
            # the kernels guard the cache write but attend to kv_len rows: past max_seq that
            # would read beyond the cache
            raise ValueError(f"{P} prompt + {n_new - 1} decode positions exceed the cache of "
                             f"{self.max_seq} rows")
        first = self.prefill(ids)
        out = [first]
        self.set_step(first, P, 0)
        if self.graph is None:
            self.capture()
            self.set_step(first, P, 0)
        for _ in range(n_new - 1):
            self.graph.replay()
            if sync_every_step:
                out.append(int(self.tok.item()))
        if not sync_every_step:
            out.extend(self.tok_log[:n_new - 1].tolist())
        self.check_status()
        return out


class Llama31Optimized(DenseDecoder):
    """Drop-in for the reference's Llama31Optimized (models/llama31-8b/llama31_optimized.py:317)."""


class Qwen3Optimized(DenseDecoder):
    """Drop-in for the reference's Qwen3Optimized (models/qwen3-4b/qwen3_optimized.py:312)."""
