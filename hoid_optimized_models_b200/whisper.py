"""Whisper-large-v3-architecture encoder and cached greedy decoder on the b200 ops.

Mirrors the reference's `OptimizedWhisperEncoder` (models/whisper-large-v3/whisper_optimized.py:518-671)
and `OptimizedWhisperDecoder` (whisper_decoder_optimized.py:181-476): static buffers, CUDA-graph
capture, `set_encoder()` to project the window's cross-attention K/V, one graph replay per token.

Encoder dataflow (all tensor-core GEMMs with fused epilogues):
    mel^T (time-major, zero-padded) -> conv1 as a GEMM over an overlapping-row view (+ bias + GELU)
    -> conv2 (stride 2) the same way (+ bias + GELU + positional embedding as the residual)
    -> 32 x [gemm q|k|v + bias, flash_prefill (bidirectional), gemm out + bias, residual + layernorm,
             gemm fc1 + bias + GELU, gemm fc2 + bias, residual + layernorm]
The convolutions need no im2col: a k=3 window over a time-major [T, C] buffer is three adjacent
rows, i.e. one row of a [T_out, 3 C] matrix whose row stride is (stride * C) elements.

Decoder step (fp32 activations, weights streamed once per token):
    embed + position -> 32 x [layernorm, gemv q|k|v + bias, cache write, flash_decode (self),
    gemv out + bias + residual, layernorm, gemv cross-q + bias, flash_decode over the encoder K/V
    (row stride 1280), gemv out + bias + residual, layernorm, gemv fc1 + bias + GELU,
    gemv fc2 + bias + residual] -> layernorm -> gemv tied head -> argmax -> greedy_advance
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from . import ops
from .configs import WhisperConfig


def _conv_as_gemm_weight(w: torch.Tensor) -> torch.Tensor:
    """[C_out, C_in, 3] -> [C_out, 3 * C_in] with the tap index major, matching a window of three
    adjacent time-major rows."""
    return w.permute(0, 2, 1).reshape(w.shape[0], -1).contiguous()


def load_checkpoint(weights_dir: str, device="cuda") -> Dict[str, torch.Tensor]:
    """The `model.*` tensors of a HuggingFace `WhisperForConditionalGeneration` safetensors
    checkpoint (the names models/whisper-large-v3/whisper_decoder_optimized.py:189-228 reads), as
    both engines below take them."""
    from . import checkpoint
    return checkpoint.load_weights(weights_dir, device=device,
                                   keep=lambda n: n.startswith("model."))


class WhisperEncoder:
    def __init__(self, cfg: WhisperConfig, weights: Dict[str, torch.Tensor], device="cuda"):
        self.cfg, self.device = cfg, torch.device(device)
        dev, D = self.device, cfg.d_model
        g = lambda n: weights["model.encoder." + n].to(dev)
        self.w1, self.b1 = _conv_as_gemm_weight(g("conv1.weight")), g("conv1.bias")
        self.w2, self.b2 = _conv_as_gemm_weight(g("conv2.weight")), g("conv2.bias")
        self.pos = g("embed_positions.weight")
        self.layers: List[Dict[str, torch.Tensor]] = []
        for i in range(cfg.enc_layers):
            p = f"layers.{i}."
            a = p + "self_attn."
            self.layers.append({
                "ln1": (g(p + "self_attn_layer_norm.weight"), g(p + "self_attn_layer_norm.bias")),
                "wqkv": torch.cat([g(a + n + ".weight") for n in ("q_proj", "k_proj", "v_proj")], 0).contiguous(),
                "bqkv": torch.cat([g(a + "q_proj.bias"), torch.zeros(D, dtype=torch.bfloat16, device=dev),
                                   g(a + "v_proj.bias")], 0).contiguous(),
                "wo": g(a + "out_proj.weight"), "bo": g(a + "out_proj.bias"),
                "ln2": (g(p + "final_layer_norm.weight"), g(p + "final_layer_norm.bias")),
                "wf1": g(p + "fc1.weight"), "bf1": g(p + "fc1.bias"),
                "wf2": g(p + "fc2.weight"), "bf2": g(p + "fc2.bias"),
            })
        self.ln_f = (g("layer_norm.weight"), g("layer_norm.bias"))
        T, S = cfg.n_frames, cfg.n_ctx
        bf = lambda *s: torch.zeros(*s, dtype=torch.bfloat16, device=dev)
        # time-major inputs with one zero row of padding on each side
        self.x0 = bf(T + 2, cfg.n_mels)
        self.x1 = bf(T + 2, D)
        self.a0 = torch.as_strided(self.x0, (T, 3 * cfg.n_mels), (cfg.n_mels, 1))
        self.a1 = torch.as_strided(self.x1, (S, 3 * D), (2 * D, 1))
        self.x, self.h = bf(S, D), bf(S, D)
        self.qkv, self.ctx, self.act = bf(S, 3 * D), bf(S, D), bf(S, cfg.ffn)
        self.out, self.o = bf(S, D), bf(S, D)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.launches_per_forward = 2 + 7 * cfg.enc_layers + 1

    def load_inputs(self, mel: torch.Tensor) -> None:
        """mel: [n_mels, n_frames] log-mel features."""
        self.x0[1:-1].copy_(mel.t())

    def forward_static(self, collect: Optional[list] = None) -> torch.Tensor:
        cfg = self.cfg
        S, D, nh, hd = cfg.n_ctx, cfg.d_model, cfg.heads, cfg.head_dim
        ops.gemm(self.x1[1:-1], self.a0, self.w1, bias=self.b1, epilogue=ops.EPI_GELU)
        ops.gemm(self.x, self.a1, self.w2, bias=self.b2, resid=self.pos, epilogue=ops.EPI_GELU)
        x, h = self.x, self.h
        qkv4 = self.qkv.view(1, S, 3, nh, hd)
        q, k, v = qkv4[:, :, 0], qkv4[:, :, 1].permute(0, 2, 1, 3), qkv4[:, :, 2].permute(0, 2, 1, 3)
        ctx4 = self.ctx.view(1, S, nh, hd)
        # Pre-LN blocks: every GEMM output o is folded into the residual stream by the next
        # LayerNorm launch (x += o; h = LN(x)), which is memory-bound and coalesced, instead of by
        # the epilogue of these short-K GEMMs.
        o = self.o
        ops.layernorm(h, x, self.layers[0]["ln1"][0], self.layers[0]["ln1"][1], cfg.eps)
        for i, L in enumerate(self.layers):
            ops.gemm(self.qkv, h, L["wqkv"], bias=L["bqkv"])
            ops.flash_prefill(ctx4, q, k, v, S, False, hd ** -0.5)
            ops.gemm(o, self.ctx, L["wo"], bias=L["bo"])
            ops.add_layernorm(h, x, o, L["ln2"][0], L["ln2"][1], cfg.eps, resid=x)
            ops.gemm(self.act, h, L["wf1"], bias=L["bf1"], epilogue=ops.EPI_GELU)
            ops.gemm(o, self.act, L["wf2"], bias=L["bf2"])
            nxt = self.layers[i + 1]["ln1"] if i + 1 < len(self.layers) else self.ln_f
            dst = h if i + 1 < len(self.layers) else self.out
            ops.add_layernorm(dst, x, o, nxt[0], nxt[1], cfg.eps, resid=x)
            if collect is not None:
                collect.append(x.clone())
        return self.out

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
    def encode(self, mel: torch.Tensor) -> torch.Tensor:
        self.load_inputs(mel)
        if self.graph is not None:
            self.graph.replay()
        else:
            self.forward_static()
        return self.out


class WhisperDecoder:
    def __init__(self, cfg: WhisperConfig, weights: Dict[str, torch.Tensor], device="cuda",
                 max_new_tokens: int = 448, suppress_tokens: Optional[Sequence[int]] = None,
                 begin_suppress_tokens: Optional[Sequence[int]] = None):
        """suppress_tokens / begin_suppress_tokens: token ids whose logit is forced to -inf at
        every step / at the first generated token only (the `mask` and `begin_mask` the reference
        adds to the logits before its argmax, models/whisper-large-v3/best_hoid.py:88-104).  The
        mask rides as the bias of the logits GEMV, so the on-device greedy selection sees it."""
        self.cfg, self.device = cfg, torch.device(device)
        dev, D, H, hd = self.device, cfg.d_model, cfg.heads, cfg.head_dim
        g = lambda n: weights["model.decoder." + n].to(dev)
        zero_b = torch.zeros(D, dtype=torch.bfloat16, device=dev)
        self.embed_tok, self.embed_pos = g("embed_tokens.weight"), g("embed_positions.weight")
        self.layers: List[Dict[str, torch.Tensor]] = []
        for i in range(cfg.dec_layers):
            p = f"layers.{i}."
            a, c = p + "self_attn.", p + "encoder_attn."
            self.layers.append({
                "ln1": (g(p + "self_attn_layer_norm.weight"), g(p + "self_attn_layer_norm.bias")),
                "wqkv": torch.cat([g(a + n + ".weight") for n in ("q_proj", "k_proj", "v_proj")], 0).contiguous(),
                "bqkv": torch.cat([g(a + "q_proj.bias"), zero_b, g(a + "v_proj.bias")], 0).contiguous(),
                "wo": g(a + "out_proj.weight"), "bo": g(a + "out_proj.bias"),
                "ln2": (g(p + "encoder_attn_layer_norm.weight"), g(p + "encoder_attn_layer_norm.bias")),
                "wcq": g(c + "q_proj.weight"), "bcq": g(c + "q_proj.bias"),
                "wck": g(c + "k_proj.weight"),
                "wcv": g(c + "v_proj.weight"), "bcv": g(c + "v_proj.bias"),
                "wco": g(c + "out_proj.weight"), "bco": g(c + "out_proj.bias"),
                "ln3": (g(p + "final_layer_norm.weight"), g(p + "final_layer_norm.bias")),
                "wf1": g(p + "fc1.weight"), "bf1": g(p + "fc1.bias"),
                "wf2": g(p + "fc2.weight"), "bf2": g(p + "fc2.bias"),
            })
        self.ln_f = (g("layer_norm.weight"), g("layer_norm.bias"))
        L, T, S = cfg.dec_layers, cfg.max_target, cfg.n_ctx
        self.kv = torch.zeros(L, 2, H, T, hd, dtype=torch.bfloat16, device=dev)      # self-attention cache
        self.cross_k = torch.zeros(L, S, D, dtype=torch.bfloat16, device=dev)         # per window
        self.cross_v = torch.zeros(L, S, D, dtype=torch.bfloat16, device=dev)
        # the cache-write op rotates by (cos, sin): identity tables make it a plain write
        self.cos = torch.ones(T, hd // 2, dtype=torch.float32, device=dev)
        self.sin = torch.zeros(T, hd // 2, dtype=torch.float32, device=dev)
        f32 = lambda *s: torch.zeros(*s, dtype=torch.float32, device=dev)
        self.state = torch.zeros(4, dtype=torch.int32, device=dev)      # {position, kv_len, generated}
        self.pos, self.kv_len = self.state[0:1], self.state[1:2]
        self.enc_len = torch.full((1,), S, dtype=torch.int32, device=dev)
        self.tok = torch.zeros(1, dtype=torch.int32, device=dev)
        self.tok_log = torch.zeros(max_new_tokens, dtype=torch.int32, device=dev)
        self.e_tok, self.e_pos = f32(D), f32(D)
        self.x, self.h = f32(D), f32(D)
        self.qkv, self.q, self.attn, self.cq = f32(3 * D), f32(D), f32(D), f32(D)
        self.act = f32(cfg.ffn)
        self.logits = f32(cfg.vocab)
        self.cand = f32(2)
        self.logit_bias = self._steady_bias = self._begin_bias = None
        if suppress_tokens or begin_suppress_tokens:
            def mask(ids):
                m = torch.zeros(cfg.vocab, dtype=torch.bfloat16, device=dev)
                if ids:
                    m[torch.tensor(sorted(set(ids)), dtype=torch.long, device=dev)] = float("-inf")
                return m
            self._steady_bias = mask(list(suppress_tokens or []))
            self._begin_bias = mask(list(suppress_tokens or []) + list(begin_suppress_tokens or []))
            self.logit_bias = self._steady_bias.clone()      # the buffer the captured graph reads
        self.self_splits = max(1, min(148 // H, (T + 63) // 64))
        self.cross_splits = max(1, min(148 // H, (S + 63) // 64))
        self.ws_self = ops.flash_decode_workspace(H, H, hd, self.self_splits, dev)
        self.ws_cross = ops.flash_decode_workspace(H, H, hd, self.cross_splits, dev)
        self.am_ws = ops.argmax_workspace(dev)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self._pbuf: Dict[int, Dict[str, torch.Tensor]] = {}      # prefix-prefill buffers by length
        self._pgraphs: Dict[tuple, torch.cuda.CUDAGraph] = {}
        self.launches_per_step = 4 + 9 * cfg.dec_layers + 3

    @torch.no_grad()
    def set_encoder(self, enc_out: torch.Tensor) -> None:
        """Project the window's encoder states [n_ctx, D] (bf16) to every layer's cross K / V."""
        for i, L in enumerate(self.layers):
            ops.gemm(self.cross_k[i], enc_out, L["wck"])
            ops.gemm(self.cross_v[i], enc_out, L["wcv"], bias=L["bcv"])

    def step_static(self) -> None:
        cfg = self.cfg
        D, H, hd = cfg.d_model, cfg.heads, cfg.head_dim
        scale = hd ** -0.5
        ops.embed_gather(self.e_tok, self.embed_tok, self.tok)
        ops.embed_gather(self.e_pos, self.embed_pos, self.pos)
        x, h = self.x, self.h
        first = True
        for i, L in enumerate(self.layers):
            # every LayerNorm is the prologue of the GEMV that consumes it; identity cos / sin
            # tables turn the fused RoPE + cache-append + attention launch into Whisper's
            # position-free self-attention
            if first:   # residual stream = token + position embedding, fused with the first norm
                ops.add_layernorm(h, x, self.e_tok, L["ln1"][0], L["ln1"][1], cfg.eps, resid=self.e_pos)
                ops.gemv(self.qkv, h, L["wqkv"], bias=L["bqkv"])
                first = False
            else:
                ops.gemv(self.qkv, x, L["wqkv"], bias=L["bqkv"], norm_w=L["ln1"][0],
                         norm_b=L["ln1"][1], eps=cfg.eps)
            ops.rope_flash_decode(self.attn, self.kv[i, 0], self.kv[i, 1], self.ws_self, self.qkv,
                                  self.cos, self.sin, self.kv_len, H, H, self.self_splits, scale)
            ops.gemv(x, self.attn, L["wo"], bias=L["bo"], resid=x)
            ops.gemv(self.cq, x, L["wcq"], bias=L["bcq"], norm_w=L["ln2"][0], norm_b=L["ln2"][1],
                     eps=cfg.eps)
            ops.flash_decode(self.attn, self.cq, self.cross_k[i], self.cross_v[i], self.enc_len,
                             self.ws_cross, H, H, self.cross_splits, scale,
                             kv_head_stride=hd, kv_row_stride=D)
            ops.gemv(x, self.attn, L["wco"], bias=L["bco"], resid=x)
            ops.gemv(self.act, x, L["wf1"], bias=L["bf1"], epilogue=ops.EPI_GELU,
                     norm_w=L["ln3"][0], norm_b=L["ln3"][1], eps=cfg.eps)
            ops.gemv(x, self.act, L["wf2"], bias=L["bf2"], resid=x)
        ops.gemv(self.logits, x, self.embed_tok, norm_w=self.ln_f[0], norm_b=self.ln_f[1],
                 eps=cfg.eps, bias=self.logit_bias)
        ops.argmax(self.cand, self.logits, self.am_ws)
        ops.greedy_advance(self.tok, self.state, self.tok_log, self.cand)

    def capture(self, warmup: int = 2) -> None:
        saved = (self.state.clone(), self.tok.clone(), self.tok_log.clone())
        self.state.zero_()
        self.state[1] = 1
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(warmup):
                self.step_static()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph), torch.no_grad():
            self.step_static()
        torch.cuda.synchronize()
        self.state.copy_(saved[0]); self.tok.copy_(saved[1]); self.tok_log.copy_(saved[2])

    def _prefill_launches(self, b: Dict[str, torch.Tensor], s: int, enc_out: Optional[torch.Tensor]) -> None:
        """Every launch of one prefix prefill over the buffers `b` (no host synchronisation)."""
        cfg = self.cfg
        D, H, hd = cfg.d_model, cfg.heads, cfg.head_dim
        if enc_out is not None:
            self.set_encoder(enc_out)
        x, h, att = b["x"], b["h"], b["att"]
        scale = hd ** -0.5
        att4 = att.view(1, s, H, hd)
        ops.embed_gather(b["e_tok"], self.embed_tok, b["ids"])
        ops.embed_gather(b["e_pos"], self.embed_pos, b["pos_ids"])
        for i, L in enumerate(self.layers):
            if i == 0:    # residual stream = token + position embedding, fused with the first norm
                ops.add_layernorm(h, x, b["e_tok"], L["ln1"][0], L["ln1"][1], cfg.eps, resid=b["e_pos"])
            else:
                ops.layernorm(h, x, L["ln1"][0], L["ln1"][1], cfg.eps)
            ops.gemm(b["qkv"], h, L["wqkv"], bias=L["bqkv"])
            # identity cos / sin tables: a plain write of the k / v rows into cache rows 0 .. s - 1
            ops.qk_rope_cache(b["q"], self.kv[i, 0], self.kv[i, 1], b["qkv"], self.cos, self.sin,
                              b["pos0"], H, H)
            ops.flash_prefill(att4, b["q"].view(1, s, H, hd), self.kv[i, 0].unsqueeze(0),
                              self.kv[i, 1].unsqueeze(0), s, True, scale)
            ops.gemm(x, att, L["wo"], bias=L["bo"], resid=x)
            ops.layernorm(h, x, L["ln2"][0], L["ln2"][1], cfg.eps)
            ops.gemm(b["cq"], h, L["wcq"], bias=L["bcq"])
            ck = self.cross_k[i].view(1, cfg.n_ctx, H, hd).permute(0, 2, 1, 3)
            cv = self.cross_v[i].view(1, cfg.n_ctx, H, hd).permute(0, 2, 1, 3)
            ops.flash_prefill(att4, b["cq"].view(1, s, H, hd), ck, cv, cfg.n_ctx, False, scale)
            ops.gemm(x, att, L["wco"], bias=L["bco"], resid=x)
            ops.layernorm(h, x, L["ln3"][0], L["ln3"][1], cfg.eps)
            ops.gemm(b["act"], h, L["wf1"], bias=L["bf1"], epilogue=ops.EPI_GELU)
            ops.gemm(x, b["act"], L["wf2"], bias=L["bf2"], resid=x)
        # logits of the last prefix position only; it yields the first new token
        ops.gemv(self.logits, x[s - 1], self.embed_tok, norm_w=self.ln_f[0], norm_b=self.ln_f[1],
                 eps=cfg.eps, bias=self.logit_bias)
        ops.argmax(self.cand, self.logits, self.am_ws)
        ops.greedy_select(self.tok, self.cand)

    @torch.no_grad()
    def prefill(self, prefix: List[int], enc_out: Optional[torch.Tensor] = None,
                graph: Optional[bool] = None) -> int:
        """The forced prefix in ONE pass over all its positions (and, with enc_out, the window's
        cross K / V projection in front of it), as the reference's decoder prefill does
        (models/whisper-large-v3/whisper_decoder_optimized.py:285-331): bf16 rows through the
        tensor-core GEMMs and the prefill attention instead of one decode step per prefix token.
        Fills the self-attention cache rows 0 .. len(prefix) - 1, leaves the step state at the next
        position and returns the first generated token."""
        cfg, dev = self.cfg, self.device
        s, D, H, hd = len(prefix), cfg.d_model, cfg.heads, cfg.head_dim
        if s < 1 or s > cfg.max_target:
            raise ValueError(f"a prefix of {s} tokens does not fit the {cfg.max_target}-token window")
        b = self._pbuf.get(s)
        if b is None:
            bf = lambda *sh: torch.zeros(*sh, dtype=torch.bfloat16, device=dev)
            b = self._pbuf[s] = {
                "ids": torch.zeros(s, dtype=torch.int32, device=dev),
                "pos_ids": torch.arange(s, dtype=torch.int32, device=dev),
                "pos0": torch.zeros(1, dtype=torch.int32, device=dev),
                "e_tok": bf(s, D), "e_pos": bf(s, D), "x": bf(s, D), "h": bf(s, D),
                "qkv": bf(s, 3 * D), "q": bf(s, D), "att": bf(s, D), "cq": bf(s, D), "act": bf(s, cfg.ffn),
            }
        b["ids"].copy_(torch.tensor(prefix, dtype=torch.int32))
        if self.logit_bias is not None:
            self.logit_bias.copy_(self._begin_bias)      # this pass yields the first new token
        # ~15 launches per layer for a handful of rows: replayed from a CUDA graph captured per
        # (prefix length, encoder buffer), the pass is bound by the kernels, not by the host
        use_graph = graph if graph is not None else self.device.type == "cuda"
        if use_graph:
            key = (s, enc_out.data_ptr() if enc_out is not None else 0)
            g = self._pgraphs.get(key)
            if g is None:
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    self._prefill_launches(b, s, enc_out)            # warm-up outside the capture
                torch.cuda.current_stream().wait_stream(side)
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    self._prefill_launches(b, s, enc_out)
                self._pgraphs[key] = g
            g.replay()
        else:
            self._prefill_launches(b, s, enc_out)
        first = int(self.tok.item())
        if self.logit_bias is not None:
            self.logit_bias.copy_(self._steady_bias)
        self.state.copy_(torch.tensor([s, s + 1, 0, 0], dtype=torch.int32))
        ops.check_status(dev)
        return first

    def set_step(self, tok: int, pos: int, generated: int = 0) -> None:
        if pos < 0 or pos + 1 > self.cfg.max_target:
            raise ValueError(f"position {pos} is outside the {self.cfg.max_target}-token window")
        self.tok.fill_(tok)
        self.state.copy_(torch.tensor([pos, pos + 1, generated, 0], dtype=torch.int32))

    def _run(self) -> None:
        if self.graph is not None:
            self.graph.replay()
        else:
            self.step_static()

    @torch.no_grad()
    def generate(self, prefix: List[int], n_new: int, collect_logits: Optional[list] = None,
                 prefix_prefill: bool = True) -> List[int]:
        """Runs the forced prefix (one prefill pass; token by token when the logits of every
        position are collected or prefix_prefill is off), then decodes n_new tokens greedily.
        Returns the generated tokens."""
        if n_new > self.tok_log.numel() + 1:
            raise ValueError("n_new exceeds max_new_tokens")
        if len(prefix) + n_new - 1 > self.cfg.max_target:
            # positions index the learned position table and the self-attention cache
            raise ValueError(f"{len(prefix)} prefix + {n_new - 1} decode positions exceed the "
                             f"{self.cfg.max_target}-token window")
        if prefix_prefill and collect_logits is None:
            out = [self.prefill(prefix)]
        else:
            for p, t in enumerate(prefix):
                self.set_step(t, p, 0)
                if self.logit_bias is not None and p == len(prefix) - 1:
                    self.logit_bias.copy_(self._begin_bias)      # this step yields the first new token
                self._run()
                if collect_logits is not None:
                    collect_logits.append(self.logits.float().cpu().clone())
            # the step for the last prefix token has already produced the first new token
            out = [int(self.tok.item())]
            if self.logit_bias is not None:
                self.logit_bias.copy_(self._steady_bias)
            pos = len(prefix)
            self.state.copy_(torch.tensor([pos, pos + 1, 0, 0], dtype=torch.int32))
        for _ in range(n_new - 1):
            self._run()
            if collect_logits is not None:
                collect_logits.append(self.logits.float().cpu().clone())
        out.extend(self.tok_log[:n_new - 1].tolist())
        ops.check_status(self.device)
        return out


class OptimizedWhisperEncoder(WhisperEncoder):
    """Name-compatible with models/whisper-large-v3/whisper_optimized.py:518."""


class OptimizedWhisperDecoder(WhisperDecoder):
    """Name-compatible with models/whisper-large-v3/whisper_decoder_optimized.py:181."""
