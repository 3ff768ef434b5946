"""TEST INFRASTRUCTURE — CPU fp32 oracle for the decoder hot path.  Never imported by the product.

Two oracles live here:

1. `hf_model(cfg, weights)`: the reference's parity authority itself — the HuggingFace
   `transformers` eager model (LlamaForCausalLM / Qwen3ForCausalLM), instantiated from config
   (no download) and loaded with the same bf16-rounded seeded weights upcast to fp32.  The
   reference gates its engines on exactly this model
   (models/llama31-8b/best_hoid.py:27-37,69-77; models/llama31-8b/common.py:60-67).
   transformers is a third-party dependency of the reference (pinned 5.15.0 in
   models/llama31-8b/pyproject.toml:8; this image has 5.5.0 — the version is recorded in
   every fixture).

2. `decoder_forward(...)`: a plain-torch fp32 restatement of the same forward
   (transformers/models/llama/modeling_llama.py: LlamaRMSNorm.forward, apply_rotary_pos_emb,
   eager_attention_forward, LlamaMLP.forward, LlamaDecoderLayer.forward; qwen3/modeling_qwen3.py
   for the per-head q/k RMSNorm), layer-streamed and query-chunked so that full-size models
   fit host memory.  tests/test_oracle.py pins it against (1) and against the committed
   golden vectors in tests/golden/.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch
import torch.nn.functional as F


# ----------------------------------------------------------------------------- HF authority
def hf_model(cfg, weights: Dict[str, torch.Tensor]):
    """Eager fp32 HuggingFace model carrying `weights` (bf16 tensors under HF names)."""
    import transformers

    common = dict(
        vocab_size=cfg.vocab, hidden_size=cfg.hidden, intermediate_size=cfg.inter or cfg.moe_inter,
        num_hidden_layers=cfg.layers, num_attention_heads=cfg.n_q, num_key_value_heads=cfg.n_kv,
        head_dim=cfg.head_dim, rms_norm_eps=cfg.eps, max_position_embeddings=131072,
        tie_word_embeddings=cfg.tied, attention_bias=False)
    if cfg.rope_scaling is not None:
        rope = dict(rope_type="llama3", rope_theta=cfg.rope_theta, **cfg.rope_scaling)
    else:
        rope = dict(rope_type="default", rope_theta=cfg.rope_theta)
    if cfg.n_experts:
        conf = transformers.Qwen3MoeConfig(
            **common, rope_parameters=rope, num_experts=cfg.n_experts,
            num_experts_per_tok=cfg.top_k, moe_intermediate_size=cfg.moe_inter,
            norm_topk_prob=True, decoder_sparse_step=1, mlp_only_layers=[])
        cls = transformers.Qwen3MoeForCausalLM
    elif cfg.qk_norm:
        conf = transformers.Qwen3Config(**common, rope_parameters=rope)
        cls = transformers.Qwen3ForCausalLM
    else:
        conf = transformers.LlamaConfig(**common, rope_parameters=rope, mlp_bias=False)
        cls = transformers.LlamaForCausalLM
    conf._attn_implementation = "eager"
    model = cls(conf).float()
    sd = {k: v.float() for k, v in weights.items()}
    if cfg.tied:
        sd["lm_head.weight"] = sd["model.embed_tokens.weight"]
    missing, unexpected = model.load_state_dict(sd, strict=False)
    if missing or unexpected:
        raise RuntimeError(f"weight names do not match HF: missing={missing} unexpected={unexpected}")
    return model.eval()


@torch.no_grad()
def hf_forward(model, ids: torch.Tensor):
    """(per-layer hidden states [L+1][S, H] with the final norm applied to the last, logits [S, V])."""
    out = model(ids.view(1, -1).long(), output_hidden_states=True, use_cache=False)
    hs = [h[0] for h in out.hidden_states]
    return hs, out.logits[0]


@torch.no_grad()
def hf_greedy(model, ids: torch.Tensor, n_new: int) -> List[int]:
    out = model.generate(ids.view(1, -1).long(), max_new_tokens=n_new, do_sample=False,
                         use_cache=True, pad_token_id=0)
    return out[0, ids.numel():].tolist()


# ----------------------------------------------------------------------------- restatement
def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """LlamaRMSNorm.forward in fp32: x * rsqrt(mean(x^2) + eps) * w."""
    var = x.pow(2).mean(-1, keepdim=True)
    return x * torch.rsqrt(var + eps) * w


def rope_rotate(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """apply_rotary_pos_emb with rotate_half: x is [S, heads, hd], cos/sin [S, hd/2]."""
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat((x1 * c - x2 * s, x2 * c + x1 * s), dim=-1)


def inv_freq(cfg) -> torch.Tensor:
    """float64 RoPE inverse frequencies (modeling_rope_utils: default and llama3 rules)."""
    hd = cfg.head_dim
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, hd, 2, dtype=torch.float64) / hd))
    sc = cfg.rope_scaling
    if sc is None:
        return inv
    factor, lo, hi = sc["factor"], sc["low_freq_factor"], sc["high_freq_factor"]
    old = sc["original_max_position_embeddings"]
    low_wl, high_wl = old / lo, old / hi
    wl = 2 * math.pi / inv
    out = torch.where(wl > low_wl, inv / factor, inv)
    smooth = (old / wl - lo) / (hi - lo)
    smoothed = (1 - smooth) * out / factor + smooth * out
    mid = ~(wl < high_wl) & ~(wl > low_wl)
    return torch.where(mid, smoothed, out)


def causal_attention(q, k, v, scale: float, q_pos0: int = 0, chunk: int = 1024) -> torch.Tensor:
    """q [S, n_q, hd]; k, v [L, n_kv, hd]; query i sees keys <= q_pos0 + i.  fp32, query-chunked."""
    S, n_q, hd = q.shape
    L, n_kv, _ = k.shape
    g = n_q // n_kv
    kk = k.permute(1, 0, 2).repeat_interleave(g, dim=0)          # [n_q, L, hd]
    vv = v.permute(1, 0, 2).repeat_interleave(g, dim=0)
    out = torch.empty(S, n_q, hd, dtype=q.dtype)
    keys = torch.arange(L)
    for s0 in range(0, S, chunk):
        s1 = min(S, s0 + chunk)
        qq = q[s0:s1].permute(1, 0, 2)                              # [n_q, c, hd]
        sc = torch.matmul(qq, kk.transpose(1, 2)) * scale           # [n_q, c, L]
        mask = keys[None, :] > (q_pos0 + torch.arange(s0, s1))[:, None]
        sc = sc.masked_fill(mask[None], float("-inf"))
        p = torch.softmax(sc, dim=-1, dtype=torch.float32)
        out[s0:s1] = torch.matmul(p, vv).permute(1, 0, 2)
    return out


def moe_route(logits: torch.Tensor, top_k: int):
    """Qwen3MoeTopKRouter semantics: fp32 softmax over experts -> top-k -> renormalise over
    the selected experts (models/qwen3-30b-a3b/qwen3_optimized.py:569-572)."""
    probs = torch.softmax(logits.float(), dim=-1)
    w, ids = torch.topk(probs, top_k, dim=-1)
    w = w / w.sum(-1, keepdim=True)
    return ids, w


def layer_weights(weights, i: int, name: str) -> torch.Tensor:
    return weights[f"model.layers.{i}.{name}"].float()


@torch.no_grad()
def decoder_forward(cfg, weights: Dict[str, torch.Tensor], ids: torch.Tensor,
                    logits_rows: Optional[Sequence[int]] = None, keep_hidden: bool = True,
                    act_dtype: Optional[torch.dtype] = None):
    """Full-sequence causal forward in fp32, one layer resident at a time.

    With act_dtype=torch.bfloat16 every tensor an eager bf16 run materialises (norm output, each
    linear output, the rotated q/k, the attention output, silu(gate), silu(gate)*up, each
    residual sum) is rounded to bf16 while all arithmetic inside an op stays fp32 - the numerics
    of the reference's own bf16 eager path (and of HuggingFace in torch_dtype=bfloat16).  The
    distance of that run from the fp32 run is the error floor any bf16-operand pipeline has at
    a given depth; the full-size parity test measures the CUDA path against it.

    Returns (hidden, logits, router): hidden[l] is the residual stream after l layers ([S, H];
    the last entry has the final norm applied, like HF's output_hidden_states), logits are
    the rows `logits_rows` (default: all) and router[l] the per-layer router logits (MoE)."""
    S = ids.numel()
    H, hd = cfg.hidden, cfg.head_dim
    r = (lambda t: t) if act_dtype is None else (lambda t: t.to(act_dtype).float())
    x = weights["model.embed_tokens.weight"][ids.long()].float()
    ang = torch.arange(S, dtype=torch.float64)[:, None] * inv_freq(cfg)[None, :]
    cos, sin = ang.cos().float(), ang.sin().float()
    hidden = [x.clone()] if keep_hidden else []
    router = []
    for i in range(cfg.layers):
        L = lambda n: layer_weights(weights, i, n)
        hn = r(rmsnorm(x, L("input_layernorm.weight"), cfg.eps))
        q = r(hn @ L("self_attn.q_proj.weight").T).view(S, cfg.n_q, hd)
        k = r(hn @ L("self_attn.k_proj.weight").T).view(S, cfg.n_kv, hd)
        v = r(hn @ L("self_attn.v_proj.weight").T).view(S, cfg.n_kv, hd)
        if cfg.qk_norm:
            q = r(rmsnorm(q, L("self_attn.q_norm.weight"), cfg.eps))
            k = r(rmsnorm(k, L("self_attn.k_norm.weight"), cfg.eps))
        q, k = r(rope_rotate(q, cos, sin)), r(rope_rotate(k, cos, sin))
        att = r(causal_attention(q, k, v, hd ** -0.5).reshape(S, cfg.n_q * hd))
        x = r(x + r(att @ L("self_attn.o_proj.weight").T))
        hn = r(rmsnorm(x, L("post_attention_layernorm.weight"), cfg.eps))
        if cfg.n_experts:
            rl = hn @ L("mlp.gate.weight").T
            router.append(rl)
            eids, ew = moe_route(rl, cfg.top_k)
            gu = L("mlp.experts.gate_up_proj")
            dn = L("mlp.experts.down_proj")
            y = torch.zeros_like(x)
            for e in eids.unique().tolist():
                tok, slot = (eids == e).nonzero(as_tuple=True)
                t = r(hn[tok] @ gu[e].T)
                a = r(r(F.silu(t[:, :cfg.moe_inter])) * t[:, cfg.moe_inter:])
                y.index_add_(0, tok, r(r(a @ dn[e].T) * ew[tok, slot][:, None]))
            x = r(x + r(y))
        else:
            g = r(hn @ L("mlp.gate_proj.weight").T)
            u = r(hn @ L("mlp.up_proj.weight").T)
            a = r(r(F.silu(g)) * u)
            x = r(x + r(a @ L("mlp.down_proj.weight").T))
        if keep_hidden and i + 1 < cfg.layers:
            hidden.append(x.clone())
    xn = rmsnorm(x, weights["model.norm.weight"].float(), cfg.eps)
    if keep_hidden:
        hidden.append(xn)
    head = weights["model.embed_tokens.weight" if cfg.tied else "lm_head.weight"].float()
    rows = list(range(S)) if logits_rows is None else list(logits_rows)
    logits = xn[rows] @ head.T
    return hidden, logits, router
