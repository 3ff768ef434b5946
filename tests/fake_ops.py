"""TEST INFRASTRUCTURE - a plain-torch CPU stand-in for `hoid_optimized_models_b200.ops`.

The engines (`decoder.py`, `encoder.py`, `whisper.py`) are host logic over the op layer: buffer
ownership, weight packing, launch order, device-side step state, tensor- / expert- / data-parallel
sharding and which all-reduce feeds which GEMV.  These functions re-state every op the engines
call with the same signature and the same in/out semantics on CPU tensors, so that logic runs in the CPU test suite
(single process and world_size-2 gloo) against the fp32 oracle.  Nothing in the product imports
this file, and it is no fallback: `hoid_optimized_models_b200.ops` itself refuses CPU tensors.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

EPI_NONE, EPI_SWIGLU, EPI_GELU, EPI_GEGLU = 0, 1, 2, 3
Tensor = torch.Tensor
_STATUS = torch.zeros(1, dtype=torch.int32)


def set_pdl(enabled: bool) -> None:
    pass


def status_word(device) -> Tensor:
    return _STATUS


def check_status(device) -> None:
    assert int(_STATUS) == 0


def _store(dst: Tensor, src: Tensor) -> None:
    dst.copy_(src.reshape(dst.shape).to(dst.dtype))


def _rms(x: Tensor, w: Optional[Tensor], eps: float) -> Tensor:
    x = x.float()
    if w is None:
        return x
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w.float()


def _epilogue(y: Tensor, epilogue: int) -> Tensor:
    if epilogue == EPI_SWIGLU:                  # interleaved rows: 2j = gate_j, 2j + 1 = up_j
        return F.silu(y[..., 0::2]) * y[..., 1::2]
    if epilogue == EPI_GELU:
        return F.gelu(y)
    if epilogue == EPI_GEGLU:                   # stock projection: value half first, gate half second
        half = y.shape[-1] // 2
        return y[..., :half] * F.gelu(y[..., half:])
    return y


# ----------------------------------------------------------------------------- GEMV / GEMM
def gemv(y, x, w, norm_w=None, eps=0.0, bias=None, resid=None, epilogue=EPI_NONE, norm_b=None):
    xin = x.float().reshape(-1)
    if norm_b is not None:
        xin = F.layer_norm(xin, xin.shape, norm_w.float(), norm_b.float(), eps)
    else:
        xin = _rms(xin, norm_w, eps)
    out = w.float() @ xin
    if bias is not None:
        out = out + bias.float()
    out = _epilogue(out, epilogue)
    if resid is not None:
        out = out + resid.float().reshape(-1)
    _store(y, out)


def gemm(y, x, w, bias=None, resid=None, epilogue=EPI_NONE):
    out = x.float() @ w.float().T
    if bias is not None:
        out = out + bias.float()
    out = _epilogue(out, epilogue)
    if resid is not None:
        out = out + resid.float()
    _store(y, out)


def moe_grouped_gemm(y, x, w, offsets, epilogue=EPI_NONE):
    E = w.shape[0]
    out = torch.zeros(x.shape[0], w.shape[1] // (2 if epilogue == EPI_SWIGLU else 1))
    for e in range(E):
        a, b = int(offsets[e]), int(offsets[e + 1])
        if b > a:
            out[a:b] = _epilogue(x[a:b].float() @ w[e].float().T, epilogue)
    y[: x.shape[0]].copy_(out.to(y.dtype))


# ----------------------------------------------------------------------------- norms
def rmsnorm(norm_out, a, w, eps):
    _store(norm_out, _rms(a, w, eps))


def add_rmsnorm(norm_out, resid_out, a, b, w, eps):
    s = (a.float() + b.float()).to(resid_out.dtype)        # the stream stores the rounded sum
    resid_out.copy_(s)
    _store(norm_out, _rms(s, w, eps))


def _ln_sum(x, bias, resid, rounded: bool):
    """x (+ bias) (+ resid); with bf16 inputs every addition is rounded to bf16 like the kernel."""
    r = (lambda t: t.to(torch.bfloat16).float()) if rounded else (lambda t: t)
    v = x.float()
    if bias is not None:
        v = r(v + bias.float())
    if resid is not None:
        v = r(v + resid.float().reshape(v.shape))
    return v


def layernorm(norm_out, x, gamma, beta, eps, bias=None, resid=None):
    v = _ln_sum(x, bias, resid, x.dtype == torch.bfloat16)
    _store(norm_out, F.layer_norm(v, v.shape[-1:], gamma.float(), beta.float(), eps))


def add_layernorm(norm_out, resid_out, x, gamma, beta, eps, bias=None, resid=None):
    v = _ln_sum(x, bias, resid, x.dtype == torch.bfloat16)
    _store(resid_out, v)
    v = resid_out.float().reshape(v.shape)
    _store(norm_out, F.layer_norm(v, v.shape[-1:], gamma.float(), beta.float(), eps))


def cls_pool_l2(out, x, seq_len, eps=1e-12):
    first = x.float().reshape(-1, seq_len, x.shape[-1])[:, 0]
    _store(out, first / first.norm(dim=-1, keepdim=True).clamp_min(eps))


def silu_mul(out, gate, up):
    _store(out, F.silu(gate.float()) * up.float())


# ----------------------------------------------------------------------------- rope / attention
def _rope(x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), -1)


def qk_rope_cache(q_out, kcache, vcache, qkv, cos, sin, pos, n_q, n_kv, eps=0.0, qn_w=None,
                  kn_w=None):
    hd = kcache.shape[-1]
    rows = qkv.float().reshape(-1, n_q + 2 * n_kv, hd)
    s, p0 = rows.shape[0], int(pos)
    q, k, v = rows[:, :n_q], rows[:, n_q:n_q + n_kv], rows[:, n_q + n_kv:]
    if qn_w is not None:
        q, k = _rms(q, qn_w, eps), _rms(k, kn_w, eps)
    c, sn = cos[p0:p0 + s, None, :], sin[p0:p0 + s, None, :]
    _store(q_out, _rope(q, c, sn))
    kcache[:, p0:p0 + s] = _rope(k, c, sn).permute(1, 0, 2).to(kcache.dtype)
    vcache[:, p0:p0 + s] = v.permute(1, 0, 2).to(vcache.dtype)


def flash_decode_workspace(n_q, n_kv, hd, n_splits, device):
    return torch.zeros(4, dtype=torch.float32)


def flash_decode(out, q, kcache, vcache, kv_len, workspace, n_q, n_kv, n_splits, scale,
                 kv_head_stride=-1, kv_row_stride=-1):
    L = int(kv_len)
    hd = q.numel() // n_q
    if kv_row_stride > 0 and kcache.dim() == 2:
        # rows of [L, n_kv * hd] projections: head h of row j starts at j * row_stride + h * hd
        kcache = kcache.reshape(kcache.shape[0], n_kv, hd).permute(1, 0, 2)
        vcache = vcache.reshape(vcache.shape[0], n_kv, hd).permute(1, 0, 2)
    g = n_q // n_kv
    qq = q.float().reshape(n_q, hd)
    kk = kcache[:, :L].float().repeat_interleave(g, 0)
    vv = vcache[:, :L].float().repeat_interleave(g, 0)
    p = torch.softmax(torch.einsum("hd,hkd->hk", qq, kk) * scale, -1)
    _store(out, torch.einsum("hk,hkd->hd", p, vv))


def rope_flash_decode(out, kcache, vcache, workspace, qkv, cos, sin, kv_len, n_q, n_kv, n_splits,
                      scale, eps=0.0, qn_w=None, kn_w=None):
    hd = kcache.shape[-1]
    q = torch.empty(n_q * hd)
    pos = (kv_len - 1).to(torch.int32)
    qk_rope_cache(q, kcache, vcache, qkv, cos, sin, pos, n_q, n_kv, eps, qn_w, kn_w)
    flash_decode(out, q, kcache, vcache, kv_len, workspace, n_q, n_kv, n_splits, scale)


def flash_prefill(out, q, k, v, kv_len, causal, scale, q_pos0=0, impl="tc"):
    B, S, n_q, hd = q.shape
    n_kv = k.shape[1]
    g = n_q // n_kv
    qq = q.float().permute(0, 2, 1, 3)                                   # [B, n_q, S, hd]
    kk = k[:, :, :kv_len].float().repeat_interleave(g, 1)
    vv = v[:, :, :kv_len].float().repeat_interleave(g, 1)
    sc = torch.matmul(qq, kk.transpose(-1, -2)) * scale
    if causal:
        keys = torch.arange(kv_len)[None, :]
        rows = (q_pos0 + torch.arange(S))[:, None]
        sc = sc.masked_fill(keys > rows, float("-inf"))
    o = torch.matmul(torch.softmax(sc, -1), vv).permute(0, 2, 1, 3)
    out.copy_(o.to(out.dtype))


# ----------------------------------------------------------------------------- MoE
def moe_router(ids, wts, logits, round_bf16=False):
    lg = logits.float().reshape(-1, logits.shape[-1])
    k = ids.numel() // lg.shape[0]
    p = torch.softmax(lg, -1)
    # descending probability, ties to the lowest index: a stable sort of -p
    order = torch.sort(-p, dim=-1, stable=True).indices[:, :k]
    w = torch.gather(p, 1, order)
    w = w / w.sum(-1, keepdim=True)
    if round_bf16:
        w = w.to(torch.bfloat16).float()
    _store(ids, order.to(torch.int32))
    _store(wts, w)


def moe_permute_workspace(pairs, E, device):
    return torch.zeros(1, dtype=torch.int32)


def moe_permute(order, inv, offsets, workspace, ids):
    flat = ids.reshape(-1).long()
    o = torch.sort(flat, stable=True).indices
    order.copy_(o.to(torch.int32))
    inv.reshape(-1)[o] = torch.arange(o.numel(), dtype=torch.int32)
    counts = torch.bincount(flat, minlength=offsets.numel() - 1)
    offsets[0] = 0
    offsets[1:] = torch.cumsum(counts, 0).to(torch.int32)


def moe_gather_rows(xg, x, order, top_k):
    xg.copy_(x[(order.long() // top_k)])


def moe_combine(out, y, inv, wts, resid=None, ids=None, expert_lo=0, n_local=0):
    tokens, top_k = wts.shape
    rows = y.float()[inv.reshape(tokens, top_k).long()]                  # [tokens, k, H]
    w = wts.float().clone()
    if ids is not None:
        local = (ids.reshape(tokens, top_k) >= expert_lo) & (ids.reshape(tokens, top_k) < expert_lo + n_local)
        w = w * local
    acc = (rows * w[..., None]).sum(1)
    if resid is not None:
        acc = acc + resid.float()
    out.copy_(acc.to(out.dtype))


def moe_decode_gate_up(act, x, w_gu, ids, wts, norm_w=None, eps=0.0, expert_lo=0):
    E = w_gu.shape[0]
    xin = _rms(x.float().reshape(-1), norm_w, eps)
    rows = []
    for slot in range(ids.numel()):
        e = int(ids[slot]) - expert_lo
        if 0 <= e < E:
            rows.append(_epilogue(w_gu[e].float() @ xin, EPI_SWIGLU) * float(wts[slot]))
        else:                                    # the expert lives on another rank
            rows.append(torch.zeros(w_gu.shape[1] // 2))
    _store(act, torch.stack(rows))


def _moe_down(act, w_down, ids, resid, expert_lo):
    E, H, I = w_down.shape
    a = act.float().reshape(ids.numel(), I)
    out = torch.zeros(H)
    for slot in range(ids.numel()):
        e = int(ids[slot]) - expert_lo
        if 0 <= e < E:
            out = out + w_down[e].float() @ a[slot]
    if resid is not None:
        out = out + resid.float().reshape(-1)
    return out


def moe_decode_down(y, act, w_down, ids, resid=None, expert_lo=0):
    _store(y, _moe_down(act, w_down, ids, resid, expert_lo))


# ----------------------------------------------------------------------------- small ops
def embed_gather(out, table, ids):
    _store(out, table[ids.long().reshape(-1)].float())


def argmax_workspace(device):
    return torch.zeros(1, dtype=torch.int32)


def argmax(cand, logits, workspace, idx_base=0):
    i = int(torch.argmax(logits))                # torch returns the first maximum: lowest index
    cand[0] = logits[i]
    cand.view(torch.int32)[1] = i + idx_base


def _best(cand):
    c = cand.reshape(-1, 2)
    vals, idx = c[:, 0], c.view(torch.int32)[:, 1]
    best = 0
    for r in range(1, c.shape[0]):
        if vals[r] > vals[best] or (vals[r] == vals[best] and idx[r] < idx[best]):
            best = r
    return int(idx[best])


def greedy_select(tok_out, cand):
    tok_out[0] = _best(cand)


def greedy_advance(tok_out, state, log, cand):
    t = _best(cand)
    tok_out[0] = t
    k = int(state[2])
    if k < log.numel():
        log[k] = t
    state[0] += 1
    state[1] += 1
    state[2] = k + 1


# ----------------------------------------------------------------------------- fused all-reduce
# The peer-memory exchange is re-stated with torch.distributed: publish keeps this rank's share,
# consume sums the shares of all ranks.  What the test checks is the engine's numbering: every
# consume must name the all-reduce its producer published, in the same order on every rank.
_PUBLISHED = {}


def gemv_tp_publish(x, w, ctx, tp_out, resid=None, bias=None):
    y = torch.empty(w.shape[0])
    gemv(y, x, w, bias=bias, resid=resid)
    assert tp_out not in _PUBLISHED, f"all-reduce {tp_out} published twice"
    _PUBLISHED[tp_out] = y


def moe_decode_down_tp_publish(act, w_down, ids, ctx, tp_out, resid=None, expert_lo=0):
    assert tp_out not in _PUBLISHED, f"all-reduce {tp_out} published twice"
    _PUBLISHED[tp_out] = _moe_down(act, w_down, ids, resid, expert_lo)


def gemv_tp_consume(y, w, ctx, tp_in, x_out=None, norm_w=None, eps=0.0, epilogue=EPI_NONE):
    import torch.distributed as dist
    x = _PUBLISHED.pop(tp_in)                    # KeyError: consumed before it was published
    dist.all_reduce(x)
    if x_out is not None:
        _store(x_out, x)
    gemv(y, x, w, norm_w=norm_w, eps=eps, epilogue=epilogue)


def tp_advance(ctx, inc):
    assert not _PUBLISHED, f"all-reduces {sorted(_PUBLISHED)} were published but never consumed"


# ----------------------------------------------------------------------------- whole-step kernel
class _Plan:
    pass


def decode_layers_plan(wqkv, wo, wgu, wd, ln1, ln2, kv, qn, kn, h, tp_ctx=-1):
    p = _Plan()
    p.__dict__.update(locals())
    q_size = wo[0].shape[1]
    p.qkv, p.attn, p.act = torch.zeros(wqkv[0].shape[0]), torch.zeros(q_size), torch.zeros(wd[0].shape[1])
    return p


def decode_layers(plan, cos, sin, kv_len, workspace, n_q, n_kv, n_splits, scale, eps):
    """The five phases of every layer, as the persistent kernel orders them; with a link the two
    all-reduces of layer i carry the numbers 2 i and 2 i + 1 and the last one is left published."""
    p = plan
    tp = p.tp_ctx >= 0
    import torch.distributed as dist
    lead = not tp or dist.get_rank() == 0
    for i in range(len(p.wqkv)):
        if tp and i > 0:
            gemv_tp_consume(p.qkv, p.wqkv[i], p.tp_ctx, 2 * i - 1, x_out=p.h, norm_w=p.ln1[i], eps=eps)
        else:
            gemv(p.qkv, p.h, p.wqkv[i], norm_w=p.ln1[i], eps=eps)
        rope_flash_decode(p.attn, p.kv[i, 0], p.kv[i, 1], workspace, p.qkv, cos, sin, kv_len, n_q,
                          n_kv, n_splits, scale, eps=eps, qn_w=p.qn[i], kn_w=p.kn[i])
        if tp:
            gemv_tp_publish(p.attn, p.wo[i], p.tp_ctx, 2 * i, resid=p.h if lead else None)
            gemv_tp_consume(p.act, p.wgu[i], p.tp_ctx, 2 * i, x_out=p.h, norm_w=p.ln2[i], eps=eps,
                            epilogue=EPI_SWIGLU)
            gemv_tp_publish(p.act, p.wd[i], p.tp_ctx, 2 * i + 1, resid=p.h if lead else None)
        else:
            gemv(p.h, p.attn, p.wo[i], resid=p.h)
            gemv(p.act, p.h, p.wgu[i], norm_w=p.ln2[i], eps=eps, epilogue=EPI_SWIGLU)
            gemv(p.h, p.act, p.wd[i], resid=p.h)
