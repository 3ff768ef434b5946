"""torch custom ops `b200::<op>` over the C ABI.

Every op is out-parameter style (the caller owns all buffers, as in the
reference engines: models/llama31-8b/llama31_optimized.py:347-376), launches on
the current torch stream, allocates nothing and is safe inside
`torch.cuda.graph` capture.  The ops keep the reference's module boundaries
(norm, prepare_qkv, decode attention, GEMV, ...), see include/b200ops.h.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib
from ._lib import BF16, F32, FLAG_PDL, EPI_NONE, EPI_SWIGLU, EPI_GELU, EPI_GEGLU, check

Tensor = torch.Tensor

_PDL = False


def set_pdl(enabled: bool) -> None:
    """Enable programmatic dependent launch on every op launched afterwards."""
    global _PDL
    _PDL = bool(enabled)


def set_nvtx(enabled: bool) -> None:
    """Wrap every library call in an NVTX range named after its C entry point (off by default;
    also B200OPS_NVTX=1).  For timelines: `ncu --nvtx` attributes each kernel to its call."""
    _lib.set_nvtx(enabled)


def set_tuning(key: int, value: int) -> None:
    """Process-wide kernel tuning knob (the B200_TUNE_* keys of include/b200ops.h)."""
    check(_lib.lib().b200_set_tuning(key, value), "b200_set_tuning")


def _flags() -> int:
    return FLAG_PDL if _PDL else 0


def _dt(t: Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return BF16
    if t.dtype == torch.float32:
        return F32
    raise TypeError(f"unsupported dtype {t.dtype}")


def _ptr(t: Optional[Tensor]) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise RuntimeError("b200 ops take CUDA tensors only (there is no CPU path)")
    if not t.is_contiguous():
        raise RuntimeError("b200 ops take contiguous tensors")
    return t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _bf16(t: Optional[Tensor], name: str) -> None:
    if t is not None and t.dtype != torch.bfloat16:
        raise TypeError(f"{name} must be bfloat16")


# ----------------------------------------------------------------------------- GEMV
@torch.library.custom_op("b200::gemv", mutates_args=("y",))
def gemv(y: Tensor, x: Tensor, w: Tensor, norm_w: Optional[Tensor] = None, eps: float = 0.0,
         bias: Optional[Tensor] = None, resid: Optional[Tensor] = None,
         epilogue: int = EPI_NONE, norm_b: Optional[Tensor] = None) -> None:
    """y = W x with optional RMSNorm (norm_w) or LayerNorm (norm_w, norm_b) prologue, bias,
    residual and SwiGLU/GELU epilogue.  w is the HuggingFace [N, K] weight; x is [K] or [1, K]."""
    _bf16(w, "w"); _bf16(norm_w, "norm_w"); _bf16(norm_b, "norm_b"); _bf16(bias, "bias")
    N, K = w.shape
    if x.numel() != K:
        raise RuntimeError(f"x has {x.numel()} elements, expected {K}")
    n_out = N // 2 if epilogue == EPI_SWIGLU else N
    if y.numel() != n_out:
        raise RuntimeError(f"y has {y.numel()} elements, expected {n_out}")
    check(_lib.lib().b200_gemv_bf16(
        _ptr(x), _dt(x), _ptr(w), _ptr(y), _dt(y), K, N, w.stride(0),
        _ptr(norm_w), _ptr(norm_b), eps, _ptr(bias), _ptr(resid),
        _dt(resid) if resid is not None else 0, epilogue, _flags(), _stream()), "b200_gemv_bf16")


# ----------------------------------------------------------------------------- fused TP GEMV
# Plain functions (not custom ops): they write peer memory / read inboxes that torch does not
# know about.  All tensors are fp32 activations and bf16 weights.
def gemv_tp_publish(x: Tensor, w: Tensor, ctx: int, tp_out: int, resid: Optional[Tensor] = None,
                    bias: Optional[Tensor] = None) -> None:
    """This rank's share of all-reduce `tp_out`: (resid +) W x (+ bias) pushed to every rank."""
    N, K = w.shape
    check(_lib.lib().b200_gemv_bf16_tp(
        _ptr(x), _ptr(w), None, K, N, w.stride(0), None, 0.0, _ptr(bias), _ptr(resid), EPI_NONE,
        ctx, -1, tp_out, None, status_word(x.device).data_ptr(), _flags(), _stream()),
        "b200_gemv_bf16_tp")


def gemv_tp_consume(y: Tensor, w: Tensor, ctx: int, tp_in: int, x_out: Optional[Tensor] = None,
                    norm_w: Optional[Tensor] = None, eps: float = 0.0,
                    epilogue: int = EPI_NONE) -> None:
    """y = W (rmsnorm of) x with x = the sum over ranks of all-reduce `tp_in`; x_out gets x."""
    N, K = w.shape
    check(_lib.lib().b200_gemv_bf16_tp(
        None, _ptr(w), _ptr(y), K, N, w.stride(0), _ptr(norm_w), eps, None, None, epilogue,
        ctx, tp_in, -1, _ptr(x_out), status_word(y.device).data_ptr(), _flags(), _stream()),
        "b200_gemv_bf16_tp")


def moe_decode_down_tp_publish(act: Tensor, w_down: Tensor, ids: Tensor, ctx: int, tp_out: int,
                               resid: Optional[Tensor] = None, expert_lo: int = 0) -> None:
    """This rank's experts' share of the layer output (+ resid) as all-reduce `tp_out`."""
    _bf16(w_down, "w_down")
    E, H, I = w_down.shape
    check(_lib.lib().b200_moe_decode_down_tp(
        _ptr(act), _ptr(w_down), _ptr(ids), ids.numel(), I, H, expert_lo, E, _ptr(resid), ctx,
        tp_out, status_word(act.device).data_ptr(), _flags(), _stream()),
        "b200_moe_decode_down_tp")


def tp_advance(ctx: int, inc: int) -> None:
    check(_lib.lib().b200_tp_advance(ctx, inc, _flags(), _stream()), "b200_tp_advance")


# ----------------------------------------------------------------------------- whole-step kernel
class DecodePlan:
    """Phase table of b200_decode_layers on the device, its synchronisation workspace (launch
    counter + the tagged vectors the phases hand to one another), and references to every tensor
    the table points at (so that none of them is freed while the plan lives)."""

    def __init__(self, table: Tensor, sync: Tensor, n_layers: int, tp_ctx: int, keep: tuple):
        self.table, self.sync, self.n_layers, self.tp_ctx, self.keep = table, sync, n_layers, tp_ctx, keep


def decode_layers_plan(wqkv, wo, wgu, wd, ln1, ln2, kv: Tensor, qn, kn, h: Tensor,
                       tp_ctx: int = -1) -> DecodePlan:
    """Set-up of the persistent decode kernel: per-layer weight lists (packed q|k|v, o_proj,
    interleaved gate|up, down; RMSNorm weights; QK-norm weights or lists of None), the KV cache
    [layers, 2, n_kv, max_seq, hd] and the fp32 residual-stream vector of the step."""
    import ctypes as C
    L = len(wqkv)
    for t in (*wqkv, *wo, *wgu, *wd, *ln1, *ln2):
        _bf16(t, "weights")
    if h.dtype != torch.float32:
        raise TypeError("the residual stream must be float32")
    _bf16(kv, "kv")

    def arr(ts):
        return (C.c_void_p * L)(*[_ptr(t) for t in ts])

    has_qk = qn[0] is not None
    lib = _lib.lib()
    dev = h.device
    H = h.numel()
    q_size = wo[0].shape[1]
    kv_size = (wqkv[0].shape[0] - q_size) // 2
    inter = wd[0].shape[1]
    table = torch.zeros(lib.b200_decode_layers_plan_bytes(L), dtype=torch.uint8, device=dev)
    sync = torch.zeros(lib.b200_decode_layers_sync_bytes(H, q_size, kv_size, inter) // 8,
                       dtype=torch.int64, device=dev)
    check(lib.b200_decode_layers_plan(
        _ptr(table), _ptr(sync), L, arr(wqkv), arr(wo), arr(wgu), arr(wd), arr(ln1), arr(ln2),
        arr([kv[i, 0] for i in range(L)]), arr([kv[i, 1] for i in range(L)]),
        arr(qn) if has_qk else None, arr(kn) if has_qk else None,
        _ptr(h), H, q_size, kv_size, inter, tp_ctx), "b200_decode_layers_plan")
    return DecodePlan(table, sync, L, tp_ctx, (wqkv, wo, wgu, wd, ln1, ln2, kv, qn, kn, h))


def decode_layers(plan: DecodePlan, cos: Tensor, sin: Tensor, kv_len: Tensor, workspace: Tensor,
                  n_q: int, n_kv: int, n_splits: int, scale: float, eps: float) -> None:
    """Every layer of one decode step in one launch: h (the embedded token) -> h after the last
    layer, the new position's k / v rows appended to the cache.  With a tensor-parallel plan h is
    not written: the last all-reduce (number 2 * layers - 1) is left for `gemv_tp_consume`."""
    kv = plan.keep[6]
    hd = kv.shape[-1]
    check(_lib.lib().b200_decode_layers(
        _ptr(plan.table), plan.n_layers, _ptr(cos), _ptr(sin), _ptr(kv_len),
        _ptr(workspace), _ptr(plan.sync), n_q, n_kv, hd, kv.stride(-3), kv.stride(-2),
        kv.shape[-2], n_splits, scale, eps, plan.tp_ctx, status_word(kv.device).data_ptr(),
        _flags(), _stream()), "b200_decode_layers")


def reset_decode_plan(plan: DecodePlan) -> None:
    """After a B200_ERR_TIMEOUT nothing needs repair (every launch tags its vectors with its own
    number); kept so that callers have one place to put recovery."""


# ----------------------------------------------------------------------------- norms
def _rmsnorm_call(resid_out, norm_out, a, b, w, eps):
    _bf16(w, "w")
    N = w.numel()
    rows = a.numel() // N
    if resid_out is not None and resid_out.dtype != a.dtype:
        raise TypeError("resid_out and a (the residual stream) must share a dtype")
    check(_lib.lib().b200_add_rmsnorm(
        _ptr(resid_out), _ptr(norm_out), _dt(norm_out), _ptr(a), _dt(a), _ptr(b),
        _dt(b) if b is not None else _dt(a), _ptr(w), rows, N, eps, _flags(), _stream()),
        "b200_add_rmsnorm")


# Mutated arguments of a custom op are always leading, required, positional parameters.
@torch.library.custom_op("b200::rmsnorm", mutates_args=("norm_out",))
def rmsnorm(norm_out: Tensor, a: Tensor, w: Tensor, eps: float) -> None:
    """norm_out = rmsnorm(a) * w."""
    _rmsnorm_call(None, norm_out, a, None, w, eps)


@torch.library.custom_op("b200::add_rmsnorm", mutates_args=("norm_out", "resid_out"))
def add_rmsnorm(norm_out: Tensor, resid_out: Tensor, a: Tensor, b: Tensor, w: Tensor,
                eps: float) -> None:
    """resid_out = a + b (rounded to its dtype); norm_out = rmsnorm(resid_out) * w.
    resid_out may alias a; a / resid_out may be fp32 with b and norm_out bf16."""
    _rmsnorm_call(resid_out, norm_out, a, b, w, eps)


def _layernorm_call(resid_out, norm_out, x, gamma, beta, eps, bias, resid):
    _bf16(gamma, "gamma"); _bf16(beta, "beta"); _bf16(bias, "bias")
    N = gamma.numel()
    rows = x.numel() // N
    if resid is not None and resid.dtype != x.dtype:
        raise TypeError("x and resid must share a dtype")
    check(_lib.lib().b200_add_layernorm(
        _ptr(resid_out), _ptr(norm_out), _dt(norm_out), _ptr(x), _ptr(bias), _ptr(resid), _dt(x),
        _ptr(gamma), _ptr(beta), rows, N, eps, _flags(), _stream()), "b200_add_layernorm")


@torch.library.custom_op("b200::layernorm", mutates_args=("norm_out",))
def layernorm(norm_out: Tensor, x: Tensor, gamma: Tensor, beta: Tensor, eps: float,
              bias: Optional[Tensor] = None, resid: Optional[Tensor] = None) -> None:
    """norm_out = LayerNorm(x (+ bias) (+ resid))."""
    _layernorm_call(None, norm_out, x, gamma, beta, eps, bias, resid)


@torch.library.custom_op("b200::add_layernorm", mutates_args=("norm_out", "resid_out"))
def add_layernorm(norm_out: Tensor, resid_out: Tensor, x: Tensor, gamma: Tensor, beta: Tensor,
                  eps: float, bias: Optional[Tensor] = None,
                  resid: Optional[Tensor] = None) -> None:
    """resid_out = x (+ bias) (+ resid); norm_out = LayerNorm(resid_out)."""
    _layernorm_call(resid_out, norm_out, x, gamma, beta, eps, bias, resid)


# ----------------------------------------------------------------------------- rope + cache
@torch.library.custom_op("b200::qk_rope_cache", mutates_args=("q_out", "kcache", "vcache"))
def qk_rope_cache(q_out: Tensor, kcache: Tensor, vcache: Tensor, qkv: Tensor, cos: Tensor,
                  sin: Tensor, pos: Tensor, n_q: int, n_kv: int, eps: float = 0.0,
                  qn_w: Optional[Tensor] = None, kn_w: Optional[Tensor] = None) -> None:
    """(QK-RMSNorm +) RoPE on the packed q|k|v rows; q -> q_out, k/v -> cache rows pos + t.
    kcache / vcache are [n_kv, max_seq, hd] bf16; pos is a device int32 scalar tensor."""
    _bf16(kcache, "kcache"); _bf16(vcache, "vcache"); _bf16(qn_w, "qn_w"); _bf16(kn_w, "kn_w")
    hd = kcache.shape[-1]
    max_seq = kcache.shape[-2]
    s = qkv.numel() // ((n_q + 2 * n_kv) * hd)
    if pos.dtype != torch.int32 or cos.dtype != torch.float32 or sin.dtype != torch.float32:
        raise TypeError("pos must be int32 and cos/sin float32")
    if cos.shape[0] < max_seq or cos.shape[-1] != hd // 2:
        raise RuntimeError("cos/sin tables must be [>= max_seq, hd/2]")
    check(_lib.lib().b200_qk_rope_cache(
        _ptr(q_out), _dt(q_out), _ptr(kcache), _ptr(vcache), _ptr(qkv), _dt(qkv),
        _ptr(qn_w), _ptr(kn_w), _ptr(cos), _ptr(sin), _ptr(pos), s, n_q, n_kv, hd, max_seq,
        eps, _flags(), _stream()), "b200_qk_rope_cache")


# ----------------------------------------------------------------------------- flash decode
def flash_decode_workspace(n_q: int, n_kv: int, hd: int, n_splits: int, device) -> Tensor:
    """Zero-initialised scratch for `flash_decode` (arrival counters + split records)."""
    nbytes = _lib.lib().b200_flash_decode_workspace_bytes(n_q, n_kv, hd, n_splits)
    return torch.zeros((nbytes + 3) // 4, dtype=torch.float32, device=device)


@torch.library.custom_op("b200::flash_decode", mutates_args=("out", "workspace"))
def flash_decode(out: Tensor, q: Tensor, kcache: Tensor, vcache: Tensor, kv_len: Tensor,
                 workspace: Tensor, n_q: int, n_kv: int, n_splits: int, scale: float,
                 kv_head_stride: int = -1, kv_row_stride: int = -1) -> None:
    """out[n_q, hd] = softmax(q K^T * scale) V over the first kv_len cache rows of each kv head.
    Default strides describe a contiguous [n_kv, max_seq, hd] cache."""
    _bf16(kcache, "kcache"); _bf16(vcache, "vcache")
    hd = q.numel() // n_q
    if kv_row_stride < 0:
        kv_row_stride = kcache.stride(-2)
    if kv_head_stride < 0:
        kv_head_stride = kcache.stride(-3) if kcache.dim() >= 3 else hd
    if kv_len.dtype != torch.int32:
        raise TypeError("kv_len must be int32")
    need = _lib.lib().b200_flash_decode_workspace_bytes(n_q, n_kv, hd, n_splits)
    if workspace.numel() * workspace.element_size() < need:
        raise RuntimeError("flash_decode workspace too small")
    check(_lib.lib().b200_flash_decode(
        _ptr(out), _dt(out), _ptr(q), _dt(q), _ptr(kcache), _ptr(vcache), _ptr(kv_len),
        _ptr(workspace), n_q, n_kv, hd, kv_head_stride, kv_row_stride, n_splits, scale,
        _flags(), _stream()), "b200_flash_decode")


@torch.library.custom_op("b200::rope_flash_decode",
                         mutates_args=("out", "kcache", "vcache", "workspace"))
def rope_flash_decode(out: Tensor, kcache: Tensor, vcache: Tensor, workspace: Tensor, qkv: Tensor,
                      cos: Tensor, sin: Tensor, kv_len: Tensor, n_q: int, n_kv: int,
                      n_splits: int, scale: float, eps: float = 0.0,
                      qn_w: Optional[Tensor] = None, kn_w: Optional[Tensor] = None) -> None:
    """qk_rope_cache + flash_decode in one launch: the packed fp32 q|k|v row of position
    kv_len - 1 is normalised / rotated in the attention kernel, its k / v row appended to the
    [n_kv, max_seq, hd] bf16 cache, and out[n_q, hd] attends to rows [0, kv_len)."""
    _bf16(kcache, "kcache"); _bf16(vcache, "vcache"); _bf16(qn_w, "qn_w"); _bf16(kn_w, "kn_w")
    if qkv.dtype != torch.float32 or cos.dtype != torch.float32 or sin.dtype != torch.float32:
        raise TypeError("qkv, cos and sin must be float32")
    if kv_len.dtype != torch.int32:
        raise TypeError("kv_len must be int32")
    hd = qkv.numel() // (n_q + 2 * n_kv)
    max_seq = kcache.shape[-2]
    need = _lib.lib().b200_flash_decode_workspace_bytes(n_q, n_kv, hd, n_splits)
    if workspace.numel() * workspace.element_size() < need:
        raise RuntimeError("flash_decode workspace too small")
    check(_lib.lib().b200_rope_flash_decode(
        _ptr(out), _dt(out), _ptr(qkv), _ptr(kcache), _ptr(vcache), _ptr(cos), _ptr(sin),
        _ptr(qn_w), _ptr(kn_w), eps, _ptr(kv_len), _ptr(workspace), n_q, n_kv, hd,
        kcache.stride(-3), kcache.stride(-2), max_seq, n_splits, scale, _flags(), _stream()),
        "b200_rope_flash_decode")


# ----------------------------------------------------------------------------- GEMM
_STATUS = {}


def status_word(device) -> Tensor:
    """Device int32 the kernels report through: B200_ERR_TIMEOUT when a bounded wait expired,
    B200_ERR_NUMERIC / B200_ERR_ARG when the router or the expert sort met a bad input."""
    key = torch.device(device).index or 0
    if key not in _STATUS:
        _STATUS[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _STATUS[key]


def check_status(device) -> None:
    """Synchronising check of the status word: the engines call it wherever they synchronise with
    the device anyway (after a prefill, when the generated tokens are read back)."""
    v = int(status_word(device).item())
    if v != 0:
        status_word(device).zero_()
        check(v, "device status word")


@torch.library.custom_op("b200::gemm", mutates_args=("y",))
def gemm(y: Tensor, x: Tensor, w: Tensor, bias: Optional[Tensor] = None,
         resid: Optional[Tensor] = None, epilogue: int = EPI_NONE) -> None:
    """y[M, N] = x[M, K] w[N, K]^T (+ bias) (+ resid) with optional SwiGLU / GELU epilogue, or
    EPI_GEGLU: w is a stock [2 O, K] GEGLU projection (value half first) and
    y[M, O] = (x Wv^T + bv) * gelu(x Wg^T + bg)."""
    for t, n in ((x, "x"), (w, "w"), (bias, "bias"), (resid, "resid")):
        _bf16(t, n)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise RuntimeError("x / w inner dimensions differ")
    n_out = N // 2 if epilogue in (EPI_SWIGLU, EPI_GEGLU) else N
    if y.shape[0] != M or y.shape[1] != n_out:
        raise RuntimeError(f"y must be [{M}, {n_out}]")
    if x.stride(1) != 1 or w.stride(1) != 1 or y.stride(1) != 1:
        raise RuntimeError("innermost dimensions must be contiguous")
    check(_lib.lib().b200_gemm_bf16(
        x.data_ptr(), w.data_ptr(), y.data_ptr(), _dt(y), M, N, K, x.stride(0), w.stride(0), y.stride(0),
        _ptr(bias), resid.data_ptr() if resid is not None else None,
        resid.stride(0) if resid is not None else 0, epilogue,
        status_word(x.device).data_ptr(), _flags(), _stream()), "b200_gemm_bf16")


@torch.library.custom_op("b200::moe_grouped_gemm", mutates_args=("y",))
def moe_grouped_gemm(y: Tensor, x: Tensor, w: Tensor, offsets: Tensor,
                     epilogue: int = EPI_NONE) -> None:
    """y[r] = x[r] w[e(r)]^T for rows sorted by expert; offsets is int32 [E + 1]; w is [E, N, K]."""
    for t, n in ((y, "y"), (x, "x"), (w, "w")):
        _bf16(t, n)
    E, N, K = w.shape
    rows = x.shape[0]
    if offsets.dtype != torch.int32 or offsets.numel() != E + 1:
        raise TypeError("offsets must be int32 [E + 1]")
    check(_lib.lib().b200_moe_grouped_gemm(
        _ptr(x), _ptr(w), _ptr(y), _ptr(offsets), E, rows, N, K, x.stride(0), y.stride(0),
        epilogue, status_word(x.device).data_ptr(), _flags(), _stream()), "b200_moe_grouped_gemm")


# ----------------------------------------------------------------------------- MoE
@torch.library.custom_op("b200::moe_router", mutates_args=("ids", "wts"))
def moe_router(ids: Tensor, wts: Tensor, logits: Tensor, round_bf16: bool = False) -> None:
    """ids int32 [s, k], wts fp32 [s, k] = top-k of softmax(logits [s, E]), renormalised."""
    if ids.dtype != torch.int32 or wts.dtype != torch.float32:
        raise TypeError("ids must be int32 and wts float32")
    s, E = logits.shape[-2] if logits.dim() > 1 else 1, logits.shape[-1]
    k = ids.numel() // s
    check(_lib.lib().b200_moe_router(_ptr(ids), _ptr(wts), _ptr(logits), _dt(logits), s, E, k,
                                     1 if round_bf16 else 0, status_word(ids.device).data_ptr(),
                                     _flags(), _stream()), "b200_moe_router")


def moe_permute_workspace(pairs: int, E: int, device) -> Tensor:
    n = _lib.lib().b200_moe_permute_workspace_bytes(pairs, E)
    return torch.zeros((n + 3) // 4, dtype=torch.int32, device=device)


@torch.library.custom_op("b200::moe_permute", mutates_args=("order", "inv", "offsets", "workspace"))
def moe_permute(order: Tensor, inv: Tensor, offsets: Tensor, workspace: Tensor, ids: Tensor) -> None:
    """Stable expert-major sort of the flattened (token, slot) pairs; offsets is int32 [E + 1]."""
    for t in (order, inv, offsets, ids):
        if t.dtype != torch.int32:
            raise TypeError("moe_permute works on int32 tensors")
    check(_lib.lib().b200_moe_permute(_ptr(order), _ptr(inv), _ptr(offsets), _ptr(ids), ids.numel(),
                                      offsets.numel() - 1, _ptr(workspace),
                                      status_word(ids.device).data_ptr(), _flags(), _stream()),
          "b200_moe_permute")


@torch.library.custom_op("b200::moe_gather_rows", mutates_args=("xg",))
def moe_gather_rows(xg: Tensor, x: Tensor, order: Tensor, top_k: int) -> None:
    _bf16(xg, "xg"); _bf16(x, "x")
    check(_lib.lib().b200_moe_gather_rows(_ptr(xg), _ptr(x), _ptr(order), order.numel(), top_k,
                                          x.shape[-1], _flags(), _stream()), "b200_moe_gather_rows")


@torch.library.custom_op("b200::moe_combine", mutates_args=("out",))
def moe_combine(out: Tensor, y: Tensor, inv: Tensor, wts: Tensor,
                resid: Optional[Tensor] = None, ids: Optional[Tensor] = None,
                expert_lo: int = 0, n_local: int = 0) -> None:
    """out[t] = (resid[t] +) sum_slot wts[t, slot] * y[inv[t, slot]]; out may alias resid.
    With ids, only pairs routed to experts [expert_lo, expert_lo + n_local) are summed."""
    _bf16(out, "out"); _bf16(y, "y"); _bf16(resid, "resid")
    tokens, top_k = wts.shape
    check(_lib.lib().b200_moe_combine(_ptr(out), _ptr(y), _ptr(inv), _ptr(wts), _ptr(resid),
                                      _ptr(ids), expert_lo, n_local, tokens, top_k, y.shape[-1], _flags(), _stream()), "b200_moe_combine")


@torch.library.custom_op("b200::moe_decode_gate_up", mutates_args=("act",))
def moe_decode_gate_up(act: Tensor, x: Tensor, w_gu: Tensor, ids: Tensor, wts: Tensor,
                       norm_w: Optional[Tensor] = None, eps: float = 0.0,
                       expert_lo: int = 0) -> None:
    """act[slot, j] = wts[slot] * silu(gate_j) * up_j for the experts ids[slot]; w_gu is
    [E, 2I, H] with interleaved gate/up rows."""
    _bf16(w_gu, "w_gu"); _bf16(norm_w, "norm_w")
    E, two_i, H = w_gu.shape
    if act.dtype != torch.float32:
        raise TypeError("act must be float32")
    check(_lib.lib().b200_moe_decode_gate_up(
        _ptr(act), _ptr(x), _dt(x), _ptr(norm_w), eps, _ptr(w_gu), _ptr(ids), _ptr(wts),
        ids.numel(), two_i // 2, H, expert_lo, E, _flags(), _stream()), "b200_moe_decode_gate_up")


@torch.library.custom_op("b200::moe_decode_down", mutates_args=("y",))
def moe_decode_down(y: Tensor, act: Tensor, w_down: Tensor, ids: Tensor,
                    resid: Optional[Tensor] = None, expert_lo: int = 0) -> None:
    """y[d] = (resid[d] +) sum_slot w_down[ids[slot]][d] . act[slot]; w_down is [E, H, I]."""
    _bf16(w_down, "w_down")
    E, H, I = w_down.shape
    check(_lib.lib().b200_moe_decode_down(
        _ptr(y), _dt(y), _ptr(act), _ptr(w_down), _ptr(ids), ids.numel(), I, H, expert_lo, E,
        _ptr(resid),
        _dt(resid) if resid is not None else 0, _flags(), _stream()), "b200_moe_decode_down")


# ----------------------------------------------------------------------------- flash prefill
@torch.library.custom_op("b200::flash_prefill", mutates_args=("out",))
def flash_prefill(out: Tensor, q: Tensor, k: Tensor, v: Tensor, kv_len: int, causal: bool,
                  scale: float, q_pos0: int = 0) -> None:
    """Flash attention over strided views (persistent tcgen05 / TMEM kernel).

    q / out: [B, S, n_q, hd] views; k / v: [B, n_kv, L, hd] views (any strides with a
    contiguous last dimension), attending to the first kv_len of L keys.  A decode cache
    [n_kv, max_seq, hd] is passed as cache.unsqueeze(0).  Causal: query row i sees keys up to
    q_pos0 + i.  hd is 64 or 128, q_pos0 >= 0, kv_len >= 1, scale > 0."""
    for t, n in ((out, "out"), (q, "q"), (k, "k"), (v, "v")):
        _bf16(t, n)
        if t.stride(-1) != 1:
            raise RuntimeError("last dimension must be contiguous")
    B, S, n_q, hd = q.shape
    n_kv = k.shape[1]
    check(_lib.lib().b200_flash_prefill_tc(
        out.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), B, S, kv_len, q_pos0, n_q,
        n_kv, hd, q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(2), k.stride(1),
        v.stride(0), v.stride(2), v.stride(1), out.stride(0), out.stride(1), out.stride(2),
        1 if causal else 0, scale, status_word(q.device).data_ptr(), _flags(), _stream()),
        "b200_flash_prefill_tc")


# ----------------------------------------------------------------------------- small ops
@torch.library.custom_op("b200::embed_gather", mutates_args=("out",))
def embed_gather(out: Tensor, table: Tensor, ids: Tensor) -> None:
    _bf16(table, "table")
    if ids.dtype != torch.int32:
        raise TypeError("ids must be int32")
    check(_lib.lib().b200_embed_gather(_ptr(out), _dt(out), _ptr(table), _ptr(ids), ids.numel(),
                                       table.shape[1], _flags(), _stream()), "b200_embed_gather")


@torch.library.custom_op("b200::cls_pool_l2", mutates_args=("out",))
def cls_pool_l2(out: Tensor, x: Tensor, seq_len: int, eps: float = 1e-12) -> None:
    """out[b] = L2-normalised first token of sequence b; x is bf16 [batch * seq_len, H]."""
    _bf16(x, "x")
    H = x.shape[-1]
    if out.dtype != torch.float32:
        raise TypeError("out must be float32")
    check(_lib.lib().b200_cls_pool_l2(_ptr(out), _ptr(x), out.shape[0], seq_len * H, H, eps,
                                      _flags(), _stream()), "b200_cls_pool_l2")


@torch.library.custom_op("b200::silu_mul", mutates_args=("out",))
def silu_mul(out: Tensor, gate: Tensor, up: Tensor) -> None:
    _bf16(out, "out"); _bf16(gate, "gate"); _bf16(up, "up")
    check(_lib.lib().b200_silu_mul(_ptr(out), _ptr(gate), _ptr(up), gate.numel(), _flags(),
                                   _stream()), "b200_silu_mul")


def argmax_workspace(device) -> Tensor:
    nbytes = _lib.lib().b200_argmax_workspace_bytes(0)
    return torch.zeros((nbytes + 3) // 4, dtype=torch.int32, device=device)


@torch.library.custom_op("b200::argmax", mutates_args=("cand", "workspace"))
def argmax(cand: Tensor, logits: Tensor, workspace: Tensor, idx_base: int = 0) -> None:
    """cand (float32 [2]) = {max logit, bit pattern of int32 argmax + idx_base}; lowest index
    wins ties.  `cand.view(torch.int32)[1]` is the token id."""
    if logits.dtype != torch.float32 or cand.dtype != torch.float32 or cand.numel() != 2:
        raise TypeError("argmax takes float32 logits and a float32 [2] candidate record")
    base = _ptr(cand)
    check(_lib.lib().b200_argmax_f32(base + 4, base, _ptr(logits), logits.numel(), idx_base,
                                     _ptr(workspace), _flags(), _stream()), "b200_argmax_f32")


def _greedy_call(tok_out, cand, state, log):
    if tok_out.dtype != torch.int32 or cand.dtype != torch.float32:
        raise TypeError("greedy_select takes an int32 token and float32 candidates")
    check(_lib.lib().b200_greedy_select(_ptr(tok_out), _ptr(cand), cand.numel() // 2, _ptr(state),
                                        _ptr(log), log.numel() if log is not None else 0,
                                        _flags(), _stream()), "b200_greedy_select")


@torch.library.custom_op("b200::greedy_select", mutates_args=("tok_out",))
def greedy_select(tok_out: Tensor, cand: Tensor) -> None:
    """tok_out[0] = index of the best of the candidate records in cand (float32 [n, 2])."""
    _greedy_call(tok_out, cand, None, None)


@torch.library.custom_op("b200::greedy_advance", mutates_args=("tok_out", "state", "log"))
def greedy_advance(tok_out: Tensor, state: Tensor, log: Tensor, cand: Tensor) -> None:
    """greedy_select, then log[state[2]] = token and state = {position, kv_len, generated}
    (int32 [3+]) advances by one: the next graph replay continues without the host."""
    _greedy_call(tok_out, cand, state, log)
