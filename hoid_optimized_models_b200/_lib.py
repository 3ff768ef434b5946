"""ctypes binding of libb200ops.so (the C ABI declared in include/b200ops.h).

There is no fallback: if the shared library is missing the import fails with
instructions to build it, and every non-zero return code raises.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# B200OPS_LIB points at another build of the same library (A/B runs of kernel variants)
LIB_PATH = os.environ.get("B200OPS_LIB") or os.path.join(HERE, "libb200ops.so")

BF16, F32 = 0, 1
FLAG_PDL = 1
EPI_NONE, EPI_SWIGLU, EPI_GELU, EPI_GEGLU = 0, 1, 2, 3

ERRORS = {
    -1: "B200_ERR_SHAPE (unsupported size / divisibility)",
    -2: "B200_ERR_ALIGN (pointer or leading dimension not 16-byte aligned)",
    -3: "B200_ERR_LAUNCH (CUDA launch error)",
    -4: "B200_ERR_ARG (null pointer / bad enum)",
    -5: "B200_ERR_TIMEOUT (bounded device-side wait expired)",
    -6: "B200_ERR_DRIVER (driver entry point unavailable)",
    -7: "B200_ERR_SCRATCH (request exceeds the library's fixed scratch array)",
    -8: "B200_ERR_NUMERIC (non-finite input where an index is derived from it)",
}

_p, _i, _f, _l = C.c_void_p, C.c_int, C.c_float, C.c_int64

# name -> (restype, argtypes); must list every symbol include/b200ops.h declares
SIGNATURES = {
    "b200_version": (_i, []),
    "b200_sm_count": (_i, []),
    "b200_set_tuning": (_i, [_i, _i]),
    "b200_gemv_bf16": (_i, [_p, _i, _p, _p, _i, _i, _i, _i, _p, _p, _f, _p, _p, _i, _i, _i, _p]),
    "b200_tp_buffer_bytes": (_l, [_i, _i]),
    "b200_tp_alloc": (_i, [_p, _p, _l]),
    "b200_tp_open": (_i, [_p, _p]),
    "b200_tp_create": (_i, [_p, _i, _i, _i]),
    "b200_tp_advance": (_i, [_i, _i, _i, _p]),
    "b200_gemv_bf16_tp": (_i, [_p, _p, _p, _i, _i, _i, _p, _f, _p, _p, _i, _i, _i, _i, _p, _p, _i, _p]),
    "b200_moe_decode_down_tp": (_i, [_p, _p, _p, _i, _i, _i, _i, _i, _p, _i, _i, _p, _i, _p]),
    "b200_decode_layers_plan_bytes": (_l, [_i]),
    "b200_decode_layers_sync_bytes": (_l, [_i, _i, _i, _i]),
    "b200_decode_layers_plan": (_i, [_p, _p, _i] + [_p] * 10 + [_p] + [_i] * 5),
    "b200_decode_layers": (_i, [_p, _i, _p, _p, _p, _p, _p, _i, _i, _i, _l, _l, _i, _i, _f, _f, _i,
                                _p, _i, _p]),
    "b200_add_rmsnorm": (_i, [_p, _p, _i, _p, _i, _p, _i, _p, _i, _i, _f, _i, _p]),
    "b200_add_layernorm": (_i, [_p, _p, _i, _p, _p, _p, _i, _p, _p, _i, _i, _f, _i, _p]),
    "b200_qk_rope_cache": (_i, [_p, _i, _p, _p, _p, _i, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i,
                                _f, _i, _p]),
    "b200_flash_decode_workspace_bytes": (_l, [_i, _i, _i, _i]),
    "b200_rope_flash_decode": (_i, [_p, _i, _p, _p, _p, _p, _p, _p, _p, _f, _p, _p, _i, _i, _i, _l, _l,
                                    _i, _i, _f, _i, _p]),
    "b200_flash_decode": (_i, [_p, _i, _p, _i, _p, _p, _p, _p, _i, _i, _i, _l, _l, _i, _f, _i, _p]),
    "b200_flash_decode_static_max_bytes": (_l, []),
    "b200_flash_decode_static": (_i, [_p, _i, _p, _i, _p, _p, _p, _i, _i, _i, _l, _l, _i, _f, _i, _p]),
    "b200_gemm_bf16": (_i, [_p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _p, _p, _i, _i, _p, _i, _p]),
    "b200_moe_grouped_gemm": (_i, [_p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _p, _i, _p]),
    "b200_moe_router": (_i, [_p, _p, _p, _i, _i, _i, _i, _i, _p, _i, _p]),
    "b200_moe_permute_workspace_bytes": (_l, [_i, _i]),
    "b200_moe_permute": (_i, [_p, _p, _p, _p, _i, _i, _p, _p, _i, _p]),
    "b200_moe_gather_rows": (_i, [_p, _p, _p, _i, _i, _i, _i, _p]),
    "b200_moe_combine": (_i, [_p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _p]),
    "b200_moe_decode_gate_up": (_i, [_p, _p, _i, _p, _f, _p, _p, _p, _i, _i, _i, _i, _i, _i, _p]),
    "b200_moe_decode_down": (_i, [_p, _i, _p, _p, _p, _i, _i, _i, _i, _i, _p, _i, _i, _p]),
    "b200_flash_prefill_tc": (_i, [_p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i] + [_l] * 12 + [_i, _f, _p, _i, _p]),
    "b200_embed_gather": (_i, [_p, _i, _p, _p, _i, _i, _i, _p]),
    "b200_cls_pool_l2": (_i, [_p, _p, _i, _l, _i, _f, _i, _p]),
    "b200_silu_mul": (_i, [_p, _p, _p, _l, _i, _p]),
    "b200_argmax_workspace_bytes": (_l, [_i]),
    "b200_argmax_f32": (_i, [_p, _p, _p, _i, _i, _p, _i, _p]),
    "b200_greedy_select": (_i, [_p, _p, _i, _p, _p, _i, _i, _p]),
}


class B200Error(RuntimeError):
    pass


def load(path: str = LIB_PATH) -> C.CDLL:
    if not os.path.exists(path):
        raise ImportError(
            f"{path} is missing: build it with `python -m hoid_optimized_models_b200.build` "
            "(needs nvcc); there is no CPU or PyTorch fallback for these ops")
    lib = C.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    return lib


_LIB = None
_NVTX = os.environ.get("B200OPS_NVTX", "0") == "1"
_NVTX_PROXY = None


class _NvtxProxy:
    """The loaded library with every entry point wrapped in an NVTX range named after it, so that
    a timeline (ncu --nvtx, or any NVTX consumer) attributes kernels to the C-ABI call that launched
    them.  Ranges cost nothing on the device; the Python wrapper costs about a microsecond per call,
    which is why it is opt-in (set_nvtx(True) or B200OPS_NVTX=1)."""

    def __init__(self, raw: C.CDLL):
        self._raw = raw
        self._wrapped = {}

    def __getattr__(self, name):
        fn = self._wrapped.get(name)
        if fn is None:
            raw_fn = getattr(self._raw, name)
            import torch

            def fn(*args, _raw_fn=raw_fn, _name=name):
                torch.cuda.nvtx.range_push(_name)
                try:
                    return _raw_fn(*args)
                finally:
                    torch.cuda.nvtx.range_pop()
            self._wrapped[name] = fn
        return fn


def set_nvtx(enabled: bool) -> None:
    """NVTX range per C-ABI call (off by default)."""
    global _NVTX
    _NVTX = bool(enabled)


def lib():
    global _LIB, _NVTX_PROXY
    if _LIB is None:
        _LIB = load()
    if _NVTX:
        if _NVTX_PROXY is None or _NVTX_PROXY._raw is not _LIB:
            _NVTX_PROXY = _NvtxProxy(_LIB)
        return _NVTX_PROXY
    return _LIB


def check(code: int, what: str) -> None:
    if code != 0:
        raise B200Error(f"{what} failed: {ERRORS.get(code, code)}")
