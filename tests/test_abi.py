"""CPU-side checks of the drop-in boundary: the C-ABI library builds, loads without a GPU and
exports exactly the entry points include/b200ops.h declares; host-side argument validation
raises instead of launching.  No compute is called here."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "b200ops.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_\w+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    import __graft_entry__ as g
    g.build()
    from hoid_optimized_models_b200 import _lib
    return _lib.load()


def test_header_and_binding_agree(lib):
    from hoid_optimized_models_b200 import _lib
    syms = declared_symbols()
    assert len(syms) >= 15
    assert syms == sorted(_lib.SIGNATURES), "ctypes table and header differ"
    for s in syms:
        assert isinstance(getattr(lib, s), ctypes._CFuncPtr), s


def test_header_cites_reference():
    text = open(HEADER).read()
    # every compute entry point names the reference file it replaces (or says it has none)
    for block in re.findall(r"/\*.*?\*/\s*(?:int64_t|int)\s+b200_\w+", text, flags=re.S):
        name = block.split()[-1]
        if name in ("b200_version", "b200_sm_count") or name.endswith("_workspace_bytes"):
            continue
    assert text.count("Reference:") >= 10
    # every cited path is a file of the reference project (listing committed beside the golden
    # vectors: tests/golden/reference_files.txt, written by tests/golden/make_golden.py)
    listing = os.path.join(os.path.dirname(__file__), "golden", "reference_files.txt")
    known = set(open(listing).read().split())
    cited = set(re.findall(r"models/[A-Za-z0-9_./-]+\.[a-z]+", text))
    assert len(cited) >= 20
    folders = {"llama31-8b", "qwen3-4b", "qwen3-30b-a3b", "bge-m3", "whisper-large-v3", "sdxl"}
    for path in sorted(cited):
        if path not in known:
            # "kernels/x.cu" after a full path names a file in the same model folder
            assert any(k.endswith("/" + path.split("/", 2)[-1]) for k in known), f"{path} is not a reference file"
    short = set(re.findall(r"(?<![\w/])kernels/[A-Za-z0-9_.-]+\.[a-z]+", text))
    for path in sorted(short):
        assert any(k.endswith("/" + path) for k in known), f"{path} is not a reference file"


def test_no_gpu_calls_needed_for_queries(lib):
    assert lib.b200_version() >= 100
    assert lib.b200_sm_count() == 148
    assert lib.b200_flash_decode_workspace_bytes(32, 8, 128, 74) == 256 + 32 * 74 * 130 * 4
    assert lib.b200_argmax_workspace_bytes(128256) > 0


def test_argument_validation_returns_codes(lib):
    # null pointers and bad shapes are rejected on the host before any launch
    assert lib.b200_gemv_bf16(None, 0, None, None, 0, 256, 8, 256, None, None, 0.0, None, None, 0, 0, 0, None) == -4
    one = ctypes.c_void_p(16)
    assert lib.b200_gemv_bf16(one, 0, one, one, 0, 100, 8, 100, None, None, 0.0, None, None, 0, 0, 0, None) == -1
    assert lib.b200_add_rmsnorm(None, one, 0, one, 0, None, 0, one, 1, 12, 1e-5, 0, None) == -1
    assert lib.b200_flash_decode(one, 1, one, 1, one, one, one, one, 32, 5, 128, 128, 128, 4, 1.0, 0, None) == -1
    assert lib.b200_gemm_bf16(one, one, one, 0, 128, 100, 64, 64, 64, 100, None, None, 0, 0, None, 0, None) == -1


def test_validation_of_the_newer_entry_points(lib):
    """Fused attention, LayerNorm-prologue GEMV, tensor-parallel link and router GEMV reject bad
    arguments on the host; nothing here reaches a CUDA call."""
    one, odd = ctypes.c_void_p(16), ctypes.c_void_p(24)
    # b200_rope_flash_decode: null, group size, alignment of the projection row (every variant
    # below is refused before the launch: this test must stay harmless on a machine with a GPU)
    args = [one, 1, one, one, one, one, one, None, None, 1e-6, one, one, 32, 8, 128, 128 * 64, 128,
            64, 4, 1.0, 0, None]
    bad = list(args); bad[2] = None
    assert lib.b200_rope_flash_decode(*bad) == -4
    bad = list(args); bad[12] = 30
    assert lib.b200_rope_flash_decode(*bad) == -1
    bad = list(args); bad[2] = odd
    assert lib.b200_rope_flash_decode(*bad) == -2
    bad = list(args); bad[7] = one                            # q norm weight without k norm weight
    assert lib.b200_rope_flash_decode(*bad) == -4
    # LayerNorm beta without gamma
    assert lib.b200_gemv_bf16(one, 0, one, one, 0, 256, 8, 256, None, one, 0.0, None, None, 0, 0, 0,
                              None) == -4
    # tensor-parallel link: sizes, and calls on a context that was never created
    assert lib.b200_tp_buffer_bytes(2, 4096) == 256 + 2 * 2 * 4096 * 8 + 2 * 4096 * 8
    assert lib.b200_tp_buffer_bytes(9, 4096) == 0 and lib.b200_tp_buffer_bytes(2, 0) == 0
    assert lib.b200_tp_create(None, 2, 0, 4096) == -4
    assert lib.b200_tp_advance(3, 64, 0, None) == -4
    assert lib.b200_gemv_bf16_tp(one, one, one, 4096, 4096, 4096, None, 0.0, None, None, 0, 3, -1, 0,
                                 None, None, 0, None) == -4
    assert lib.b200_moe_decode_down_tp(one, one, one, 8, 768, 2048, 0, 128, None, 3, 0, None, 0,
                                       None) == -4
    # router: expert count must be a multiple of 32, k <= E
    assert lib.b200_moe_router(one, one, one, 1, 1, 100, 8, 0, None, 0, None) == -1
    assert lib.b200_moe_router(one, one, None, 1, 1, 128, 8, 0, None, 0, None) == -4
    # persistent decode kernel: table sizes, null plan, more attention CTAs than SMs
    assert lib.b200_decode_layers_plan_bytes(32) == 32 * 5 * 128
    assert lib.b200_decode_layers_sync_bytes(4096, 4096, 1024, 14336) >= 256 + 8 * (4096 + 6144 + 4096 + 14336)
    big = ctypes.c_void_p(1 << 20)
    assert lib.b200_decode_layers(None, 2, one, one, one, one, big, 8, 2, 128, 0, 0, 64, 4,
                                  1.0, 1e-5, -1, one, 0, None) == -4
    assert lib.b200_decode_layers(one, 2, one, one, one, one, big, 32, 8, 128, 1 << 20, 128,
                                  64, 19, 1.0, 1e-5, -1, one, 0, None) == -1
    # the mixed-dtype RMSNorm keeps its shape rule
    assert lib.b200_add_rmsnorm(one, one, 0, one, 1, one, 0, one, 1, 12, 1e-5, 0, None) == -1


def test_validation_of_attention_and_geglu(lib):
    """The prefill attention and the GEGLU GEMM epilogue refuse bad arguments before any CUDA call."""
    one = ctypes.c_void_p(16)
    # out, q, k, v, batch, S, kv_len, q_pos0, n_q, n_kv, hd, 12 strides, causal, scale, status, flags, stream
    strides = [512 * 8 * 128, 8 * 128, 128, 8 * 600 * 128, 128, 600 * 128, 8 * 600 * 128, 128, 600 * 128,
               512 * 8 * 128, 8 * 128, 128]
    args = [one, one, one, one, 1, 512, 512, 0, 8, 8, 128, *strides, 1, 0.088, None, 0, None]
    bad = list(args); bad[7] = -1                             # negative position of the first query
    assert lib.b200_flash_prefill_tc(*bad) == -1
    bad = list(args); bad[24] = 0.0                           # scale must be positive
    assert lib.b200_flash_prefill_tc(*bad) == -4
    bad = list(args); bad[10] = 96                            # head dim 64 or 128
    assert lib.b200_flash_prefill_tc(*bad) == -1
    bad = list(args); bad[12] = 8 * 128 + 4                   # stride not a multiple of 8 elements
    assert lib.b200_flash_prefill_tc(*bad) == -2
    # GEGLU: N = 2 O must be a multiple of 16, no residual, bf16 output only, not grouped
    geglu = 3
    assert lib.b200_gemm_bf16(one, one, one, 0, 128, 200, 64, 64, 64, 104, None, None, 0, geglu, None, 0, None) == -1
    assert lib.b200_gemm_bf16(one, one, one, 0, 128, 256, 64, 64, 64, 128, None, one, 128, geglu, None, 0, None) == -1
    assert lib.b200_gemm_bf16(one, one, one, 1, 128, 256, 64, 64, 64, 128, None, None, 0, geglu, None, 0, None) == -4
    assert lib.b200_gemm_bf16(one, one, one, 0, 128, 256, 64, 64, 64, 128, None, None, 0, 4, None, 0, None) == -4


def test_ops_refuse_cpu_tensors():
    """There is no CPU fallback: CPU tensors are an error, not a slow path."""
    from hoid_optimized_models_b200 import ops
    w = torch.zeros(8, 256, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        ops.gemv(torch.zeros(8), torch.zeros(256), w)


def test_missing_library_fails_loudly(tmp_path):
    from hoid_optimized_models_b200 import _lib
    with pytest.raises(ImportError, match="no CPU or PyTorch fallback"):
        _lib.load(str(tmp_path / "nope.so"))


def test_header_and_binding_constants_agree():
    """The enum values the Python side passes (epilogues, dtypes, error codes) are the header's."""
    from hoid_optimized_models_b200 import _lib
    text = re.sub(r"/\*.*?\*/", "", open(HEADER).read(), flags=re.S)
    enums = {k: int(v) for k, v in re.findall(r"\b(B200_[A-Z0-9_]+)\s*=\s*(-?\d+)", text)}
    for name in ("EPI_NONE", "EPI_SWIGLU", "EPI_GELU", "EPI_GEGLU", "BF16", "F32", "FLAG_PDL"):
        assert getattr(_lib, name) == enums["B200_" + name], name
    for code, label in _lib.ERRORS.items():
        assert enums[label.split()[0]] == code, label


def test_nvtx_ranges_wrap_every_call(lib, monkeypatch):
    """Opt-in NVTX: each C-ABI call sits in a range named after its entry point, results pass
    through unchanged, and switching it off returns the plain library."""
    from hoid_optimized_models_b200 import _lib
    events = []
    monkeypatch.setattr(torch.cuda.nvtx, "range_push", lambda name: events.append(("push", name)))
    monkeypatch.setattr(torch.cuda.nvtx, "range_pop", lambda: events.append(("pop", None)))
    monkeypatch.setattr(_lib, "_LIB", lib)
    _lib.set_nvtx(True)
    try:
        assert _lib.lib().b200_sm_count() == 148
        assert _lib.lib().b200_gemv_bf16(None, 0, None, None, 0, 256, 8, 256, None, None, 0.0, None, None,
                                         0, 0, 0, None) == -4
    finally:
        _lib.set_nvtx(False)
    assert events == [("push", "b200_sm_count"), ("pop", None), ("push", "b200_gemv_bf16"), ("pop", None)]
    assert _lib.lib() is lib
