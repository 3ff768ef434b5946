"""The five benchmark configurations at full size, shared by the GPU-side dump and the CPU-side
comparison (tests/full_size/dump_gpu.py, tests/full_size/compare_cpu.py)."""
import torch

from hoid_optimized_models_b200 import configs as C

N_NEW = 33          # first token from the prefill + 32 decode steps

# name -> (config, prompt tokens, seed)
DECODERS = {
    "qwen3-4b": (C.QWEN3_4B, 1024, 1),
    "llama-3.1-8b": (C.LLAMA31_8B, 8192, 2),
    "qwen3-30b-a3b": (C.QWEN3_30B_A3B, 1024, 3),
}
XLMR = ("xlm-roberta-large", C.XLMR_LARGE, 64, 512, 4)
WHISPER = ("whisper-large-v3", C.WHISPER_LARGE_V3, 5)
WHISPER_PREFIX = [50258, 50259, 50360, 50364]
WHISPER_STEPS = 224
WHISPER_LOGIT_ROWS = 68      # logit rows carried to the oracle (prefix + first decode steps)


def prompt(cfg, P, seed):
    return torch.randint(0, cfg.vocab, (P,), generator=torch.Generator().manual_seed(seed))


def probe_rows(P, seed, n=32):
    """Token rows whose per-layer hidden states are carried from the GPU run to the oracle: the
    first and last positions plus a seeded sample (all P rows of all layers would be GBs)."""
    g = torch.Generator().manual_seed(1000 + seed)
    extra = torch.randperm(P, generator=g)[:n].tolist()
    return sorted(set([0, 1, 2, P // 2, P - 3, P - 2, P - 1] + extra))[:n]
