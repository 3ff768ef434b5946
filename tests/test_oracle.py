"""Pins the CPU oracle (oracle/ref_decoder.py) that the GPU parity tests trust:

1. against the committed golden vectors produced by the HuggingFace eager fp32 models (the
   reference's parity authority) — tests/golden/make_golden.py;
2. live against the same HuggingFace models when transformers is importable;
3. the engine's RoPE tables against the oracle's / HuggingFace's frequency rule.
Tolerances: fp32 against fp32 with a different summation order -> 1e-4 relative."""
import os
from dataclasses import replace

import numpy as np
import pytest
import torch

from hoid_optimized_models_b200.configs import LLAMA31_8B, QWEN3_4B, QWEN3_30B_A3B
from hoid_optimized_models_b200.weights import make_decoder_weights, rope_inv_freq
from oracle import ref_decoder as R

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
FAMILIES = {"llama": LLAMA31_8B, "qwen3": QWEN3_4B, "qwen3moe": QWEN3_30B_A3B}


def tiny(base):
    moe = bool(base.n_experts)
    return replace(base, name=base.name + "-tiny", hidden=128, layers=2, n_q=4, n_kv=2, head_dim=32,
                   inter=0 if moe else 256, vocab=512, n_experts=8 if moe else 0,
                   top_k=2 if moe else 0, moe_inter=64 if moe else 0)


@pytest.mark.parametrize("fam", sorted(FAMILIES))
def test_restatement_matches_golden(fam):
    cfg = tiny(FAMILIES[fam])
    gold = np.load(os.path.join(GOLD, f"decoder_{fam}.npz"))
    w = make_decoder_weights(cfg, 1234)
    ids = torch.from_numpy(gold["ids"])
    hidden, logits, router = R.decoder_forward(cfg, w, ids)
    got = torch.stack([h[-1] for h in hidden]).numpy()
    assert np.abs(got - gold["hidden_last"]).max() <= 1e-4 * np.abs(gold["hidden_last"]).max()
    assert np.abs(logits[-4:].numpy() - gold["logits_tail"]).max() <= 1e-4 * np.abs(gold["logits_tail"]).max()
    # greedy continuation by re-running the oracle on the growing sequence
    seq = ids.clone()
    out = []
    for _ in range(len(gold["greedy"])):
        _, lg, _ = R.decoder_forward(cfg, w, seq, logits_rows=[seq.numel() - 1], keep_hidden=False)
        out.append(int(lg.argmax()))
        seq = torch.cat((seq, torch.tensor([out[-1]])))
    assert out == gold["greedy"].tolist()
    if cfg.n_experts:
        ids_k = torch.stack([R.moe_route(r, cfg.top_k)[0].sort(-1).values for r in router]).numpy()
        assert np.array_equal(ids_k, gold["router_ids"])   # expert choice is bit-exact


@pytest.mark.parametrize("fam", sorted(FAMILIES))
def test_restatement_matches_live_hf(fam):
    pytest.importorskip("transformers")
    cfg = replace(tiny(FAMILIES[fam]), layers=3)
    w = make_decoder_weights(cfg, 77)
    ids = torch.randint(0, cfg.vocab, (40,), generator=torch.Generator().manual_seed(5))
    hs, logits = R.hf_forward(R.hf_model(cfg, w), ids)
    hidden, lg, _ = R.decoder_forward(cfg, w, ids)
    for a, b in zip(hs, hidden):
        assert float((a - b).abs().max()) <= 1e-4 * float(a.abs().max())
    assert float((logits - lg).abs().max()) <= 1e-4 * float(logits.abs().max())


def test_rope_tables_follow_llama3_rule():
    for cfg in (LLAMA31_8B, QWEN3_4B):
        a, b = rope_inv_freq(cfg), R.inv_freq(cfg)
        assert float((a - b).abs().max()) < 1e-15
    # the scaled band really is scaled: lowest frequency is divided by the factor
    base = replace(LLAMA31_8B, rope_scaling=None)
    assert abs(float(rope_inv_freq(LLAMA31_8B)[-1] * 8 / rope_inv_freq(base)[-1]) - 1) < 1e-12
    assert float(rope_inv_freq(LLAMA31_8B)[0]) == float(rope_inv_freq(base)[0])


def test_chunked_attention_is_chunk_invariant():
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(50, 4, 16, generator=g), torch.randn(50, 2, 16, generator=g),
               torch.randn(50, 2, 16, generator=g))
    a = R.causal_attention(q, k, v, 0.25, chunk=7)
    b = R.causal_attention(q, k, v, 0.25, chunk=1024)
    assert float((a - b).abs().max()) < 1e-6


def test_algorithmic_bytes_match_derivation():
    # 15 009 849 344 B of weights + 131 072 B of KV per cached position (Llama-3.1-8B)
    assert LLAMA31_8B.decode_bytes_per_token(0) == 15_009_849_344
    assert LLAMA31_8B.decode_bytes_per_token(8192) - LLAMA31_8B.decode_bytes_per_token(0) == 131072 * 8192


def test_encoder_restatement_matches_golden_and_hf():
    from hoid_optimized_models_b200.configs import XLMR_LARGE
    from hoid_optimized_models_b200.weights import make_encoder_weights
    from oracle import ref_encoder as E
    cfg = replace(XLMR_LARGE, name="xlmr-tiny", hidden=128, layers=2, heads=4, inter=256, vocab=600,
                  max_pos=64)
    gold = np.load(os.path.join(GOLD, "encoder_xlmr.npz"))
    w = make_encoder_weights(cfg, 1234)
    ids = torch.from_numpy(gold["ids"])
    hidden, pooled = E.encoder_forward(cfg, w, ids)
    got = torch.stack([h[:, 0] for h in hidden]).numpy()
    assert np.abs(got - gold["hidden_cls"]).max() <= 1e-4 * np.abs(gold["hidden_cls"]).max()
    assert np.abs(pooled.numpy() - gold["pooled"]).max() <= 1e-5
    pytest.importorskip("transformers")
    hs, p2 = E.hf_forward(E.hf_model(cfg, w), ids)
    assert float((p2 - pooled).abs().max()) <= 1e-5


def test_whisper_restatement_matches_golden_and_hf():
    from hoid_optimized_models_b200.configs import WHISPER_LARGE_V3
    from hoid_optimized_models_b200.weights import make_whisper_weights
    from oracle import ref_whisper as W
    cfg = replace(WHISPER_LARGE_V3, name="whisper-tiny", d_model=128, enc_layers=2, dec_layers=2,
                  heads=4, ffn=256, n_mels=16, n_frames=60, n_ctx=30, max_target=24, vocab=300)
    gold = np.load(os.path.join(GOLD, "whisper.npz"))
    w = make_whisper_weights(cfg, 1234)
    mel, ids = torch.from_numpy(gold["mel"]), torch.from_numpy(gold["dec_ids"])
    enc = W.encoder_forward(cfg, w, mel)
    lg = W.decoder_forward(cfg, w, enc, ids)
    assert np.abs(enc[-4:].numpy() - gold["enc_tail"]).max() <= 1e-4 * np.abs(gold["enc_tail"]).max()
    assert np.abs(lg[-2:].numpy() - gold["logits_tail"]).max() <= 1e-4 * np.abs(gold["logits_tail"]).max()
    pytest.importorskip("transformers")
    enc2, lg2 = W.hf_forward(W.hf_model(cfg, w), mel, ids)
    assert float((enc2 - enc).abs().max()) <= 1e-4 * float(enc2.abs().max())
    assert float((lg2 - lg).abs().max()) <= 1e-4 * float(lg2.abs().max())


def test_bf16_eager_mode_is_a_depth_dependent_floor():
    """decoder_forward(act_dtype=bfloat16) restates the reference's bf16 eager numerics: same
    function as the fp32 run up to rounding, and its distance from fp32 grows with depth (the
    full-size GPU test measures the CUDA path against this run)."""
    from dataclasses import replace
    from hoid_optimized_models_b200.configs import LLAMA31_8B
    from hoid_optimized_models_b200.weights import make_decoder_weights
    from oracle.ref_decoder import decoder_forward
    cfg = replace(LLAMA31_8B, name="floor-test", hidden=512, inter=1536, n_q=4, n_kv=2, layers=6,
                  vocab=512)
    w = make_decoder_weights(cfg, 5)
    ids = torch.randint(0, cfg.vocab, (48,), generator=torch.Generator().manual_seed(5))
    h32, l32, _ = decoder_forward(cfg, w, ids)
    h16, l16, _ = decoder_forward(cfg, w, ids, act_dtype=torch.bfloat16)
    err = [float((a - b).abs().max() / b.abs().max()) for a, b in zip(h16[1:-1], h32[1:-1])]
    assert all(0 < e < 5e-2 for e in err), err            # bf16 rounding, not a different function
    assert err[-1] > err[0]                                # and it accumulates over layers
    cos = torch.nn.functional.cosine_similarity(l16, l32, dim=-1)
    assert float(cos.min()) > 0.99
    # the default is untouched fp32
    h32b, _, _ = decoder_forward(cfg, w, ids, act_dtype=None)
    assert torch.equal(h32b[3], h32[3])


def test_bf16_eager_mode_matches_hf_run_in_bf16():
    """Pins the floor itself: HuggingFace's eager model run in torch.bfloat16 on the CPU sits at
    the same distance from the fp32 run as the restatement with act_dtype=bfloat16 (the two round
    at slightly different places, so they are compared by their distance from fp32, per layer)."""
    from dataclasses import replace
    from hoid_optimized_models_b200.configs import LLAMA31_8B
    from hoid_optimized_models_b200.weights import make_decoder_weights
    from oracle.ref_decoder import decoder_forward, hf_forward, hf_model
    cfg = replace(LLAMA31_8B, name="floor-test", hidden=512, inter=1536, n_q=4, n_kv=2, layers=6,
                  vocab=512)
    w = make_decoder_weights(cfg, 5)
    ids = torch.randint(0, cfg.vocab, (48,), generator=torch.Generator().manual_seed(5))
    h32, _, _ = decoder_forward(cfg, w, ids)
    h16, _, _ = decoder_forward(cfg, w, ids, act_dtype=torch.bfloat16)
    hs, _ = hf_forward(hf_model(cfg, w).to(torch.bfloat16), ids)
    for l in range(1, cfg.layers):
        ref = h32[l]
        mine = float((h16[l] - ref).abs().max() / ref.abs().max())
        hf = float((hs[l].float() - ref).abs().max() / ref.abs().max())
        assert 0.5 < mine / hf < 2.0, (l, mine, hf)
