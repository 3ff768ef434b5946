"""XLM-RoBERTa-large-architecture encoder on the GPU against the fp32 CPU oracle: real layer
widths (hidden 1024, 16 heads, FFN 4096), reduced depth and vocabulary.  Tolerances: per-layer
hidden states <= 2e-2 max relative error, pooled embeddings cosine >= 0.999 (the reference's
own gate is SNR >= 15 dB / cosine >= 0.95, models/bge-m3/best_hoid.py:59-92)."""
from dataclasses import replace

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B,S", [(4, 512), (3, 77)])
def test_xlmr_arch(dev, B, S):
    from hoid_optimized_models_b200.configs import XLMR_LARGE
    from hoid_optimized_models_b200.encoder import XlmrEncoder
    from hoid_optimized_models_b200.weights import make_encoder_weights
    from hoid_optimized_models_b200 import ops
    from oracle.ref_encoder import encoder_forward
    cfg = replace(XLMR_LARGE, name="xlmr-L3", layers=3, vocab=5000, max_pos=600)
    w = make_encoder_weights(cfg, 4)
    ids = torch.randint(3, cfg.vocab, (B, S), generator=torch.Generator().manual_seed(4))
    eng = XlmrEncoder(cfg, w, batch=B, seq=S, device=dev)
    eng.load_inputs(ids.to(dev))
    hid = []
    pooled = eng.forward_static(collect=hid).cpu().clone()
    ops.check_status(dev)
    hidden, pooled_ref = encoder_forward(cfg, w, ids)
    for l in range(cfg.layers):
        ref = hidden[l + 1].reshape(B * S, -1)
        err = float((hid[l].float().cpu() - ref).abs().max() / ref.abs().max())
        assert err < 2e-2, f"layer {l}: {err}"
    cos = torch.nn.functional.cosine_similarity(pooled, pooled_ref, dim=-1)
    assert float(cos.min()) >= 0.999
    assert float((pooled.norm(dim=-1) - 1).abs().max()) < 1e-3
    # graph replay gives the same embeddings
    eng.capture()
    again = eng.embed(ids.to(dev)).cpu()
    assert torch.equal(again, pooled)
