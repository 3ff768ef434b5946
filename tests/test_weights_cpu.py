"""The seeded synthetic checkpoints: every tensor has its own generator, so the whole-dict builder,
the thread-pool builder and the lazy layer-at-a-time view (which the full-size parity check walks
a 61 GB model with) must give bit-identical tensors."""
from dataclasses import replace

import torch


def test_lazy_and_parallel_builders_equal_the_plain_one():
    from hoid_optimized_models_b200 import weights as W
    from hoid_optimized_models_b200.configs import QWEN3_30B_A3B, QWEN3_4B
    for base in (QWEN3_30B_A3B, QWEN3_4B):
        moe = bool(base.n_experts)
        cfg = replace(base, name="w-test", layers=3, vocab=512, hidden=256, n_q=4, n_kv=2, head_dim=64,
                      inter=0 if moe else 384, n_experts=8 if moe else 0, top_k=2 if moe else 0,
                      moe_inter=64 if moe else 0)
        plain = W.make_decoder_weights(cfg, 7)
        lazy = W.LazyDecoderWeights(cfg, 7)
        pool = W.make_decoder_weights_parallel(cfg, 7, "cpu", threads=4)
        assert set(plain) == set(lazy.keys()) == set(pool)
        for name in plain:                                  # layer order: the lazy view drops old layers
            assert torch.equal(plain[name], lazy[name]) and torch.equal(plain[name], pool[name]), name
        # only the layer in use (and the tensors outside the layers) stays resident
        resident = [k for k in dict.keys(lazy) if k.startswith("model.layers.")]
        assert resident and all(k.startswith(f"model.layers.{cfg.layers - 1}.") for k in resident)
        # going back to an earlier layer regenerates it, identically
        assert torch.equal(lazy["model.layers.0.self_attn.q_proj.weight"],
                           plain["model.layers.0.self_attn.q_proj.weight"])
