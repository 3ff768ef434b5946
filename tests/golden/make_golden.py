"""Generates tests/golden/decoder_<family>.npz from the HuggingFace eager fp32 models (the
reference's parity authority) on tiny seeded configurations.

    python tests/golden/make_golden.py
    python tests/golden/make_golden.py --reference-listing <checkout of the reference project>

The second form only writes reference_files.txt, the list of the reference project's file paths
that tests/test_abi.py checks the header's citations against.

Each file holds the token ids, the HF per-layer hidden state of the last position, the HF
logits of the last four positions, 8 HF greedy tokens and (MoE) the HF router's top-k expert
ids; the transformers / torch versions are recorded alongside."""
import json
import os
import sys
from dataclasses import replace

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from hoid_optimized_models_b200.configs import LLAMA31_8B, QWEN3_4B, QWEN3_30B_A3B  # noqa: E402
from hoid_optimized_models_b200.weights import make_decoder_weights  # noqa: E402
from oracle import ref_decoder as R  # noqa: E402

SEED = 1234


def tiny(base):
    moe = bool(base.n_experts)
    return replace(base, name=base.name + "-tiny", hidden=128, layers=2, n_q=4, n_kv=2, head_dim=32,
                   inter=0 if moe else 256, vocab=512, n_experts=8 if moe else 0,
                   top_k=2 if moe else 0, moe_inter=64 if moe else 0)


FAMILIES = {"llama": LLAMA31_8B, "qwen3": QWEN3_4B, "qwen3moe": QWEN3_30B_A3B}


def main():
    import transformers
    meta = {"transformers": transformers.__version__, "torch": torch.__version__, "seed": SEED}
    for fam, base in FAMILIES.items():
        cfg = tiny(base)
        w = make_decoder_weights(cfg, SEED)
        ids = torch.randint(0, cfg.vocab, (24,), generator=torch.Generator().manual_seed(SEED))
        model = R.hf_model(cfg, w)
        hs, logits = R.hf_forward(model, ids)
        out = {"ids": ids.numpy(), "hidden_last": torch.stack([h[-1] for h in hs]).numpy(),
               "logits_tail": logits[-4:].numpy(),
               "greedy": np.array(R.hf_greedy(model, ids, 8))}
        if cfg.n_experts:
            captured = []
            hooks = [l.mlp.gate.register_forward_hook(lambda m, i, o: captured.append(o))
                     for l in model.model.layers]
            R.hf_forward(model, ids)
            for h in hooks:
                h.remove()
            # router output layout differs between transformers versions; keep the index tensor
            idx = [c for o in captured for c in (o if isinstance(o, tuple) else (o,))
                   if c.dtype in (torch.int64, torch.int32)]
            out["router_ids"] = torch.stack([i.sort(-1).values for i in idx]).numpy()
        np.savez_compressed(os.path.join(HERE, f"decoder_{fam}.npz"), **out)
        print(fam, {k: v.shape for k, v in out.items()})
    # encoder (XLM-RoBERTa architecture)
    from hoid_optimized_models_b200.configs import XLMR_LARGE
    from hoid_optimized_models_b200.weights import make_encoder_weights
    from oracle import ref_encoder as E
    ecfg = replace(XLMR_LARGE, name="xlmr-tiny", hidden=128, layers=2, heads=4, inter=256, vocab=600,
                   max_pos=64)
    ew = make_encoder_weights(ecfg, SEED)
    eids = torch.randint(3, ecfg.vocab, (3, 20), generator=torch.Generator().manual_seed(SEED))
    hs, pooled = E.hf_forward(E.hf_model(ecfg, ew), eids)
    np.savez_compressed(os.path.join(HERE, "encoder_xlmr.npz"), ids=eids.numpy(),
                        hidden_cls=torch.stack([h[:, 0] for h in hs]).numpy(), pooled=pooled.numpy())
    print("xlmr", pooled.shape)
    # Whisper architecture (encoder + teacher-forced decoder)
    from hoid_optimized_models_b200.configs import WHISPER_LARGE_V3
    from hoid_optimized_models_b200.weights import make_whisper_weights
    from oracle import ref_whisper as W
    wcfg = replace(WHISPER_LARGE_V3, name="whisper-tiny", d_model=128, enc_layers=2, dec_layers=2,
                   heads=4, ffn=256, n_mels=16, n_frames=60, n_ctx=30, max_target=24, vocab=300)
    ww = make_whisper_weights(wcfg, SEED)
    mel = torch.randn(16, 60, generator=torch.Generator().manual_seed(SEED)).clamp(-1.5, 1.5)
    dids = torch.randint(3, 300, (9,), generator=torch.Generator().manual_seed(SEED + 1))
    enc, lg = W.hf_forward(W.hf_model(wcfg, ww), mel, dids)
    np.savez_compressed(os.path.join(HERE, "whisper.npz"), mel=mel.numpy(), dec_ids=dids.numpy(),
                        enc_tail=enc[-4:].numpy(), logits_tail=lg[-2:].numpy())
    print("whisper", enc.shape, lg.shape)
    with open(os.path.join(HERE, "versions.json"), "w") as f:
        json.dump(meta, f, indent=1)


def write_reference_listing(root: str) -> None:
    paths = []
    for d, dirs, files in os.walk(root):
        dirs[:] = [x for x in dirs if x != ".git"]
        paths += [os.path.relpath(os.path.join(d, f), root) for f in files]
    with open(os.path.join(HERE, "reference_files.txt"), "w") as f:
        f.write("\n".join(sorted(paths)) + "\n")


if __name__ == "__main__":
    if len(sys.argv) == 3 and sys.argv[1] == "--reference-listing":
        write_reference_listing(sys.argv[2])
    else:
        main()
