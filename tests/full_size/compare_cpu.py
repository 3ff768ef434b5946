"""CPU half of the full-size parity check: regenerates the seeded weights layer by layer, runs the
fp32 oracle (teacher-forced over the prompt + the tokens the GPU generated) and compares it with
the .npz that tests/full_size/dump_gpu.py wrote on the GPU box.  Prints one markdown table row
per configuration (collected in profiles/parity_full_size.md).

    python -m tests.full_size.compare_cpu <dump.npz> [--floor]

--floor also runs the oracle with the reference's bf16-eager numerics (every materialised tensor
rounded to bf16) and reports that run's own distance from fp32 beside ours.
"""
import sys
import time

import numpy as np
import torch

from tests.full_size import cases


def _cos_min(a, b):
    return float(torch.nn.functional.cosine_similarity(a, b, dim=-1).min())


def compare_decoder(d, floor):
    import transformers
    from hoid_optimized_models_b200.weights import LazyDecoderWeights, _normal, decoder_weight_specs
    from oracle.ref_decoder import decoder_forward, moe_route
    name = str(d["config"])
    cfg, P, seed = cases.DECODERS[name]
    N = cases.N_NEW
    w = LazyDecoderWeights(cfg, seed)
    # the GPU box generated the same weights
    spec = {n: (s, l, k, m) for n, s, l, k, m in decoder_weight_specs(cfg)}
    probe = ["model.embed_tokens.weight", "model.layers.0.self_attn.q_proj.weight",
             f"model.layers.{cfg.layers - 1}.self_attn.o_proj.weight", "model.norm.weight"]
    mine = np.array([float(_normal(spec[n][0], seed, spec[n][1], spec[n][2], "cpu", mean=spec[n][3]).double().sum())
                     for n in probe])
    assert np.allclose(mine, d["weight_checksum"], rtol=1e-9, atol=1e-6), (mine, d["weight_checksum"])
    toks = d["toks"].tolist()
    assert toks == d["toks_device_loop"].tolist(), "host-driven and device-driven generation differ"
    ids = cases.prompt(cfg, P, seed)
    full = torch.cat((ids, torch.tensor(toks[:-1])))
    rows = list(range(P - 1, P + N - 1))
    t0 = time.time()
    hidden, logits_ref, router_ref = decoder_forward(cfg, w, full, logits_rows=rows)
    t_or = time.time() - t0
    sel = torch.tensor(d["rows"].tolist())
    got_h = torch.from_numpy(d["prefill_hidden"].astype(np.float32))   # [L, R, H]
    keep = torch.ones(len(sel), dtype=torch.bool)
    rerouted = 0
    exhausted = None
    errs = []
    for l in range(cfg.layers - 1):
        if cfg.n_experts:
            ids_ref, _ = moe_route(router_ref[l][sel], cfg.top_k)
            got_r = torch.from_numpy(d["routed"][l]).long()
            same = (got_r.sort(-1).values == ids_ref.sort(-1).values).all(-1)
            probs = torch.softmax(router_ref[l][sel].float(), -1).topk(cfg.top_k + 1, -1).values
            margin = (probs[:, cfg.top_k - 1] - probs[:, cfg.top_k]) / probs[:, cfg.top_k - 1]
            bad = margin[~same & keep]
            assert bad.numel() == 0 or float(bad.max()) < 3e-2, f"layer {l}: routing differs at margin {float(bad.max())}"
            keep &= same
            rerouted = int((~keep).sum())
        ref = hidden[l + 1][:P]
        dd = (got_h[l] - ref[sel])[keep]
        if dd.numel() == 0:         # every sampled row has met a router near-tie by this depth
            exhausted = l if exhausted is None else exhausted
            continue
        errs.append(float(dd.abs().max() / ref.abs().max()))
    step_h = torch.from_numpy(d["step_hidden"])
    step_errs = [float((step_h[l] - hidden[l + 1][P]).abs().max() / hidden[l + 1][P].abs().max())
                 for l in range(cfg.layers - 1)]
    got = torch.from_numpy(d["logits"].astype(np.float32))
    ref_steps = logits_ref[1:]
    cos = _cos_min(got, ref_steps)
    lerr = (got - ref_steps).abs().max(-1).values
    greedy_ref = logits_ref.argmax(-1).tolist()
    top2 = logits_ref.topk(2, -1).values
    margin = top2[:, 0] - top2[:, 1]
    noise = torch.cat((lerr[:1], lerr))
    flips = [(j, round(float(margin[j]), 4), round(float(noise[j]), 4)) for j in range(N) if toks[j] != greedy_ref[j]]
    fl = ""
    if floor:
        h16, l16, _ = decoder_forward(cfg, w, full, logits_rows=rows, act_dtype=torch.bfloat16)
        f_h = max(float((h16[l + 1][:P] - hidden[l + 1][:P]).abs().max() / hidden[l + 1][:P].abs().max())
                  for l in range(cfg.layers - 1))
        fl = (f" | bf16-eager floor: hidden {f_h:.2e}, cosine {_cos_min(l16[1:], ref_steps):.5f}, "
              f"logit err {float((l16[1:] - ref_steps).abs().max()):.3f}")
    first_over = next((l for l, e in enumerate(errs) if e >= 2e-2), None)
    print(f"| {name} | {cfg.layers} L, P={P}, {N - 1} steps | {max(errs):.2e} (layer {int(np.argmax(errs))}; "
          f"first layer >= 2e-2: {first_over}) | {max(step_errs):.2e} | {cos:.5f} | {float(lerr.max()):.3f} | "
          f"{len(flips)} {flips} | {rerouted}{'' if exhausted is None else f' (all sampled rows by layer {exhausted})'} | transformers {transformers.__version__}, oracle {t_or:.0f} s, "
          f"persistent kernel {bool(d['persistent_kernel'])}{fl} |", flush=True)


def compare_xlmr(d):
    from hoid_optimized_models_b200.weights import make_encoder_weights
    from oracle.ref_encoder import encoder_forward
    name, cfg, B, S, seed = cases.XLMR
    w = make_encoder_weights(cfg, seed)
    ids = torch.randint(3, cfg.vocab, (B, S), generator=torch.Generator().manual_seed(seed))
    t0 = time.time()
    hidden, pooled_ref = encoder_forward(cfg, w, ids)
    sel = torch.tensor(d["rows"].tolist())
    got = torch.from_numpy(d["hidden"].astype(np.float32))
    errs = []
    for l in range(cfg.layers):
        ref = hidden[l + 1].reshape(B * S, -1)
        errs.append(float((got[l] - ref[sel]).abs().max() / ref.abs().max()))
    pooled = torch.from_numpy(d["pooled"])
    assert np.array_equal(d["pooled"], d["pooled_graph"])
    snr = 10 * torch.log10(pooled_ref.pow(2).sum() / (pooled - pooled_ref).pow(2).sum())
    first_over = next((l for l, e in enumerate(errs) if e >= 2e-2), None)
    print(f"| {name} | {cfg.layers} L, {B} x {S} | {max(errs):.2e} (layer {int(np.argmax(errs))}; first layer "
          f">= 2e-2: {first_over}) | - | pooled {_cos_min(pooled, pooled_ref):.5f} | SNR {float(snr):.1f} dB | - | - | "
          f"oracle {time.time() - t0:.0f} s |", flush=True)


def compare_whisper(d):
    from hoid_optimized_models_b200.weights import make_whisper_weights
    from oracle import ref_whisper as W
    name, cfg, seed = cases.WHISPER
    w = make_whisper_weights(cfg, seed)
    mel = torch.randn(cfg.n_mels, cfg.n_frames, generator=torch.Generator().manual_seed(seed)).clamp(-1.5, 1.5)
    t0 = time.time()
    ref_out, ref_hid = W.encoder_forward(cfg, w, mel.to(torch.bfloat16).float(), keep_hidden=True)
    sel = torch.tensor(d["rows"].tolist())
    got_h = torch.from_numpy(d["enc_hidden"].astype(np.float32))
    errs = [float((got_h[l] - ref_hid[l][sel]).abs().max() / ref_hid[l].abs().max()) for l in range(cfg.enc_layers)]
    enc_out = torch.from_numpy(d["enc_out"].astype(np.float32))
    e_out = float((enc_out - ref_out).abs().max() / ref_out.abs().max())
    toks = d["toks"].tolist()
    prefix = cases.WHISPER_PREFIX
    seq = torch.tensor(prefix + toks[:-1])
    # the oracle decoder sees the GPU's own (bf16) encoder output: only the decoder is compared
    lg_ref = W.decoder_forward(cfg, w, enc_out, seq)
    got = torch.from_numpy(d["logits"].astype(np.float32))              # the first rows only
    R = got.shape[0]
    cos = _cos_min(got, lg_ref[:R])
    lerr = (got - lg_ref[:R]).abs().max(-1).values
    top2 = lg_ref.topk(2, -1).values
    margin = top2[:, 0] - top2[:, 1]
    ref_toks = lg_ref.argmax(-1).tolist()[len(prefix) - 1:]
    # every one of the generated tokens is checked; a flip is judged against the oracle's margin
    flips = [(j, round(float(margin[len(prefix) - 1 + j]), 4)) for j, (a, b) in enumerate(zip(toks, ref_toks)) if a != b]
    first_over = next((l for l, e in enumerate(errs) if e >= 2e-2), None)
    print(f"| {name} | {cfg.enc_layers}+{cfg.dec_layers} L, {len(toks)} steps | encoder {max(errs):.2e} (first layer "
          f">= 2e-2: {first_over}), output {e_out:.2e} | - | {cos:.5f} | {float(lerr.max()):.3f} | "
          f"{len(flips)} {flips[:6]} | - | oracle {time.time() - t0:.0f} s |", flush=True)


if __name__ == "__main__":
    d = np.load(sys.argv[1])
    which = str(d["config"])
    with torch.no_grad():
        if which in cases.DECODERS:
            compare_decoder(d, "--floor" in sys.argv)
        elif which == cases.XLMR[0]:
            compare_xlmr(d)
        else:
            compare_whisper(d)
