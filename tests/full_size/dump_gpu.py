"""GPU half of the full-size parity check: runs one benchmark configuration at full depth and
width on cuda:0 with the seeded weights the oracle can regenerate, and writes what the oracle
comparison needs to a small .npz (generated tokens, the logits of every decode step in fp16,
per-layer hidden states of a sample of prompt rows (fp16) and of the first decode step, MoE routing
of the sampled rows).  The CPU half is tests/full_size/compare_cpu.py.

    python -m tests.full_size.dump_gpu <config> <out.npz>
    config: qwen3-4b | llama-3.1-8b | qwen3-30b-a3b | xlm-roberta-large | whisper-large-v3
"""
import os
import sys
import time

import numpy as np
import torch

from tests.full_size import cases


def _checksum(w, names):
    return np.array([float(w[n].double().sum()) for n in names])


def dump_decoder(name, out):
    from hoid_optimized_models_b200 import ops
    from hoid_optimized_models_b200.decoder import DenseDecoder
    from hoid_optimized_models_b200.weights import make_decoder_weights_parallel
    cfg, P, seed = cases.DECODERS[name]
    dev = torch.device("cuda:0")
    t0 = time.time()
    w = make_decoder_weights_parallel(cfg, seed, dev, threads=min(16, os.cpu_count() or 8))
    probe = ["model.embed_tokens.weight", "model.layers.0.self_attn.q_proj.weight",
             f"model.layers.{cfg.layers - 1}.self_attn.o_proj.weight", "model.norm.weight"]
    check = _checksum(w, probe)
    print(f"weights in {time.time() - t0:.0f} s", flush=True)
    ids = cases.prompt(cfg, P, seed)
    N = cases.N_NEW
    eng = DenseDecoder(cfg, w, max_seq=P + N + 2, device=dev, free_source_weights=True)
    del w
    torch.cuda.empty_cache()
    rows = cases.probe_rows(P, seed)
    hid, routed = [], []
    first = eng.prefill(ids.to(dev), collect=hid, collect_router=routed)
    prefill_hidden = torch.stack([h[rows].float().cpu() for h in hid])           # [L, R, H]
    routed_rows = torch.stack([r[rows].cpu() for r in routed]) if routed else torch.zeros(0)
    del hid, routed
    eng.capture()
    toks, logits, step_hidden, tok = [first], [], None, first
    for j in range(N - 1):
        if j == 0:
            step_hidden = []
            eng.set_step(tok, P)
            eng.step_static(collect=step_hidden)      # launch-per-phase path, to look inside
            lg = eng.logits
        else:
            lg = eng.step(tok, P + j)                 # captured graph (persistent kernel if dense)
        logits.append(lg.float().cpu().to(torch.float16))
        tok = int(eng.tok.item())
        assert tok == int(lg.argmax())
        toks.append(tok)
    toks2 = eng.generate(ids.to(dev), N)              # device-driven loop, no host round trip
    ops.check_status(dev)
    np.savez(out, config=name, toks=np.array(toks), toks_device_loop=np.array(toks2),
             logits=torch.stack(logits).numpy(), rows=np.array(rows),
             prefill_hidden=prefill_hidden.to(torch.float16).numpy(), routed=routed_rows.numpy(),
             step_hidden=torch.stack([h.float().cpu() for h in step_hidden]).numpy(),
             weight_checksum=check, persistent_kernel=eng.plan is not None)
    print(f"{name}: tokens {toks[:8]}... device loop equal: {toks2 == toks}", flush=True)


def dump_xlmr(out):
    from hoid_optimized_models_b200 import ops
    from hoid_optimized_models_b200.encoder import XlmrEncoder
    from hoid_optimized_models_b200.weights import make_encoder_weights
    name, cfg, B, S, seed = cases.XLMR
    dev = torch.device("cuda:0")
    w = make_encoder_weights(cfg, seed)
    ids = torch.randint(3, cfg.vocab, (B, S), generator=torch.Generator().manual_seed(seed))
    eng = XlmrEncoder(cfg, w, batch=B, seq=S, device=dev)
    eng.load_inputs(ids.to(dev))
    hid = []
    pooled = eng.forward_static(collect=hid).cpu().clone()
    ops.check_status(dev)
    rows = cases.probe_rows(B * S, seed, 128)
    eng.capture()
    again = eng.embed(ids.to(dev)).cpu()
    np.savez(out, config=name, pooled=pooled.numpy(), pooled_graph=again.numpy(), rows=np.array(rows),
             hidden=torch.stack([h[rows].float().cpu() for h in hid]).to(torch.float16).numpy())
    print(f"{name}: pooled {tuple(pooled.shape)}, graph replay equal: {torch.equal(again, pooled)}")


def dump_whisper(out):
    from hoid_optimized_models_b200 import ops
    from hoid_optimized_models_b200.weights import make_whisper_weights
    from hoid_optimized_models_b200.whisper import WhisperDecoder, WhisperEncoder
    name, cfg, seed = cases.WHISPER
    dev = torch.device("cuda:0")
    w = make_whisper_weights(cfg, seed)
    mel = torch.randn(cfg.n_mels, cfg.n_frames, generator=torch.Generator().manual_seed(seed)).clamp(-1.5, 1.5)
    enc = WhisperEncoder(cfg, w, device=dev)
    enc.load_inputs(mel.to(dev).to(torch.bfloat16))
    hid = []
    enc_out = enc.forward_static(collect=hid).float().cpu()
    ops.check_status(dev)
    rows = cases.probe_rows(cfg.n_ctx, seed, 64)
    dec = WhisperDecoder(cfg, w, device=dev, max_new_tokens=cases.WHISPER_STEPS + 8)
    dec.set_encoder(enc.out)
    dec.capture()
    logits = []
    toks = dec.generate(cases.WHISPER_PREFIX, cases.WHISPER_STEPS, collect_logits=logits)
    got = torch.stack(logits)                            # [prefix + steps - 1, V]
    np.savez(out, config=name, toks=np.array(toks), logits=got[:cases.WHISPER_LOGIT_ROWS].to(torch.float16).numpy(),
             enc_out=enc_out.to(torch.float16).numpy(), rows=np.array(rows),
             enc_hidden=torch.stack([h[rows].float().cpu() for h in hid]).to(torch.float16).numpy())
    print(f"{name}: {len(toks)} tokens {toks[:8]}...")


if __name__ == "__main__":
    which, out = sys.argv[1], sys.argv[2]
    os.makedirs(os.path.dirname(os.path.abspath(out)), exist_ok=True)
    with torch.no_grad():
        if which in cases.DECODERS:
            dump_decoder(which, out)
        elif which == cases.XLMR[0]:
            dump_xlmr(out)
        elif which == cases.WHISPER[0]:
            dump_whisper(out)
        else:
            raise SystemExit(f"unknown configuration {which}")
