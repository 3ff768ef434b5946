"""Host logic of the encoder and Whisper engines on the CPU over tests/fake_ops.py, against the
fp32 oracle: weight packing, the conv front-end as GEMMs over overlapping-row views, LayerNorm
prologues, cross-attention over strided projections, the decode step state, and the two-rank
data-parallel encoder on gloo."""
import os
import socket
from dataclasses import replace

import pytest
import torch
import torch.multiprocessing as mp

from tests import fake_ops


@pytest.fixture(autouse=True)
def _patch_ops():
    import hoid_optimized_models_b200.encoder as E
    import hoid_optimized_models_b200.whisper as Wh
    real = (E.ops, Wh.ops)
    E.ops = Wh.ops = fake_ops
    yield
    E.ops, Wh.ops = real


def _enc_case():
    from hoid_optimized_models_b200.configs import XLMR_LARGE
    from hoid_optimized_models_b200.weights import make_encoder_weights
    cfg = replace(XLMR_LARGE, name="host-xlmr", hidden=128, heads=4, inter=256, layers=2, vocab=300,
                  max_pos=80)
    B, S = 4, 40
    ids = torch.randint(3, cfg.vocab, (B, S), generator=torch.Generator().manual_seed(8))
    return cfg, make_encoder_weights(cfg, 8), B, S, ids


def test_encoder_matches_oracle_on_cpu():
    from hoid_optimized_models_b200.encoder import XlmrEncoder
    from oracle.ref_encoder import encoder_forward
    cfg, w, B, S, ids = _enc_case()
    eng = XlmrEncoder(cfg, w, batch=B, seq=S, device="cpu")
    eng.load_inputs(ids)
    hid = []
    pooled = eng.forward_static(collect=hid).clone()
    hidden, pooled_ref = encoder_forward(cfg, w, ids)
    for l in range(cfg.layers):
        ref = hidden[l + 1].reshape(B * S, -1)
        assert float((hid[l].float() - ref).abs().max() / ref.abs().max()) < 2e-2, l
    assert float(torch.nn.functional.cosine_similarity(pooled, pooled_ref, dim=-1).min()) > 0.999


def _port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _dp_worker(rank, size, port, out):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=size)
    try:
        import hoid_optimized_models_b200.encoder as E
        E.ops = fake_ops
        torch.set_num_threads(2)
        cfg, w, B, S, ids = _enc_case()
        eng = E.XlmrEncoder(cfg, w, batch=B, seq=S, device="cpu", dp_rank=rank, dp_size=size,
                            group=dist.group.WORLD)
        per = B // size
        emb = eng.embed(ids[rank * per:(rank + 1) * per])
        out.put((rank, emb.tolist()))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_encoder_data_parallel_on_two_gloo_ranks():
    from hoid_optimized_models_b200.encoder import XlmrEncoder
    cfg, w, B, S, ids = _enc_case()
    ref = XlmrEncoder(cfg, w, batch=B, seq=S, device="cpu").embed(ids).clone()
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _port()
    procs = [ctx.Process(target=_dp_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    res = [out.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, emb in res:                         # every rank ends up with the whole batch
        assert float((torch.tensor(emb) - ref).abs().max()) < 1e-5, rank


def test_whisper_matches_oracle_on_cpu():
    from hoid_optimized_models_b200.configs import WHISPER_LARGE_V3
    from hoid_optimized_models_b200.weights import make_whisper_weights
    from hoid_optimized_models_b200.whisper import WhisperDecoder, WhisperEncoder
    from oracle import ref_whisper as W
    cfg = replace(WHISPER_LARGE_V3, name="host-whisper", d_model=128, heads=4, ffn=256, n_mels=16,
                  n_frames=120, n_ctx=60, enc_layers=2, dec_layers=2, vocab=300, max_target=32)
    w = make_whisper_weights(cfg, 6)
    mel = torch.randn(cfg.n_mels, cfg.n_frames, generator=torch.Generator().manual_seed(6)).clamp(-1.5, 1.5)
    mel = mel.to(torch.bfloat16)
    enc = WhisperEncoder(cfg, w, device="cpu")
    enc.load_inputs(mel)
    hid = []
    out = enc.forward_static(collect=hid).float()
    ref_out, ref_hid = W.encoder_forward(cfg, w, mel.float(), keep_hidden=True)
    for l in range(cfg.enc_layers):
        assert float((hid[l].float() - ref_hid[l]).abs().max() / ref_hid[l].abs().max()) < 2e-2, l
    assert float((out - ref_out).abs().max() / ref_out.abs().max()) < 2e-2

    dec = WhisperDecoder(cfg, w, device="cpu")
    dec.set_encoder(enc.out)
    prefix, n_new = [7, 100, 33, 250], 8
    logits = []
    toks = dec.generate(prefix, n_new, collect_logits=logits)
    seq = torch.tensor(prefix + toks[:-1])
    lg_ref = W.decoder_forward(cfg, w, enc.out.float(), seq)
    got = torch.stack(logits)
    cos = torch.nn.functional.cosine_similarity(got, lg_ref, dim=-1)
    assert float(cos.min()) > 0.999
    top2 = lg_ref.topk(2, -1).values
    ref_toks = lg_ref.argmax(-1).tolist()[len(prefix) - 1:]
    for j, (a, b) in enumerate(zip(toks, ref_toks)):
        k = len(prefix) - 1 + j
        assert a == b or float(top2[k, 0] - top2[k, 1]) < 2e-2, (j, toks, ref_toks)
    # the forced prefix as one prefill pass: same cache rows, same first token and continuation
    # (bf16 rows against fp32 vectors: a token may differ only at an oracle near-tie)
    kv_steps = dec.kv[:, :, :, :len(prefix)].float().clone()
    dec.kv.zero_()
    toks2 = dec.generate(prefix, n_new)
    assert float((dec.kv[:, :, :, :len(prefix)].float() - kv_steps).abs().max()) < 2e-2 * float(kv_steps.abs().max())
    for j, (a, b) in enumerate(zip(toks2, ref_toks)):
        k = len(prefix) - 1 + j
        assert a == b or float(top2[k, 0] - top2[k, 1]) < 2e-2, (j, toks2, ref_toks)
        if a != b:
            break                                        # teacher forcing ends at the first flip


def test_encoder_and_whisper_from_checkpoints_on_cpu(tmp_path):
    """Safetensors directories (one with a wrapper prefix on the stored names) -> engines with the
    same outputs as the engines built from the in-memory weights."""
    from hoid_optimized_models_b200 import checkpoint
    from hoid_optimized_models_b200.encoder import XlmrEncoder
    import hoid_optimized_models_b200.whisper as Wh
    from hoid_optimized_models_b200.configs import WHISPER_LARGE_V3
    from hoid_optimized_models_b200.weights import make_whisper_weights
    cfg, w, B, S, ids = _enc_case()
    (tmp_path / "enc").mkdir()
    checkpoint.save_file(str(tmp_path / "enc" / "model.safetensors"), {"roberta." + n: t for n, t in w.items()})
    a = XlmrEncoder(cfg, w, batch=B, seq=S, device="cpu").embed(ids).clone()
    b = XlmrEncoder.from_checkpoint(cfg, str(tmp_path / "enc"), B, S, device="cpu",
                                    strip_prefix="roberta.").embed(ids)
    assert torch.equal(a, b)

    wc = replace(WHISPER_LARGE_V3, name="host-whisper", d_model=128, heads=4, ffn=256, n_mels=16,
                 n_frames=120, n_ctx=60, enc_layers=1, dec_layers=1, vocab=300, max_target=32)
    ww = make_whisper_weights(wc, 6)
    (tmp_path / "whisper").mkdir()
    checkpoint.save_file(str(tmp_path / "whisper" / "model.safetensors"), {**ww, "proj_out.weight": ww["model.decoder.embed_tokens.weight"]})
    got = Wh.load_checkpoint(str(tmp_path / "whisper"), device="cpu")
    assert set(got) == set(ww) and all(torch.equal(got[n], ww[n]) for n in ww)
    mel = torch.randn(wc.n_mels, wc.n_frames, generator=torch.Generator().manual_seed(6)).to(torch.bfloat16)
    e1, e2 = Wh.WhisperEncoder(wc, ww, device="cpu"), Wh.WhisperEncoder(wc, got, device="cpu")
    assert torch.equal(e1.encode(mel), e2.encode(mel))


def test_whisper_suppression_masks_ride_in_the_logits_bias():
    """suppress_tokens hold at every step, begin_suppress_tokens at the first generated token only;
    without either the decoder is unchanged."""
    from hoid_optimized_models_b200.configs import WHISPER_LARGE_V3
    from hoid_optimized_models_b200.weights import make_whisper_weights
    from hoid_optimized_models_b200.whisper import WhisperDecoder
    cfg = replace(WHISPER_LARGE_V3, name="host-whisper", d_model=128, heads=4, ffn=256, n_mels=16,
                  n_frames=120, n_ctx=60, enc_layers=1, dec_layers=2, vocab=300, max_target=32)
    w = make_whisper_weights(cfg, 6)
    enc_out = (torch.randn(cfg.n_ctx, cfg.d_model, generator=torch.Generator().manual_seed(1)) * 0.5).to(torch.bfloat16)
    prefix, n_new = [7, 100, 33], 6

    def run(**kw):
        dec = WhisperDecoder(cfg, w, device="cpu", **kw)
        dec.set_encoder(enc_out)
        logits = []
        return dec.generate(prefix, n_new, collect_logits=logits), torch.stack(logits)

    base, lg0 = run()
    banned_first = base[0]
    others = [t for t in base[1:] if t != banned_first]
    banned_always = others[0] if others else (banned_first + 1) % cfg.vocab
    toks, lg = run(suppress_tokens=[banned_always], begin_suppress_tokens=[banned_first])
    assert toks[0] != banned_first and banned_always not in toks
    first = len(prefix) - 1                         # row of the first generated token
    assert torch.isinf(lg[first, banned_first]) and torch.isinf(lg[first:, banned_always]).all()
    assert not torch.isinf(lg[first + 1:, banned_first]).any()      # begin mask: first token only
    keep = torch.ones(cfg.vocab, dtype=torch.bool)
    keep[[banned_first, banned_always]] = False
    assert torch.allclose(lg[first][keep], lg0[first][keep])        # everything else untouched
