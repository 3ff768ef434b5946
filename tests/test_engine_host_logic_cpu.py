"""Host logic of the decoder engines on the CPU: `decoder.py` runs unchanged over a plain-torch
stand-in for the op layer (tests/fake_ops.py) and is compared with the fp32 oracle - weight
packing (q|k|v, interleaved gate|up, expert layouts), launch order, the device-side step state,
prefill -> decode hand-over - and, on two gloo ranks, tensor- and expert-parallel sharding with
the all-reduce through the collective calls and through the fused publish / consume numbering."""
import os
import socket
from dataclasses import replace

import pytest
import torch
import torch.multiprocessing as mp

from tests import fake_ops

N_NEW = 6
P = 24


def _cfg(kind):
    from hoid_optimized_models_b200.configs import LLAMA31_8B, QWEN3_4B, QWEN3_30B_A3B
    if kind == "llama":
        return replace(LLAMA31_8B, name="host-llama", hidden=256, inter=512, n_q=4, n_kv=2, layers=3,
                       vocab=512)
    if kind == "qwen3":
        return replace(QWEN3_4B, name="host-qwen3", hidden=256, inter=512, n_q=4, n_kv=2, layers=2,
                       vocab=512)
    return replace(QWEN3_30B_A3B, name="host-moe", hidden=256, moe_inter=256, n_q=4, n_kv=2, layers=2,
                   vocab=512, n_experts=8, top_k=2)


def _engine(cfg, w, monkeypatch=None, **kw):
    import hoid_optimized_models_b200.decoder as D
    D.ops = fake_ops                       # the engine's only door to the GPU
    return D.DenseDecoder(cfg, w, max_seq=P + N_NEW + 2, device="cpu", **kw)


def _generate(eng, ids):
    """prefill + host-driven eager steps (no CUDA graph on the CPU)."""
    tok = eng.prefill(ids)
    toks = [tok]
    for j in range(N_NEW - 1):
        eng.step(tok, P + j)
        tok = int(eng.tok)
        toks.append(tok)
    return toks


@pytest.fixture(autouse=True)
def _restore_ops():
    import hoid_optimized_models_b200.decoder as D
    real = D.ops
    yield
    D.ops = real
    fake_ops._PUBLISHED.clear()


@pytest.mark.parametrize("kind", ["llama", "qwen3", "moe"])
@pytest.mark.parametrize("fuse_rope", [True, False])
def test_engine_matches_oracle_on_cpu(kind, fuse_rope):
    from hoid_optimized_models_b200.weights import make_decoder_weights
    from oracle.ref_decoder import decoder_forward
    cfg = _cfg(kind)
    w = make_decoder_weights(cfg, 3)
    ids = torch.randint(0, cfg.vocab, (P,), generator=torch.Generator().manual_seed(3))
    eng = _engine(cfg, dict(w), fuse_rope=fuse_rope)
    toks = _generate(eng, ids)
    full = torch.cat((ids, torch.tensor(toks[:-1])))
    _, logits, _ = decoder_forward(cfg, w, full, logits_rows=range(P - 1, P + N_NEW - 1),
                                   keep_hidden=False)
    top2 = logits.topk(2, -1).values
    ref = logits.argmax(-1).tolist()
    for j, (a, b) in enumerate(zip(toks, ref)):          # bf16 prefill activations: near-ties may flip
        assert a == b or float(top2[j, 0] - top2[j, 1]) < 2e-2, (j, toks, ref)
    # the device-side bookkeeping: position, length, generated count and the token log
    assert eng.state[:3].tolist() == [P + N_NEW - 1, P + N_NEW, 1]
    assert int(eng.tok_log[0]) == toks[-1]


def _port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class _FakeLink:
    ctx = 0


def _worker(rank, size, port, kind, fused, out):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=size)
    try:
        import hoid_optimized_models_b200.comm as comm
        from hoid_optimized_models_b200.weights import make_decoder_weights
        comm.PeerLink = lambda *a, **k: _FakeLink()      # no CUDA IPC on the CPU
        torch.set_num_threads(2)
        cfg = _cfg(kind.split("-")[0])
        w = make_decoder_weights(cfg, 3)
        ids = torch.randint(0, cfg.vocab, (P,), generator=torch.Generator().manual_seed(3))
        eng = _engine(cfg, w, tp_rank=rank, tp_size=size, group=dist.group.WORLD,
                      fused_allreduce=fused, ep_all_to_all=kind.endswith("-a2a"))
        assert eng._ep_dispatch(P) == kind.endswith("-a2a")
        assert (eng.link is not None) == fused
        toks = _generate(eng, ids)
        out.put((rank, toks, eng.logits.float().tolist()))
        dist.barrier()
    finally:
        dist.destroy_process_group()


# "moe-a2a": expert-parallel prefill with the all-to-all dispatch / combine of token rows
@pytest.mark.parametrize("kind,fused", [("llama", False), ("llama", True), ("moe", False), ("moe", True),
                                        ("moe-a2a", True)])
def test_two_gloo_ranks_match_one(kind, fused):
    from hoid_optimized_models_b200.weights import make_decoder_weights
    cfg = _cfg(kind.split("-")[0])
    w = make_decoder_weights(cfg, 3)
    ids = torch.randint(0, cfg.vocab, (P,), generator=torch.Generator().manual_seed(3))
    ref_eng = _engine(cfg, dict(w))
    toks_ref = _generate(ref_eng, ids)
    logits_ref = ref_eng.logits.float().clone()
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, kind, fused, out)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted([out.get(timeout=300) for _ in procs], key=lambda r: r[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, toks, _ in res:
        assert toks == toks_ref, f"rank {rank}: {toks} vs {toks_ref}"
    # dense: the vocabulary is sharded over the ranks; MoE: every rank holds all logits
    full = torch.tensor(res[0][2]) if kind.startswith("moe") else torch.cat([torch.tensor(r[2]) for r in res])
    assert float((full - logits_ref).abs().max() / logits_ref.abs().max()) < 2e-2


def test_engine_from_checkpoint_on_cpu(tmp_path):
    """The real-weight path end to end: sharded safetensors directory -> from_checkpoint ->
    the same tokens as the engine built from the in-memory weights."""
    import hoid_optimized_models_b200.decoder as D
    from hoid_optimized_models_b200 import checkpoint
    from hoid_optimized_models_b200.weights import make_decoder_weights
    D.ops = fake_ops
    cfg = _cfg("qwen3")
    w = make_decoder_weights(cfg, 3)
    names = sorted(w)
    checkpoint.save_file(str(tmp_path / "model-00001-of-00002.safetensors"), {n: w[n] for n in names[::2]})
    checkpoint.save_file(str(tmp_path / "model-00002-of-00002.safetensors"), {n: w[n] for n in names[1::2]})
    ids = torch.randint(0, cfg.vocab, (P,), generator=torch.Generator().manual_seed(3))
    a = _generate(_engine(cfg, dict(w)), ids)
    eng = D.Qwen3Optimized.from_checkpoint(cfg, str(tmp_path), max_seq=P + N_NEW + 2, device="cpu")
    assert _generate(eng, ids) == a
