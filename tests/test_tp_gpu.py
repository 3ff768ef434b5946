"""Multi-GPU engines against the fp32 CPU oracle and against the single-GPU engine.

Tensor parallel (Llama architecture) with the all-reduce inside the persistent decode kernel,
fused into the per-phase GEMVs, or through NCCL; expert parallel (Qwen3-MoE architecture);
data parallel (XLM-R architecture).  World sizes 2, 4 and 8 - a case is skipped when fewer GPUs
are visible.  Greedy tokens must equal the single-GPU engine's, logits must agree with it within
1e-2 relative (the multi-rank prefill all-reduces bf16 partial projections, a rounding the
single-GPU prefill does not have) and with the oracle's teacher-forced logits at cosine >= 0.999.

Also here, on one GPU: bounded device-side waits made to run out (a peer that never publishes),
which must end in an error status, never in a hang.
"""
import os
import socket
from dataclasses import replace

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

N_NEW = 9
P = 152          # divisible by 2, 4 and 8: the all-to-all prefill splits the prompt over the ranks


def _port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _cfg(moe):
    from hoid_optimized_models_b200.configs import LLAMA31_8B, QWEN3_30B_A3B
    if moe:
        return replace(QWEN3_30B_A3B, name="moe-ep-test", layers=2, vocab=4096, n_experts=32)
    return replace(LLAMA31_8B, name="llama-tp-test", layers=2, vocab=4096)


def _engine_kwargs(mode):
    # "layers": persistent kernel with the exchange inside; "gemv": one launch per phase with the
    # exchange fused into the GEMVs; "nccl": one launch per phase and library all-reduces
    # "a2a": expert-parallel prefill with the all-to-all dispatch / combine of token rows
    return {"layers": dict(fused_allreduce=True, fused_layers=True),
            "gemv": dict(fused_allreduce=True, fused_layers=False),
            "nccl": dict(fused_allreduce=False, fused_layers=False),
            "a2a": dict(fused_allreduce=True, ep_all_to_all=True)}[mode]


def _worker(rank, size, port, moe, mode, out):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=size, device_id=dev)
    try:
        from hoid_optimized_models_b200 import ops
        from hoid_optimized_models_b200.decoder import DenseDecoder
        from hoid_optimized_models_b200.weights import make_decoder_weights
        cfg = _cfg(moe)
        w = make_decoder_weights(cfg, 21)
        ids = torch.randint(0, cfg.vocab, (P,), generator=torch.Generator().manual_seed(21)).to(dev)
        eng = DenseDecoder(cfg, w, max_seq=P + N_NEW + 2, device=dev, tp_rank=rank, tp_size=size,
                           group=dist.group.WORLD, **_engine_kwargs(mode))
        assert (eng.link is not None) == (mode != "nccl")
        assert (eng.plan is not None) == (mode == "layers" and not moe)
        # host-driven steps, so that every step's logits can be compared with the oracle
        first = eng.prefill(ids)
        eng.capture()
        toks, rows, tok = [first], [], first
        for j in range(N_NEW - 1):
            rows.append(eng.step(tok, P + j).float().cpu().tolist())
            tok = int(eng.tok.item())
            toks.append(tok)
        ops.check_status(dev)                        # no bounded wait gave up
        out.put((rank, toks, rows))                  # plain data: the child exits right after
        out.close()
        out.join_thread()
        # a captured graph holds NCCL kernels: drop it before the communicator goes away, and
        # leave without the communicator teardown (it can block while graphs are alive)
        eng.graph = None
        del eng
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
    finally:
        os._exit(0)


def _run_ranks(target, size, args):
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _port()
    procs = [ctx.Process(target=target, args=(r, size, port, *args, out)) for r in range(size)]
    for p in procs:
        p.start()
    res, waited = [], 0
    while len(res) < len(procs):
        try:
            res.append(out.get(timeout=5))
        except Exception:                                    # queue.Empty
            waited += 5
            dead = [p.exitcode for p in procs if p.exitcode not in (None, 0)]
            if dead or waited > 400:                         # a rank crashed: do not wait for it
                for p in procs:
                    if p.is_alive():
                        p.kill()
                pytest.fail(f"rank exit codes {[p.exitcode for p in procs]} after {waited} s")
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    return sorted(res, key=lambda r: r[0])


# World sizes that fit the visible GPUs, decided at collection: on a one-GPU machine the eighteen
# engine cases and the three encoder cases below collapse into one skipped placeholder each instead
# of twenty-one skips that say the same thing.
_N_GPUS = torch.cuda.device_count() if torch.cuda.is_available() else 0
_WORLDS = [w for w in (2, 4, 8) if w <= _N_GPUS]
_NEEDS_GPUS = pytest.mark.skip(reason="multi-rank cases (world 2, 4 and 8) need at least two GPUs")
_MODES = [(False, "layers", "dense-layers"), (False, "gemv", "dense-gemv"), (False, "nccl", "dense-nccl"),
          (True, "gemv", "moe-fused"), (True, "nccl", "moe-nccl"), (True, "a2a", "moe-all-to-all")]
_ENGINE_CASES = [pytest.param(w, moe, mode, id=f"{name}-{w}") for w in _WORLDS for moe, mode, name in _MODES] or \
    [pytest.param(2, False, "gemv", id="needs-2-gpus", marks=_NEEDS_GPUS)]
_DP_CASES = [pytest.param(w, id=str(w)) for w in _WORLDS] or [pytest.param(2, id="needs-2-gpus", marks=_NEEDS_GPUS)]


@pytest.mark.parametrize("world,moe,mode", _ENGINE_CASES)
def test_ranks_match_oracle_and_one_rank(dev, world, moe, mode):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    from hoid_optimized_models_b200.decoder import DenseDecoder
    from hoid_optimized_models_b200.weights import make_decoder_weights
    from oracle.ref_decoder import decoder_forward
    cfg = _cfg(moe)
    w = make_decoder_weights(cfg, 21)
    ids_cpu = torch.randint(0, cfg.vocab, (P,), generator=torch.Generator().manual_seed(21))
    ids = ids_cpu.to(dev)
    ref = DenseDecoder(cfg, w, max_seq=P + N_NEW + 2, device=dev)
    first = ref.prefill(ids)
    ref.capture()
    toks_ref, rows_ref, tok = [first], [], first
    for j in range(N_NEW - 1):
        rows_ref.append(ref.step(tok, P + j).float().cpu())
        tok = int(ref.tok.item())
        toks_ref.append(tok)
    logits_ref = torch.stack(rows_ref)
    del ref
    res = _run_ranks(_worker, world, (moe, mode))
    for rank, toks, _ in res:
        assert toks == toks_ref, f"rank {rank}: {toks} vs {toks_ref}"
    # dense: vocabulary-sharded logits, one slice per rank
    full = (torch.tensor(res[0][2]) if moe
            else torch.cat([torch.tensor(r[2]) for r in res], dim=-1))
    err = float((full - logits_ref).abs().max() / logits_ref.abs().max())
    assert err < 1e-2, err
    # the oracle, teacher-forced over the tokens the ranks generated
    seq = torch.cat((ids_cpu, torch.tensor(toks_ref[:-1])))
    _, logits_or, _ = decoder_forward(cfg, w, seq, logits_rows=range(P, P + N_NEW - 1),
                                      keep_hidden=False)
    cos = torch.nn.functional.cosine_similarity(full, logits_or, dim=-1)
    if moe:
        # a decode step whose token is routed to a different expert at a near-tie of the router
        # (bf16 router input against the fp32 oracle; the one-rank engine does the same, see the
        # bound above) shows in the logits: allowed on a few steps, as in tests/test_decoder_gpu.py
        assert int((cos < 0.999).sum()) <= 3 and float(cos.min()) >= 0.99, cos.tolist()
    else:
        assert float(cos.min()) >= 0.999, float(cos.min())
    top2 = logits_or.topk(2, -1).values
    noise = (full - logits_or).abs().max(-1).values
    for j in range(N_NEW - 1):                               # greedy parity, near-ties excepted
        if toks_ref[j + 1] != int(logits_or[j].argmax()):
            assert float(top2[j, 0] - top2[j, 1]) <= 2 * float(noise[j]), f"step {j}"


def _dp_worker(rank, size, port, out):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=size, device_id=dev)
    try:
        from hoid_optimized_models_b200.encoder import XlmrEncoder
        from hoid_optimized_models_b200.weights import make_encoder_weights
        cfg, B, S, ids = _enc_case()
        eng = XlmrEncoder(cfg, make_encoder_weights(cfg, 31), batch=B, seq=S, device=dev,
                          dp_rank=rank, dp_size=size, group=dist.group.WORLD)
        per = B // size
        emb = eng.embed(ids[rank * per:(rank + 1) * per].to(dev))
        out.put((rank, emb.float().cpu().tolist()))
        out.close()
        out.join_thread()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
    finally:
        os._exit(0)


def _enc_case():
    from hoid_optimized_models_b200.configs import XLMR_LARGE
    cfg = replace(XLMR_LARGE, name="xlmr-dp-test", layers=2, vocab=4096)
    B, S = 8, 128
    ids = torch.randint(3, cfg.vocab, (B, S), generator=torch.Generator().manual_seed(31))
    return cfg, B, S, ids


@pytest.mark.parametrize("world", _DP_CASES)
def test_encoder_data_parallel_matches_oracle(dev, world):
    """Batch split over the ranks + all-gather of the pooled rows, against the fp32 oracle and the
    one-rank encoder."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    from hoid_optimized_models_b200.encoder import XlmrEncoder
    from hoid_optimized_models_b200.weights import make_encoder_weights
    from oracle.ref_encoder import encoder_forward
    cfg, B, S, ids = _enc_case()
    w = make_encoder_weights(cfg, 31)
    ref = XlmrEncoder(cfg, w, batch=B, seq=S, device=dev)
    emb_ref = ref.embed(ids.to(dev)).float().cpu()
    emb_or = encoder_forward(cfg, w, ids)[1]
    assert float(torch.nn.functional.cosine_similarity(emb_ref, emb_or, dim=-1).min()) > 0.999
    res = _run_ranks(_dp_worker, world, ())
    for rank, emb in res:                                    # every rank holds the whole batch
        e = torch.tensor(emb)
        assert float((e - emb_ref).abs().max()) < 1e-3, rank
        assert float(torch.nn.functional.cosine_similarity(e, emb_or, dim=-1).min()) > 0.999


# ----------------------------------------------------------------------------- bounded waits
def _silent_peer_link(dev, hidden):
    """A world-2 link whose second 'rank' is a buffer on this GPU that nothing ever writes:
    every wait on it must run out."""
    import ctypes as C
    from hoid_optimized_models_b200 import _lib
    lib = _lib.lib()
    nbytes = lib.b200_tp_buffer_bytes(2, hidden)
    bufs = (C.c_void_p * 2)()
    for i in range(2):
        p, h = C.c_void_p(), C.create_string_buffer(64)
        _lib.check(lib.b200_tp_alloc(C.byref(p), h, nbytes), "b200_tp_alloc")
        bufs[i] = p.value
    ctx = lib.b200_tp_create(bufs, 2, 0, hidden)
    assert ctx >= 0
    return ctx


def test_wait_on_a_silent_peer_times_out(dev):
    """gemv_tp_consume polls the peer's share of an all-reduce that is never published.  With a
    short budget the launch must return, report B200_ERR_TIMEOUT, and leave the GPU usable."""
    from hoid_optimized_models_b200 import ops
    from hoid_optimized_models_b200._lib import B200Error
    H, N = 1024, 512
    ctx = _silent_peer_link(dev, H)
    g = torch.Generator().manual_seed(5)
    w = (torch.randn(N, H, generator=g) * 0.02).to(torch.bfloat16).to(dev)
    x = torch.randn(H, generator=g).to(dev)
    y = torch.zeros(N, device=dev)
    ops.check_status(dev)
    try:
        ops.set_tuning(5, 200)                   # B200_TUNE_WAIT_KTICKS: ~0.1 ms
        ops.gemv_tp_consume(y, w, ctx, 0)
        torch.cuda.synchronize()
        with pytest.raises(B200Error, match="TIMEOUT"):
            ops.check_status(dev)
    finally:
        ops.set_tuning(5, 0)
    ops.gemv(y, x, w)                            # the context is intact
    ref = w.float().cpu() @ x.cpu()
    assert float((y.cpu() - ref).abs().max() / ref.abs().max()) < 1e-4
    ops.check_status(dev)


def test_persistent_kernel_wait_times_out(dev):
    """The persistent decode kernel on the same silent link: its gate|up phase waits for the
    peer's share of the o_proj all-reduce.  The wait runs out, every later wait falls through,
    the kernel ends, and the status word says why."""
    from hoid_optimized_models_b200 import ops
    from hoid_optimized_models_b200._lib import B200Error
    from hoid_optimized_models_b200.weights import rope_tables
    from hoid_optimized_models_b200.configs import LLAMA31_8B
    H, n_q, n_kv, hd, inter, L, max_seq = 1024, 8, 2, 128, 1024, 2, 64
    ctx = _silent_peer_link(dev, H)
    g = torch.Generator().manual_seed(6)
    bf = lambda *s: (torch.randn(*s, generator=g) * 0.02).to(torch.bfloat16).to(dev)
    wqkv = [bf((n_q + 2 * n_kv) * hd, H) for _ in range(L)]
    wo = [bf(H, n_q * hd) for _ in range(L)]
    wgu = [bf(2 * inter, H) for _ in range(L)]
    wd = [bf(H, inter) for _ in range(L)]
    ln = [torch.ones(H, dtype=torch.bfloat16, device=dev) for _ in range(L)]
    kv = torch.zeros(L, 2, n_kv, max_seq, hd, dtype=torch.bfloat16, device=dev)
    h = torch.randn(H, generator=g).to(dev)
    plan = ops.decode_layers_plan(wqkv, wo, wgu, wd, ln, ln, kv, [None] * L, [None] * L, h, tp_ctx=ctx)
    cos, sin = rope_tables(replace(LLAMA31_8B, head_dim=hd), max_seq, dev)
    kv_len = torch.tensor([5], dtype=torch.int32, device=dev)
    ws = ops.flash_decode_workspace(n_q, n_kv, hd, 2, dev)
    ops.check_status(dev)
    try:
        ops.set_tuning(5, 200)
        ops.decode_layers(plan, cos, sin, kv_len, ws, n_q, n_kv, 2, hd ** -0.5, 1e-5)
        torch.cuda.synchronize()
        with pytest.raises(B200Error, match="TIMEOUT"):
            ops.check_status(dev)
    finally:
        ops.set_tuning(5, 0)
    y = torch.zeros(H, device=dev)
    ops.gemv(y, h, wo[0])                        # the context is intact
    torch.cuda.synchronize()
    ops.check_status(dev)
