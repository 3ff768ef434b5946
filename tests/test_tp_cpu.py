"""Multi-rank host logic on CPU (gloo, world_size 2): the head / expert / vocabulary shards of
hoid_optimized_models_b200.tp, combined with the collectives the engine issues (all-reduce
after o_proj and down_proj or after the expert sum, all-gather of per-rank argmax records),
reproduce the unsharded fp32 oracle layer and the same greedy token."""
import os
import socket
from dataclasses import replace

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from hoid_optimized_models_b200 import tp
from hoid_optimized_models_b200.configs import LLAMA31_8B, QWEN3_30B_A3B
from hoid_optimized_models_b200.weights import make_decoder_weights
from oracle import ref_decoder as R


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _cfg(moe):
    base = QWEN3_30B_A3B if moe else LLAMA31_8B
    return replace(base, name="tp-test", hidden=128, layers=1, n_q=4, n_kv=2, head_dim=32,
                   inter=0 if moe else 256, vocab=512, n_experts=8 if moe else 0,
                   top_k=2 if moe else 0, moe_inter=64 if moe else 0)


def _layer_sharded(cfg, w, x, rank, size, cos, sin):
    """One decoder layer the way the engine runs it on `rank`, in fp32 on the CPU."""
    S, hd = x.shape[0], cfg.head_dim
    att = 1 if cfg.n_experts else size
    r = rank if att > 1 else 0
    wqkv, wo = tp.shard_attention(cfg, w, 0, r, att)
    nq, nkv = cfg.n_q // att, cfg.n_kv // att
    hn = R.rmsnorm(x, w["model.layers.0.input_layernorm.weight"].float(), cfg.eps)
    qkv = hn @ wqkv.float().T
    q = qkv[:, :nq * hd].view(S, nq, hd)
    k = qkv[:, nq * hd:(nq + nkv) * hd].view(S, nkv, hd)
    v = qkv[:, (nq + nkv) * hd:].view(S, nkv, hd)
    if cfg.qk_norm:
        q = R.rmsnorm(q, w["model.layers.0.self_attn.q_norm.weight"].float(), cfg.eps)
        k = R.rmsnorm(k, w["model.layers.0.self_attn.k_norm.weight"].float(), cfg.eps)
    q, k = R.rope_rotate(q, cos, sin), R.rope_rotate(k, cos, sin)
    a = R.causal_attention(q, k, v, hd ** -0.5).reshape(S, nq * hd)
    part = a @ wo.float().T
    if att > 1:
        if rank == 0:
            part = part + x                     # the residual is added once, on the lead rank
        dist.all_reduce(part)
        x = part
    else:
        x = x + part
    hn = R.rmsnorm(x, w["model.layers.0.post_attention_layernorm.weight"].float(), cfg.eps)
    if cfg.n_experts:
        gu, dn, lo = tp.shard_experts(cfg, w, 0, rank, size)
        ids, wt = R.moe_route(hn @ w["model.layers.0.mlp.gate.weight"].float().T, cfg.top_k)
        y = torch.zeros_like(x)
        for t in range(S):
            for s in range(cfg.top_k):
                e = int(ids[t, s]) - lo
                if 0 <= e < gu.shape[0]:
                    z = gu[e].float() @ hn[t]                   # interleaved gate / up rows
                    act = torch.nn.functional.silu(z[0::2]) * z[1::2] * wt[t, s]
                    y[t] += dn[e].float() @ act
        if rank == 0:
            y = y + x
        dist.all_reduce(y)
        return y
    gu, dn = tp.shard_mlp(cfg, w, 0, rank, size)
    z = hn @ gu.float().T
    part = (torch.nn.functional.silu(z[:, 0::2]) * z[:, 1::2]) @ dn.float().T
    if rank == 0:
        part = part + x
    dist.all_reduce(part)
    return part


def _worker(rank, size, port, moe, out):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=size)
    try:
        torch.set_num_threads(1)
        cfg = _cfg(moe)
        w = make_decoder_weights(cfg, 11)
        ids = torch.randint(0, cfg.vocab, (12,), generator=torch.Generator().manual_seed(1))
        hidden, logits, _ = R.decoder_forward(cfg, w, ids)
        x0 = hidden[0]
        ang = torch.arange(12, dtype=torch.float64)[:, None] * R.inv_freq(cfg)[None]
        x1 = _layer_sharded(cfg, w, x0, rank, size, ang.cos().float(), ang.sin().float())
        xn = R.rmsnorm(x1, w["model.norm.weight"].float(), cfg.eps)
        err = float((xn - hidden[1]).abs().max() / hidden[1].abs().max())
        # vocabulary-sharded head + all-gather of (max, argmax) records
        head = tp.shard_vocab(w["lm_head.weight"], rank, size).float()
        lg = head @ xn[-1]
        cand = torch.zeros(1, 2)
        cand[0, 0] = lg.max()
        cand.view(torch.int32)[0, 1] = int(lg.argmax()) + rank * head.shape[0]
        allc = torch.zeros(size, 2)
        dist.all_gather_into_tensor(allc, cand)
        tok = tp.merge_candidates(allc)
        out.put((rank, err, tok, int(logits[-1].argmax())))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("moe", [False, True])
def test_sharded_layer_matches_unsharded_oracle(moe):
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, moe, out)) for r in range(2)]
    for p in procs:
        p.start()
    res = [out.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err, tok, ref_tok in res:
        assert err < 1e-5, f"rank {rank}: {err}"
        assert tok == ref_tok


def test_divisibility_is_checked():
    with pytest.raises(ValueError):
        tp.check_divisible(LLAMA31_8B, 3)
    with pytest.raises(ValueError):
        tp.check_divisible(QWEN3_30B_A3B, 5)
    tp.check_divisible(LLAMA31_8B, 8)
    tp.check_divisible(QWEN3_30B_A3B, 8)


def test_merge_candidates_tie_rule():
    c = torch.zeros(3, 2)
    c[:, 0] = torch.tensor([2.0, 5.0, 5.0])
    ci = c.view(torch.int32)
    ci[0, 1], ci[1, 1], ci[2, 1] = 1, 900, 40
    assert tp.merge_candidates(c) == 40
