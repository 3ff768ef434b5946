"""MoE path on the GPU: router, permutation, gather / combine, decode experts and the
Qwen3-MoE-architecture engine.  Integer outputs (expert ids, permutation, offsets) are
bit-exact against torch on the CPU given identical router logits; floating-point outputs
use the tolerances stated in each test."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def bf(t):
    return t.to(torch.bfloat16)


def rel_err(a, b):
    return float((a.float().cpu() - b.float().cpu()).abs().max() / b.float().abs().max().clamp_min(1e-30))


@pytest.mark.parametrize("s,E,k", [(1, 128, 8), (77, 128, 8), (1000, 128, 8), (5, 32, 4), (3, 256, 2)])
def test_router_matches_torch_topk(dev, s, E, k):
    from hoid_optimized_models_b200 import ops
    from oracle.ref_decoder import moe_route
    g = torch.Generator().manual_seed(s + E)
    logits = torch.randn(s, E, generator=g) * 2
    ids_ref, w_ref = moe_route(logits, k)
    ids = torch.zeros(s, k, dtype=torch.int32, device=dev)
    w = torch.zeros(s, k, dtype=torch.float32, device=dev)
    ops.moe_router(ids, w, logits.to(dev))
    assert torch.equal(ids.cpu().long(), ids_ref), "expert ids must be bit-exact"
    assert rel_err(w, w_ref) < 1e-5
    # bf16 logits (the reference's router input dtype) and bf16-rounded weights
    lb = bf(logits)
    ids_ref2, w_ref2 = moe_route(lb.float(), k)
    # remove rows with exact ties between the k-th and (k+1)-th logit: torch.topk does not
    # promise an order there; the tie rule is tested separately below
    srt = lb.float().sort(-1, descending=True).values
    ok = srt[:, k - 1] != srt[:, k]
    for j in range(k - 1):
        ok &= srt[:, j] != srt[:, j + 1]
    ops.moe_router(ids, w, lb.to(dev), round_bf16=True)
    assert torch.equal(ids.cpu().long()[ok], ids_ref2[ok])
    assert rel_err(w.cpu()[ok], bf(w_ref2).float()[ok]) < 1e-2


def test_router_tie_break_is_lowest_index(dev):
    from hoid_optimized_models_b200 import ops
    logits = torch.zeros(2, 128)
    logits[0, [5, 90, 17, 64]] = 3.0            # four-way tie at the top, then zeros
    logits[1, :] = 1.0                          # all equal
    ids = torch.zeros(2, 8, dtype=torch.int32, device=dev)
    w = torch.zeros(2, 8, dtype=torch.float32, device=dev)
    ops.moe_router(ids, w, logits.to(dev))
    # stable descending sort = (value desc, index asc)
    ref = torch.sort(logits, dim=-1, descending=True, stable=True).indices[:, :8]
    assert torch.equal(ids.cpu().long(), ref)
    assert abs(float(w[1].sum()) - 1.0) < 1e-6


def test_router_non_finite_logit_reports_and_stays_in_range(dev):
    """One NaN logit turns the whole softmax row into NaN.  The router must still write valid
    expert numbers (the row's probabilities count as zero), flag the status word, and leave the
    other tokens alone; the expert sort downstream indexes shared memory with these ids."""
    from hoid_optimized_models_b200 import ops
    from hoid_optimized_models_b200._lib import B200Error
    g = torch.Generator().manual_seed(3)
    logits = torch.randn(5, 128, generator=g)
    logits[2, 77] = float("nan")
    logits[4, 3] = float("inf")
    ids = torch.full((5, 8), -7, dtype=torch.int32, device=dev)
    w = torch.zeros(5, 8, dtype=torch.float32, device=dev)
    ops.check_status(dev)
    ops.moe_router(ids, w, logits.to(dev))
    with pytest.raises(B200Error, match="NUMERIC"):
        ops.check_status(dev)
    ops.check_status(dev)                                # the word was cleared
    got = ids.cpu()
    assert int(got.min()) >= 0 and int(got.max()) < 128
    good = [0, 1, 3]
    ref = torch.sort(logits[good], dim=-1, descending=True, stable=True).indices[:, :8]
    assert torch.equal(got[good].long(), ref)
    assert torch.isfinite(w.cpu()).all()
    # and the sort takes them without a fault
    order = torch.zeros(40, dtype=torch.int32, device=dev)
    inv = torch.zeros(40, dtype=torch.int32, device=dev)
    offs = torch.zeros(129, dtype=torch.int32, device=dev)
    ops.moe_permute(order, inv, offs, ops.moe_permute_workspace(40, 128, dev), ids)
    ops.check_status(dev)
    assert int(offs[128]) == 40


def test_permute_reports_out_of_range_ids(dev):
    """Expert ids outside [0, E) are a caller error: they are sorted as expert 0 (every index
    stays in range) and the status word says so."""
    from hoid_optimized_models_b200 import ops
    from hoid_optimized_models_b200._lib import B200Error
    ids = torch.tensor([[3, 0x7fffffff], [-5, 1]], dtype=torch.int32, device=dev)
    order = torch.zeros(4, dtype=torch.int32, device=dev)
    inv = torch.zeros(4, dtype=torch.int32, device=dev)
    offs = torch.zeros(9, dtype=torch.int32, device=dev)
    ops.check_status(dev)
    ops.moe_permute(order, inv, offs, ops.moe_permute_workspace(4, 8, dev), ids)
    with pytest.raises(B200Error, match="ARG"):
        ops.check_status(dev)
    assert offs.cpu().tolist() == [0, 2, 3, 3, 4, 4, 4, 4, 4]
    assert sorted(order.cpu().tolist()) == [0, 1, 2, 3]


@pytest.mark.parametrize("S,E,k", [(1, 128, 8), (333, 128, 8), (8192, 128, 8), (50, 16, 2)])
def test_permute_matches_stable_argsort(dev, S, E, k):
    from hoid_optimized_models_b200 import ops
    g = torch.Generator().manual_seed(S)
    # realistic routing: k distinct experts per token, some experts empty
    scores = torch.randn(S, E, generator=g)
    scores[:, E // 3] = -100.0
    ids = scores.topk(k, -1).indices.to(torch.int32)
    flat = ids.reshape(-1)
    order_ref = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat.long(), minlength=E)
    offs_ref = torch.cat((torch.zeros(1, dtype=torch.long), counts.cumsum(0)))
    pairs = S * k
    order = torch.zeros(pairs, dtype=torch.int32, device=dev)
    inv = torch.zeros(pairs, dtype=torch.int32, device=dev)
    offs = torch.zeros(E + 1, dtype=torch.int32, device=dev)
    ws = ops.moe_permute_workspace(pairs, E, dev)
    ops.moe_permute(order, inv, offs, ws, ids.to(dev))
    assert torch.equal(order.cpu().long(), order_ref)
    assert torch.equal(offs.cpu().long(), offs_ref)
    assert torch.equal(inv.cpu().long()[order_ref], torch.arange(pairs))
    # gather + combine round trip: combining the gathered rows with weights w gives sum(w) * x
    H = 256
    x = bf(torch.randn(S, H, generator=g))
    wts = torch.rand(S, k, generator=g)
    xg = torch.empty(pairs, H, dtype=torch.bfloat16, device=dev)
    ops.moe_gather_rows(xg, x.to(dev), order, k)
    assert torch.equal(xg.cpu(), x[(order_ref // k)])
    out = torch.empty(S, H, dtype=torch.bfloat16, device=dev)
    ops.moe_combine(out, xg, inv, wts.to(dev), x.to(dev))
    ref = x.float() * (1 + wts.sum(-1, keepdim=True))
    assert rel_err(out, ref) < 1e-2
    # expert-parallel masking: the two halves of the experts sum to the whole
    parts = []
    for lo in (0, E // 2):
        o = torch.empty(S, H, dtype=torch.float32, device=dev).to(torch.bfloat16)
        ops.moe_combine(o, xg, inv, wts.to(dev), None, ids.to(dev), lo, E // 2)
        parts.append(o.float().cpu())
    assert rel_err(parts[0] + parts[1], x.float() * wts.sum(-1, keepdim=True)) < 2e-2


def test_decode_experts(dev):
    from hoid_optimized_models_b200 import ops
    from oracle.ref_decoder import rmsnorm
    g = torch.Generator().manual_seed(4)
    E, I, H, k = 16, 768, 2048, 8
    gu = bf(torch.randn(E, 2 * I, H, generator=g) * 0.03)      # HF layout: gate rows, then up rows
    dn = bf(torch.randn(E, H, I, generator=g) * 0.03)
    x = torch.randn(H, generator=g)
    nw = bf(1 + 0.1 * torch.randn(H, generator=g))
    ids = torch.tensor([3, 15, 0, 7, 8, 1, 12, 5], dtype=torch.int32)
    wts = torch.rand(k, generator=g)
    wts /= wts.sum()
    xn = rmsnorm(x, nw.float(), 1e-6)
    act_ref = torch.stack([wts[s] * torch.nn.functional.silu(gu[ids[s], :I].float() @ xn) *
                           (gu[ids[s], I:].float() @ xn) for s in range(k)])
    y_ref = x + sum(dn[ids[s]].float() @ act_ref[s] for s in range(k))
    gu_il = torch.stack((gu[:, :I], gu[:, I:]), dim=2).reshape(E, 2 * I, H).contiguous().to(dev)
    act = torch.empty(k, I, dtype=torch.float32, device=dev)
    ops.moe_decode_gate_up(act, x.to(dev), gu_il, ids.to(dev), wts.to(dev), norm_w=nw.to(dev), eps=1e-6)
    assert rel_err(act, act_ref) < 2e-4
    y = x.clone().to(dev)
    ops.moe_decode_down(y, act, dn.to(dev), ids.to(dev), resid=y)
    assert rel_err(y, y_ref) < 2e-4
    # expert parallel: two ranks holding half the experts each sum to the same result
    tot = torch.zeros(H)
    for lo in (0, E // 2):
        a2 = torch.empty(k, I, dtype=torch.float32, device=dev)
        ops.moe_decode_gate_up(a2, x.to(dev), gu_il[lo:lo + E // 2].contiguous(), ids.to(dev),
                               wts.to(dev), norm_w=nw.to(dev), eps=1e-6, expert_lo=lo)
        y2 = torch.empty(H, dtype=torch.float32, device=dev)
        ops.moe_decode_down(y2, a2, dn[lo:lo + E // 2].contiguous().to(dev), ids.to(dev),
                            expert_lo=lo)
        tot += y2.cpu()
    assert rel_err(x + tot, y_ref) < 2e-4


def test_qwen3_moe_arch(dev):
    from dataclasses import replace
    from hoid_optimized_models_b200.configs import QWEN3_30B_A3B
    from tests.test_decoder_gpu import _run
    cfg = replace(QWEN3_30B_A3B, name="qwen3-moe-L2", layers=2, vocab=8192, n_experts=32)
    _run(dev, cfg, P=200, seed=3)
