"""Per-op parity on the GPU: every b200 op against the same math in fp32 torch on the CPU
(oracle/ref_decoder.py helpers where they exist).  Tolerances are stated per test."""
import math

import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def bf(t):
    return t.to(torch.bfloat16)


def rel_err(a, b):
    return float((a.float().cpu() - b.float().cpu()).abs().max() / b.float().abs().max().clamp_min(1e-30))


# ----------------------------------------------------------------------------- GEMV
@pytest.mark.parametrize("K,N", [(4096, 4096), (4096, 6144), (14336, 4096), (2560, 9728 * 2),
                                 (2048, 128), (1280, 51866), (768, 2048), (256, 7)])
@pytest.mark.parametrize("xdt", [torch.float32, torch.bfloat16])
def test_gemv_plain(dev, K, N, xdt):
    from hoid_optimized_models_b200 import ops
    g = torch.Generator().manual_seed(K + N)
    w = bf(torch.randn(N, K, generator=g) * 0.02)
    x = torch.randn(K, generator=g).to(xdt)
    ref = w.float() @ x.float()
    y = torch.empty(N, dtype=torch.float32, device=dev)
    ops.gemv(y, x.to(dev), w.to(dev))
    torch.cuda.synchronize()
    # fp32 accumulation in a different order: 1e-4 of the output scale
    assert rel_err(y, ref) < 1e-4
    y2 = torch.empty(N, dtype=torch.float32, device=dev)
    ops.gemv(y2, x.to(dev), w.to(dev))
    assert torch.equal(y, y2), "GEMV must be bit-reproducible"


def test_gemv_fusions(dev):
    from hoid_optimized_models_b200 import ops
    from oracle.ref_decoder import rmsnorm
    g = torch.Generator().manual_seed(7)
    K, I = 4096, 14336
    h = torch.randn(K, generator=g)
    nw = bf(1 + 0.02 * torch.randn(K, generator=g))
    gate = bf(torch.randn(I, K, generator=g) * 0.02)
    up = bf(torch.randn(I, K, generator=g) * 0.02)
    xn = rmsnorm(h, nw.float(), 1e-5)
    ref = torch.nn.functional.silu(gate.float() @ xn) * (up.float() @ xn)
    wgu = torch.stack((gate, up), dim=1).reshape(2 * I, K).contiguous().to(dev)
    act = torch.empty(I, dtype=torch.float32, device=dev)
    ops.gemv(act, h.to(dev), wgu, norm_w=nw.to(dev), eps=1e-5, epilogue=ops.EPI_SWIGLU)
    assert rel_err(act, ref) < 2e-4
    # residual epilogue, in place, plus bias and bf16 output
    wd = bf(torch.randn(K, I, generator=g) * 0.02)
    bias = bf(torch.randn(K, generator=g))
    hres = h.clone().to(dev)
    ops.gemv(hres, act, wd.to(dev), resid=hres, bias=bias.to(dev))
    ref2 = h + wd.float() @ act.float().cpu() + bias.float()
    assert rel_err(hres, ref2) < 2e-4
    yb = torch.empty(K, dtype=torch.bfloat16, device=dev)
    ops.gemv(yb, act, wd.to(dev), epilogue=ops.EPI_GELU)
    ref3 = torch.nn.functional.gelu(wd.float() @ act.float().cpu())
    assert rel_err(yb, ref3) < 1e-2  # bf16 output rounding


def test_gemv_rejects_bad_shapes(dev):
    from hoid_optimized_models_b200 import ops
    from hoid_optimized_models_b200._lib import B200Error
    w = torch.zeros(8, 100, dtype=torch.bfloat16, device=dev)
    with pytest.raises(B200Error):
        ops.gemv(torch.zeros(8, device=dev), torch.zeros(100, device=dev), w)


# ----------------------------------------------------------------------------- norms
@pytest.mark.parametrize("rows,N", [(1, 4096), (5, 2560), (64, 2048), (3, 1024), (2, 1280), (1, 128)])
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float32])
def test_add_rmsnorm(dev, rows, N, dt):
    from hoid_optimized_models_b200 import ops
    from oracle.ref_decoder import rmsnorm
    g = torch.Generator().manual_seed(rows * N)
    a = torch.randn(rows, N, generator=g).to(dt)
    b = torch.randn(rows, N, generator=g).to(dt)
    w = bf(1 + 0.1 * torch.randn(N, generator=g))
    s = (a.float() + b.float()).to(dt)       # the stored residual is rounded first
    ref = rmsnorm(s.float(), w.float(), 1e-6)
    res = torch.empty(rows, N, dtype=dt, device=dev)
    out = torch.empty(rows, N, dtype=dt, device=dev)
    ops.add_rmsnorm(out, res, a.to(dev), b.to(dev), w.to(dev), 1e-6)
    assert torch.equal(res.cpu(), s)
    tol = 1e-2 if dt == torch.bfloat16 else 1e-5
    assert rel_err(out, ref) < tol
    out2 = torch.empty_like(out)
    ops.rmsnorm(out2, a.to(dev), w.to(dev), 1e-6)
    assert rel_err(out2, rmsnorm(a.float(), w.float(), 1e-6)) < tol


@pytest.mark.parametrize("rows,N", [(5, 4096), (3, 2560), (2, 2048)])
def test_add_rmsnorm_fp32_stream(dev, rows, N):
    """fp32 residual stream, bf16 delta, bf16 normalised output (the prefill layout)."""
    from hoid_optimized_models_b200 import ops
    from oracle.ref_decoder import rmsnorm
    g = torch.Generator().manual_seed(rows + N)
    a = torch.randn(rows, N, generator=g)
    b = bf(torch.randn(rows, N, generator=g))
    w = bf(1 + 0.1 * torch.randn(N, generator=g))
    s = a + b.float()
    res = a.clone().to(dev)
    out = torch.empty(rows, N, dtype=torch.bfloat16, device=dev)
    ops.add_rmsnorm(out, res, res, b.to(dev), w.to(dev), 1e-6)     # in place on the stream
    assert torch.equal(res.cpu(), s)
    assert rel_err(out, rmsnorm(s, w.float(), 1e-6)) < 1e-2
    out2 = torch.empty_like(out)
    ops.rmsnorm(out2, res, w.to(dev), 1e-6)
    assert torch.equal(out2, out)


@pytest.mark.parametrize("rows,N", [(7, 1024), (3, 1280), (1, 4096)])
def test_add_layernorm(dev, rows, N):
    from hoid_optimized_models_b200 import ops
    g = torch.Generator().manual_seed(N)
    x = bf(torch.randn(rows, N, generator=g))
    bias = bf(torch.randn(N, generator=g))
    r = bf(torch.randn(rows, N, generator=g))
    gamma = bf(1 + 0.1 * torch.randn(N, generator=g))
    beta = bf(0.1 * torch.randn(N, generator=g))
    s = bf(bf(x.float() + bias.float()).float() + r.float())   # reference rounds each addition
    ref = torch.nn.functional.layer_norm(s.float(), (N,), gamma.float(), beta.float(), 1e-5)
    res = torch.empty(rows, N, dtype=torch.bfloat16, device=dev)
    out = torch.empty(rows, N, dtype=torch.bfloat16, device=dev)
    ops.add_layernorm(out, res, x.to(dev), gamma.to(dev), beta.to(dev), 1e-5, bias=bias.to(dev),
                      resid=r.to(dev))
    assert torch.equal(res.cpu(), s)
    assert rel_err(out, ref) < 1e-2
    # plain fp32 LayerNorm
    xf = torch.randn(rows, N, generator=g)
    outf = torch.empty(rows, N, dtype=torch.float32, device=dev)
    ops.layernorm(outf, xf.to(dev), gamma.to(dev), beta.to(dev), 1e-5)
    reff = torch.nn.functional.layer_norm(xf, (N,), gamma.float(), beta.float(), 1e-5)
    assert rel_err(outf, reff) < 1e-5


# ----------------------------------------------------------------------------- rope + cache
@pytest.mark.parametrize("s,n_q,n_kv,hd,qk_norm", [(1, 32, 8, 128, False), (5, 32, 8, 128, True),
                                                   (3, 32, 4, 128, True), (2, 4, 4, 64, False)])
def test_qk_rope_cache(dev, s, n_q, n_kv, hd, qk_norm):
    from hoid_optimized_models_b200 import ops
    from oracle.ref_decoder import rmsnorm, rope_rotate
    g = torch.Generator().manual_seed(s + n_q)
    max_seq, pos0 = 40, 9
    qkv = torch.randn(s, (n_q + 2 * n_kv) * hd, generator=g)
    qn = bf(1 + 0.1 * torch.randn(hd, generator=g))
    kn = bf(1 + 0.1 * torch.randn(hd, generator=g))
    ang = torch.arange(max_seq, dtype=torch.float64)[:, None] * (
        1e4 ** (-torch.arange(0, hd, 2, dtype=torch.float64) / hd))[None]
    cos, sin = ang.cos().float(), ang.sin().float()
    q = qkv[:, :n_q * hd].view(s, n_q, hd)
    k = qkv[:, n_q * hd:(n_q + n_kv) * hd].view(s, n_kv, hd)
    v = qkv[:, (n_q + n_kv) * hd:].view(s, n_kv, hd)
    if qk_norm:
        q, k = rmsnorm(q, qn.float(), 1e-6), rmsnorm(k, kn.float(), 1e-6)
    qr = rope_rotate(q, cos[pos0:pos0 + s], sin[pos0:pos0 + s])
    kr = rope_rotate(k, cos[pos0:pos0 + s], sin[pos0:pos0 + s])
    kc = torch.zeros(n_kv, max_seq, hd, dtype=torch.bfloat16, device=dev)
    vc = torch.zeros_like(kc)
    qo = torch.empty(s, n_q * hd, dtype=torch.float32, device=dev)
    pos = torch.tensor([pos0], dtype=torch.int32, device=dev)
    ops.qk_rope_cache(qo, kc, vc, qkv.to(dev), cos.to(dev), sin.to(dev), pos, n_q, n_kv, eps=1e-6,
                      qn_w=qn.to(dev) if qk_norm else None, kn_w=kn.to(dev) if qk_norm else None)
    assert rel_err(qo.view(s, n_q, hd), qr) < 1e-5
    assert torch.equal(kc[:, pos0:pos0 + s].cpu(), bf(kr.permute(1, 0, 2))) or \
        rel_err(kc[:, pos0:pos0 + s], kr.permute(1, 0, 2)) < 1e-2
    assert torch.equal(vc[:, pos0:pos0 + s].cpu(), bf(v.permute(1, 0, 2)))
    # rows outside [pos0, pos0 + s) stay untouched
    assert float(kc[:, :pos0].abs().max()) == 0 and float(kc[:, pos0 + s:].abs().max()) == 0


# ----------------------------------------------------------------------------- flash decode
@pytest.mark.parametrize("n_q,n_kv,hd,kv_len,n_splits", [
    (32, 8, 128, 1, 4), (32, 8, 128, 37, 16), (32, 8, 128, 1500, 37), (32, 4, 128, 1025, 64),
    (20, 20, 64, 1500, 8), (20, 20, 64, 5, 8), (4, 1, 128, 700, 74), (8, 4, 64, 333, 5)])
def test_flash_decode(dev, n_q, n_kv, hd, kv_len, n_splits):
    from hoid_optimized_models_b200 import ops
    g = torch.Generator().manual_seed(kv_len)
    max_seq = kv_len + 3
    q = torch.randn(n_q, hd, generator=g)
    kc = bf(torch.randn(n_kv, max_seq, hd, generator=g))
    vc = bf(torch.randn(n_kv, max_seq, hd, generator=g))
    G = n_q // n_kv
    kk = kc[:, :kv_len].float().repeat_interleave(G, 0)
    vv = vc[:, :kv_len].float().repeat_interleave(G, 0)
    p = torch.softmax(torch.einsum("hd,hkd->hk", q, kk) * hd ** -0.5, -1)
    ref = torch.einsum("hk,hkd->hd", p, vv)
    out = torch.empty(n_q, hd, dtype=torch.float32, device=dev)
    ws = ops.flash_decode_workspace(n_q, n_kv, hd, n_splits, dev)
    kl = torch.tensor([kv_len], dtype=torch.int32, device=dev)
    for _ in range(2):  # second call checks that the arrival counters were left at zero
        out.zero_()
        ops.flash_decode(out, q.to(dev), kc.to(dev), vc.to(dev), kl, ws, n_q, n_kv, n_splits,
                         hd ** -0.5)
        # the tensor-core kernel carries q and P as bf16 high + low parts (~16 mantissa bits)
        assert rel_err(out, ref) < 5e-5


@pytest.mark.parametrize("n_q,n_kv,hd,kv_len,n_splits,qk_norm", [
    (32, 8, 128, 1, 4, False), (32, 8, 128, 37, 16, False), (32, 8, 128, 1500, 37, False),
    (32, 8, 128, 8193, 18, False), (32, 8, 128, 1024, 16, True), (32, 4, 128, 1025, 37, True),
    (16, 4, 128, 129, 8, False), (20, 20, 64, 300, 7, False), (8, 4, 64, 333, 5, True),
    (4, 1, 128, 700, 74, False)])
def test_rope_flash_decode_matches_two_kernels(dev, n_q, n_kv, hd, kv_len, n_splits, qk_norm):
    """The fused launch against qk_rope_cache followed by flash_decode: same attention output,
    same appended cache row, every other cache row untouched."""
    from hoid_optimized_models_b200 import ops
    g = torch.Generator().manual_seed(kv_len + n_splits)
    max_seq = kv_len + 2
    pos = kv_len - 1
    qkv = torch.randn((n_q + 2 * n_kv) * hd, generator=g).to(dev)
    kc = bf(torch.randn(n_kv, max_seq, hd, generator=g)).to(dev)
    vc = bf(torch.randn(n_kv, max_seq, hd, generator=g)).to(dev)
    ang = torch.arange(max_seq, dtype=torch.float64)[:, None] * \
        (10000.0 ** (-torch.arange(hd // 2, dtype=torch.float64) * 2 / hd))[None, :]
    cos, sin = ang.cos().float().to(dev), ang.sin().float().to(dev)
    qn = bf(1 + 0.1 * torch.randn(hd, generator=g)).to(dev) if qk_norm else None
    kn = bf(1 + 0.1 * torch.randn(hd, generator=g)).to(dev) if qk_norm else None
    kl = torch.tensor([kv_len], dtype=torch.int32, device=dev)
    pd = torch.tensor([pos], dtype=torch.int32, device=dev)
    ws = ops.flash_decode_workspace(n_q, n_kv, hd, n_splits, dev)
    # two kernels
    k2, v2 = kc.clone(), vc.clone()
    q2 = torch.empty(n_q * hd, dtype=torch.float32, device=dev)
    out2 = torch.empty(n_q, hd, dtype=torch.float32, device=dev)
    ops.qk_rope_cache(q2, k2, v2, qkv, cos, sin, pd, n_q, n_kv, eps=1e-6, qn_w=qn, kn_w=kn)
    ops.flash_decode(out2, q2, k2, v2, kl, ws, n_q, n_kv, n_splits, hd ** -0.5)
    # one kernel, twice (the second call checks the counters and overwrites the same row)
    k1, v1 = kc.clone(), vc.clone()
    out1 = torch.empty(n_q, hd, dtype=torch.float32, device=dev)
    for _ in range(2):
        out1.zero_()
        ops.rope_flash_decode(out1, k1, v1, ws, qkv, cos, sin, kl, n_q, n_kv, n_splits,
                              hd ** -0.5, eps=1e-6, qn_w=qn, kn_w=kn)
        assert rel_err(out1, out2.cpu()) < 5e-5
        # the appended row: bf16 of the same fp32 arithmetic (an fma contraction may move one ulp)
        assert rel_err(k1[:, pos], k2[:, pos].cpu()) < 1e-2
        assert torch.equal(v1, v2)
        keep = torch.ones(max_seq, dtype=torch.bool, device=dev)
        keep[pos] = False
        assert torch.equal(k1[:, keep], kc[:, keep])


def test_flash_decode_strided_cross_kv(dev):
    """Whisper cross-attention layout: K/V rows are [1500, 20 * 64] projections."""
    from hoid_optimized_models_b200 import ops
    g = torch.Generator().manual_seed(3)
    H, hd, L = 20, 64, 1500
    q = torch.randn(H, hd, generator=g)
    k = bf(torch.randn(L, H * hd, generator=g))
    v = bf(torch.randn(L, H * hd, generator=g))
    kk = k.float().view(L, H, hd).permute(1, 0, 2)
    vv = v.float().view(L, H, hd).permute(1, 0, 2)
    p = torch.softmax(torch.einsum("hd,hkd->hk", q, kk) * hd ** -0.5, -1)
    ref = torch.einsum("hk,hkd->hd", p, vv)
    out = torch.empty(H, hd, dtype=torch.float32, device=dev)
    ws = ops.flash_decode_workspace(H, H, hd, 16, dev)
    kl = torch.tensor([L], dtype=torch.int32, device=dev)
    ops.flash_decode(out, q.to(dev), k.to(dev), v.to(dev), kl, ws, H, H, 16, hd ** -0.5,
                     kv_head_stride=hd, kv_row_stride=H * hd)
    assert rel_err(out, ref) < 5e-5


# ----------------------------------------------------------------------------- small ops
def test_embed_silu_argmax(dev):
    from hoid_optimized_models_b200 import ops
    g = torch.Generator().manual_seed(11)
    table = bf(torch.randn(1000, 2560, generator=g))
    ids = torch.tensor([3, 999, 0, 512, 3], dtype=torch.int32)
    o32 = torch.empty(5, 2560, dtype=torch.float32, device=dev)
    o16 = torch.empty(5, 2560, dtype=torch.bfloat16, device=dev)
    ops.embed_gather(o32, table.to(dev), ids.to(dev))
    ops.embed_gather(o16, table.to(dev), ids.to(dev))
    assert torch.equal(o32.cpu(), table[ids.long()].float())
    assert torch.equal(o16.cpu(), table[ids.long()])
    a, b = bf(torch.randn(3, 14336, generator=g)), bf(torch.randn(3, 14336, generator=g))
    o = torch.empty(3, 14336, dtype=torch.bfloat16, device=dev)
    ops.silu_mul(o, a.to(dev), b.to(dev))
    assert rel_err(o, torch.nn.functional.silu(a.float()) * b.float()) < 1e-2
    ws = ops.argmax_workspace(dev)
    for n in (1, 5, 4096, 128256, 151936):
        x = torch.randn(n, generator=g)
        x[n // 2] = 50.0
        if n > 4:
            x[n - 2] = 50.0           # tie: the lower index must win
        cand = torch.zeros(2, dtype=torch.float32, device=dev)
        ops.argmax(cand, x.to(dev), ws, idx_base=7)
        assert int(cand.view(torch.int32)[1]) == n // 2 + 7
        assert float(cand[0]) == 50.0
    # greedy_select across "ranks" + state advance
    cands = torch.tensor([[1.0, 0], [3.0, 0], [3.0, 0]], dtype=torch.float32)
    ci = cands.view(torch.int32)
    ci[0, 1], ci[1, 1], ci[2, 1] = 5, 900, 40
    tok = torch.zeros(1, dtype=torch.int32, device=dev)
    state = torch.tensor([10, 11, 2, 0], dtype=torch.int32, device=dev)
    log = torch.zeros(8, dtype=torch.int32, device=dev)
    ops.greedy_advance(tok, state, log, cands.to(dev))
    assert int(tok) == 40 and state.tolist() == [11, 12, 3, 0] and int(log[2]) == 40


# ----------------------------------------------------------------------------- GEMM (tcgen05)
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 512), (256, 512, 4096), (1500, 1280, 1280),
                                   (8192, 6144, 4096), (77, 136, 72), (300, 28672, 4096)])
def test_gemm_plain(dev, M, N, K):
    from hoid_optimized_models_b200 import ops
    g = torch.Generator(device=dev).manual_seed(M + N + K)
    x = bf(torch.randn(M, K, generator=g, device=dev))
    w = bf(torch.randn(N, K, generator=g, device=dev) * 0.05)
    y = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    ops.gemm(y, x, w)
    ops.check_status(dev)
    # fp32 reference on a sample of rows (full product for small cases)
    rows = torch.arange(M) if M * N * K < 2 ** 32 else torch.randint(0, M, (64,))
    ref = x[rows.to(dev)].float() @ w.float().T
    assert rel_err(y[rows.to(dev)], ref) < 8e-3   # one bf16 rounding of the output


@pytest.mark.parametrize("bn", [256, 128, 64])
def test_gemm_tile_widths(dev, bn):
    """Every tile width, forced through the tuning knob, on shapes with M / N / K tails."""
    from hoid_optimized_models_b200 import ops, _lib
    g = torch.Generator(device=dev).manual_seed(bn)
    try:
        _lib.lib().b200_set_tuning(1, bn)
        for (M, N, K) in [(300, 1280, 1280), (1500, 136, 72), (129, 512, 4096)]:
            x = bf(torch.randn(M, K, generator=g, device=dev))
            w = bf(torch.randn(N, K, generator=g, device=dev) * 0.05)
            b = bf(torch.randn(N, generator=g, device=dev))
            r = bf(torch.randn(M, N, generator=g, device=dev))
            y = r.clone()
            ops.gemm(y, x, w, bias=b, resid=y)
            ops.check_status(dev)
            ref = r.float() + x.float() @ w.float().T + b.float()
            assert rel_err(y, ref) < 1e-2, (bn, M, N, K)
            yf = torch.empty(M, N, dtype=torch.float32, device=dev)
            ops.gemm(yf, x, w)
            assert rel_err(yf, x.float() @ w.float().T) < 1e-4, (bn, M, N, K)
    finally:
        _lib.lib().b200_set_tuning(1, 0)


def test_gemm_epilogues(dev):
    from hoid_optimized_models_b200 import ops
    g = torch.Generator(device=dev).manual_seed(5)
    M, K, I = 333, 1024, 1536
    x = bf(torch.randn(M, K, generator=g, device=dev))
    gate = bf(torch.randn(I, K, generator=g, device=dev) * 0.03)
    up = bf(torch.randn(I, K, generator=g, device=dev) * 0.03)
    wgu = torch.stack((gate, up), 1).reshape(2 * I, K).contiguous()
    act = torch.empty(M, I, dtype=torch.bfloat16, device=dev)
    ops.gemm(act, x, wgu, epilogue=ops.EPI_SWIGLU)
    ref = torch.nn.functional.silu(x.float() @ gate.float().T) * (x.float() @ up.float().T)
    assert rel_err(act, ref) < 1e-2
    wd = bf(torch.randn(K, I, generator=g, device=dev) * 0.03)
    bias = bf(torch.randn(K, generator=g, device=dev))
    res = bf(torch.randn(M, K, generator=g, device=dev))
    y = res.clone()
    ops.gemm(y, act, wd, bias=bias, resid=y)
    ref2 = res.float() + act.float() @ wd.float().T + bias.float()
    assert rel_err(y, ref2) < 1e-2
    y3 = torch.empty(M, K, dtype=torch.bfloat16, device=dev)
    ops.gemm(y3, act, wd, bias=bias, epilogue=ops.EPI_GELU)
    ref3 = torch.nn.functional.gelu(act.float() @ wd.float().T + bias.float())
    assert rel_err(y3, ref3) < 1e-2
    ops.check_status(dev)


def test_moe_grouped_gemm(dev):
    from hoid_optimized_models_b200 import ops
    g = torch.Generator(device=dev).manual_seed(9)
    E, K, N = 16, 2048, 1536
    counts = torch.tensor([0, 5, 300, 128, 1, 0, 129, 64, 700, 3, 0, 0, 256, 17, 90, 2])
    offs = torch.zeros(E + 1, dtype=torch.int32)
    offs[1:] = counts.cumsum(0)
    rows = int(offs[-1])
    x = bf(torch.randn(rows, K, generator=g, device=dev))
    w = bf(torch.randn(E, N, K, generator=g, device=dev) * 0.03)
    y = torch.full((rows, N), float("nan"), dtype=torch.bfloat16, device=dev)
    ops.moe_grouped_gemm(y, x, w, offs.to(dev))
    ops.check_status(dev)
    for e in range(E):
        a, b = int(offs[e]), int(offs[e + 1])
        if b > a:
            ref = x[a:b].float() @ w[e].float().T
            assert rel_err(y[a:b], ref) < 1e-2, f"expert {e}"


@pytest.mark.parametrize("M,K,O", [(300, 640, 2560), (4096, 1280, 5120), (130, 64, 200)])
def test_gemm_geglu(dev, M, K, O):
    """Stock GEGLU projection [2 O, K], value half first: (x Wv^T + bv) * gelu(x Wg^T + bg) from one
    GEMM launch (the dual-GEMM of models/sdxl/kernels/dual_geglu.cutedsl.py)."""
    from hoid_optimized_models_b200 import ops
    g = torch.Generator().manual_seed(M + O)
    x = bf(torch.randn(M, K, generator=g)).to(dev)
    w = bf(torch.randn(2 * O, K, generator=g) * K ** -0.5).to(dev)
    b = bf(torch.randn(2 * O, generator=g) * 0.1).to(dev)
    y = torch.full((M, O), float("nan"), dtype=torch.bfloat16, device=dev)
    ops.gemm(y, x, w, bias=b, epilogue=ops.EPI_GEGLU)
    ops.check_status(dev)
    full = x.float() @ w.float().T + b.float()
    ref = full[:, :O] * torch.nn.functional.gelu(full[:, O:])
    assert rel_err(y, ref) < 1e-2


# ----------------------------------------------------------------------------- flash prefill
@pytest.mark.parametrize("S,n_q,n_kv,hd,causal", [(64, 4, 1, 128, True), (200, 8, 2, 128, True),
                                                  (1000, 32, 8, 128, True), (512, 16, 16, 64, False),
                                                  (77, 4, 4, 64, False), (1500, 20, 20, 64, False)])
def test_flash_prefill(dev, S, n_q, n_kv, hd, causal):
    from hoid_optimized_models_b200 import ops
    from oracle.ref_decoder import causal_attention
    g = torch.Generator().manual_seed(S)
    max_seq = S + 5
    q = bf(torch.randn(S, n_q, hd, generator=g))
    kc = bf(torch.randn(n_kv, max_seq, hd, generator=g))
    vc = bf(torch.randn(n_kv, max_seq, hd, generator=g))
    k = kc[:, :S].float().permute(1, 0, 2)
    v = vc[:, :S].float().permute(1, 0, 2)
    if causal:
        ref = causal_attention(q.float(), k, v, hd ** -0.5)
    else:
        G = n_q // n_kv
        kk = k.permute(1, 0, 2).repeat_interleave(G, 0)
        vv = v.permute(1, 0, 2).repeat_interleave(G, 0)
        p = torch.softmax(torch.einsum("shd,hkd->hsk", q.float(), kk) * hd ** -0.5, -1)
        ref = torch.einsum("hsk,hkd->shd", p, vv)
    out = torch.empty(1, S, n_q, hd, dtype=torch.bfloat16, device=dev)
    ops.flash_prefill(out, q.to(dev).view(1, S, n_q, hd), kc.to(dev).unsqueeze(0),
                      vc.to(dev).unsqueeze(0), S, causal, hd ** -0.5)
    ops.check_status(dev)
    # P and the output are rounded to bf16
    assert rel_err(out[0], ref) < 2e-2


@pytest.mark.parametrize("S,n_q,n_kv,hd,causal", [(640, 4, 2, 128, False), (900, 4, 4, 64, False),
                                                  (1100, 8, 2, 128, True)])
def test_flash_prefill_growing_row_maxima(dev, S, n_q, n_kv, hd, causal):
    """Keys grow with position, so the row maxima rise by far more than 2^8 from one key tile to
    the next: every tile takes the path that rescales the output accumulator in tensor memory
    (with well-scaled inputs the reference maximum is almost never raised after the first tile)."""
    from hoid_optimized_models_b200 import ops
    g = torch.Generator().manual_seed(S)
    q = bf(torch.randn(1, S, n_q, hd, generator=g) * 2.0)
    grow = (1.0 + 7.0 * torch.arange(S + 2) / S).view(1, 1, S + 2, 1)
    kc = bf(torch.randn(1, n_kv, S + 2, hd, generator=g) * grow)
    vc = bf(torch.randn(1, n_kv, S + 2, hd, generator=g))
    G = n_q // n_kv
    kk = kc[:, :, :S].float().repeat_interleave(G, 1)
    vv = vc[:, :, :S].float().repeat_interleave(G, 1)
    sc = torch.einsum("bshd,bhkd->bhsk", q.float(), kk) * hd ** -0.5
    if causal:
        sc = sc.masked_fill(torch.ones(S, S, dtype=torch.bool).triu(1), float("-inf"))
    # the scores really do outgrow the lazy-rescale threshold (8 in log2 units) tile after tile
    tile_max = torch.stack([sc[..., j:j + 128].amax(-1) for j in range(0, S - 127, 128)], -1) * 1.4427
    last_rows = tile_max[:, :, -64:]                    # these see every key tile, causal or not
    assert float((last_rows[..., -1] - last_rows[..., 0]).median()) > 16
    ref = torch.einsum("bhsk,bhkd->bshd", torch.softmax(sc, -1), vv)
    out = torch.full((1, S, n_q, hd), float("nan"), dtype=torch.bfloat16, device=dev)
    ops.flash_prefill(out, q.to(dev), kc.to(dev), vc.to(dev), S, causal, hd ** -0.5)
    ops.check_status(dev)
    assert rel_err(out, ref) < 2e-2


@pytest.mark.parametrize("B,S,n_q,n_kv,hd,causal", [(12, 512, 16, 16, 64, False), (5, 700, 8, 2, 128, True),
                                                     (3, 130, 6, 6, 64, False),
                                                     # three query tiles per head: every second work item has
                                                     # no rows for its second stream, and with more items than
                                                     # SMs a CTA walks both kinds back to back
                                                     (8, 300, 16, 4, 128, True), (10, 300, 16, 16, 64, False)])
def test_flash_prefill_batched_many_rounds(dev, B, S, n_q, n_kv, hd, causal):
    """More work items than SMs: every CTA walks several (batch, head, query tile) items back
    to back, with the Q / K / V rings and the S accumulators carried across item boundaries."""
    from hoid_optimized_models_b200 import ops
    g = torch.Generator().manual_seed(B * S)
    q = bf(torch.randn(B, S, n_q, hd, generator=g))
    kc = bf(torch.randn(B, n_kv, S + 3, hd, generator=g))
    vc = bf(torch.randn(B, n_kv, S + 3, hd, generator=g))
    G = n_q // n_kv
    kk = kc[:, :, :S].float().repeat_interleave(G, 1)
    vv = vc[:, :, :S].float().repeat_interleave(G, 1)
    sc = torch.einsum("bshd,bhkd->bhsk", q.float(), kk) * hd ** -0.5
    if causal:
        sc = sc.masked_fill(torch.ones(S, S, dtype=torch.bool).triu(1), float("-inf"))
    ref = torch.einsum("bhsk,bhkd->bshd", torch.softmax(sc, -1), vv)
    out = torch.full((B, S, n_q, hd), float("nan"), dtype=torch.bfloat16, device=dev)
    ops.flash_prefill(out, q.to(dev), kc.to(dev), vc.to(dev), S, causal, hd ** -0.5)
    ops.check_status(dev)
    assert rel_err(out, ref) < 2e-2
