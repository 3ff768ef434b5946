"""The allocation-free flash-decode entry point, called through the C ABI.

It serves callers that may not allocate device memory (a plugin living inside another
framework's memory pool, a serving loop that forbids allocation after start-up), so its
scratch is a fixed array inside the library.  The check: on two calls in a row its output
equals the workspace-taking entry point's within the tolerance the flash-decode tests use
(2e-5 relative), and an oversized request is refused with B200_ERR_SCRATCH.  The file sorts
last so that a run stopping at the first failure has already executed every other test."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_pair(lib, dev, n_q, n_kv, hd, kv_len, n_splits, seed):
    g = torch.Generator().manual_seed(seed)
    max_seq = kv_len + 5
    q = torch.randn(n_q, hd, generator=g).to(dev)
    kc = torch.randn(n_kv, max_seq, hd, generator=g).to(torch.bfloat16).to(dev)
    vc = torch.randn(n_kv, max_seq, hd, generator=g).to(torch.bfloat16).to(dev)
    kl = torch.tensor([kv_len], dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    scale = hd ** -0.5
    # existing entry point: the caller brings a zeroed workspace
    nbytes = lib.b200_flash_decode_workspace_bytes(n_q, n_kv, hd, n_splits)
    ws = torch.zeros((nbytes + 3) // 4, dtype=torch.float32, device=dev)
    ref = torch.empty(n_q, hd, dtype=torch.float32, device=dev)
    rc = lib.b200_flash_decode(ref.data_ptr(), 1, q.data_ptr(), 1, kc.data_ptr(), vc.data_ptr(),
                               kl.data_ptr(), ws.data_ptr(), n_q, n_kv, hd, max_seq * hd, hd,
                               n_splits, scale, 0, stream)
    assert rc == 0
    out = torch.full((n_q, hd), float("nan"), dtype=torch.float32, device=dev)
    rc = lib.b200_flash_decode_static(out.data_ptr(), 1, q.data_ptr(), 1, kc.data_ptr(),
                                      vc.data_ptr(), kl.data_ptr(), n_q, n_kv, hd, max_seq * hd,
                                      hd, n_splits, scale, 0, stream)
    assert rc == 0
    torch.cuda.synchronize()
    err = float((out - ref).abs().max() / ref.abs().max())
    assert err < 2e-5, err


def test_static_scratch_matches_workspace_entry_point(dev):
    from hoid_optimized_models_b200 import _lib
    lib = _lib.lib()
    # two calls in a row with different shapes: the second finds the first's leftovers
    _call_pair(lib, dev, 32, 8, 128, 1500, 18, seed=1)
    _call_pair(lib, dev, 32, 8, 128, 777, 18, seed=2)
    _call_pair(lib, dev, 20, 20, 64, 300, 7, seed=3)


def test_static_scratch_rejects_oversized_requests(dev):
    from hoid_optimized_models_b200 import _lib
    lib = _lib.lib()
    cap = lib.b200_flash_decode_static_max_bytes()
    assert cap == 2 << 20
    n_q, n_kv, hd, n_splits = 64, 8, 128, 1024          # 8 * 1024 * (8*128 + 16) * 4 B > 2 MiB
    assert lib.b200_flash_decode_workspace_bytes(n_q, n_kv, hd, n_splits) > cap
    x = torch.zeros(n_q * hd, dtype=torch.float32, device=dev)
    kv = torch.zeros(n_kv, 8, hd, dtype=torch.bfloat16, device=dev)
    kl = torch.ones(1, dtype=torch.int32, device=dev)
    rc = lib.b200_flash_decode_static(x.data_ptr(), 1, x.data_ptr(), 1, kv.data_ptr(), kv.data_ptr(),
                                      kl.data_ptr(), n_q, n_kv, hd, 8 * hd, hd, n_splits, 0.1, 0,
                                      torch.cuda.current_stream().cuda_stream)
    assert rc == -7
