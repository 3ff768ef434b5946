"""Host-side helpers of bench.py that can be checked without a GPU: the peak lookup, the parsing
of the clock / throttle samples, and the bounded CPU arm's record."""
import importlib.util
import json
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_peak_lookup_prefers_the_measured_file(tmp_path):
    b = _bench()
    b.ROOT = str(tmp_path)
    assert b.measured_peaks() == (6650.0, "fallback")
    with open(tmp_path / "MEASURED_PEAKS.json", "w") as f:
        json.dump({"hbm_gbs": 6538.6, "bf16_tflops": 1615.9}, f)
    assert b.measured_peaks() == (6538.6, "measured")


def test_clock_samples_are_summarised(tmp_path):
    b = _bench()
    s = b.ClockSampler(0)
    s.path = str(tmp_path / "clocks.csv")
    with open(s.path, "w") as f:
        f.write("0, 1905, 1965, 812.4, 0x0000000000000004, Not Active, Not Active, Not Active, Active\n")
        f.write("0, 1875, 1965, 955.0, 0x0000000000000004, Not Active, Not Active, Not Active, Active\n")
        f.write("0, 1920, 1965, 700.1, 0x0000000000000000, Not Active, Not Active, Not Active, Not Active\n")
        f.write("garbage line\n")
    out = s.summary()
    assert out == {"sm_mhz": 1905.0, "sm_max_mhz": 1965.0, "reasons": ["sw_power_cap"], "samples": 3}
    assert not os.path.exists(s.path)
    # no samples (nvidia-smi missing): an explicit empty record, not an exception
    assert b.ClockSampler(0).summary()["samples"] == 0


def test_cpu_arm_record_on_a_tiny_model():
    from dataclasses import replace
    from hoid_optimized_models_b200.configs import LLAMA31_8B
    b = _bench()
    cfg = replace(LLAMA31_8B, name="cpu-arm-test", hidden=128, inter=256, n_q=4, n_kv=2, layers=8,
                  vocab=256)
    rec = b.cpu_reference(cfg, ctx=32, steps=2, warmup=1, sample_layers=2)
    assert rec["kind"] == "reference" and rec["unit"] == "tok/s" and rec["cores"] >= 1
    assert rec["value"] > 0 and abs(rec["ms_per_step"] - 1e3 / rec["value"]) < 1e-6
    assert "2 of 8 layers" in rec["sample"] and "scaled x4" in rec["sample"]


def test_traffic_is_read_from_the_tracked_figures_file(tmp_path):
    """roofline.traffic comes from profiles/ncu_traffic.json (written beside the ncu summaries),
    scaled by depth when the capture was taken on a reduced-depth model; no file, no number."""
    b = _bench()
    tracked = b.ncu_traffic("gemv_kernel_gate_up", 32)
    assert tracked is not None and 2.3e8 < tracked < 2.5e8          # the committed capture
    b.ROOT = str(tmp_path)
    assert b.ncu_traffic("gemv_kernel_gate_up", 32) is None
    os.makedirs(tmp_path / "profiles")
    with open(tmp_path / "profiles" / "ncu_traffic.json", "w") as f:
        json.dump({"k": {"dram_bytes_per_launch": 100.0, "layers": 2}, "flat": {"dram_bytes_per_launch": 7.0}}, f)
    assert b.ncu_traffic("k", 32) == 1600.0 and b.ncu_traffic("flat", 32) == 7.0
    assert b.ncu_traffic("missing", 32) is None


def test_fake_gemm_epilogues_follow_the_abi_conventions():
    """The CPU stand-in of ops.gemm used by the host-logic tests implements the same epilogue
    conventions as the library: SwiGLU over interleaved gate / up rows, GEGLU over a stock
    [value half; gate half] projection."""
    import torch
    from tests import fake_ops
    g = torch.Generator().manual_seed(3)
    x = torch.randn(5, 16, generator=g)
    w = torch.randn(24, 16, generator=g)
    b = torch.randn(24, generator=g)
    full = x @ w.T + b
    y = torch.empty(5, 12)
    fake_ops.gemm(y, x, w, bias=b, epilogue=fake_ops.EPI_GEGLU)
    assert torch.allclose(y, full[:, :12] * torch.nn.functional.gelu(full[:, 12:]), atol=1e-5)
    fake_ops.gemm(y, x, w, bias=b, epilogue=fake_ops.EPI_SWIGLU)
    assert torch.allclose(y, torch.nn.functional.silu(full[:, 0::2]) * full[:, 1::2], atol=1e-5)
