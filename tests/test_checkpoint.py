"""Real-weight path on the CPU: the safetensors reader / writer against the `safetensors` library,
sharded directories, expert fusion, and a decoder checkpoint round trip under the HF names."""
import json
import os
from dataclasses import replace

import pytest
import torch

from hoid_optimized_models_b200 import checkpoint as ck


def _tensors():
    g = torch.Generator().manual_seed(0)
    return {
        "model.a.weight": torch.randn(7, 12, generator=g).to(torch.bfloat16),
        "model.b.bias": torch.randn(5, generator=g),
        "model.half": torch.randn(3, 4, generator=g).to(torch.float16),
        "ids": torch.arange(10, dtype=torch.int64).view(2, 5),
        "flags": torch.tensor([True, False, True]),
        "scalar": torch.tensor(3.5),
        "empty": torch.empty(0, 4),
    }


def test_reader_matches_the_safetensors_library(tmp_path):
    from safetensors import safe_open
    from safetensors.torch import save_file
    t = _tensors()
    path = str(tmp_path / "lib.safetensors")
    save_file(t, path, metadata={"format": "pt"})
    got = {n: x.clone() for n, x in ck.iter_tensors(path)}
    assert set(got) == set(t)
    for n in t:
        assert got[n].dtype == t[n].dtype and got[n].shape == t[n].shape
        assert torch.equal(got[n], t[n]), n
    # and the other way round: a file from this writer, read by the library
    mine = str(tmp_path / "mine.safetensors")
    ck.save_file(mine, t, metadata={"format": "pt"})
    with safe_open(mine, framework="pt", device="cpu") as f:
        assert set(f.keys()) == set(t)
        for n in t:
            assert torch.equal(f.get_tensor(n), t[n]), n


def test_keep_filter_and_malformed_files(tmp_path):
    path = str(tmp_path / "x.safetensors")
    ck.save_file(path, _tensors())
    names = [n for n, _ in ck.iter_tensors(path, keep=lambda n: n.startswith("model."))]
    assert sorted(names) == ["model.a.weight", "model.b.bias", "model.half"]
    bad = tmp_path / "bad.safetensors"
    bad.write_bytes(b"\x01\x02")
    with pytest.raises(ValueError):
        ck.read_header(str(bad))
    with pytest.raises(FileNotFoundError):
        ck.checkpoint_files(str(tmp_path / "nowhere")) if os.path.isdir(tmp_path / "nowhere") else \
            ck.checkpoint_files(str(_empty_dir(tmp_path)))


def _empty_dir(tmp_path):
    d = tmp_path / "empty"
    d.mkdir()
    return d


def test_sharded_decoder_checkpoint_round_trip(tmp_path):
    from hoid_optimized_models_b200.configs import QWEN3_4B
    from hoid_optimized_models_b200.weights import make_decoder_weights
    cfg = replace(QWEN3_4B, name="ckpt-test", hidden=256, inter=512, n_q=4, n_kv=2, layers=3, vocab=384)
    w = make_decoder_weights(cfg, 9)
    names = sorted(w)
    half = len(names) // 2
    shards = {"model-00001-of-00002.safetensors": names[:half],
              "model-00002-of-00002.safetensors": names[half:]}
    for fn, ns in shards.items():
        ck.save_file(str(tmp_path / fn), {n: w[n] for n in ns})
    (tmp_path / "stale.safetensors").write_bytes(b"not part of the checkpoint")   # index wins
    with open(tmp_path / "model.safetensors.index.json", "w") as f:
        json.dump({"weight_map": {n: fn for fn, ns in shards.items() for n in ns}}, f)
    got = ck.load_weights(str(tmp_path), device="cpu")
    assert set(got) == set(w)
    for n in w:
        assert got[n].dtype == torch.bfloat16 and torch.equal(got[n], w[n]), n
    ck.check_decoder_names(cfg, got)
    del got["model.layers.1.self_attn.q_norm.weight"]
    got["model.norm.weight"] = got["model.norm.weight"][:-1]
    with pytest.raises(ValueError, match="q_norm.weight: missing"):
        ck.check_decoder_names(cfg, got)


def test_per_expert_tensors_are_fused_into_the_engine_layout(tmp_path):
    from hoid_optimized_models_b200.configs import QWEN3_30B_A3B
    from hoid_optimized_models_b200.weights import make_decoder_weights
    cfg = replace(QWEN3_30B_A3B, name="ckpt-moe-test", hidden=128, moe_inter=64, n_q=4, n_kv=2,
                  layers=2, vocab=256, n_experts=8, top_k=2)
    w = make_decoder_weights(cfg, 11)
    on_disk = {}
    for n, t in w.items():
        if n.endswith("mlp.experts.gate_up_proj"):
            p = n[: -len(".gate_up_proj")]
            for e in range(cfg.n_experts):
                on_disk[f"{p}.{e}.gate_proj.weight"] = t[e, : cfg.moe_inter].clone()
                on_disk[f"{p}.{e}.up_proj.weight"] = t[e, cfg.moe_inter:].clone()
        elif n.endswith("mlp.experts.down_proj"):
            p = n[: -len(".down_proj")]
            for e in range(cfg.n_experts):
                on_disk[f"{p}.{e}.down_proj.weight"] = t[e].clone()
        else:
            on_disk[n] = t
    ck.save_file(str(tmp_path / "model.safetensors"), on_disk)
    got = ck.load_weights(str(tmp_path), device="cpu")
    assert set(got) == set(w)
    for n in w:
        assert torch.equal(got[n], w[n]), n
    ck.check_decoder_names(cfg, got)
    # an incomplete expert set is an error, not a silently smaller model
    del on_disk["model.layers.0.mlp.experts.3.up_proj.weight"]
    with pytest.raises(ValueError, match="incomplete expert set"):
        ck.fuse_experts(on_disk)


def test_float32_checkpoint_is_cast_and_other_dtypes_kept(tmp_path):
    ck.save_file(str(tmp_path / "model.safetensors"),
                 {"model.w": torch.full((4, 4), 1.00390625), "model.idx": torch.arange(4)})
    got = ck.load_weights(str(tmp_path), device="cpu")
    assert got["model.w"].dtype == torch.bfloat16 and got["model.idx"].dtype == torch.int64
    raw = ck.load_weights(str(tmp_path), device="cpu", dtype=None)
    assert raw["model.w"].dtype == torch.float32
    enc = ck.load_weights(str(tmp_path), device="cpu", keep=lambda n: True, strip_prefix="model.")
    assert set(enc) == {"w", "idx"}
