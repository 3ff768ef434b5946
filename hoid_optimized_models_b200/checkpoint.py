"""Real-weight path: HuggingFace safetensors checkpoints -> {name: tensor} under the names the
engines read (the ones `weights.py` generates synthetically).

Same job as the reference's loaders (models/llama31-8b/llama31_optimized.py:294-310 walks the
`*.safetensors` files of a directory and keeps `model.*` and `lm_head.weight` as bf16;
models/qwen3-30b-a3b/qwen3_optimized.py:359-371 takes the fused expert tensors
`gate_up_proj [E, 2I, H]` / `down_proj [E, H, I]`).  The file format is read directly - an 8-byte
little-endian header length, a JSON header {name: {dtype, shape, data_offsets}}, then the raw
tensor bytes - so the loader needs nothing beyond numpy and torch and memory-maps the files: a
tensor's bytes are touched once, when it is copied to the device.

Checkpoints that store Mixture-of-Experts weights per expert
(`...mlp.experts.<e>.{gate,up,down}_proj.weight`) are fused into the two tensors above.
"""
from __future__ import annotations

import json
import os
import re
import struct
import warnings
from typing import Callable, Dict, Iterator, Optional, Tuple

import numpy as np
import torch

# safetensors dtype tag -> (torch dtype, bytes per element)
_DTYPES = {
    "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2), "F32": (torch.float32, 4),
    "F64": (torch.float64, 8), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_TAGS = {v[0]: k for k, v in _DTYPES.items()}


def read_header(path: str) -> Tuple[Dict[str, dict], int]:
    """(header without `__metadata__`, offset of the data section)."""
    with open(path, "rb") as f:
        raw = f.read(8)
        if len(raw) != 8:
            raise ValueError(f"{path}: not a safetensors file (too short)")
        (n,) = struct.unpack("<Q", raw)
        if n <= 0 or n > 100 * 1024 * 1024:
            raise ValueError(f"{path}: implausible header length {n}")
        header = json.loads(f.read(n).decode("utf-8"))
    header.pop("__metadata__", None)
    return header, 8 + n


def iter_tensors(path: str, keep: Optional[Callable[[str], bool]] = None
                 ) -> Iterator[Tuple[str, torch.Tensor]]:
    """Yields (name, CPU tensor) for every kept tensor of one file.  The tensors are views of a
    read-only memory map: copy (`.to(device)`, `.clone()`) before the map goes away."""
    header, base = read_header(path)
    size = os.path.getsize(path)
    mm = np.memmap(path, dtype=np.uint8, mode="r") if size > base else np.zeros(0, np.uint8)
    for name, meta in header.items():
        if keep is not None and not keep(name):
            continue
        if meta["dtype"] not in _DTYPES:
            raise ValueError(f"{path}: tensor {name} has unsupported dtype {meta['dtype']}")
        dtype, width = _DTYPES[meta["dtype"]]
        b, e = meta["data_offsets"]
        shape = tuple(meta["shape"])
        count = int(np.prod(shape, dtype=np.int64)) if shape else 1
        if e - b != count * width or base + e > size:
            raise ValueError(f"{path}: tensor {name} has inconsistent offsets")
        if count == 0:
            yield name, torch.empty(shape, dtype=dtype)
            continue
        buf = mm[base + b: base + e]
        # numpy has no bfloat16: go through a same-width integer view
        carrier = {1: np.uint8, 2: np.int16, 4: np.int32, 8: np.int64}[width]
        with warnings.catch_warnings():          # the map is read-only by design; nothing writes
            warnings.simplefilter("ignore", UserWarning)
            t = torch.from_numpy(buf.view(carrier))
        t = t.view(torch.uint8).view(dtype) if dtype == torch.bool else t.view(dtype)
        yield name, t.reshape(shape)


def save_file(path: str, tensors: Dict[str, torch.Tensor], metadata: Optional[dict] = None) -> None:
    """Minimal writer of the same format (tests, and exporting the synthetic checkpoints)."""
    header, offset, blobs = {}, 0, []
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _TAGS:
            raise ValueError(f"unsupported dtype {t.dtype}")
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _TAGS[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * (-len(hj) % 8)                      # keep the data section 8-byte aligned
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for raw in blobs:
            f.write(raw)


def checkpoint_files(weights_dir: str) -> list:
    """The `*.safetensors` files of a checkpoint directory: those the index names if there is a
    `*.safetensors.index.json`, otherwise all of them, sorted."""
    names = sorted(os.listdir(weights_dir))
    index = [n for n in names if n.endswith(".safetensors.index.json")]
    if index:
        with open(os.path.join(weights_dir, index[0])) as f:
            files = sorted(set(json.load(f)["weight_map"].values()))
    else:
        files = [n for n in names if n.endswith(".safetensors")]
    if not files:
        raise FileNotFoundError(f"no safetensors files under {weights_dir}")
    return [os.path.join(weights_dir, n) for n in files]


_EXPERT = re.compile(r"^(.*\.mlp\.experts)\.(\d+)\.(gate_proj|up_proj|down_proj)\.weight$")


def fuse_experts(w: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """Per-expert `...experts.<e>.{gate,up,down}_proj.weight` -> `...experts.gate_up_proj`
    [E, 2I, H] (gate rows first) and `...experts.down_proj` [E, H, I]; other names pass through."""
    groups: Dict[str, Dict[str, Dict[int, torch.Tensor]]] = {}
    out: Dict[str, torch.Tensor] = {}
    for name, t in w.items():
        m = _EXPERT.match(name)
        if m is None:
            out[name] = t
        else:
            groups.setdefault(m.group(1), {}).setdefault(m.group(3), {})[int(m.group(2))] = t
    for prefix, parts in groups.items():
        n = len(parts.get("gate_proj", {}))
        for kind in ("gate_proj", "up_proj", "down_proj"):
            if sorted(parts.get(kind, {})) != list(range(n)) or n == 0:
                raise ValueError(f"{prefix}: incomplete expert set for {kind}")
        gate = torch.stack([parts["gate_proj"][e] for e in range(n)])
        up = torch.stack([parts["up_proj"][e] for e in range(n)])
        out[prefix + ".gate_up_proj"] = torch.cat((gate, up), dim=1).contiguous()
        out[prefix + ".down_proj"] = torch.stack([parts["down_proj"][e] for e in range(n)]).contiguous()
    return out


def load_weights(weights_dir: str, device="cuda", dtype: Optional[torch.dtype] = torch.bfloat16,
                 keep: Optional[Callable[[str], bool]] = None,
                 strip_prefix: str = "") -> Dict[str, torch.Tensor]:
    """Every kept tensor of the checkpoint on `device`, floating-point ones cast to `dtype`
    (None keeps the stored dtypes).  Default `keep`: `model.*` and `lm_head.weight`, the decoder
    engines' names; pass `keep=lambda n: True, strip_prefix="roberta."` and the like for encoder
    checkpoints whose names carry a wrapper prefix."""
    if keep is None:
        keep = lambda n: n.startswith("model.") or n == "lm_head.weight"   # noqa: E731
    w: Dict[str, torch.Tensor] = {}
    for path in checkpoint_files(weights_dir):
        for name, t in iter_tensors(path, keep):
            if strip_prefix and name.startswith(strip_prefix):
                name = name[len(strip_prefix):]
            if name in w:
                raise ValueError(f"tensor {name} appears in more than one file")
            out = t.to(device=device, dtype=dtype) if dtype is not None and t.is_floating_point() \
                else t.to(device=device)
            if out.device.type == "cpu" and out.data_ptr() == t.data_ptr():
                out = out.clone()                    # do not hand out views of the read-only map
            w[name] = out
    if not w:
        raise ValueError(f"no tensor under {weights_dir} matched")
    return fuse_experts(w)


def check_decoder_names(cfg, w: Dict[str, torch.Tensor]) -> None:
    """Raises with the list of missing / mis-shaped tensors for a decoder config (the engine would
    otherwise fail on the first missing name, deep inside its constructor)."""
    H, hd = cfg.hidden, cfg.head_dim
    want = {"model.embed_tokens.weight": (cfg.vocab, H), "model.norm.weight": (H,)}
    if not cfg.tied:
        want["lm_head.weight"] = (cfg.vocab, H)
    for i in range(cfg.layers):
        p = f"model.layers.{i}."
        want[p + "input_layernorm.weight"] = (H,)
        want[p + "post_attention_layernorm.weight"] = (H,)
        want[p + "self_attn.q_proj.weight"] = (cfg.q_size, H)
        want[p + "self_attn.k_proj.weight"] = (cfg.kv_size, H)
        want[p + "self_attn.v_proj.weight"] = (cfg.kv_size, H)
        want[p + "self_attn.o_proj.weight"] = (H, cfg.q_size)
        if cfg.qk_norm:
            want[p + "self_attn.q_norm.weight"] = (hd,)
            want[p + "self_attn.k_norm.weight"] = (hd,)
        if cfg.n_experts:
            want[p + "mlp.gate.weight"] = (cfg.n_experts, H)
            want[p + "mlp.experts.gate_up_proj"] = (cfg.n_experts, 2 * cfg.moe_inter, H)
            want[p + "mlp.experts.down_proj"] = (cfg.n_experts, H, cfg.moe_inter)
        else:
            want[p + "mlp.gate_proj.weight"] = (cfg.inter, H)
            want[p + "mlp.up_proj.weight"] = (cfg.inter, H)
            want[p + "mlp.down_proj.weight"] = (H, cfg.inter)
    bad = [f"{n}: missing" for n in want if n not in w]
    bad += [f"{n}: shape {tuple(w[n].shape)} != {s}" for n, s in want.items()
            if n in w and tuple(w[n].shape) != s]
    if bad:
        raise ValueError("checkpoint does not match the configuration:\n  " + "\n  ".join(bad[:20]))
