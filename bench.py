#!/usr/bin/env python
"""Headline benchmark: batch-1 Llama-3.1-8B-architecture decode tok/s (+ TTFT) at an 8192-token
prompt on N B200s (head-sharded tensor parallel for N > 1).

    python bench.py --gpus 1 --steps 64 --warmup 8
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference          # the reference's eager PyTorch path on host cores

One JSON line on stdout (rank 0).  A "step" is one decode token: one replay of the captured
whole-step CUDA graph (every weight byte + the KV cache read once).  Weights are seeded
random-init N(0, 0.02) in bf16 and the prompt is uniform-random token ids (synthetic data).
Protocol follows the reference's: warm steps, then timed steps with CUDA events
(models/llama31-8b/best_hoid.py:83-100).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PROMPT = 8192
SMI_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def ncu_traffic(kernel: str, layers: int):
    """DRAM bytes per launch of `kernel` from profiles/ncu_traffic.json (written beside the ncu
    summaries from the captures they describe).  An entry measured on a reduced-depth model
    carries its depth, and the traffic of the layer phases scales with the number of layers."""
    path = os.path.join(ROOT, "profiles", "ncu_traffic.json")
    try:
        with open(path) as f:
            e = json.load(f)[kernel]
        per = float(e["dram_bytes_per_launch"])
        return per * layers / e["layers"] if e.get("layers") else per
    except (OSError, KeyError, ValueError, TypeError):
        return None


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""

    def __init__(self, gpu_index: int):
        self.path = f"/tmp/b200_clocks_{os.getpid()}.csv"
        self.gpu = gpu_index
        self.proc = None

    def __enter__(self):
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={SMI_QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100", "-i", str(self.gpu)], stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()   # the exact child we started
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.f.close()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            with open(self.path) as f:
                for line in f:
                    c = [x.strip() for x in line.split(",")]
                    if len(c) < 9:
                        continue
                    sm.append(float(c[1])); mx.append(float(c[2]))
                    for n, v in zip(names, c[5:9]):
                        if v.lower().startswith("active"):
                            reasons.add(n)
            os.remove(self.path)
        except (OSError, ValueError):
            pass
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------------------ CPU arm
def cpu_reference(cfg, ctx: int, steps: int, warmup: int, sample_layers: int = 4):
    """The reference's eager PyTorch path (HuggingFace LlamaForCausalLM, fp32) on the host cores.

    Bounded sample: `sample_layers` of the model's layers plus the full lm_head, decoding one
    token against a synthetic `ctx`-position KV cache; the per-layer time is scaled to the
    full depth (the layers are identical in shape)."""
    from hoid_optimized_models_b200.configs import reduced
    from hoid_optimized_models_b200.weights import make_decoder_weights
    from oracle.ref_decoder import hf_model
    import transformers

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    small = reduced(cfg, layers=sample_layers)
    model = hf_model(small, make_decoder_weights(small, 1234, "cpu"))
    g = torch.Generator().manual_seed(3)

    def fresh_cache():
        cache = transformers.DynamicCache(config=model.config)
        for l in range(sample_layers):
            k = torch.randn(1, cfg.n_kv, ctx, cfg.head_dim, generator=g)
            v = torch.randn(1, cfg.n_kv, ctx, cfg.head_dim, generator=g)
            cache.update(k, v, l)
        return cache

    tok = torch.randint(0, cfg.vocab, (1, 1), generator=g)
    times = []
    with torch.no_grad():
        cache = fresh_cache()
        for i in range(warmup + steps):
            t0 = time.perf_counter()
            out = model(tok, past_key_values=cache, use_cache=True)
            tok = out.logits[:, -1:].argmax(-1)
            dt = time.perf_counter() - t0
            if i >= warmup:
                times.append(dt)
        # the head alone (final norm + lm_head), to scale only the layer part
        h = torch.randn(1, 1, cfg.hidden, generator=g)
        ht = []
        for i in range(3):
            t0 = time.perf_counter()
            model.lm_head(model.model.norm(h))
            ht.append(time.perf_counter() - t0)
    t_step = statistics.median(times)
    t_head = min(statistics.median(ht), t_step)
    full = (t_step - t_head) * (cfg.layers / sample_layers) + t_head
    return {
        "value": 1.0 / full, "unit": "tok/s", "cores": cores, "kind": "reference",
        "sample": (f"HF transformers {transformers.__version__} LlamaForCausalLM eager fp32, "
                   f"{sample_layers} of {cfg.layers} layers + full lm_head, ctx {ctx} synthetic KV, "
                   f"p50 of {steps} decode steps, layer time scaled x{cfg.layers // sample_layers} "
                   f"(extrapolated)"),
        "ms_per_step": full * 1e3,
    }


# ------------------------------------------------------------------------------ other configs
def _no_switch_multicast():
    """The ranks leave with os._exit while captured graphs still hold communicator kernels (see
    leave()), i.e. without the communicator teardown.  Memory bound to an NVLink multicast object
    must not outlive its process that way, so the collective library's in-switch path is left off
    whatever the caller's environment says; the decode exchange does not go through the library
    anyway."""
    os.environ["NCCL_NVLS_ENABLE"] = "0"


def _time_graph(graph, steps, warmup):
    for _ in range(warmup):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def run_secondary(args):
    """The other benchmark configurations: same protocol, one JSON line each.  The two decoders
    also run multi-rank (Qwen3-4B head-sharded, Qwen3-30B-A3B expert-parallel); the encoder and
    Whisper lines are single GPU.  Published reference numbers (one B200, real checkpoints) are
    quoted for context."""
    from hoid_optimized_models_b200 import ops
    from hoid_optimized_models_b200 import configs as C
    from hoid_optimized_models_b200 import weights as Wt
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    ops.set_pdl(not args.no_pdl)
    for kv in args.tune:
        ops.set_tuning(*(int(t) for t in kv.split("=")))
    peak, peak_kind = measured_peaks()
    K, W = args.steps, max(args.warmup, 3)
    name = args.workload
    group = None
    if world > 1:
        if name not in ("qwen3-4b", "qwen3-30b-a3b", "xlm-roberta-large"):
            raise SystemExit(f"{name} runs on one GPU")
        import torch.distributed as dist
        if os.environ.get("NCCL_DEBUG", "").upper() in ("VERSION", "WARN"):
            del os.environ["NCCL_DEBUG"]
        _no_switch_multicast()
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD

    def over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        return float(t.item())

    def sync():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    line = {"workload": name, "n_gpus": world, "steps": K, "warmup": W, "dtype": "bf16", "data": "synthetic"}
    if name in ("qwen3-4b", "qwen3-30b-a3b"):
        from hoid_optimized_models_b200.decoder import DenseDecoder
        cfg = C.QWEN3_4B if name == "qwen3-4b" else C.QWEN3_30B_A3B
        P = args.prompt or 1024                    # the reference quotes these two at 1k tokens
        w = Wt.make_decoder_weights(cfg, 1234, dev)
        settle = 96 if world > 1 else 0            # untimed replays before the warm-up, see main()
        eng = DenseDecoder(cfg, w, max_seq=P + settle + W + K + 8, device=dev,
                           max_new_tokens=settle + W + K + 8,
                           free_source_weights=True, tp_rank=rank, tp_size=world, group=group,
                           fused_allreduce=args.tp_allreduce != "nccl",
                           fused_layers=args.persistent_layers,
                           ep_all_to_all=args.ep_all_to_all)
        del w
        torch.cuda.empty_cache()
        ids = torch.randint(0, cfg.vocab, (P,), generator=torch.Generator().manual_seed(1)).to(dev)
        first = eng.prefill(ids)
        ttft = []
        for _ in range(args.ttft_runs):
            sync()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); first = eng.prefill(ids); e1.record(); sync()
            ttft.append(over_ranks(e0.elapsed_time(e1)))
        ops.check_status(dev)
        eng.capture()
        eng.set_step(first, P, 0)
        if settle:
            for _ in range(settle):
                eng.graph.replay()
            eng.set_step(first, P, 0)
        line["settle_steps"] = settle
        sync()
        ms = over_ranks(_time_graph(eng.graph, K, W))
        sync()
        ops.check_status(dev)
        line["parallelism"] = ("ep" if cfg.n_experts else "tp") + str(world)
        line["tp_allreduce"] = args.tp_allreduce if world > 1 else None
        if cfg.n_experts and world > 1:
            line["ep_prefill"] = "all-to-all" if eng._ep_dispatch(P) else "replicated routing + all-reduce"
        nbytes = cfg.decode_bytes_per_token(P + W + K // 2)
        ref = {"qwen3-4b": {"decode_tok_per_s": 269.8, "ttft_ms": 9.58},
               "qwen3-30b-a3b": {"decode_tok_per_s": 241.1, "ttft_ms": 28.66}}[name]
        line.update({"metric": "decode_tok_per_s", "value": 1e3 / ms, "unit": "tok/s", "ms_per_step": ms,
                     "ttft_ms": statistics.median(ttft), "prompt_tokens": P,
                     "gpu_launches": eng.launches_per_step * K,
                     "published_reference": ref})
        if world == 1:                # per-rank bytes are not a plain 1/N share under EP
            line["step_roofline"] = {"bytes_per_step": nbytes, "achieved_gbs": nbytes / ms / 1e6,
                                     "frac_of_peak": nbytes / ms / 1e6 / peak, "peak_kind": peak_kind}
    elif name == "xlm-roberta-large":
        from hoid_optimized_models_b200.encoder import XlmrEncoder
        cfg, B, S = C.XLMR_LARGE, 64, 512
        # data parallel: the 64 sequences are split over the ranks, the pooled rows all-gathered
        eng = XlmrEncoder(cfg, Wt.make_encoder_weights(cfg, 1234, dev), batch=B, seq=S, device=dev,
                          dp_rank=rank, dp_size=world, group=group)
        ids = torch.randint(3, cfg.vocab, (B // world, S),
                            generator=torch.Generator().manual_seed(4 + rank)).to(dev)
        eng.load_inputs(ids)
        eng.capture()
        ops.check_status(dev)

        def one_forward():
            eng.graph.replay()
            if world > 1:
                torch.distributed.all_gather_into_tensor(eng.pooled_all, eng.pooled, group=group)

        for _ in range(W):
            one_forward()
        sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(K):
            one_forward()
        e1.record()
        sync()
        ms = over_ranks(e0.elapsed_time(e1) / K)
        flops = 21.44e12
        line.update({"metric": "sequences_per_s", "value": B / ms * 1e3, "unit": "seq/s",
                     "ms_per_step": ms, "gpu_launches": eng.launches_per_forward * K,
                     "parallelism": f"dp{world}", "scaling": "strong",
                     "roofline": {"bound": "tensor", "achieved": flops / world / ms / 1e9,
                                  "unit": "TFLOP/s per GPU"},
                     "published_reference": {"sequences_per_s": 2721.3, "forward_ms": 23.52}})
    elif name == "whisper-large-v3":
        from hoid_optimized_models_b200.whisper import WhisperDecoder, WhisperEncoder
        cfg = C.WHISPER_LARGE_V3
        w = Wt.make_whisper_weights(cfg, 1234, dev)
        enc, dec = WhisperEncoder(cfg, w, device=dev), WhisperDecoder(cfg, w, device=dev)
        mel = torch.randn(cfg.n_mels, cfg.n_frames, generator=torch.Generator().manual_seed(5)).clamp(-1.5, 1.5)
        enc.load_inputs(mel.to(dev).to(torch.bfloat16))
        enc.capture()
        enc_ms = _time_graph(enc.graph, max(8, K // 4), W)
        dec.set_encoder(enc.out)
        ops.check_status(dev)
        # cross K / V projection + the 4-token forced prefix as one prefill pass
        prefix = [50258, 50259, 50360, 50364]
        dec.prefill(prefix, enc_out=enc.out)
        pre = []
        for _ in range(5):
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); dec.prefill(prefix, enc_out=enc.out); e1.record(); torch.cuda.synchronize()
            pre.append(e0.elapsed_time(e1))
        dec.capture()
        dec.set_step(7, 0, 0)
        n = min(K, 224)
        ms = _time_graph(dec.graph, n, W)   # positions 0 .. W + n of the 448-slot window
        line.update({"metric": "decode_tok_per_s", "value": 1e3 / ms, "unit": "tok/s", "ms_per_step": ms,
                     "encoder_forward_ms": enc_ms, "prefix_prefill_ms": statistics.median(pre),
                     "gpu_launches": dec.launches_per_step * n,
                     "published_reference": {"decode_tok_per_s": 499.7, "decode_step_ms": 1.8219,
                                             "encoder_forward_ms": 3.525}})
    else:
        raise SystemExit(f"unknown workload {name}")
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        # graphs hold communicator kernels: drop them, meet, and leave without the teardown
        eng.graph = None
        torch.cuda.synchronize()
        torch.distributed.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


# ------------------------------------------------------------------------------ main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--prompt", type=int, default=None,
                    help=f"prompt tokens (default {PROMPT}; 1024 for the Qwen3 workloads)")
    ap.add_argument("--layers", type=int, default=0, help="debug: reduced depth (invalid as a result)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-pdl", action="store_true")
    ap.add_argument("--ttft-runs", type=int, default=3)
    ap.add_argument("--tp-allreduce", default="fused", choices=["fused", "nccl"],
                    help="N>1: all-reduce fused into the decode kernels over peer memory, or NCCL calls")
    ap.add_argument("--ep-all-to-all", action="store_true",
                    help="expert-parallel prefill with an all-to-all dispatch / combine of token rows "
                         "instead of replicated routing + all-reduce (A/B; measured slower)")
    ap.add_argument("--persistent-layers", action="store_true",
                    help="all layers of a decode step as one persistent launch instead of one launch "
                         "per phase (A/B; measured slower at 1 and 2 GPUs)")
    ap.add_argument("--workload", default="llama-3.1-8b",
                    help="llama-3.1-8b (headline) | qwen3-4b | qwen3-30b-a3b | xlm-roberta-large | whisper-large-v3")
    ap.add_argument("--tune", action="append", default=[], metavar="KEY=VALUE",
                    help="kernel tuning knob (B200_TUNE_* key number = value), repeatable")
    ap.add_argument("--skip-prefill", action="store_true",
                    help="profiling aid: random KV cache instead of a prefill, decode timing only")
    args = ap.parse_args()

    if args.workload != "llama-3.1-8b" and args.impl == "b200":
        run_secondary(args)
        return
    args.prompt = args.prompt or PROMPT
    from hoid_optimized_models_b200.configs import LLAMA31_8B, reduced
    cfg = LLAMA31_8B if not args.layers else reduced(LLAMA31_8B, layers=args.layers)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    W = max(args.warmup, 3)
    K = args.steps
    config = {"workload": f"{cfg.name} batch-1 greedy decode, {args.prompt}-token prompt + {K + W} steps "
                          f"(the reference's headline configuration)", "prompt_tokens": args.prompt,
              "parallelism": f"tp{world}",
              "tp_allreduce": (args.tp_allreduce if world > 1 else None), "settle_steps": (96 if world > 1 else 0),
              "cache_policy": "inputs larger than L2 "
              "(every step streams all weights, 15 GB / TP)"}

    if args.impl == "reference":
        if rank != 0:
            return
        base = cpu_reference(cfg, args.prompt, K, W)       # exactly K timed steps after W warm ones
        line = {"impl": "reference", "metric": "decode_tok_per_s", "value": base["value"],
                "unit": "tok/s", "n_gpus": args.gpus, "steps": K, "warmup": W,
                "ms_per_step": base["ms_per_step"], "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
                "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
                "e2e": {"value": base["value"], "unit": "tok/s", "h2d_bytes_per_step": 0,
                        "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line))
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the b200 ops have no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    group = None
    if world > 1:
        import torch.distributed as dist
        if os.environ.get("NCCL_DEBUG", "").upper() in ("VERSION", "WARN"):
            del os.environ["NCCL_DEBUG"]           # keep stdout to the one JSON line
        _no_switch_multicast()
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD

    from hoid_optimized_models_b200 import ops
    from hoid_optimized_models_b200.decoder import Llama31Optimized
    from hoid_optimized_models_b200.weights import make_decoder_weights
    ops.set_pdl(not args.no_pdl)
    for kv in args.tune:
        ops.set_tuning(*(int(t) for t in kv.split("=")))

    weights = make_decoder_weights(cfg, 1234, dev)
    # Multi-GPU: some untimed replays before the W warm-up steps (config.settle_steps in the JSON
    # line).  The first job on a fresh multi-GPU box measured up to 5 % slower at 2 GPUs than the
    # same binary run again, and W = 8 warm-up steps last only ~20 ms.
    settle = 96 if world > 1 else 0
    max_seq = args.prompt + settle + W + K + 8
    eng = Llama31Optimized(cfg, weights, max_seq=max_seq, device=dev, tp_rank=rank, tp_size=world,
                           group=group, max_new_tokens=settle + W + K + 8, free_source_weights=True,
                           fused_allreduce=args.tp_allreduce != "nccl",
                           fused_layers=args.persistent_layers)
    del weights
    torch.cuda.empty_cache()
    ids = torch.randint(0, cfg.vocab, (args.prompt,), generator=torch.Generator().manual_seed(2))
    ids_dev = ids.to(dev)

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        return float(t.item())

    # ---- TTFT: prompt -> first token (p50 over runs, after one warm run) ----
    ttft = []
    if args.skip_prefill:
        eng.kv.normal_(0, 1)
        first, ttft = 1, [float("nan")]
    else:
        first = eng.prefill(ids_dev)
    for _ in range(0 if args.skip_prefill else args.ttft_runs):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        first = eng.prefill(ids_dev)
        e1.record()
        torch.cuda.synchronize()
        ttft.append(max_over_ranks(e0.elapsed_time(e1)))
    ttft_ms = statistics.median(ttft)
    ops.check_status(dev)

    # ---- decode: device-timed graph replays ----
    eng.capture()
    eng.set_step(first, args.prompt, 0)
    if settle:
        for _ in range(settle):
            eng.graph.replay()
        eng.set_step(first, args.prompt, 0)      # the timed steps run at the configured context
    for _ in range(W):
        eng.graph.replay()
    barrier()
    with ClockSampler(local) as clocks:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(K):
            eng.graph.replay()
        e1.record()
        barrier()
        dec_ms = max_over_ranks(e0.elapsed_time(e1))
        # keep sampling long enough for at least a few readings on short runs
        if dec_ms < 500:
            t_end = time.time() + 0.6
            while time.time() < t_end:
                eng.graph.replay()
            torch.cuda.synchronize()
    clk = clocks.summary()
    ms_per_step = dec_ms / K
    tok_s = 1e3 / ms_per_step

    if args.skip_prefill:
        if rank == 0:
            print(json.dumps({"profiling_only": True, "ms_per_step": ms_per_step, "tok_s": tok_s,
                              "clocks": clk}))
        if world > 1:
            eng.graph = None
            torch.cuda.synchronize()
            torch.distributed.barrier()
            sys.stdout.flush()
            os._exit(0)
        return

    # ---- end to end through the public host-driven step (DenseDecoder.step_host): per step the
    # token + step state go up from pinned host memory, the graph replays, the token comes back ----
    pos = args.prompt + W + K
    KE = max(8, min(K, 32))
    tok = first
    barrier()
    t0 = time.perf_counter()
    for j in range(KE):
        tok = eng.step_host(tok, pos - KE + j)
    e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3) / KE

    # ---- roofline of the dominant kernel, timed live with CUDA events on the launching stream.
    # With the persistent kernel that is decode_layers_kernel (every layer's weights + the KV
    # cache, all but the lm_head of the step's bytes); on the per-phase path the gate|up GEMV. ----
    peak, peak_kind = measured_peaks()
    ctx_mid = args.prompt + W + K // 2
    step_bytes = cfg.decode_bytes_per_token(ctx_mid) / world
    step_gbs = step_bytes / (ms_per_step * 1e-3) / 1e9
    ops.check_status(dev)
    reps = 16
    if eng.plan is not None:
        kernel_name = "decode_layers_kernel (all layers of the step: q|k|v, attention, o, gate|up, down)"
        head_bytes = 2 * (cfg.vocab * cfg.hidden + cfg.hidden) / world
        kernel_bytes = step_bytes - head_bytes
        eng.set_step(first, ctx_mid - 1, 0)
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
        barrier()
        for it in range(3 + reps):
            ops.embed_gather(eng.h, eng.embed, eng.tok)
            if it >= 3:
                ev[it - 3][0].record()
            ops.decode_layers(eng.plan, eng.cos, eng.sin, eng.kv_len, eng.fd_ws, eng.n_q, eng.n_kv,
                              eng.n_splits, eng.scale, cfg.eps)
            if it >= 3:
                ev[it - 3][1].record()
            if eng.link is not None:      # finish the step's exchange so that the sequence advances
                ops.gemv_tp_consume(eng.logits, eng.lm_head, eng.link.ctx, 2 * cfg.layers - 1,
                                    x_out=eng.h, norm_w=eng.final_norm_w, eps=cfg.eps)
                ops.tp_advance(eng.link.ctx, 2 * cfg.layers)
        torch.cuda.synchronize()
        kernel_ms = max_over_ranks(statistics.median(a.elapsed_time(b) for a, b in ev))
        launches_timed = 1
    else:
        kernel_name = "gemv_kernel (gate|up + SwiGLU, N=28672/tp K=4096)"
        # the launches of all layers inside one captured graph (32 different matrices, so nothing
        # is served from L2), replayed: the time is the kernels', not the host's launch rate
        x = torch.randn(cfg.hidden, dtype=torch.float32, device=dev)

        def all_layers():
            for i in range(cfg.layers):
                ops.gemv(eng.act, x, eng.wgu[i], norm_w=eng.ln2[i], eps=cfg.eps, epilogue=ops.EPI_SWIGLU)

        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            all_layers()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            all_layers()
        kernel_ms = max_over_ranks(_time_graph(g, 8, 3) / cfg.layers)
        del g
        kernel_bytes = eng.wgu[0].numel() * 2 + cfg.hidden * 4 + cfg.hidden * 2 + eng.inter * 4
        launches_timed = 1
    ops.check_status(dev)
    achieved = kernel_bytes / (kernel_ms * 1e-3) / 1e9
    traffic = ncu_traffic("decode_layers_kernel" if eng.plan is not None else "gemv_kernel_gate_up",
                          cfg.layers) if world == 1 else None

    def leave():
        """Multi-rank exit: the captured graph holds NCCL kernels, so drop it, meet the other
        ranks, flush and leave without the communicator teardown (which can block while graphs
        that reference the communicator are alive)."""
        if world > 1:
            eng.graph = None
            torch.cuda.synchronize()
            torch.distributed.barrier()
            torch.cuda.synchronize()
            sys.stdout.flush()
            sys.stderr.flush()
            os._exit(0)

    if rank != 0:
        leave()
        return

    line = {
        "metric": "decode_tok_per_s", "value": tok_s, "unit": "tok/s", "n_gpus": world,
        "steps": K, "warmup": W, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong",
        # the reference engine's published 185.6 tok/s for this model / prompt on one B200
        # (real checkpoint; timing does not depend on weight values)
        "vs_baseline": (tok_s / 185.6) if world == 1 else None,
        "dtype": "bf16", "data": "synthetic",
        "config": config,
        "ttft_ms": ttft_ms,
        "e2e": {"value": 1e3 / e2e_ms, "unit": "tok/s", "h2d_bytes_per_step": 20,
                "d2h_bytes_per_step": 4, "ms_per_step": e2e_ms, "steps": KE},
        "gpu_launches": eng.launches_per_step * K,
        "clocks": clk,
        "roofline": {"bound": "hbm", "kernel": kernel_name,
                     "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_kind": f"of {peak_kind}",
                     # dram__bytes_read.sum + dram__bytes_write.sum per launch, read from the
                     # figures file kept beside the ncu summary under profiles/
                     "traffic": traffic,
                     "bytes_per_launch": kernel_bytes, "ms_per_launch": kernel_ms},
        "step_roofline": {"bytes_per_step_per_gpu": step_bytes, "achieved_gbs": step_gbs,
                          "frac_of_peak": step_gbs / peak, "frac_of_8tbs": step_gbs / 8000.0},
        "published_reference": {"decode_tok_per_s": 185.6, "ttft_ms": 119.53,
                                "note": "reference engine on 1xB200, real weights (its published table)"},
    }
    if world == 1 and not args.no_cpu_baseline:
        try:
            base = cpu_reference(cfg, args.prompt, 4, 1)
            line["cpu_baseline"] = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")}
        except Exception as e:  # the baseline is reported, never a gate
            line["cpu_baseline"] = {"value": None, "unit": "tok/s", "cores": os.cpu_count(),
                                    "kind": "reference", "sample": f"failed: {e!r}"}
    print(json.dumps(line))
    leave()


if __name__ == "__main__":
    main()
