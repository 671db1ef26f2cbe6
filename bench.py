#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Qwen3-8B layer sizes with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--impl ours|reference]

One step is one decode step of the whole batch.  The default run: 36 layers of the
8B sizes, bfloat16, a batch of 8 sequences with 1,024-token random prompts in a
4,096-token context, W untimed then K timed decode steps replayed from CUDA graphs
and timed with CUDA events.  One JSON line is printed:

  value      decoded tokens a second, timed on the device (tokens stay on the device)
  e2e        the same through ``generate`` (host token lists in, host token lists out;
             every step copies its input ids from pinned host memory and reads the sampled ids back)
  prefill    one prompt of 2,048 tokens: tokens a second, and flops / time / peak
  roofline   decode: (every weight once + the live sequences' cache) / step time, against the HBM peak
  points     decode tokens a second at batch 1 and 64

Peaks come from MEASURED_PEAKS.json beside this file when it is there ("of measured"),
else from the fallback figures 6.65 TB/s and 1.59 PFLOP/s ("of fallback").  Every decode
step reads more than 15 GB of weights, far more than the 126 MB L2, so no L2 flush is needed
between timed steps (config.l2 says so).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = {                     # the layer sizes of Qwen3-8B: the model this benchmark is quoted on
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 36, "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 128, "intermediate_size": 12288, "vocab_size": 151936, "rope_theta": 1e6,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 4096,
}
N_CTX = 4096
PROMPT_LEN = 1024
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        def number(v):                       # a plain number, or an object that holds one under "value"
            return float(v["value"] if isinstance(v, dict) else v)
        peaks = {k: number(d[k]) for k in ("hbm_gbs", "bf16_tflops") if k in d}
        if len(peaks) == 2 and all(v > 0 for v in peaks.values()):
            peaks["bf16_tflops_sustained"] = number(d.get("bf16_tflops_sustained", peaks["bf16_tflops"]))
            return peaks, "measured"
    except Exception:                            # an unreadable file is no reason to lose the run: fall back
        pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while a timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for name, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def weight_bytes(engine) -> int:
    """Bytes of every weight a decode step reads once (the embedding table is only gathered from)."""
    total = 0
    for block in engine.model.blocks:
        total += block.mixer.w_qkv.numel() * block.mixer.w_qkv.element_size()
        total += block.mixer.w_o.numel() * block.mixer.w_o.element_size()
        total += block.ffn.w_gate_up.numel() * block.ffn.w_gate_up.element_size()
        total += block.ffn.w_down.numel() * block.ffn.w_down.element_size()
    total += engine.model.head.weight.numel() * engine.model.head.weight.element_size()
    return total


def kv_bytes_per_token(cfg, n_layers, elem=2) -> int:
    return 2 * n_layers * cfg["num_key_value_heads"] * cfg["head_dim"] * elem


def prefill_flops(cfg, n_layers, T) -> float:
    D, Hq, Hkv, hd, F, V = (cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"],
                            cfg["head_dim"], cfg["intermediate_size"], cfg["vocab_size"])
    per_token = 2 * (D * (Hq + 2 * Hkv) * hd + Hq * hd * D + 3 * D * F)
    attn = 2 * 2 * Hq * hd * (T * (T + 1) / 2)            # causal QK^T and PV
    return n_layers * (T * per_token + attn) + 2 * D * V   # the head runs on one row


def decode_run(engine, torch, batch, warmup, steps, rng, count_launches=False):
    """Prefill `batch` prompts of PROMPT_LEN, then time `steps` graph-replayed decode steps."""
    from questwend_b200.engine.engine import StepEntry
    from questwend_b200.sampling.params import GREEDY
    from questwend_b200.kernels import ops
    V = engine.vocab_size
    prompts = [rng.integers(0, V, PROMPT_LEN).tolist() for _ in range(batch)]
    slots = engine.open_sequences(batch)
    first = []
    for i in range(0, batch, 8):                       # prompts in groups of 8: bounded activation memory
        grp = list(range(i, min(batch, i + 8)))
        lg = engine.step([StepEntry(slots[j], prompts[j], [PROMPT_LEN - 1]) for j in grp])
        first += lg.argmax(-1).tolist()
    runner = engine.decode_runner(batch, GREEDY)
    runner.bind(slots, first, list(range(batch)), 1)
    for _ in range(warmup):
        runner.step()
    torch.cuda.synchronize()
    launches_before = ops.LAUNCHES[0]
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ctx0 = engine.cache.length(slots[0])
    start.record()
    for _ in range(steps):
        runner.step()
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end)
    ctx1 = engine.cache.length(slots[0])
    per_step = runner.launches_per_step
    engine.close_sequences(slots)
    return {"ms_per_step": ms / steps, "tok_s": batch * steps / (ms / 1e3), "mean_ctx": (ctx0 + ctx1) / 2.0,
            "launches_per_step": per_step, "eager_launches": ops.LAUNCHES[0] - launches_before}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=QWEN3_8B["num_hidden_layers"])
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-points", action="store_true", help="leave out batch 1 / 64 and the e2e run")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "kishida/questwend is a CMake C++ project with no Python package: pip install of the "
                          "reference fails offline (no setup.py / pyproject.toml), so there is nothing to import"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    warmup = max(3, args.warmup)
    steps = max(1, args.steps)
    if PROMPT_LEN + warmup + steps + 1 > N_CTX:
        print(f"bench.py: {PROMPT_LEN} prompt tokens + {warmup} + {steps} steps exceed the context of {N_CTX}")
        return 2

    import numpy as np
    import torch
    import questwend_b200 as qw
    from questwend_b200.config.registry import config_from_dict
    from questwend_b200.engine.engine import Engine, StepEntry
    from questwend_b200.kernels import ops

    peaks, peak_source = load_peaks()
    cfgd = dict(QWEN3_8B)
    cfgd["num_hidden_layers"] = args.layers
    cfg = config_from_dict(cfgd)
    max_batch = max(args.batch, 1 if args.skip_points else 64)
    engine = Engine.from_config(cfg, seed=0, dtype="bfloat16", max_tokens=max_batch * (PROMPT_LEN + 512),
                                max_seq_len=N_CTX, max_batch=max_batch)
    rng = np.random.default_rng(0)
    wbytes = weight_bytes(engine)
    kv_tok = kv_bytes_per_token(cfgd, args.layers)

    # ---- the headline: decode at the given batch, device-timed
    clocks = ClockSampler()
    clocks.start()
    main_run = decode_run(engine, torch, args.batch, warmup, steps, rng)
    clock_info = clocks.stop()
    step_s = main_run["ms_per_step"] / 1e3
    step_bytes = wbytes + args.batch * main_run["mean_ctx"] * kv_tok
    achieved = step_bytes / step_s / 1e9

    # ---- prefill of one 2,048-token prompt
    times = []
    for _ in range(4):
        slot = engine.open_sequences(1)[0]
        prompt = rng.integers(0, engine.vocab_size, PREFILL_TOKENS).tolist()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        engine.step([StepEntry(slot, prompt, [PREFILL_TOKENS - 1])])
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
        engine.close_sequences([slot])
    pf_ms = statistics.median(times[1:])
    pf_flops = prefill_flops(cfgd, args.layers, PREFILL_TOKENS)
    prefill = {"value": PREFILL_TOKENS / (pf_ms / 1e3), "tokens": PREFILL_TOKENS, "ms": pf_ms,
               "frac": pf_flops / (pf_ms / 1e3) / (peaks["bf16_tflops"] * 1e12)}

    # ---- other batch sizes, and the same batch through the Python entry point
    points, e2e = {}, None
    if not args.skip_points:
        for b in (1, 64):
            r = decode_run(engine, torch, b, 3, 32, rng)
            points[f"decode_b{b}"] = r["tok_s"]
        prompts = [rng.integers(0, engine.vocab_size, PROMPT_LEN).tolist() for _ in range(args.batch)]
        stats = qw.GenerationStats()
        qw.generate(engine, prompts, max_new_tokens=warmup + 1, ignore_eos=True)          # warm the graphs
        qw.generate(engine, prompts, max_new_tokens=steps + 1, ignore_eos=True, stats=stats)
        e2e = {"value": args.batch * stats.steps / stats.decode_seconds, "unit": "tokens/s",
               "h2d_bytes_per_step": 4 * args.batch, "d2h_bytes_per_step": 4 * args.batch}

    out = {
        "metric": "decode tokens/s (Qwen3-8B sizes, random bf16 weights, batch %d, n_ctx %d)" % (args.batch, N_CTX),
        "value": main_run["tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": main_run["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random weights and uniform random token ids",
        "config": {"model": "qwen3-8b-sizes", "layers": args.layers, "layers_full": QWEN3_8B["num_hidden_layers"],
                   "hidden_size": cfgd["hidden_size"], "heads": cfgd["num_attention_heads"],
                   "kv_heads": cfgd["num_key_value_heads"], "head_dim": cfgd["head_dim"],
                   "intermediate_size": cfgd["intermediate_size"], "vocab_size": cfgd["vocab_size"],
                   "global_batch": args.batch, "seq_len": N_CTX, "prompt_len": PROMPT_LEN,
                   "mean_ctx_timed": main_run["mean_ctx"], "parallelism": "single-gpu",
                   "l2": "inputs_exceed_l2", "cuda_graph": True, "peaks": peak_source},
        "clocks": clock_info, "e2e": e2e, "gpu_launches": main_run["launches_per_step"] * steps,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peaks["hbm_gbs"], "of": peak_source},
        "points": points,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
