#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Qwen3 layer sizes with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--impl ours|reference] [--model 8b|0.6b|32b]

One step is one decode step of the whole batch.  The default run: 36 layers of the 8B sizes, bfloat16, a batch of 8
sequences with 1,024-token random prompts in a 4,096-token context, W untimed then K timed decode steps replayed from
CUDA graphs and timed with CUDA events.  One JSON line is printed:

  value      decoded tokens a second, timed on the device (tokens stay on the device)
  e2e        the same through ``generate`` (host token lists in, host token lists out; every step copies its input
             ids from pinned host memory and reads the sampled ids back): one call that runs the prompts, W untimed
             decode steps and the K timed ones, by the loop's own clock around each step (``value_all_steps``: over
             all W + K; the first dozen steps after a prompt step run at the clocks the prompt left)
  prefill    one prompt of 2,048 tokens: tokens a second, and flops / time / peak
  roofline   decode: (every weight once + the live sequences' cache) / step time, against the HBM peak
  points     decode tokens a second at batch 1 and 64 with their roofline fractions, prefill of 4,096 tokens (the context),
             and the benchmark's two other workloads (left out with --skip-other-models): Qwen3-0.6B sizes, 16 prompts
             with lengths uniform in [1, 2048] in one prefill step, then 128 decode steps; Qwen3-32B sizes, all 64
             layers, a 2,048-token prefill and decode at batch 1, 8 and 16 from 1,024-token prompts

``--model 0.6b`` or ``--model 32b`` runs one of those workloads alone and prints a line of its own.
``--impl reference`` runs kishida/questwend itself (built by baseline/build_reference.py into baseline/_ref/) on the
same sizes: it holds one sequence, so the batch is run as that many sequences one after the other.

Peaks come from MEASURED_PEAKS.json beside this file when it is there ("of measured"),
else from the fallback figures 6.65 TB/s and 1.59 PFLOP/s ("of fallback").  Every decode
step reads more than 15 GB of weights, far more than the 126 MB L2, so no L2 flush is needed
between timed steps (config.l2 says so).
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import shutil
import statistics
import subprocess
import sys
import tempfile
import threading

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = {                     # the layer sizes of Qwen3-8B: the model this benchmark is quoted on
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 36, "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 128, "intermediate_size": 12288, "vocab_size": 151936, "rope_theta": 1e6,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 4096,
}
QWEN3_06B = dict(QWEN3_8B, num_hidden_layers=28, hidden_size=1024, num_attention_heads=16, num_key_value_heads=8,
                 intermediate_size=3072, tie_word_embeddings=True)
QWEN3_32B = dict(QWEN3_8B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, num_key_value_heads=8,
                 intermediate_size=25600)
MODELS = {"8b": QWEN3_8B, "0.6b": QWEN3_06B, "32b": QWEN3_32B}
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
    engine.check_kernels()                             # no bounded wait inside a kernel gave up
    ctx1 = engine.cache.length(slots[0])
    per_step = runner.launches_per_step
    engine.close_sequences(slots)
    return {"ms_per_step": ms / steps, "tok_s": batch * steps / (ms / 1e3), "mean_ctx": (ctx0 + ctx1) / 2.0,
            "launches_per_step": per_step, "eager_launches": ops.LAUNCHES[0] - launches_before}


def time_prefill(engine, torch, rng, n_tokens, reps=4) -> float:
    """Median milliseconds of one prompt of ``n_tokens`` in one step (the first run is not counted)."""
    from questwend_b200.engine.engine import StepEntry
    times = []
    for _ in range(reps):
        slot = engine.open_sequences(1)[0]
        prompt = rng.integers(0, engine.vocab_size, n_tokens).tolist()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        engine.step([StepEntry(slot, prompt, [n_tokens - 1])])
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
        engine.close_sequences([slot])
    return statistics.median(times[1:])


def make_engine(cfgd, layers, max_batch, tokens_each, n_ctx=N_CTX):
    from questwend_b200.config.registry import config_from_dict
    from questwend_b200.engine.engine import Engine
    d = dict(cfgd)
    d["num_hidden_layers"] = layers
    return Engine.from_config(config_from_dict(d), seed=0, dtype="bfloat16", max_tokens=max_batch * tokens_each,
                              max_seq_len=n_ctx, max_batch=max_batch), d


def release(engine, torch):
    """Give the engine's device memory back (weights, cache, graphs) whoever still holds the object."""
    engine._runners.clear()
    engine.model = engine.cache = engine.unit_caches = None
    gc.collect()
    torch.cuda.empty_cache()


def small_model_workload(torch, np, peaks) -> dict:
    """Qwen3-0.6B sizes: 16 prompts with lengths uniform in [1, 2048] in ONE prefill step, then 128 decode steps."""
    from questwend_b200.engine.engine import StepEntry
    from questwend_b200.sampling.params import GREEDY
    engine, d = make_engine(QWEN3_06B, QWEN3_06B["num_hidden_layers"], 16, 2048 + 256)
    rng = np.random.default_rng(6)
    lengths = rng.integers(1, 2049, 16).tolist()
    out = {}
    pf = []
    for rep in range(3):
        prompts = [rng.integers(0, engine.vocab_size, n).tolist() for n in lengths]
        slots = engine.open_sequences(16)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        lg = engine.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
        b.record()
        torch.cuda.synchronize()
        pf.append(a.elapsed_time(b))
        if rep < 2:
            engine.close_sequences(slots)
    pf_ms = min(pf[1:])
    runner = engine.decode_runner(16, GREEDY)
    runner.bind(slots, lg.argmax(-1).tolist(), list(range(16)), 1)
    for _ in range(4):
        runner.step()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    len0 = sum(engine.cache.length(s) for s in slots)
    a.record()
    for _ in range(128):
        runner.step()
    b.record()
    torch.cuda.synchronize()
    len1 = sum(engine.cache.length(s) for s in slots)
    ms = a.elapsed_time(b) / 128
    step_bytes = weight_bytes(engine) + (len0 + len1) / 2 * kv_bytes_per_token(d, d["num_hidden_layers"])
    T = sum(lengths)
    flops = sum(prefill_flops(d, d["num_hidden_layers"], n) for n in lengths)
    out = {"m06b_b16_decode": 16 / (ms / 1e3), "m06b_b16_decode_ms": ms,
           "m06b_b16_decode_frac": step_bytes / (ms / 1e3) / 1e9 / peaks["hbm_gbs"],
           "m06b_b16_launches_per_step": runner.launches_per_step, "m06b_prefill": T / (pf_ms / 1e3),
           "m06b_prefill_tokens": T, "m06b_prefill_ms": pf_ms,
           "m06b_prefill_frac": flops / (pf_ms / 1e3) / (peaks["bf16_tflops"] * 1e12)}
    engine.close_sequences(slots)
    release(engine, torch)
    return out


def large_model_workload(torch, np, peaks) -> dict:
    """Qwen3-32B sizes, all 64 layers: a 2,048-token prefill, and decode at batch 1, 8 and 16 from 1,024-token prompts."""
    if True:
        engine, d = make_engine(QWEN3_32B, QWEN3_32B["num_hidden_layers"], 16, PROMPT_LEN + 256)
        rng = np.random.default_rng(32)
        out = {"m32b_weights_gb": weight_bytes(engine) / 1e9}
        for b in (1, 8, 16):
            r = decode_run(engine, torch, b, 3, 16, rng)
            step_bytes = weight_bytes(engine) + b * r["mean_ctx"] * kv_bytes_per_token(d, d["num_hidden_layers"])
            out[f"m32b_decode_b{b}"] = r["tok_s"]
            out[f"m32b_decode_b{b}_frac"] = step_bytes / (r["ms_per_step"] / 1e3) / 1e9 / peaks["hbm_gbs"]
        pf_ms = time_prefill(engine, torch, rng, PREFILL_TOKENS, reps=3)
        out["m32b_prefill"] = PREFILL_TOKENS / (pf_ms / 1e3)
        out["m32b_prefill_ms"] = pf_ms
        out["m32b_prefill_frac"] = (prefill_flops(d, d["num_hidden_layers"], PREFILL_TOKENS) / (pf_ms / 1e3)
                                    / (peaks["bf16_tflops"] * 1e12))
        out["m32b_peak_memory_gb"] = torch.cuda.max_memory_allocated() / 1e9
        release(engine, torch)
    return out


def reference_arm(args) -> int:
    """kishida/questwend itself, unmodified, through its own public classes (baseline/ref_bench.cpp), on the same sizes.
    Nothing of questwend_b200 is imported on this path."""
    def unavailable(why: str) -> int:
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0
    exe = os.path.join(ROOT, "baseline", "_ref", "bin", "qw_ref_bench")
    if not os.path.exists(exe):
        return unavailable("the reference's CUDA build is not in baseline/_ref/bin (python baseline/build_reference.py "
                           "makes it from the CMake project; pip cannot install a project without setup.py or pyproject.toml)")
    if args.gpus != 1:
        return unavailable("kishida/questwend runs on one GPU")
    cfgd = MODELS[args.model]
    layers = args.layers or cfgd["num_hidden_layers"]
    need = 2 * (layers * (cfgd["hidden_size"] * (cfgd["num_attention_heads"] + 2 * cfgd["num_key_value_heads"]) * cfgd["head_dim"]
                          + cfgd["num_attention_heads"] * cfgd["head_dim"] * cfgd["hidden_size"]
                          + 3 * cfgd["hidden_size"] * cfgd["intermediate_size"])
                + 2 * cfgd["vocab_size"] * cfgd["hidden_size"]) + (1 << 30)
    place = None
    for cand in ("/dev/shm", tempfile.gettempdir()):
        try:
            if shutil.disk_usage(cand).free > need:
                place = cand
                break
        except OSError:
            pass
    if place is None:
        return unavailable(f"no room for a {need / 1e9:.0f} GB GGUF of random weights in /dev/shm or the temporary folder")
    warmup, steps = max(3, args.warmup), max(1, args.steps)
    peaks, peak_source = load_peaks()
    tmp = tempfile.mkdtemp(prefix="qw_ref_bench_", dir=place)
    gguf = os.path.join(tmp, "random.gguf")
    cmd = [exe, "--gguf", gguf, "--layers", str(layers), "--hidden", str(cfgd["hidden_size"]),
           "--heads", str(cfgd["num_attention_heads"]), "--kv-heads", str(cfgd["num_key_value_heads"]),
           "--head-dim", str(cfgd["head_dim"]), "--inter", str(cfgd["intermediate_size"]), "--vocab", str(cfgd["vocab_size"]),
           "--n-ctx", str(N_CTX), "--prompt", str(args.ref_prompt or PROMPT_LEN), "--prefill", str(PREFILL_TOKENS),
           "--sequences", str(args.batch), "--steps", str(steps), "--warmup", str(warmup)]
    clocks = ClockSampler()
    clocks.start()
    try:
        proc = subprocess.run(cmd, capture_output=True, text=True, timeout=1500)
    except subprocess.TimeoutExpired:
        clocks.stop()
        shutil.rmtree(tmp, ignore_errors=True)
        return unavailable("the reference's program did not finish within 1500 s")
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    clock_info = clocks.stop()
    sys.stderr.write(proc.stderr[-2000:])
    if proc.returncode != 0:
        last = (proc.stderr.strip().splitlines() or ["no message"])[-1]
        return unavailable(f"the reference's program ended with code {proc.returncode}: {last[:200]}")
    r = json.loads(proc.stdout.strip().splitlines()[-1])
    prompt = args.ref_prompt or PROMPT_LEN
    ctx = prompt + warmup + steps / 2.0
    wbytes = need - (1 << 30) - 2 * cfgd["vocab_size"] * cfgd["hidden_size"]          # the embedding table is only gathered from
    step_bytes = wbytes + ctx * kv_bytes_per_token(cfgd, layers)
    achieved = step_bytes * r["decode_tok_s"] / 1e9
    bucket = -(-int(ctx) // 32) * 32
    out = {"impl": "reference",
           "metric": "decode tokens/s (Qwen3-%s sizes, random bf16 weights, batch %d, n_ctx %d)" % (args.model.upper(), args.batch, N_CTX),
           "value": r["decode_tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
           "ms_per_step": r["ms_per_token"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
           "data": "synthetic: seeded random weights in a GGUF written for the run, uniform random token ids",
           "config": {"model": f"qwen3-{args.model}-sizes", "layers": layers, "layers_full": cfgd["num_hidden_layers"],
                      "hidden_size": cfgd["hidden_size"], "heads": cfgd["num_attention_heads"],
                      "kv_heads": cfgd["num_key_value_heads"], "head_dim": cfgd["head_dim"],
                      "intermediate_size": cfgd["intermediate_size"], "vocab_size": cfgd["vocab_size"],
                      "global_batch": args.batch, "seq_len": N_CTX, "prompt_len": prompt,
                      "batching": "none in the reference: the sequences run one after the other, one token a step",
                      "parallelism": "single-gpu", "l2": "inputs_exceed_l2", "cuda_graph": "ggml's own", "peaks": peak_source,
                      "timing": "host clock around Runtime::decode, which returns after the logits are on the host"},
           "clocks": clock_info,
           "e2e": {"value": r["e2e_tok_s"], "unit": "tokens/s", "h2d_bytes_per_step": 4 + 4 + 8 + 2 * bucket,
                   "d2h_bytes_per_step": 4 * cfgd["vocab_size"]},
           "gpu_launches": None,
           "prefill": {"value": r["prefill_tok_s"], "tokens": r["prefill_tokens"], "ms": r["prefill_ms"],
                       "frac": (prefill_flops(cfgd, layers, r["prefill_tokens"]) / (r["prefill_ms"] / 1e3) /
                                (peaks["bf16_tflops"] * 1e12)) if r["prefill_ms"] else None},
           "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                        "frac": achieved / peaks["hbm_gbs"], "of": peak_source},
           "points": {"decode_b1": r["decode_tok_s"]}}
    print(json.dumps(out))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--model", default="8b", choices=sorted(MODELS))
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (named in config)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-points", action="store_true", help="leave out batch 1 / 64, the e2e run and the other models")
    ap.add_argument("--skip-other-models", action="store_true", help="leave out the 0.6B and 32B workloads")
    ap.add_argument("--ref-prompt", type=int, default=0, help="reference arm: another prompt length (a first, small call)")
    args = ap.parse_args()

    if args.impl == "reference":
        return reference_arm(args)
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

    peaks, peak_source = load_peaks()
    if args.model != "8b":                      # one of the other workloads alone, as a line of its own
        points = small_model_workload(torch, np, peaks) if args.model == "0.6b" else large_model_workload(torch, np, peaks)
        print(json.dumps({"metric": f"Qwen3-{args.model.upper()} sizes workload", "n_gpus": 1, "dtype": "bf16",
                          "data": "synthetic: seeded random weights and uniform random token ids", "peaks": peak_source,
                          "points": points}))
        return 0
    layers = args.layers or QWEN3_8B["num_hidden_layers"]
    max_batch = max(args.batch, 1 if args.skip_points else 64)
    engine, cfgd = make_engine(QWEN3_8B, layers, max_batch, max(PROMPT_LEN + 512, -(-(PREFILL_TOKENS + 64) // max_batch)))
    rng = np.random.default_rng(0)
    wbytes = weight_bytes(engine)
    kv_tok = kv_bytes_per_token(cfgd, layers)

    # ---- the headline: decode at the given batch, device-timed
    clocks = ClockSampler()
    clocks.start()
    main_run = decode_run(engine, torch, args.batch, warmup, steps, rng)
    clock_info = clocks.stop()
    step_s = main_run["ms_per_step"] / 1e3
    step_bytes = wbytes + args.batch * main_run["mean_ctx"] * kv_tok
    achieved = step_bytes / step_s / 1e9

    # ---- prefill of one 2,048-token prompt
    pf_ms = time_prefill(engine, torch, rng, PREFILL_TOKENS)
    pf_flops = prefill_flops(cfgd, layers, PREFILL_TOKENS)
    prefill = {"value": PREFILL_TOKENS / (pf_ms / 1e3), "tokens": PREFILL_TOKENS, "ms": pf_ms,
               "frac": pf_flops / (pf_ms / 1e3) / (peaks["bf16_tflops"] * 1e12)}

    # ---- other batch sizes, and the same batch through the Python entry point
    points, e2e = {}, None
    if not args.skip_points:
        for b in (1, 64):
            r = decode_run(engine, torch, b, 3, 32, rng)
            points[f"decode_b{b}"] = r["tok_s"]
            points[f"decode_b{b}_frac"] = (wbytes + b * r["mean_ctx"] * kv_tok) / (r["ms_per_step"] / 1e3) / 1e9 / peaks["hbm_gbs"]
        prompts = [rng.integers(0, engine.vocab_size, PROMPT_LEN).tolist() for _ in range(args.batch)]
        stats = qw.GenerationStats()
        qw.generate(engine, prompts, max_new_tokens=warmup + 1, ignore_eos=True)          # warm the graphs
        # one call: the prompts, `warmup` untimed decode steps, then the `steps` timed ones (the loop's own clock around
        # each step: tokens from pinned host memory in, the step, its ids back on the host)
        qw.generate(engine, prompts, max_new_tokens=warmup + steps + 1, ignore_eos=True, stats=stats)
        timed = stats.step_seconds[-steps:]
        e2e = {"value": args.batch * len(timed) / sum(timed), "unit": "tokens/s",
               "h2d_bytes_per_step": 4 * args.batch, "d2h_bytes_per_step": 4 * args.batch,
               "steps": len(timed), "warmup_steps": len(stats.step_seconds) - len(timed),
               "value_all_steps": args.batch * stats.steps / stats.decode_seconds}
        for n in (4096,):          # the whole context of the benchmark's configuration
            ms = time_prefill(engine, torch, rng, n, reps=3)
            points[f"prefill_{n}"] = n / (ms / 1e3)
            points[f"prefill_{n}_frac"] = prefill_flops(cfgd, layers, n) / (ms / 1e3) / (peaks["bf16_tflops"] * 1e12)
    release(engine, torch)
    del engine
    if not (args.skip_points or args.skip_other_models):
        points.update(small_model_workload(torch, np, peaks))
        points.update(large_model_workload(torch, np, peaks))

    out = {
        "metric": "decode tokens/s (Qwen3-8B sizes, random bf16 weights, batch %d, n_ctx %d)" % (args.batch, N_CTX),
        "value": main_run["tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": main_run["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random weights and uniform random token ids",
        "config": {"model": "qwen3-8b-sizes", "layers": layers, "layers_full": QWEN3_8B["num_hidden_layers"],
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
