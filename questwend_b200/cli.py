"""qw-cli: generate from token ids on the command line.

The options that kishida/questwend's ``qw-cli`` has keep their names, meanings and defaults
(cli/main.cpp:86-124, 134-191): ``-m`` the model, ``-p`` the prompt, ``-n`` max new tokens (128),
``--n-ctx`` the context length (default: the model's trained length), ``--temp`` (0 = greedy, the
default), ``--top-p`` (0.95), ``--top-k`` (40), ``--seed`` (0 = random), ``--repeat-penalty`` (1 = off),
``--repeat-last-n`` (64), ``--log-tokens-per-sec``, ``--info``.  There is no tokenizer here, so a
prompt is a list of token ids: ``-p "1 2 3"`` (spaces or commas); ``-p`` may be given several times,
and ``--ids-file`` reads one prompt per line; the prompts then run as batches.  ``-m`` names a
folder with config.json and model.safetensors; instead of it, ``--random <config.json>`` takes a
configuration alone and draws the weights from ``--seed`` (N(0, 0.02), norms 1 + U(-0.1, 0.1)), on the
device, or, with ``--save <folder>``, on the CPU into a model folder that is written and then loaded
(the same numbers on every machine).  ``--profile-step`` prints where every decode step's time went
(the reference's QWEN_PROF, core/runtime.cpp:1769, 1821-1825).  Generation stops at the model's ``eos_token_id``
(the reference stops at its vocabulary's EOS and at <|im_end|>, cli/main.cpp:374-376) and at any
``--stop-id``; a stop token is not printed.  Output: one line of generated ids per prompt.
"""
from __future__ import annotations

import argparse
import json
import re
import sys


def parse_ids(text: str) -> list[int]:
    parts = [p for p in re.split(r"[\s,]+", text.strip()) if p]
    try:
        return [int(p) for p in parts]
    except ValueError:
        raise SystemExit(f"error: a prompt is a list of token ids, got: {text!r}") from None


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="qw-cli", description="generate from token ids with a Qwen3 model on one B200")
    ap.add_argument("-m", dest="model", help="model folder (config.json + model.safetensors)")
    ap.add_argument("--random", metavar="CONFIG_JSON", help="instead of -m: a config.json; the weights are drawn from --seed")
    ap.add_argument("--save", metavar="DIR", help="with --random: write the model folder there (config.json + model.safetensors)")
    ap.add_argument("-p", dest="prompts", action="append", default=[], help="prompt as token ids, e.g. \"1 2 3\"")
    ap.add_argument("--ids-file", help="file with one prompt (token ids) per line")
    ap.add_argument("-n", dest="max_tokens", type=int, default=128, help="max new tokens (default 128)")
    ap.add_argument("--n-ctx", type=int, default=0, help="context length (default: the model's trained length)")
    ap.add_argument("--temp", type=float, default=0.0, help="temperature (0 = greedy, default 0)")
    ap.add_argument("--top-p", type=float, default=0.95, help="nucleus top-p (default 0.95)")
    ap.add_argument("--top-k", type=int, default=40, help="top-k (default 40)")
    ap.add_argument("--seed", type=int, default=0, help="RNG seed (0 = random)")
    ap.add_argument("--repeat-penalty", type=float, default=1.0, help="repetition penalty over the last N tokens (default 1 = off)")
    ap.add_argument("--repeat-last-n", type=int, default=64, help="penalty window (default 64)")
    ap.add_argument("--presence-penalty", type=float, default=0.0)
    ap.add_argument("--frequency-penalty", type=float, default=0.0)
    ap.add_argument("--stop-id", type=int, action="append", default=None, help="token id that ends a sequence (repeatable)")
    ap.add_argument("--ignore-eos", action="store_true", help="never stop at a stop token")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--max-batch", type=int, default=64, help="most sequences generated at once")
    ap.add_argument("--log-tokens-per-sec", action="store_true", help="print speed")
    ap.add_argument("--info", action="store_true", help="print model info and exit")
    ap.add_argument("--profile-step", action="store_true", help="print where every decode step's time went")
    return ap


def model_info(config, dtype: str) -> dict:
    """The configuration, the tensors it asks for, and what the model takes in memory: the weights as the engine holds
    them and the cache per token of a live sequence (the reference's ``--info`` prints its summary, cli/main.cpp:236-239)."""
    import math

    import torch

    from .config.registry import get_architecture
    from .engine.model import Model
    from .parts.base import Runtime
    from .weights.loader import held_dtype
    plan = get_architecture(config.architecture).plan(config)
    compute = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    model = Model(plan, Runtime(torch.device("cpu"), compute))
    tensors = [t for t in model.tensors() if not (t.optional or t.ignored)]
    size = lambda dt: torch.empty((), dtype=dt).element_size()
    weight_bytes = sum(math.prod(t.shape) * size(held_dtype(t, compute, compute)) for t in tensors)
    cache_bytes = sum(2 * kv.n_kv_heads * kv.head_dim * size(compute)
                      for kv, _, cache_of in model.cache_units() if kv is not None and cache_of is None)
    state_bytes = sum(math.prod(st.shape) * size(st.dtype)
                      for _, st, cache_of in model.cache_units() if st is not None and cache_of is None)
    return {"config": config.to_dict(), "parameters": sum(math.prod(t.shape) for t in tensors), "layers": len(plan.layers),
            "tensors": len(plan.manifest()),
            "memory": {"dtype": dtype, "weight_bytes": weight_bytes, "cache_bytes_per_token": cache_bytes,
                       "state_bytes_per_sequence": state_bytes}}


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    from .config.registry import config_from_dict, load_config
    from .engine.engine import Engine
    from .engine.generate import GenerationStats, generate
    from .sampling.params import SamplingParams
    from .weights.random_init import write_model_folder

    if bool(args.model) == bool(args.random):
        raise SystemExit("error: give either -m <model folder> or --random <config.json>")
    if args.save and not args.random:
        raise SystemExit("error: --save goes with --random")
    if args.random:
        import os
        with open(args.random) as f:
            config = config_from_dict(json.load(f), args.random)
        if args.save:
            write_model_folder(args.save, config, args.seed, args.dtype)
            args.model = args.save
            if not (args.prompts or args.ids_file or args.info):
                print(os.path.abspath(args.save))
                return 0
    else:
        config = load_config(args.model)
    if args.info:
        print(json.dumps(model_info(config, args.dtype), indent=2))
        return 0
    prompts = [parse_ids(p) for p in args.prompts]
    if args.ids_file:
        with open(args.ids_file) as f:
            prompts += [parse_ids(line) for line in f if line.strip()]
    if not prompts:
        raise SystemExit("error: no prompt; give -p \"<token ids>\" or --ids-file")
    n_ctx = args.n_ctx or getattr(config, "max_position_embeddings", None) or 4096
    batch = min(args.max_batch, len(prompts))
    longest = min(n_ctx, max(len(p) for p in prompts) + args.max_tokens)
    sizes = dict(max_tokens=batch * (longest + 64), max_seq_len=n_ctx, max_batch=batch)
    if args.model:
        engine = Engine.from_folder(args.model, dtype=args.dtype, **sizes)
    else:
        engine = Engine.from_config(config, seed=args.seed, dtype=args.dtype, **sizes)
    sampling = SamplingParams(temperature=args.temp, top_p=args.top_p, top_k=args.top_k, seed=args.seed,
                              repeat_penalty=args.repeat_penalty, presence_penalty=args.presence_penalty,
                              frequency_penalty=args.frequency_penalty, repeat_last_n=args.repeat_last_n)
    stats = GenerationStats()
    stop_ids = None
    if args.stop_id is not None:
        stop_ids = tuple(args.stop_id) + tuple(engine.plan.stop_token_ids)
    results = generate(engine, prompts, max_new_tokens=args.max_tokens, sampling=sampling, stop_ids=stop_ids,
                       ignore_eos=args.ignore_eos, stats=stats, profile=True if args.profile_step else None)
    for r in results:
        print(" ".join(str(t) for t in r.tokens))
    if args.log_tokens_per_sec:
        print(stats.line(), file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
