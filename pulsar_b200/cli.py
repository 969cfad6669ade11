"""Command line: generate token ids from a model folder.

The reference has no generate command; its evaluation harness gives the house style of
the options (scripts/eval_longbench.py:887-1141: ``--model``, ``--device``,
``--gen_tokens``, ``--temperature``, ``--top_p``, ``--top_k``, ``--seed``,
``--max_chunk_size``, ``--active_buffer_size``, ``--max_pages``, ``--json``), which keep
their names, defaults and meanings here.  Prompts are token ids: tokenizers are out of
scope of this engine.
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from typing import List


def parse_args(argv=None) -> argparse.Namespace:
    ap = argparse.ArgumentParser(prog="pulsar-generate", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True, help="model folder (config.json + model.safetensors)")
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--prompt_ids", action="append", default=[],
                    help="comma-separated token ids of one prompt; repeat for a batch")
    ap.add_argument("--prompt_file", help="file with one prompt per line (token ids separated by spaces or commas), "
                                          "or a JSON list of lists")
    ap.add_argument("--gen_tokens", type=int, default=512, help="new tokens per prompt")
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top_p", type=float, default=1.0)
    ap.add_argument("--top_k", type=int, default=0)
    ap.add_argument("--seed", type=int, default=-1)
    ap.add_argument("--eos_id", type=int, default=None, help="stop token (default: the model's eos_token_id; -1 none)")
    ap.add_argument("--max_chunk_size", type=int, default=512, help="token budget of one step")
    ap.add_argument("--active_buffer_size", type=int, default=32768, help="tokens of cache per session")
    ap.add_argument("--max_sessions", type=int, default=8)
    ap.add_argument("--max_running", type=int, default=8)
    ap.add_argument("--max_pages", type=int, default=None, help="pages of the cache pool (overrides "
                                                                "max_sessions * active_buffer_size / page_size)")
    ap.add_argument("--page_size", type=int, default=16)
    ap.add_argument("--random_weights", metavar="CONFIG_JSON",
                    help="write --model from this config.json with seeded random weights first")
    ap.add_argument("--weights_seed", type=int, default=0)
    ap.add_argument("--json", action="store_true", help="print one JSON object instead of text")
    return ap.parse_args(argv)


def read_prompts(args) -> List[List[int]]:
    prompts = [[int(t) for t in p.replace(",", " ").split()] for p in args.prompt_ids]
    if args.prompt_file:
        text = open(args.prompt_file).read().strip()
        if text.startswith("["):
            prompts += [[int(t) for t in p] for p in json.loads(text)]
        else:
            prompts += [[int(t) for t in line.replace(",", " ").split()] for line in text.splitlines() if line.strip()]
    if not prompts:
        raise SystemExit("no prompt: give --prompt_ids or --prompt_file")
    return prompts


def main(argv=None) -> int:
    args = parse_args(argv)
    prompts = read_prompts(args)
    if args.random_weights:
        import torch
        from .config import config_from_dict
        from .weights import write_model_folder
        with open(args.random_weights) as f:
            write_model_folder(config_from_dict(json.load(f)), args.model, args.weights_seed,
                               store_dtype=torch.bfloat16 if args.dtype == "bfloat16" else torch.float32)
    from .config.model_config import read_config_json
    from .engine.engine import Engine
    eos = args.eos_id
    if eos is None:
        raw_eos = read_config_json(args.model).get("eos_token_id", -1)
        eos = (raw_eos[0] if isinstance(raw_eos, list) and raw_eos else raw_eos) if raw_eos is not None else -1
    config = dict(device=args.device, dtype=args.dtype, page_size=args.page_size, max_sessions=args.max_sessions,
                  active_buffer_size=args.active_buffer_size, max_running=args.max_running,
                  max_chunk_size=args.max_chunk_size, eos_id=int(eos), temperature=args.temperature,
                  top_p=args.top_p, top_k=args.top_k, seed=args.seed)
    if args.max_pages is not None:
        config["num_pages"] = args.max_pages
    engine = Engine(args.model, config)
    t0 = time.time()
    outputs = engine.generate(prompts, args.gen_tokens, seed=args.seed)
    dt = time.time() - t0
    n_new = sum(len(o) for o in outputs)
    if args.json:
        print(json.dumps({"outputs": outputs, "new_tokens": n_new, "seconds": dt, "forwards": engine.forwards}))
    else:
        for i, o in enumerate(outputs):
            print(f"[{i}] " + " ".join(str(t) for t in o))
        print(f"{n_new} tokens in {dt:.3f}s ({n_new / max(dt, 1e-9):.1f} tok/s, {engine.forwards} forwards)", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
