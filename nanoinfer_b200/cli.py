"""Command line, in the manner of the reference's demos (demo/llama.cpp:94-110,
demo/batched_infer_multi_prompts.cpp:18-25): same option names where it has them
(--model, --dtype, --temperature, --top-k, --top-p, --rep-penalty, --seed), its engine
limits as options instead of compile-time constants, and the same report (generated ids,
time to first token, prefill and decode tokens per second).  Prompts are token ids.

    bin/nanoinfer generate --model DIR --prompt-ids 1,15,7 --max-new-tokens 32
    bin/nanoinfer random-model --config config.json --seed 0 --out DIR
    bin/nanoinfer random-model --preset llama-3.2-1b --layers 4 --out DIR
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from typing import List


def _parse_ids(text: str) -> List[int]:
    return [int(x) for x in text.replace(",", " ").split()]


def _generate(args) -> int:
    import torch

    from .engine import Engine, EngineConfig
    from .sampling import SamplingParams

    cfg = EngineConfig(max_batch_size=args.max_batch_size, max_sequences=args.max_sequences,
                       prefill_chunk_size=args.prefill_chunk_size, block_size=args.block_size,
                       num_cache_blocks=args.num_cache_blocks,
                       max_num_batched_tokens=args.max_num_batched_tokens, dtype=args.dtype)
    t0 = time.perf_counter()
    engine = Engine.from_model_dir(args.model, cfg)
    print(f"model loaded in {time.perf_counter() - t0:.2f} s: {engine.runner.config.architecture}, "
          f"{engine.runner.config.num_layers} layers, dtype {args.dtype}", file=sys.stderr)
    prompts: List[List[int]] = [_parse_ids(p) for p in args.prompt_ids or []]
    if args.prompt_file:
        with open(args.prompt_file) as f:
            prompts += [_parse_ids(line) for line in f if line.strip()]
    if args.prompt_len:
        g = torch.Generator().manual_seed(0)
        prompts.append(torch.randint(0, engine.runner.config.vocab_size, (args.prompt_len,), generator=g).tolist())
    if not prompts:
        print("no prompt given (use --prompt-ids, --prompt-file or --prompt-len)", file=sys.stderr)
        return 2
    sp = SamplingParams(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p,
                        repetition_penalty=args.rep_penalty, seed=args.seed)
    ids = [engine.add_request(p, args.max_new_tokens, sp) for p in prompts]
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    engine.run()
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - t0
    n_prompt = sum(len(p) for p in prompts)
    n_new = 0
    for rid in ids:
        req = engine.get_request(rid)
        n_new += len(req.generated_tokens)
        ttft = (req.first_token_time - req.arrival_time) if req.first_token_time else float("nan")
        print(json.dumps({"request": rid, "prompt_tokens": len(req.prompt_tokens), "state": req.state.value,
                          "finish_reason": req.finish_reason, "ttft_s": round(ttft, 4),
                          "generated": req.generated_tokens}))
    print(f"{len(ids)} requests, {n_prompt} prompt tokens, {n_new} generated tokens in {elapsed:.3f} s "
          f"({engine.num_steps} steps): {(n_prompt + n_new) / elapsed:.1f} tok/s overall, "
          f"{n_new / elapsed:.1f} generated tok/s", file=sys.stderr)
    return 0


def _random_model(args) -> int:
    import torch

    from .weights import write_random_model
    if (args.config is None) == (args.preset is None):
        print("random-model: give either --config FILE or --preset NAME", file=sys.stderr)
        return 2
    if args.preset is not None:
        from .config import preset
        raw = preset(args.preset)
    else:
        with open(args.config) as f:
            raw = json.load(f)
    if args.layers is not None:
        raw = dict(raw, num_hidden_layers=args.layers)
    dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[args.dtype]
    write_random_model(args.out, raw, args.seed, args.std, dtype)
    print(f"wrote {args.out}/config.json and model.safetensors (seed {args.seed})", file=sys.stderr)
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="nanoinfer", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="command", required=True)
    g = sub.add_parser("generate", help="generate from token-id prompts")
    g.add_argument("--model", required=True, help="model folder (config.json + *.safetensors)")
    g.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    g.add_argument("--prompt-ids", action="append", help="comma separated token ids; may be repeated")
    g.add_argument("--prompt-file", help="one prompt per line, token ids separated by spaces or commas")
    g.add_argument("--prompt-len", type=int, help="add a random prompt of this many tokens")
    g.add_argument("--max-new-tokens", type=int, default=128)
    g.add_argument("--temperature", type=float, default=0.0, help="0 = greedy (the demos' default)")
    g.add_argument("--top-k", type=int, default=-1)
    g.add_argument("--top-p", type=float, default=1.0)
    g.add_argument("--rep-penalty", type=float, default=1.0)
    g.add_argument("--seed", type=int, default=-1)
    g.add_argument("--max-batch-size", type=int, default=32)
    g.add_argument("--max-sequences", type=int, default=128)
    g.add_argument("--prefill-chunk-size", type=int, default=512)
    g.add_argument("--block-size", type=int, default=16)
    g.add_argument("--num-cache-blocks", type=int, default=1024)
    g.add_argument("--max-num-batched-tokens", type=int, default=2048)
    g.set_defaults(func=_generate)
    r = sub.add_parser("random-model", help="write a model folder with random weights")
    r.add_argument("--config", help="a config.json to build the model from")
    r.add_argument("--preset", help="or one of the package's config.json files: llama-3.2-1b, llama-3.2-3b, llama-3.1-8b")
    r.add_argument("--layers", type=int, help="another number of layers than the configuration names")
    r.add_argument("--out", required=True)
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--std", type=float, default=0.02)
    r.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    r.set_defaults(func=_random_model)
    args = ap.parse_args(argv)
    return args.func(args)


if __name__ == "__main__":
    sys.exit(main())
