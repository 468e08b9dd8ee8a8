"""The command line, in the reference's manner.

The reference answers one prompt with ``bc mesh run <model> <prompt> --max-tokens 256
--temperature 0.0`` (apps/bc-cli/src/main.rs:130-144), samples with top_p 0.95 and a seed
from the clock (main.rs:542,590), and reports "N prompt tokens, first token after X ms; M
tokens in P passes, R tokens/s" (main.rs:550-554).  Its example program is ``generate
<model> "<prompt>" [tokens]`` (crates/bc-infer/examples/generate.rs).  The same words are
kept here; a prompt is a list of token ids, since text and tokenizers are outside this
library, and several prompts separated by ';' run as one batch.

    bc-infer generate <model folder> "1,2,3;7,8" --max-tokens 64 --temperature 0.8
    bc-infer random <config.json> <new folder> --seed 1       # a model folder of random weights
"""

from __future__ import annotations

import argparse
import json
import sys
import time
from typing import List


def parse_prompts(text: str) -> List[List[int]]:
    prompts = []
    for part in text.replace("\n", ";").split(";"):
        part = part.strip()
        if part:
            prompts.append([int(t) for t in part.replace(",", " ").split()])
    return prompts


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="bc-infer", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="command", required=True)
    g = sub.add_parser("generate", help="answer one prompt, or a batch of them")
    g.add_argument("model", help="a folder with config.json and model.safetensors")
    g.add_argument("prompt", nargs="?", default=None, help="token ids, e.g. '1,2,3'; several prompts separated by ';'")
    g.add_argument("--prompt-file", help="a file of prompts, one list of token ids a line")
    g.add_argument("--max-tokens", type=int, default=256)
    g.add_argument("--temperature", type=float, default=0.0)
    g.add_argument("--top-p", type=float, default=0.95)
    g.add_argument("--seed", type=int, default=None, help="sampling seed (default: from the clock)")
    g.add_argument("--stop-ids", default=None, help="token ids that end a sequence (default: the model's eos ids)")
    g.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    g.add_argument("--max-batch", type=int, default=None, help="most sequences that run together; more run as later batches")
    g.add_argument("--max-seq", type=int, default=None, help="positions a sequence can reach (default: the longest prompt plus --max-tokens)")
    g.add_argument("--include-stop", action="store_true", help="a stop id that ends a sequence is printed as its last id")
    g.add_argument("--stats", action="store_true", help="print the call's Stats as one JSON line on standard output, after the tokens")
    g.add_argument("--device", default="cuda:0")
    r = sub.add_parser("random", help="write a model folder of random weights for a config.json")
    r.add_argument("config", help="a config.json")
    r.add_argument("folder", help="the folder to write")
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    args = ap.parse_args(argv)

    if args.command == "random":
        import torch

        from .weights import write_model_folder

        with open(args.config) as f:
            config = json.load(f)
        write_model_folder(args.folder, config, args.seed, torch.bfloat16 if args.dtype == "bfloat16" else torch.float32)
        print(f"bc: wrote {args.folder}", file=sys.stderr)
        return 0

    text = args.prompt
    if args.prompt_file:
        with open(args.prompt_file) as f:
            text = f.read()
    if not text:
        ap.error("a prompt is needed (token ids), or --prompt-file")
    prompts = parse_prompts(text)
    from .local import Local
    from .sampling import Sampling

    longest = max(len(p) for p in prompts) + args.max_tokens
    if args.max_seq is not None:
        if args.max_seq < longest:
            ap.error(f"--max-seq {args.max_seq} is less than the longest prompt plus --max-tokens ({longest})")
        longest = args.max_seq
    batch = min(len(prompts), args.max_batch or len(prompts))
    model = Local.load(args.model, dtype=args.dtype, device=args.device, max_seq=longest, max_slots=batch,
                       max_tokens=batch * (-(-longest // 64) * 64))
    seed = args.seed if args.seed is not None else time.time_ns() & ((1 << 64) - 1)
    stops = None if args.stop_ids is None else [int(t) for t in args.stop_ids.replace(",", " ").split()]
    out, stats = model.generate(prompts, args.max_tokens, Sampling(args.temperature, args.top_p, seed), stop_ids=stops, max_batch=batch,
                                include_stop=args.include_stop)
    for tokens in out:
        print(",".join(str(t) for t in tokens))
    if args.stats:
        print(json.dumps({"prompt_tokens": stats.prompt_tokens, "generated": stats.generated, "passes": stats.passes,
                          "first_token_ms": round(stats.first_token_ms, 3), "total_ms": round(stats.total_ms, 3),
                          "decode_tokens_per_second": round(stats.decode_tokens_per_second, 2)}))
    print(f"bc: {stats.prompt_tokens} prompt tokens, first token after {stats.first_token_ms:.0f} ms; {stats.generated} tokens in "
          f"{stats.passes} passes, {stats.decode_tokens_per_second:.1f} tokens/s", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
