"""Offline generation from the command line, options in the reference's manner: ``--model``,
``--max-tokens``, and JSON keyword dictionaries ``--arch-kw`` / ``--engine-kw`` passed to the
declaration and the engine (Tokenomos api/server.py:211-228, bench/decode.py:32-60)::

    python -m tokenomos_b200.generate --model DIR --prompt-ids 1,2,3 --prompt-ids 7,8 \\
        --max-tokens 16 --temperature 0.8 --seed 3 --arch-kw '{"work": "bf16"}' \\
        --engine-kw '{"page": 16, "max_len": 512}'

Prints one JSON object per prompt: ``{"prompt_tokens": n, "token_ids": [...], "finish": ...,
"text": ...}``. ``--random-weights CONFIG.json`` first writes a model folder with random weights
at ``--model`` from that configuration and ``--seed-weights``.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(prog="python -m tokenomos_b200.generate")
    ap.add_argument("--model", required=True, help="model folder (config.json + safetensors)")
    ap.add_argument("--prompt-ids", action="append", default=[],
                    help="comma-separated token ids; repeat for several prompts")
    ap.add_argument("--prompt", action="append", default=[],
                    help="text prompt (needs tokenizer.json in the folder); repeatable")
    ap.add_argument("--max-tokens", type=int, default=256)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--min-p", type=float, default=0.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--stop-token-ids", default="", help="comma-separated token ids")
    ap.add_argument("--arch-kw", default="{}", help='JSON kwargs of the declaration, e.g. {"work": "fp32"}')
    ap.add_argument("--engine-kw", default="{}", help="JSON kwargs of the engine")
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--random-weights", default=None,
                    help="a config.json to write a random-weights model folder from, at --model")
    ap.add_argument("--seed-weights", type=int, default=0)
    ap.add_argument("--std", type=float, default=0.02)
    args = ap.parse_args(argv)

    import torch

    from tokenomos_b200 import models
    from tokenomos_b200.api.llm import LLM, SamplingParams
    from tokenomos_b200.weights import write_model_folder

    if args.random_weights:
        config = json.loads(Path(args.random_weights).read_text("utf-8"))
        write_model_folder(args.model, config, args.seed_weights, args.std, 0.0, torch.bfloat16)
    prompts: list = [[int(t) for t in p.split(",") if t.strip()] for p in args.prompt_ids]
    prompts += args.prompt
    if not prompts:
        ap.error("give at least one --prompt-ids or --prompt")
    stops = tuple(int(t) for t in args.stop_token_ids.split(",") if t.strip())
    params = SamplingParams(args.max_tokens, args.temperature, args.top_p, args.top_k, args.min_p,
                            args.seed, stops)
    arch = models.configure(args.model, **json.loads(args.arch_kw))
    with LLM(args.model, args.device, arch, **json.loads(args.engine_kw)) as llm:
        for out in llm.generate(prompts, params):
            print(json.dumps({"prompt_tokens": out.prompt_tokens, "token_ids": out.token_ids,
                              "finish": out.finish, "text": out.text}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
