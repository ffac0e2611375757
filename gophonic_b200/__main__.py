"""Command line: load a model folder once, reply to every input, print one JSON line each.

Flags follow gophonic's command (cmd/gophonic/main.go:28-38: ``-model``, ``-format``,
``-threads``) and its reply options (chat/chat.go:50-67; the server's request fields
internal/httpserver/chat.go:46-110: ``max_tokens``, ``temperature``, ``top_k``, ``top_p``,
``presence_penalty``, ``seed``).  Inputs are prompts as comma-separated token ids.

    python -m gophonic_b200 -model DIR -max-tokens 16 "1,2,3" "4,5"
"""
from __future__ import annotations

import argparse
import json
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="gophonic_b200", description="generate from a Qwen3 model folder")
    ap.add_argument("-model", "--model", required=True, help="model: a checkpoint directory (config.json, model.safetensors)")
    ap.add_argument("-format", "--format", default="", help="weight format: bf16 or f32 (default: bf16)")
    ap.add_argument("-threads", "--threads", type=int, default=0, help="accepted for compatibility; the engine uses no CPU workers")
    ap.add_argument("-max-tokens", "--max-tokens", type=int, default=0, help="bound of each reply (0: the context)")
    ap.add_argument("-temperature", "--temperature", type=float, default=0.0, help="0 picks the most likely token")
    ap.add_argument("-top-k", "--top-k", type=int, default=0, help="keep the k most likely tokens (0: all, at most 1024)")
    ap.add_argument("-top-p", "--top-p", type=float, default=0.0, help="nucleus probability (0 or 1: off)")
    ap.add_argument("-presence", "--presence", type=float, default=0.0, help="presence penalty")
    ap.add_argument("-seed", "--seed", type=int, default=0, help="sampling seed")
    ap.add_argument("-stop", "--stop", default=None,
                    help="comma-separated stop token ids (default: the end-of-sequence ids the model folder names; '' for none)")
    ap.add_argument("-batch", "--batch", type=int, default=8, help="sequences that start together")
    ap.add_argument("-device", "--device", default="cuda:0")
    ap.add_argument("prompts", nargs="+", help="prompts as comma-separated token ids")
    args = ap.parse_args(argv)
    if args.threads < 0:
        ap.print_usage(sys.stderr)
        return 2
    from .api import ChatOptions, Lane, Open, Options, TokensGenerator
    try:
        prompts = [[int(t) for t in p.replace(" ", "").split(",") if t] for p in args.prompts]
        stops = None if args.stop is None else [int(t) for t in args.stop.split(",") if t]
    except ValueError as e:
        print(f"gophonic_b200: {e}", file=sys.stderr)
        return 2
    try:
        model = Open(args.model, Options(Threads=args.threads, Format=args.format, Device=args.device, Batch=args.batch))
        gen = Lane(model, TokensGenerator)
        opts = ChatOptions(MaxTokens=args.max_tokens, Temperature=args.temperature, TopK=args.top_k,
                           TopP=args.top_p, Presence=args.presence, Seed=args.seed)
        replies = gen.Generate(prompts, opts, stop_ids=stops)
        for p, r in zip(prompts, replies):
            print(json.dumps({"prompt": p, "tokens": r}), flush=True)
        model.Close()
    except Exception as e:  # one line, as the reference's command prints its errors
        print(f"gophonic_b200: {e}", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
