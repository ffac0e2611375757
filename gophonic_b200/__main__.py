"""Command line: load a model once, reply to every input, print one JSON line each.

Flags follow gophonic's command (cmd/gophonic/main.go:28-38: ``-model``, ``-format``,
``-threads``) and its reply options (chat/chat.go:50-67; the server's request fields
internal/httpserver/chat.go:46-110: ``max_tokens``, ``temperature``, ``top_k``, ``top_p``,
``presence_penalty``, ``seed``).  The model is a checkpoint folder (``-model``) or a named
configuration with seeded random weights (``-random-config``, with ``-weights-seed`` and
``-layers``; ``-write-model DIR`` writes that model as a folder instead of generating).  Inputs
are prompts as comma-separated token ids on the command line or one a line in ``-prompt-ids
FILE``; where the model folder has a tokenizer, ``-prompt TEXT`` asks in text through the chat
lane and the reply is printed as text too.

    python -m gophonic_b200 -model DIR -max-tokens 16 "1,2,3" "4,5"
    python -m gophonic_b200 -random-config tinyA -weights-seed 3 -max-tokens 8 -prompt-ids prompts.txt
"""
from __future__ import annotations

import argparse
import json
import sys


def _ids(text: str):
    return [int(t) for t in text.replace(",", " ").split()]


def main(argv=None) -> int:
    from .config.presets import preset_names
    ap = argparse.ArgumentParser(prog="gophonic_b200", description="generate from a Qwen3 model folder")
    ap.add_argument("-model", "--model", default="", help="model: a checkpoint directory (config.json, model.safetensors)")
    ap.add_argument("-random-config", "--random-config", default="", choices=[""] + preset_names(),
                    help="instead of -model: a named configuration with seeded random weights")
    ap.add_argument("-weights-seed", "--weights-seed", type=int, default=0, help="seed of the random weights")
    ap.add_argument("-layers", "--layers", type=int, default=0, help="keep this many layers of the named configuration (0: all)")
    ap.add_argument("-write-model", "--write-model", default="", help="write the random model as a folder here and exit")
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
    ap.add_argument("-prompt-ids", "--prompt-ids", default="", help="a file of prompts, one a line, as token ids")
    ap.add_argument("-prompt", "--prompt", action="append", default=[], help="a question in text (needs the folder's tokenizer.json)")
    ap.add_argument("-system", "--system", default="", help="system message of the text conversation")
    ap.add_argument("prompts", nargs="*", help="prompts as comma-separated token ids")
    args = ap.parse_args(argv)
    if args.threads < 0 or bool(args.model) == bool(args.random_config):
        ap.print_usage(sys.stderr)
        print("gophonic_b200: give either -model or -random-config", file=sys.stderr)
        return 2
    from .api import ChatGeneratorLane, ChatOptions, Lane, Open, Options, TokensGenerator, random_model_path
    try:
        prompts = [_ids(p) for p in args.prompts]
        if args.prompt_ids:
            with open(args.prompt_ids) as f:
                prompts += [_ids(line) for line in f if line.strip()]
        stops = None if args.stop is None else _ids(args.stop)
    except (ValueError, OSError) as e:
        print(f"gophonic_b200: {e}", file=sys.stderr)
        return 2
    try:
        if args.write_model:
            if not args.random_config:
                raise ValueError("-write-model needs -random-config")
            from .api import _parse_random
            from .weights import write_random_model
            config, seed = _parse_random(random_model_path(args.random_config, args.weights_seed, args.layers))
            write_random_model(config, seed, args.write_model, "float32" if args.format == "f32" else "bfloat16")
            print(json.dumps({"wrote": args.write_model, "config": args.random_config, "seed": seed}), flush=True)
            return 0
        if not prompts and not args.prompt:
            raise ValueError("no prompt: give token ids, -prompt-ids FILE or -prompt TEXT")
        path = args.model or random_model_path(args.random_config, args.weights_seed, args.layers)
        model = Open(path, Options(Threads=args.threads, Format=args.format, Device=args.device, Batch=args.batch))
        opts = ChatOptions(MaxTokens=args.max_tokens, Temperature=args.temperature, TopK=args.top_k,
                           TopP=args.top_p, Presence=args.presence, Seed=args.seed)
        if prompts:
            gen = Lane(model, TokensGenerator)
            replies = gen.Generate(prompts, opts, stop_ids=stops)
            for p, r in zip(prompts, replies):
                print(json.dumps({"prompt": p, "tokens": r}), flush=True)
        if args.prompt:
            from .chat import User
            chat = Lane(model, ChatGeneratorLane)
            if chat.tokenizer is None:
                raise ValueError("-prompt needs a tokenizer.json in the model folder; give token ids instead")
            for question in args.prompt:       # each question is a conversation of its own
                session = chat.NewSession(args.system or None)
                session.Add(User, question)
                reply = session.Reply(opts)
                print(json.dumps({"prompt": question, "text": chat.tokenizer.decode(reply, skip_special=True), "tokens": reply}),
                      flush=True)
                session.Close()
            chat.Close()
        model.Close()
    except Exception as e:  # one line, as the reference's command prints its errors
        print(f"gophonic_b200: {e}", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
