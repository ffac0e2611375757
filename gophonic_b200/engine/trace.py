"""Trace replay: feed given token ids through a model step by step and write fp32 logits.

The program samples nothing and has no model code of its own: it opens the model through the
registry, makes the engine's cache, and calls the engine's step function, exactly as
generation does.  Input is one JSON object a line on standard input:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

A request that appears for the first time gets a cache slot; ``end`` gives slots back after the
step.  For a step that wants logits, ``<out>/<step>.f32`` holds them as little-endian float32,
[wanted, vocab], in the order of the entries and of each ``want``.  After every step the line
``done <step>`` is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Dict

import numpy as np


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at once, each rounded up to a multiple of 64")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)

    import torch
    from .model import Model
    from .step import Engine

    os.makedirs(args.out, exist_ok=True)
    model = Model.from_dir(args.model, dtype=args.dtype, device=args.device)
    engine = Engine(model, max_tokens=args.max_tokens)
    slots: Dict[str, int] = {}

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries, want = [], []
        fresh = []
        try:
            for e in rec.get("entries", []):
                rid = str(e["id"])
                if rid not in slots:
                    slots[rid] = engine.new_sequence()
                    fresh.append(rid)
                entries.append((slots[rid], [int(t) for t in e["tokens"]]))
                want.append([int(w) for w in e.get("want", [])])
            logits = engine.step(entries, want) if entries else None
        except Exception:
            for rid in fresh:  # a refused step leaves nothing behind
                engine.end_sequence(slots.pop(rid))
            raise
        engine.check_kernels()
        if logits is not None and logits.numel() > 0:
            arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
            arr.tofile(os.path.join(args.out, f"{step}.f32"))
        for rid in rec.get("end", []):
            rid = str(rid)
            if rid not in slots:
                raise KeyError(f"step {step}: request '{rid}' ends but never started")
            engine.end_sequence(slots.pop(rid))
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
