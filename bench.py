#!/usr/bin/env python3
"""Decode and prefill throughput of the Qwen3-8B-shaped model with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

Prints one JSON line.  ``value`` is decoded tokens per second at batch 8 with every sequence's
context filling to 4096, timed on the device over exactly K decode steps (one token per sequence
a step, token selection included).  ``e2e`` is the same loop driven as a user drives it, host
token ids in and host token ids out every step.  ``prefill`` is one prompt of 2,048 tokens,
``points`` are decode at batch 1 and 64, ``roofline`` divides the bytes a decode step has to
read (every weight once, the live sequences' keys and values) by its time.
"""
import argparse
import dataclasses
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONTEXT = 4096
PREFILL_TOKENS = 2048

# layer sizes by name, from the library's own configuration files: the default is the configuration
# the headline metric is quoted on; the others are further points, never the default
MODELS = ("8b", "1.7b", "32b")


def sizes(name):
    from gophonic_b200.config.presets import preset
    c = preset(name)
    return dict(layers=c["num_hidden_layers"], hidden=c["hidden_size"], heads=c["num_attention_heads"],
                kv_heads=c["num_key_value_heads"], head_dim=c["head_dim"], intermediate=c["intermediate_size"],
                vocab=c["vocab_size"], tied=bool(c["tie_word_embeddings"]))


def config_of(name, layers, context):
    """The named configuration with ``layers`` layers (0: all of them) and room for ``context`` positions."""
    from gophonic_b200 import registry
    from gophonic_b200.config.presets import preset
    raw = dict(preset(name))
    if layers:
        raw["num_hidden_layers"] = layers
    raw["max_position_embeddings"] = max(int(raw["max_position_embeddings"]), context)
    return registry.config_class(registry.architecture_of(raw)).from_dict(raw)


def peaks():
    """(hbm GB/s, bf16 TFLOP/s burst, which) from MEASURED_PEAKS.json, else the stated fallback."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
    except (OSError, ValueError, KeyError):
        return 6650.0, 1590.0, "fallback"


class ClockSampler:
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.file.read().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        self.file.close()
        os.unlink(self.file.name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def decode_setup(engine, batch, start_len, torch):
    """``batch`` live sequences whose caches hold ``start_len`` tokens of synthetic keys and values."""
    slots = [engine.new_sequence() for _ in range(batch)]
    grow = [(s, start_len) for s in slots]
    engine.cache.reserve(grow)
    engine.cache.commit(grow)
    return slots


def fill_cache_random(engine, torch):
    g = torch.Generator(device=engine.device)
    g.manual_seed(1)
    for planes in list(engine.cache._k.values()) + list(engine.cache._v.values()):
        for i in range(planes.shape[0]):  # plane by plane keeps the temporary small
            planes[i].normal_(0.0, 1.0, generator=g)


def time_decode(engine, sampler, batch, steps, warmup, torch, ops):
    """Device time of a decode step (CUDA events around ``steps`` steps), kernel launches per step and the live cache tokens."""
    import numpy as np
    start_len = engine.capacity - (steps + warmup) - 1
    slots = decode_setup(engine, batch, start_len, torch)
    rng = np.random.default_rng(0)
    tokens = rng.integers(0, engine.vocab, size=batch).tolist()
    rows = list(range(batch))
    from gophonic_b200.sampling import Options
    for r in rows:
        sampler.start(r, Options(), r)
    out = {}
    try:
        for _ in range(warmup):
            logits = engine.step([(s, [t]) for s, t in zip(slots, tokens)], borrow=True)
            tokens = sampler.select(logits, rows)
        torch.cuda.synchronize()
        l0 = ops.launches
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(steps):
            logits = engine.step([(s, [t]) for s, t in zip(slots, tokens)], borrow=True)
            sampler.select_device(logits, rows)
        ev1.record()
        torch.cuda.synchronize()
        out["ms"] = ev0.elapsed_time(ev1) / steps
        out["launches"] = (ops.launches - l0) / steps
        out["kv_tokens"] = sum(engine.length(s) for s in slots)
    finally:
        for s in slots:
            engine.end_sequence(s)
    return out


def time_entry_point(model, batch, steps, warmup, context, torch):
    """Decode throughput through the public entry point: ``TokenGenerator.Generate`` with prompts
    given as host lists of token ids and replies read back as host integers.  The prompts fill the
    context up to the decoded tokens, are prefilled by the generator itself (not timed), and the
    clock runs over ``steps`` decode steps between two token callbacks."""
    import numpy as np
    import gophonic_b200 as gp
    from gophonic_b200.api import TokenGenerator
    gen = TokenGenerator(model, gp.Options(Format=gp.FormatBF16, CacheTokens=batch * context, Batch=batch))
    rng = np.random.default_rng(0)
    extra = 2  # tokens after the timed window, so that the window lies wholly in the loop's steady state
    prompt_len = context - (steps + warmup + extra) - 1
    prompts = [rng.integers(0, model.spec.vocab, size=prompt_len).tolist() for _ in range(batch)]
    marks = {}
    seen = [0]

    def on_token(i, token):
        if i != 0:
            return
        seen[0] += 1
        if seen[0] == warmup + 1:          # produced by the prompt step and warmup decode steps
            marks["t0"] = time.perf_counter()
            marks["up0"] = gen.engine.stager.bytes_uploaded
        elif seen[0] == warmup + 1 + steps:
            marks["t1"] = time.perf_counter()
            marks["up1"] = gen.engine.stager.bytes_uploaded

    replies = gen.Generate(prompts, gp.ChatOptions(MaxTokens=warmup + 1 + steps + extra, Temperature=0.0), on_token=on_token)
    assert all(len(r) == warmup + 1 + steps + extra for r in replies)
    out = {"ms": (marks["t1"] - marks["t0"]) * 1e3 / steps, "h2d": (marks["up1"] - marks["up0"]) // steps, "d2h": 4 * batch}
    gen.Close()
    del gen
    torch.cuda.empty_cache()
    return out


def run_mixed_batch(model, torch, requests=16, shortest=64, longest=2048, new_tokens=256):
    """A batch of prompts of unequal lengths (seeded, uniform in [shortest, longest]) that start
    together and then decode ``new_tokens`` tokens each, through the public entry point with host
    token ids in and out; wall clock, once untimed and once timed."""
    import numpy as np
    import gophonic_b200 as gp
    from gophonic_b200.api import TokenGenerator
    gen = TokenGenerator(model, gp.Options(Format=gp.FormatBF16, CacheTokens=requests * (longest + new_tokens), Batch=requests))
    rng = np.random.default_rng(0)
    lengths = rng.integers(shortest, longest + 1, size=requests).tolist()
    prompts = [rng.integers(0, model.spec.vocab, size=n).tolist() for n in lengths]
    out = {}
    for timed in (False, True):
        marks = {}

        def on_token(i, token):
            if "first" not in marks:
                marks["first"] = time.perf_counter()

        torch.cuda.synchronize()
        t0 = time.perf_counter()
        replies = gen.Generate(prompts, gp.ChatOptions(MaxTokens=new_tokens, Temperature=0.0), on_token=on_token)
        t1 = time.perf_counter()
        assert all(len(r) == new_tokens for r in replies)
        if timed:
            out = {"workload": f"{requests} prompts of {shortest}..{longest} tokens that start together, then {new_tokens} tokens each",
                   "prompt_tokens": int(sum(lengths)), "prefill_ms": round((marks["first"] - t0) * 1e3, 2),
                   "prefill_tok_s": round(sum(lengths) / (marks["first"] - t0), 1),
                   "decode_steps": new_tokens - 1, "decode_ms_per_step": round((t1 - marks["first"]) * 1e3 / (new_tokens - 1), 4),
                   "decode_tok_s": round(requests * (new_tokens - 1) / (t1 - marks["first"]), 1),
                   "total_s": round(t1 - t0, 4)}
    gen.Close()
    return out


def time_prefill(engine, tokens, iters, warmup, torch):
    import numpy as np
    rng = np.random.default_rng(1)
    prompt = rng.integers(0, engine.vocab, size=tokens).tolist()
    times = []
    for i in range(warmup + iters):
        slot = engine.new_sequence()
        torch.cuda.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        engine.step([(slot, prompt)])
        ev1.record()
        torch.cuda.synchronize()
        engine.end_sequence(slot)
        if i >= warmup:
            times.append(ev0.elapsed_time(ev1))
    return statistics.median(times)


def further_model_points(name, steps, torch, ops, hbm_peak, tflops_peak):
    """Decode and prefill points of another named configuration (all its layers, random weights): 1.7B
    at batch 1 and 8 to context 4096, 32B at batch 1 and 32 to context 8192, each with its prefill of
    2,048 tokens; tokens a second and the fraction of the roofline, keyed by the model's name."""
    from gophonic_b200.engine import Engine, Model
    from gophonic_b200.sampling import DeviceSampler
    context, batches = (8192, (1, 32)) if name == "32b" else (4096, (1, 8))
    cfg = config_of(name, 0, context)
    model = Model.from_random(cfg, seed=0, dtype="bfloat16", device="cuda:0")
    engine = Engine(model, max_tokens=max(batches) * context, max_slots=max(batches), max_seq_tokens=context)
    fill_cache_random(engine, torch)
    sampler = DeviceSampler(cfg.vocab_size, max(batches), engine.device)
    weight_bytes, kv_bytes = model.weight_bytes_per_step(), engine.cache.bytes_per_token()
    out = {}
    for b in batches:
        d = time_decode(engine, sampler, b, steps, 16, torch, ops)
        out[f"{name}_decode_b{b}"] = round(b / (d["ms"] * 1e-3), 1)
        out[f"{name}_decode_b{b}_hbm_frac"] = round((weight_bytes + kv_bytes * d["kv_tokens"]) / (d["ms"] * 1e-3) / 1e9 / hbm_peak, 4)
    ms = time_prefill(engine, PREFILL_TOKENS, iters=3, warmup=2, torch=torch)
    T = PREFILL_TOKENS
    head_elems = cfg.vocab_size * cfg.hidden_size
    head_bytes = head_elems * 2
    params = (weight_bytes - head_bytes) // 2
    flops = 2.0 * T * params + 2.0 * cfg.num_attention_heads * cfg.head_dim * T * T * cfg.num_hidden_layers + 2.0 * head_elems
    out[f"{name}_prefill_tok_s"] = round(T / (ms * 1e-3), 1)
    out[f"{name}_prefill_frac"] = round(flops / (ms * 1e-3) / (tflops_peak * 1e12), 4)
    del engine, sampler, model
    torch.cuda.empty_cache()
    return out


def probe(name, **opts):
    """Run one kernel of the step a few times on a small, fixed workload (operands larger than L2
    where the kernel is bound by memory), for profilers.  Prints the kernel's own timing."""
    import torch
    from gophonic_b200 import ops
    dev = "cuda:0"
    bf = torch.bfloat16
    g = torch.Generator(device=dev)
    g.manual_seed(0)

    def rnd(*shape, scale=1.0):
        return (torch.randn(*shape, device=dev, generator=g) * scale).to(bf)

    if name in ("gemm_prefill", "gemm_prefill_swiglu"):
        M, N, K = 2048, 24576, 4096       # gate/up of one layer: 201 MB of weights
        a, w = rnd(M, K), rnd(N, K, scale=0.05)
        out = torch.empty((M, N // 2 if name.endswith("swiglu") else N), dtype=bf, device=dev)
        fn = (lambda: ops.gemm_swiglu(a, w, out)) if name.endswith("swiglu") else (lambda: ops.gemm(a, w, out))
        work = 2.0 * M * N * K
        unit = "TFLOP/s"
    elif name in ("gemm_decode_b8", "gemm_decode_b64", "gemm_down_b128", "gemm_o_b8"):
        M = 8 if name.endswith("b8") else 64
        N, K = 24576, 4096
        if name == "gemm_down_b128":   # the down projection of a step of 128 rows: K slices in clusters
            M, N, K = 128, 4096, 12288
        if name == "gemm_o_b8":        # the narrowest product of a decode step
            N, K = 4096, 4096
        ws = [rnd(N, K, scale=0.05) for _ in range(max(3, int(6e8 / (2.0 * N * K))))]   # rotate 600 MB of weights through L2
        a = rnd(M, K)
        out = torch.empty((M, N), dtype=bf, device=dev)
        state = {"i": 0}

        def fn():
            ops.gemm(a, ws[state["i"] % len(ws)], out)
            state["i"] += 1
        work = N * K * 2.0
        unit = "GB/s"
    elif name in ("gemm_scaled_b8", "gemm_residual_b8", "gemm_scaled_b64", "gemm_residual_b64"):
        # the two products of a decode step that carry the residual's row-wise work: gate/up with the
        # rows' norm factors and SwiGLU in its epilogue, and the down projection that adds into the
        # residual and leaves the row statistics and the next norm's rows (8 rows: the fragment-streaming
        # kernel; 64 rows: the tcgen05 decode kernel)
        M = 8 if name.endswith("b8") else 64
        N, K = (24576, 4096) if name.startswith("gemm_scaled") else (4096, 12288)
        ws = [rnd(N, K, scale=0.05) for _ in range(max(3, int(6e8 / (2.0 * N * K))))]
        x = rnd(M, K)
        stats = torch.ones((M, max(K, N) // 16), device=dev)
        state = {"i": 0}
        if name.startswith("gemm_scaled"):
            out = torch.empty((M, N // 2), dtype=bf, device=dev)

            def fn():
                ops.gemm_scaled(x, 1e-6, stats, K // (16 if M <= 8 else 128), ws[state["i"] % len(ws)], out, swiglu=True)
                state["i"] += 1
        else:
            h = torch.zeros((M, N), device=dev)
            nw, nxt = torch.ones(N, device=dev), torch.empty((M, N), dtype=bf, device=dev)

            def fn():
                ops.gemm_residual(x, ws[state["i"] % len(ws)], h, stats, nw, nxt)
                state["i"] += 1
        work = N * K * 2.0
        unit = "GB/s"
    elif name in ("attn_decode_b8", "attn_decode_b64", "attn_decode_rope_b8", "attn_prefill"):
        heads, kvh, d = 32, 8, 128
        if name == "attn_prefill":
            nseq, q_len, kv_len = 1, 2048, 2048
        else:
            nseq, q_len, kv_len = (8 if name.endswith("b8") else 64), 1, 4096
        pages_per = (kv_len + 63) // 64
        n_pages = nseq * pages_per
        k = rnd(n_pages, kvh, 64, d)
        v = rnd(n_pages, kvh, 64, d)
        table = torch.arange(n_pages, dtype=torch.int32, device=dev).reshape(nseq, pages_per)
        q = rnd(nseq * q_len, heads * d)
        out = torch.empty_like(q)
        ints = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
        slot, start = ints(list(range(nseq))), ints([i * q_len for i in range(nseq)])
        ql, kl = ints([q_len] * nseq), ints([kv_len] * nseq)
        from gophonic_b200.parts.attention import choose_splits
        splits = 1 if q_len > 1 else choose_splits(nseq * kvh, kv_len)
        scratch = torch.empty(ops.attention_scratch_floats(nseq, heads, d, splits), dtype=torch.float32, device=dev) if splits > 1 else None

        def fn():
            ops.attention(q, out, k, v, table, slot, start, ql, kl, nseq, q_len, heads, kvh, d, d ** -0.5, 0, splits, scratch)
        if name == "attn_decode_rope_b8":
            # as a decode step calls it: rows as the q/k/v product left them; the kernel norms and rotates
            # its queries, takes the token's key and value from the row and stores them in the cache
            qkv = rnd(nseq, (heads + 2 * kvh) * d)
            out = torch.empty((nseq, heads * d), dtype=bf, device=dev)
            w = torch.ones(d, device=dev)
            angles = torch.rand(kv_len, d // 2, device=dev)
            cos, sin = torch.cos(angles), torch.sin(angles)
            rope_args = (heads, kvh, d, w, w, 1e-6, cos, sin, d, ints([kv_len - 1] * nseq), slot, slot, table, k, v, True)
            attn_args = (k, v, table, slot, start, ql, kl, nseq, 1, heads, kvh, d, d ** -0.5, 0, splits, scratch)

            def fn():
                ops.attention_decode_rope(qkv, out, rope_args, attn_args)
        if q_len == 1:
            work, unit = 2.0 * n_pages * kvh * 64 * d * 2, "GB/s"
        else:
            work, unit = 2.0 * heads * d * q_len * q_len, "TFLOP/s"
    elif name in ("prefill_step", "decode_step"):
        # a whole engine step of a 4-layer model with the layer sizes of the benchmark (or of --model):
        # the launch list of a profiler then shows every kernel of a layer with its share.  --batch
        # and --context set the decode step's sequences and their length, --prompt-tokens the prompt.
        from gophonic_b200.engine import Engine, Model
        batch, context, tokens = opts.get("batch", 8), opts.get("context", CONTEXT), opts.get("prompt_tokens", PREFILL_TOKENS)
        cfg = config_of(opts.get("model", "8b"), 4, context)
        model = Model.from_random(cfg, seed=0, dtype="bfloat16", device=dev)
        engine = Engine(model, max_tokens=batch * context, max_slots=batch, max_seq_tokens=context)
        prompt = torch.randint(0, cfg.vocab_size, (tokens,), generator=torch.Generator().manual_seed(1)).tolist()
        if name == "prefill_step":
            def fn():
                slot = engine.new_sequence()
                engine.step([(slot, prompt)])
                engine.end_sequence(slot)
            work, unit = float(tokens), "tok/s"
        else:
            fill_cache_random(engine, torch)
            slots = decode_setup(engine, batch, context - 64, torch)

            def fn():
                engine.step([(s, [1]) for s in slots])
            work, unit = float(batch), "tok/s"
    else:
        raise SystemExit(f"unknown probe '{name}'")
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(3):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / 3
    rate = work / (ms * 1e-3) / {"TFLOP/s": 1e12, "GB/s": 1e9}.get(unit, 1.0)
    hbm_peak, tflops_peak, which = peaks()
    line = {"probe": name, "ms": round(ms, 4), "rate": round(rate, 1), "unit": unit, "status": ops.tc5_status()}
    if unit == "TFLOP/s":
        line.update(frac=round(rate / tflops_peak, 4), of=f"{tflops_peak:.0f} TFLOP/s bf16 ({which})")
    elif unit == "GB/s":
        line.update(frac=round(rate / hbm_peak, 4), of=f"{hbm_peak:.0f} GB/s HBM ({which})")
    print(json.dumps(line), flush=True)
    return 0


KERNEL_PROBES = ("gemm_prefill", "gemm_prefill_swiglu", "attn_prefill", "gemm_decode_b8", "gemm_scaled_b8", "gemm_residual_b8",
                 "gemm_decode_b64", "gemm_scaled_b64", "gemm_residual_b64", "gemm_down_b128", "attn_decode_b8", "attn_decode_rope_b8",
                 "attn_decode_b64")


def profile():
    """One line per hot kernel: its time on a workload of the benchmark's sizes, the bytes or flops it
    has to move, and the fraction of the roofline that is."""
    for name in KERNEL_PROBES:
        probe(name)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="run fewer layers than the configuration has (reported)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--no-points", action="store_true", help="skip batch 1 / 64 and prefill")
    ap.add_argument("--points", default="1,64", help="batch sizes of the further decode points (default 1,64)")
    ap.add_argument("--model", default="8b", choices=sorted(MODELS), help="layer sizes (default: the benchmark's own, 8b)")
    ap.add_argument("--extra-models", default="1.7b,32b",
                    help="further sizes whose decode and prefill points go into \"points\" (default 1.7b,32b; '' for none)")
    ap.add_argument("--context", type=int, default=CONTEXT, help="context length each sequence is filled to")
    ap.add_argument("--mixed", action="store_true",
                    help="instead of the headline run: 16 prompts of 64 to 2048 tokens that start together, then 256 tokens each, "
                         "through the entry point (a further point, with --model)")
    ap.add_argument("--profile", action="store_true", help="time each hot kernel alone and print its fraction of the roofline")
    ap.add_argument("--probe", default="", help="run one kernel on a small fixed workload (for profilers) and exit")
    ap.add_argument("--prompt-tokens", type=int, default=PREFILL_TOKENS, help="prompt length of --probe prefill_step")
    args = ap.parse_args()
    if args.probe:
        return probe(args.probe, model=args.model, batch=args.batch, context=args.context, prompt_tokens=args.prompt_tokens)
    if args.profile:
        return profile()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "GetStream/gophonic is a Go module (no setup.py/pyproject; pip "
                          "refuses it), there is no Go toolchain here, and its GPU paths are Metal/WebGPU only"}))
        return 0
    if args.gpus != 1:
        print(json.dumps({"error": f"this library runs on one GPU; --gpus {args.gpus} is not supported", "n_gpus": args.gpus}))
        return 2
    warmup = max(3, args.warmup)

    import torch
    from gophonic_b200 import ops
    from gophonic_b200.engine import Engine, Model
    from gophonic_b200.sampling import DeviceSampler

    sz = sizes(args.model)
    context = args.context
    full_layers = sz["layers"]
    layers = args.layers or full_layers
    cfg = config_of(args.model, args.layers, context)
    hbm_peak, tflops_peak, which = peaks()
    model = Model.from_random(cfg, seed=0, dtype="bfloat16", device="cuda:0")
    if args.mixed:
        line = run_mixed_batch(model, torch)
        line.update({"model": f"Qwen3-{args.model.upper()}-shaped", "layers": layers, "layers_full": full_layers, "dtype": "bf16",
                     "data": "synthetic: seeded random weights and token ids", "timing": "wall clock around the entry point's call"})
        print(json.dumps(line))
        return 0
    point_batches = [] if args.no_points else [int(b) for b in args.points.split(",") if b]
    max_batch = max([args.batch] + point_batches)
    engine = Engine(model, max_tokens=max_batch * context, max_slots=max_batch, max_seq_tokens=context)
    fill_cache_random(engine, torch)
    sampler = DeviceSampler(cfg.vocab_size, max_batch, engine.device)
    weight_bytes = model.weight_bytes_per_step()
    kv_bytes_per_token = engine.cache.bytes_per_token()

    clocks_all = ClockSampler()      # over everything that is timed; ``clocks`` is the headline loop alone
    clocks_all.start()
    clocks = ClockSampler()
    clocks.start()
    dev = time_decode(engine, sampler, args.batch, args.steps, warmup, torch, ops)
    clock_info = clocks.stop()
    prefill_ms, point_runs = None, {}
    if not args.no_points:
        prefill_ms = time_prefill(engine, PREFILL_TOKENS, iters=3, warmup=3, torch=torch)
        for b in point_batches:
            # after the prompt steps the GPU runs some milliseconds at the clocks of a compute-bound
            # phase: more untimed steps than the headline run needs
            point_runs[b] = time_decode(engine, sampler, b, args.steps, 16, torch, ops)
    # the entry point makes an engine and a cache of its own: give this one's memory back first
    del engine, sampler
    torch.cuda.empty_cache()
    # the generator prefills its own long prompts first (see above): 16 untimed steps here too
    e2e = time_entry_point(model, args.batch, args.steps, max(warmup, 16), context, torch)

    extra_points = {}
    if not args.no_points and args.model == "8b" and not args.layers and args.context == CONTEXT:
        # a further context length: the same model, eight sequences of 32768 tokens (39 GB of keys and values)
        long_context = 32768
        engine = Engine(model, max_tokens=args.batch * long_context, max_slots=args.batch, max_seq_tokens=long_context)
        fill_cache_random(engine, torch)
        sampler = DeviceSampler(cfg.vocab_size, args.batch, engine.device)
        run = time_decode(engine, sampler, args.batch, args.steps, 16, torch, ops)
        long_bytes = weight_bytes + kv_bytes_per_token * run["kv_tokens"]
        extra_points[f"decode_b{args.batch}_ctx{long_context}"] = round(args.batch / (run["ms"] * 1e-3), 1)
        extra_points[f"decode_b{args.batch}_ctx{long_context}_hbm_frac"] = round(long_bytes / (run["ms"] * 1e-3) / 1e9 / hbm_peak, 4)
        del engine, sampler
    if not args.no_points and args.model == "8b" and not args.layers:
        del model
        torch.cuda.empty_cache()
        for name in [m for m in args.extra_models.split(",") if m]:
            extra_points.update(further_model_points(name, args.steps, torch, ops, hbm_peak, tflops_peak))
    clock_all_info = clocks_all.stop()

    step_bytes = weight_bytes + kv_bytes_per_token * dev["kv_tokens"]
    achieved = step_bytes / (dev["ms"] * 1e-3) / 1e9
    value = args.batch / (dev["ms"] * 1e-3)
    line = {
        "metric": f"Qwen3-{args.model.upper()} decode tok/s @ batch {args.batch}, context {context} (random weights, bf16)",
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(dev["ms"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random weights, random token ids, cache pre-filled with random keys/values",
        "impl": "ours",
        "config": {"model": f"Qwen3-{args.model.upper()}-shaped", "layers": layers, "layers_full": full_layers, "hidden": sz["hidden"],
                   "heads": sz["heads"], "kv_heads": sz["kv_heads"], "head_dim": sz["head_dim"], "intermediate": sz["intermediate"],
                   "vocab": sz["vocab"], "tied_head": sz["tied"], "global_batch": args.batch, "seq_len": context,
                   "parallelism": "single-gpu", "l2": f"step reads {weight_bytes / 1e9:.1f} GB of weights, larger than L2",
                   "peaks": which},
        "e2e": {"value": round(args.batch / (e2e["ms"] * 1e-3), 1), "unit": "tok/s",
                "h2d_bytes_per_step": int(e2e["h2d"]), "d2h_bytes_per_step": int(e2e["d2h"])},
        "gpu_launches": int(round(dev["launches"] * args.steps)),
        "clocks": clock_info,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_peak, "unit": "GB/s",
                     "frac": round(achieved / hbm_peak, 4)},
    }
    line["clocks_all"] = clock_all_info
    if not args.no_points:
        ms = prefill_ms
        T = PREFILL_TOKENS
        head_elems = cfg.vocab_size * cfg.hidden_size
        params = (weight_bytes - head_elems * 2) // 2
        flops = 2.0 * T * params + 2.0 * cfg.num_attention_heads * cfg.head_dim * T * T * layers + 2.0 * head_elems
        line["prefill"] = {"value": round(T / (ms * 1e-3), 1), "tokens": T, "ms": round(ms, 3),
                           "frac": round(flops / (ms * 1e-3) / (tflops_peak * 1e12), 4)}
        points = {}
        for b, d in point_runs.items():
            points[f"decode_b{b}"] = round(b / (d["ms"] * 1e-3), 1)
            bytes_b = weight_bytes + kv_bytes_per_token * d["kv_tokens"]
            points[f"decode_b{b}_hbm_frac"] = round(bytes_b / (d["ms"] * 1e-3) / 1e9 / hbm_peak, 4)
        points.update(extra_points)
        line["points"] = points
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
