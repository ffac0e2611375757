"""The entry point, in the manner of gophonic's root package (gophonic.go:28-237):

    model = Open(path, Options(Format="bf16"))
    gen = Lane(model, "tokens.Generator")
    replies = gen.Generate([[1, 2, 3]], ChatOptions(MaxTokens=16))
    model.Close()

``Open`` loads the model at ``path`` with the first registered format that matches it; formats
registered later are tried first, so a registered format can take over paths a built-in one
matches (gophonic.go:176-186).  What a model can do is the set of lanes it provides; ``Lane``
opens one and ``Supports`` reports whether it can (gophonic.go:89-124).  The built-in format
matches a folder whose config.json names a registered architecture (qwen3/model.go:110-129 reads
``model_type`` the same way) and provides two lanes: "tokens.Generator", batched generation over
token ids, and "chat.Generator", conversations whose context stays evaluated between replies
(``gophonic_b200.chat``; text where the folder has a tokenizer.json, token ids otherwise).
"""
from __future__ import annotations

import json
import os
import threading
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

from . import registry
from .sampling.options import Options as ChatOptions

FormatBF16 = "bf16"   # bfloat16 weights and activations on the tensor cores, fp32 residual and statistics
FormatF32 = "f32"     # everything in true 32-bit, no reduced-precision matrix mode

TokensGenerator = "tokens.Generator"
ChatGeneratorLane = "chat.Generator"


class ErrUnknownFormat(ValueError):
    pass


class ErrUnsupported(ValueError):
    pass


@dataclass
class Options:
    """Configures Open.  The zero value picks each model's defaults (gophonic.go:28-39)."""
    # Threads is accepted for compatibility with gophonic.Options and must not be negative; the
    # engine runs on the GPU and uses no CPU workers.
    Threads: int = 0
    # Format names the weight format: FormatBF16 (default) or FormatF32.
    Format: str = ""
    # Device is the CUDA device the model lives on.
    Device: str = "cuda:0"
    # CacheTokens sizes the key/value cache (tokens held by live sequences at once, each rounded
    # up to 64); Batch bounds how many sequences start together.
    CacheTokens: int = 0
    Batch: int = 8


@dataclass
class Format:
    """One kind of model that Open recognizes (gophonic.go:155-172)."""
    Name: str
    Match: Callable[[str], bool]
    Open: Callable[[str, Options], "OpenedModel"]
    Provides: Sequence[str] = ()


class OpenedModel:
    """A loaded model; its weights are shared by every lane opened from it (gophonic.go:66-84)."""

    def __init__(self, name: str, path: str, close: Optional[Callable[[], None]] = None):
        self._name, self._path = name, path
        self._lanes: Dict[str, Callable[[], object]] = {}
        self._close = close

    def Name(self) -> str:
        return self._name

    def Path(self) -> str:
        return self._path

    def Provides(self) -> List[str]:
        return list(self._lanes)

    def Close(self) -> None:
        c, self._close, self._lanes = self._close, None, {}
        if c is not None:
            c()


def Provide(m: OpenedModel, lane: str, open_fn: Callable[[], object]) -> OpenedModel:
    m._lanes[lane] = open_fn
    return m


def Lane(m: OpenedModel, lane: str):
    if lane not in m._lanes:
        raise ErrUnsupported(f"gophonic_b200: {m.Name()} does not provide {lane}")
    return m._lanes[lane]()


def Supports(m: OpenedModel, lane: str) -> bool:
    return lane in m._lanes


_lock = threading.RLock()
_formats: List[Format] = []


def Register(f: Format) -> None:
    if f.Match is None or f.Open is None:
        raise ValueError("gophonic_b200: Register of a format without Match or Open")
    with _lock:
        _formats.insert(0, f)


def Formats() -> List[Format]:
    with _lock:
        return list(_formats)


def Detect(path: str) -> Optional[Format]:
    for f in Formats():
        if f.Match(path):
            return f
    return None


def Open(path: str, opts: Optional[Options] = None) -> OpenedModel:
    opts = opts or Options()
    if opts.Threads < 0:
        raise ValueError(f"gophonic_b200: invalid thread count {opts.Threads}")
    if opts.Format not in ("", FormatBF16, FormatF32):
        raise ErrUnsupported(f"gophonic_b200: unknown weight format '{opts.Format}'")
    f = Detect(path)
    if f is None:
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        raise ErrUnknownFormat(f"gophonic_b200: unrecognized model format: {path}")
    m = f.Open(path, opts)
    for lane in f.Provides:
        if not Supports(m, lane):
            m.Close()
            raise ErrUnsupported(f"gophonic_b200: format {f.Name} declares {lane}, but its model does not provide it")
    return m


# ---- the built-in format -------------------------------------------------------------------
def _is_model_dir(path: str) -> bool:
    try:
        with open(os.path.join(path, "config.json")) as fh:
            registry.architecture_of(json.load(fh))
        return True
    except (OSError, ValueError, KeyError):
        return False


def read_stop_ids(path: str) -> List[int]:
    """The end-of-sequence token ids a model folder names in ``generation_config.json`` (one id or a
    list), else in ``config.json``; none if neither says.  qwen3/chat.go:88-92 takes its stop tokens
    from the tokenizer's added tokens; this library works on ids and reads the ids the folder gives."""
    for name in ("generation_config.json", "config.json"):
        try:
            with open(os.path.join(path, name)) as fh:
                eos = json.load(fh).get("eos_token_id")
        except (OSError, ValueError):
            continue
        if isinstance(eos, bool) or eos is None:
            continue
        if isinstance(eos, int):
            return [eos]
        if isinstance(eos, list) and all(isinstance(t, int) and not isinstance(t, bool) for t in eos):
            return list(eos)
    return []


class TokenGenerator:
    """Lane "tokens.Generator": replies to prompts given as token ids."""

    def __init__(self, model, opts: Options, stop_ids: Sequence[int] = ()):
        self.stop_ids = list(stop_ids)  # the folder's own end-of-sequence ids: the default of Generate
        from .engine.generate import Generator
        from .engine.step import Engine
        from .sampling.sampler import DeviceSampler
        self.model = model
        cfg = model.config
        context = int(getattr(cfg, "max_position_embeddings", model.spec.max_positions))
        tokens = opts.CacheTokens or min(context, 4096) * opts.Batch
        self.engine = Engine(model, max_tokens=tokens, max_seq_tokens=min(context, tokens))
        self.sampler = DeviceSampler(model.spec.vocab, opts.Batch, model.rt.device)
        self.context = min(context, self.engine.capacity)
        self.batch = opts.Batch

    def Generate(self, prompts: Sequence[Sequence[int]], options=None, stop_ids: Optional[Sequence[int]] = None,
                 on_token=None) -> List[List[int]]:
        """Replies to ``prompts`` (lists of token ids), in order.  ``stop_ids``: the token ids that
        end a reply (not part of it); None takes the ids the model folder names, () none at all."""
        from .engine.generate import Generator
        g = Generator(self.engine, self.sampler, self.batch, self.context, self.stop_ids if stop_ids is None else stop_ids)
        out = g.generate(prompts, options, on_token)
        self.engine.check_kernels()
        self.stats = g.stats
        return out

    def Close(self) -> None:
        self.engine = None


def _open_chat(model, opts: Options, path: str):
    """Lane "chat.Generator" over a model: sessions that keep their context evaluated."""
    from .chat import ChatGenerator, Template
    from .engine.step import Engine
    from .sampling.sampler import DeviceSampler
    from .tokenizer import load_tokenizer
    cfg = model.config
    context = int(getattr(cfg, "max_position_embeddings", model.spec.max_positions))
    tokens = opts.CacheTokens or min(context, 4096) * opts.Batch
    engine = Engine(model, max_tokens=tokens, max_seq_tokens=min(context, tokens))
    sampler = DeviceSampler(model.spec.vocab, 1, model.rt.device)
    tokenizer = load_tokenizer(path)
    if tokenizer is not None and tokenizer.added_id("<|im_end|>") is not None:
        template = Template.qwen3(tokenizer, thinking_block=tokenizer.template_thinks)
    else:
        template = Template(stop=read_stop_ids(path))
    return ChatGenerator(engine, sampler, min(context, engine.capacity), template, tokenizer)


def _open_dir(path: str, opts: Options) -> OpenedModel:
    from .engine.model import Model
    mode = "float32" if opts.Format == FormatF32 else "bfloat16"
    model = Model.from_dir(path, dtype=mode, device=opts.Device)
    m = OpenedModel(model.spec.architecture, path)
    m.model = model
    Provide(m, TokensGenerator, lambda: TokenGenerator(model, opts, read_stop_ids(path)))
    return Provide(m, ChatGeneratorLane, lambda: _open_chat(model, opts, path))


Register(Format(Name="model-folder", Match=_is_model_dir, Open=_open_dir, Provides=(TokensGenerator, ChatGeneratorLane)))


# ---- random weights by name ---------------------------------------------------------------------
RANDOM_PREFIX = "random:"


def random_model_path(name: str, seed: int = 0, layers: int = 0) -> str:
    """The path that opens the named configuration with seeded random weights made on the device:
    ``random:NAME?seed=S&layers=L`` (``layers`` > 0 keeps that many of the configuration's layers;
    every layer keeps its size)."""
    q = [f"seed={int(seed)}"] + ([f"layers={int(layers)}"] if layers else [])
    return f"{RANDOM_PREFIX}{name}?{'&'.join(q)}"


def _parse_random(path: str):
    from .config.presets import preset
    body = path[len(RANDOM_PREFIX):]
    name, _, query = body.partition("?")
    args = {"seed": 0, "layers": 0}
    for item in filter(None, query.split("&")):
        k, _, v = item.partition("=")
        if k not in args:
            raise ValueError(f"gophonic_b200: unknown option '{k}' in {path} (seed, layers)")
        try:
            args[k] = int(v)
        except ValueError:
            raise ValueError(f"gophonic_b200: '{k}={v}' in {path} is not an integer") from None
    try:
        raw = preset(name)
    except KeyError as e:
        raise ErrUnknownFormat(f"gophonic_b200: {e.args[0]}") from None
    if args["layers"] < 0 or args["layers"] > raw["num_hidden_layers"]:
        raise ValueError(f"gophonic_b200: layers={args['layers']} of a configuration with {raw['num_hidden_layers']}")
    if args["layers"]:
        raw = dict(raw, num_hidden_layers=args["layers"])
    return registry.config_class(registry.architecture_of(raw)).from_dict(raw), args["seed"]


def _open_random(path: str, opts: Options) -> OpenedModel:
    from .engine.model import Model
    config, seed = _parse_random(path)
    mode = "float32" if opts.Format == FormatF32 else "bfloat16"
    model = Model.from_random(config, seed=seed, dtype=mode, device=opts.Device)
    m = OpenedModel(model.spec.architecture, path)
    m.model = model
    Provide(m, TokensGenerator, lambda: TokenGenerator(model, opts, ()))
    return Provide(m, ChatGeneratorLane, lambda: _open_chat(model, opts, path))


Register(Format(Name="random-weights", Match=lambda path: path.startswith(RANDOM_PREFIX), Open=_open_random,
                Provides=(TokensGenerator, ChatGeneratorLane)))
