"""Typed configuration of the Qwen3 dense decoder, read from the keys of its ``config.json``.

Keys, defaults and the rejected variants follow ``TextConfig`` and ``TextConfig.model()``
(internal/qwen3lm/weights.go:161-176, 644-698): geometry keys are required and positive,
``head_dim`` falls back to hidden/heads when absent, heads must be a multiple of kv heads, the
head width must be even, eps and theta must be positive, and scaled RoPE, attention bias, a
sliding window or an activation other than SiLU are load errors.  No size stands in code: every
number below comes from the file.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field, asdict
from typing import Any, Dict, Optional

from .spec import (AttentionSpec, EmbeddingSpec, HeadSpec, LayerSpec, ModelSpec, RMSNormSpec,
                   RotarySpec, SwiGLUSpec, default_schedule)


class ConfigError(ValueError):
    """A config.json that this library cannot run; the message names the offending key."""


_LIMIT = 16 << 20  # internal/qwen3lm/weights.go:672-677


def _need_int(d: Dict[str, Any], key: str) -> int:
    if key not in d or d[key] is None:
        raise ConfigError(f"config.json: missing key '{key}'")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"config.json: '{key}' must be an integer, got {v!r}")
    if v <= 0 or v > _LIMIT:
        raise ConfigError(f"config.json: '{key}' = {v} is outside (0, {_LIMIT}]")
    return v


def _need_pos_float(d: Dict[str, Any], key: str) -> float:
    if key not in d or d[key] is None:
        raise ConfigError(f"config.json: missing key '{key}'")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: '{key}' must be a number, got {v!r}")
    v = float(v)
    if not (v > 0) or math.isinf(v):
        raise ConfigError(f"config.json: '{key}' = {v} must be positive and finite")
    return v


@dataclass(frozen=True)
class Qwen3Config:
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool = False
    model_type: str = "qwen3"
    architecture: str = "Qwen3ForCausalLM"
    torch_dtype: str = "bfloat16"

    # ---- reading -------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "Qwen3Config":
        mt = d.get("model_type")
        if mt != "qwen3":
            raise ConfigError(f"config.json: 'model_type' must be \"qwen3\", got {mt!r}")
        if d.get("rope_scaling") is not None:
            raise ConfigError("config.json: 'rope_scaling' is set; scaled RoPE is not supported")
        if d.get("attention_bias"):
            raise ConfigError("config.json: 'attention_bias' is true; biased projections are not supported")
        if d.get("use_sliding_window"):
            raise ConfigError("config.json: 'use_sliding_window' is true; Qwen3 dense runs without a window")
        act = d.get("hidden_act", "")
        if act not in ("", None, "silu"):
            raise ConfigError(f"config.json: 'hidden_act' must be \"silu\", got {act!r}")
        hidden = _need_int(d, "hidden_size")
        layers = _need_int(d, "num_hidden_layers")
        heads = _need_int(d, "num_attention_heads")
        kv_heads = _need_int(d, "num_key_value_heads")
        if d.get("head_dim") in (None, 0):
            if hidden % heads != 0:
                raise ConfigError(f"config.json: no 'head_dim' and 'hidden_size' {hidden} is not a "
                                  f"multiple of 'num_attention_heads' {heads}")
            head_dim = hidden // heads
        else:
            head_dim = _need_int(d, "head_dim")
        inter = _need_int(d, "intermediate_size")
        vocab = _need_int(d, "vocab_size")
        max_pos = _need_int(d, "max_position_embeddings")
        eps = _need_pos_float(d, "rms_norm_eps")
        theta = _need_pos_float(d, "rope_theta")
        if heads % kv_heads != 0:
            raise ConfigError(f"config.json: 'num_attention_heads' {heads} is not a multiple of "
                              f"'num_key_value_heads' {kv_heads}")
        if head_dim % 2 != 0:
            raise ConfigError(f"config.json: 'head_dim' {head_dim} must be even")
        archs = d.get("architectures") or ["Qwen3ForCausalLM"]
        return cls(hidden_size=hidden, num_hidden_layers=layers, num_attention_heads=heads,
                   num_key_value_heads=kv_heads, head_dim=head_dim, intermediate_size=inter,
                   vocab_size=vocab, max_position_embeddings=max_pos, rms_norm_eps=eps,
                   rope_theta=theta, tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
                   architecture=str(archs[0]), torch_dtype=str(d.get("torch_dtype", "bfloat16")))

    @classmethod
    def from_json(cls, path: str) -> "Qwen3Config":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        try:
            with open(path, "r") as f:
                d = json.load(f)
        except OSError as e:
            raise ConfigError(f"cannot read {path}: {e}") from e
        except json.JSONDecodeError as e:
            raise ConfigError(f"cannot parse {path}: {e}") from e
        if not isinstance(d, dict):
            raise ConfigError(f"{path}: not a JSON object")
        return cls.from_dict(d)

    # ---- writing -------------------------------------------------------------------------
    def to_dict(self) -> Dict[str, Any]:
        return {
            "architectures": [self.architecture],
            "model_type": self.model_type,
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": None,
            "attention_bias": False,
            "hidden_act": "silu",
            "use_sliding_window": False,
            "tie_word_embeddings": self.tie_word_embeddings,
            "torch_dtype": self.torch_dtype,
        }

    # ---- derived -------------------------------------------------------------------------
    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def model_spec(self) -> ModelSpec:
        """The decoder as parts: pre-norm blocks of GQA attention (per-head q/k RMSNorm, full-head
        rotate-half RoPE, scale 1/sqrt(head_dim): internal/qwen3lm/weights.go:681-693) and a
        SwiGLU feed-forward, tensor names as the checkpoint has them
        (internal/qwen3lm/weights.go:325-351)."""
        d = self.head_dim
        layers = []
        for i in range(self.num_hidden_layers):
            layers.append(LayerSpec(
                prefix=f"model.layers.{i}.",
                mixer=AttentionSpec(
                    hidden=self.hidden_size, heads=self.num_attention_heads,
                    kv_heads=self.num_key_value_heads, head_dim=d,
                    scale=1.0 / math.sqrt(d),
                    position=RotarySpec(head_dim=d, rotary_dim=d, theta=self.rope_theta),
                    qk_norm=RMSNormSpec(size=d, eps=self.rms_norm_eps), window=0),
                feed_forward=SwiGLUSpec(hidden=self.hidden_size, intermediate=self.intermediate_size),
                mixer_norm=RMSNormSpec(size=self.hidden_size, eps=self.rms_norm_eps),
                feed_forward_norm=RMSNormSpec(size=self.hidden_size, eps=self.rms_norm_eps),
                block="prenorm"))
        spec = ModelSpec(
            architecture=self.architecture, hidden=self.hidden_size, vocab=self.vocab_size,
            max_positions=self.max_position_embeddings,
            embedding=EmbeddingSpec("model.embed_tokens.weight", self.vocab_size, self.hidden_size),
            layers=tuple(layers), schedule=default_schedule(self.num_hidden_layers),
            final_norm=RMSNormSpec(size=self.hidden_size, eps=self.rms_norm_eps),
            final_norm_name="model.norm.weight",
            head=HeadSpec("lm_head.weight", self.vocab_size, self.hidden_size,
                          tied_to="model.embed_tokens.weight"))
        spec.validate()
        return spec
