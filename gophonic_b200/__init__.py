"""gophonic_b200: a small library that runs the Qwen3 dense decoder on one NVIDIA B200.

Importing the package needs no GPU.  The kernel library is compiled and loaded the first time a
model is opened on a CUDA device.
"""
from . import chat, registry
from .api import (ChatGeneratorLane, ChatOptions, Detect, ErrUnknownFormat, ErrUnsupported, Format, FormatBF16, FormatF32, Formats,
                  Lane, Open, OpenedModel, Options, Provide, Register, Supports, TokensGenerator, random_model_path)
from .config import ConfigError, Qwen3Config

__version__ = "0.1.0"

__all__ = ["ChatGeneratorLane", "ChatOptions", "ConfigError", "Detect", "ErrUnknownFormat", "ErrUnsupported", "Format", "FormatBF16",
           "FormatF32", "Formats", "Lane", "Open", "OpenedModel", "Options", "Provide", "Qwen3Config", "Register",
           "Supports", "TokensGenerator", "chat", "random_model_path", "registry"]
