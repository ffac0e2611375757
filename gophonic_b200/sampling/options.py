"""Options of one reply, with the names and meanings of gophonic's ``chat.Options``
(chat/chat.go:50-67): the zero value decodes greedily until the model ends its message."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class Options:
    # MaxTokens bounds the reply; zero means no bound but the context.
    MaxTokens: int = 0
    # Temperature scales the logits before sampling; zero picks the most likely token every step.
    Temperature: float = 0.0
    # TopK keeps only the TopK most likely tokens; zero keeps them all (at most 1024 are
    # considered: qwen3/chat.go:796-799).
    TopK: int = 0
    # TopP keeps the smallest set of most likely tokens whose probability reaches TopP; zero or one
    # keeps them all.
    TopP: float = 0.0
    # Presence lowers the logit of every token the reply already holds by this much.
    Presence: float = 0.0
    # Seed seeds sampling; replies with equal seeds and inputs are equal.
    Seed: int = 0

    def validate(self) -> None:
        if self.MaxTokens < 0:
            raise ValueError(f"MaxTokens {self.MaxTokens} is negative")
        if self.TopK < 0:
            raise ValueError(f"TopK {self.TopK} is negative")
        if not 0.0 <= self.TopP <= 1.0:
            raise ValueError(f"TopP {self.TopP} is outside [0, 1]")
        if self.Temperature != self.Temperature or self.Temperature < 0:
            raise ValueError(f"Temperature {self.Temperature} is negative or not a number")
