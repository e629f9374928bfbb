"""Generation parameters and statistics, with FeLLM's names, meanings and defaults
(GenParams: crates/fellm-runtime/src/engine.rs:269-326; GenStats: engine.rs:211-265)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Tuple


@dataclass
class GenParams:
    max_tokens: int = 128
    temperature: float = 0.2          # <= 0 (or top_k == 1) is greedy
    top_k: int = 80                   # 0 disables
    top_p: float = 1.0                # >= 1 disables
    min_p: float = 0.0                # 0 disables
    seed: int = 0                     # draw i uses seed + i
    repetition_penalty: float = 1.05  # <= 1 disables
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    logit_bias: Dict[int, float] = field(default_factory=dict)
    priority: int = 0                 # larger runs first within decodes and within prefills
    stop_token_ids: Tuple[int, ...] = ()   # FeLLM takes these from the tokenizer (engine.rs:1295-1311)

    def is_greedy(self) -> bool:
        return self.temperature <= 0.0 or self.top_k == 1

    def uses_history(self) -> bool:
        return (self.repetition_penalty > 1.0 or self.frequency_penalty != 0.0
                or self.presence_penalty != 0.0)

    @staticmethod
    def greedy(max_tokens: int = 128, **kw) -> "GenParams":
        return GenParams(max_tokens=max_tokens, temperature=0.0, repetition_penalty=1.0, **kw)


@dataclass
class GenStats:
    """prompt_ms: time until the logits for the first sample exist; the per-second figures
    follow engine.rs:230-264."""
    prompt_tokens: int = 0
    predicted_tokens: int = 0
    prompt_ms: float = 0.0
    total_ms: float = 0.0
    time_to_first_token_ms: float = 0.0
    finish_reason: str = ""

    def prompt_tok_per_sec(self) -> float:
        return self.prompt_tokens / (self.prompt_ms / 1000.0) if self.prompt_ms > 0 else 0.0

    def generation_tok_per_sec(self) -> float:
        ms = max(self.total_ms - self.prompt_ms, 0.0)
        return self.predicted_tokens / (ms / 1000.0) if ms > 0 else 0.0

    def predicted_tok_per_sec(self) -> float:
        ms = max(self.total_ms - self.time_to_first_token_ms, 0.0)
        return (self.predicted_tokens - 1) / (ms / 1000.0) if ms > 0 and self.predicted_tokens > 1 else 0.0
