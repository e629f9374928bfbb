"""Engine options: what FeLLM calls EngineSettings (crates/fellm-runtime/src/engine.rs:46-97)
and the KV fabric's memory plan (crates/fellm-runtime/src/kv_fabric/fabric.rs:21-88)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .errors import ConfigError

DTYPES = ("bfloat16", "float32")


@dataclass
class EngineOptions:
    """n_ctx / n_batch / n_ubatch keep FeLLM's names and defaults (engine.rs:56-97):
    n_ctx 8192 clamped to the model's maximum (0 = the model's maximum), n_batch = tokens a
    scheduler iteration may run, n_ubatch = the longest portion of one prompt in a step."""
    dtype: str = "bfloat16"
    n_ctx: int = 8192
    n_batch: int = 2048
    n_ubatch: int = 512
    ctx_past_model: bool = False    # replay of given tokens: n_ctx is taken as given, not clamped to the model's maximum
    page_tokens: int = 64
    max_requests: int = 64          # state slots and block-table rows
    max_tokens: Optional[int] = None    # cache pool size in tokens; None = from memory
    kv_memory_fraction: float = 0.25    # fabric.rs:40-48 (share of free memory when max_tokens is None)
    kv_device_budget: int = 0           # bytes of cache pages when max_tokens is None; 0 = from free memory (FeLLM's --kv-device-budget)
    cuda_graphs: bool = True
    device: str = "cuda:0"

    def validate(self):
        if self.dtype not in DTYPES:
            raise ConfigError(f"dtype must be one of {DTYPES}, got {self.dtype!r}")
        if self.page_tokens < 1 or (self.page_tokens & (self.page_tokens - 1)):
            raise ConfigError(f"page_tokens must be a power of two, got {self.page_tokens}")
        if self.page_tokens > 256:
            raise ConfigError(f"page_tokens must be <= 256, got {self.page_tokens}")
        for k in ("n_batch", "n_ubatch", "max_requests"):
            if getattr(self, k) < 1:
                raise ConfigError(f"{k} must be >= 1")
        if self.kv_device_budget < 0:
            raise ConfigError("kv_device_budget must be >= 0 bytes")
        if self.n_ctx < 0:
            raise ConfigError("n_ctx must be >= 0")
        return self
