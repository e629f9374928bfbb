"""Position encodings.  Rotary: inv_freq[i] = theta^(-2i/rot_dim) in float32
(crates/fellm-model/src/rope.rs:13-21); pairs (2i, 2i+1) or (i, i+rot_dim/2)
(crates/backend-cpu/src/kernels/rope.rs:28-62).  The rotation itself happens inside the kernel
that also norms q/k and writes the cache (fellm_b200/csrc/qk_rope_write.cu)."""
from __future__ import annotations

import torch

from ..config.errors import ConfigError
from .base import PositionEncoding, register_part


@register_part("position", "none")
class NoPosition(PositionEncoding):
    def __init__(self, *, dtype: str):
        super().__init__()
        self.inv_freq = None
        self.pairing = "adjacent"

    def to(self, device):
        return self


@register_part("position", "rope")
class Rotary(PositionEncoding):
    def __init__(self, *, dtype: str, rot_dim: int, theta: float, pairing: str):
        super().__init__()
        if rot_dim % 2:
            raise ConfigError(f"rotary dimension {rot_dim} must be even")
        if pairing not in ("adjacent", "split_half"):
            raise ConfigError(f"unknown rotary pairing {pairing!r}")
        self.rot_dim, self.theta, self.pairing = int(rot_dim), float(theta), pairing
        i = torch.arange(self.rot_dim // 2, dtype=torch.float32)
        self.inv_freq = torch.pow(torch.tensor(self.theta, dtype=torch.float32),
                                  -(2.0 * i) / float(self.rot_dim))

    def to(self, device):
        self.inv_freq = self.inv_freq.to(device)
        return self
