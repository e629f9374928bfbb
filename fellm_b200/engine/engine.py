"""The engine: a model folder (or a configuration and a seed) turned into a model on the GPU,
its cache, the step function, and on top of them generation.

It keeps the names of FeLLM's Rust API (crates/fellm-runtime/src/engine.rs): `Engine::open_with`
(527) -> Engine.open, `generate` (947) -> Engine.generate, `step_batch` (1805) -> Engine.step,
`GenParams` (269-326), `GenStats` (211-265), and `Scheduler::enqueue_ids / poll_event`
(crates/fellm-runtime/src/scheduler.rs:319,381) -> Engine.scheduler().
"""
from __future__ import annotations

import time
from pathlib import Path
from typing import Iterable, List, Optional

import torch

from ..cache.manager import CacheManager
from ..config.errors import ConfigError, KernelError
from ..config.options import EngineOptions
from ..config.registry import config_from_dict, read_model_config
from ..csrc import jit
from ..models.model import build_model
from ..weights.loader import bind_tensors, load_into
from ..weights.random_init import random_tensors
from .step import StepItem, Stepper


def _require_gpu(device: str):
    if not torch.cuda.is_available():
        raise KernelError("fellm_b200 needs a CUDA device: there is no CPU path")
    major, minor = torch.cuda.get_device_capability(torch.device(device))
    if major != 10:
        raise KernelError(f"fellm_b200's kernels are built for sm_100a; {device} is sm_{major}{minor}")


class Engine:
    def __init__(self, arch, config, options: EngineOptions, *, folder=None, tensors=None):
        options.validate()
        _require_gpu(options.device)
        self.arch, self.config, self.options = arch, config, options
        self.device = torch.device(options.device)
        torch.cuda.set_device(self.device)
        spec = arch.build_spec(config)
        self.spec = spec
        self.model = build_model(spec, options.dtype)
        jit.compile_many(self.model.kernel_modules())
        if folder is not None:
            load_into(self.model, folder, self.device)
        else:
            bind_tensors(self.model, tensors, self.device)
        # context: FeLLM clamps n_ctx to the model's maximum, 0 = the maximum (engine.rs:190-197)
        n_ctx = spec.max_position if options.n_ctx == 0 else min(options.n_ctx, spec.max_position)
        self.n_ctx = n_ctx
        cache_dtype = torch.bfloat16 if options.dtype == "bfloat16" else torch.float32
        needs = self.model.cache_needs()
        max_tokens = options.max_tokens
        if max_tokens is None:
            max_tokens = self._tokens_from_memory(needs, cache_dtype)
        self.cache = CacheManager(needs, page_tokens=options.page_tokens, max_tokens=max_tokens,
                                  max_requests=options.max_requests, n_ctx=n_ctx, dtype=cache_dtype,
                                  device=self.device)
        max_rows = max(options.n_batch, options.n_ubatch) + options.max_requests
        self.stepper = Stepper(self.model, self.cache, max_rows=max_rows, max_items=options.max_requests,
                               device=self.device)

    # ---- constructors
    @classmethod
    def open(cls, folder, options: Optional[EngineOptions] = None, **settings) -> "Engine":
        """A folder with config.json and model.safetensors; the model class is chosen by
        config.json's `architectures`."""
        options = options or EngineOptions(**settings)
        arch, config = read_model_config(folder)
        if not (Path(folder) / "model.safetensors").exists():
            from ..config.errors import WeightError
            raise WeightError(f"no model.safetensors in {folder}")
        return cls(arch, config, options, folder=folder)

    @classmethod
    def random(cls, config_dict: dict, seed: int, options: Optional[EngineOptions] = None, **settings) -> "Engine":
        """Random weights from a configuration and a seed, without a folder in between (the same
        values `write_model_folder` stores)."""
        options = options or EngineOptions(**settings)
        arch, config = config_from_dict(config_dict)
        probe = build_model(arch.build_spec(config), "float32")
        tensors = random_tensors(probe, seed)
        return cls(arch, config, options, tensors=tensors)

    def _tokens_from_memory(self, needs, cache_dtype) -> int:
        """FeLLM: usable = free - reserves; budget = usable * kv_memory_fraction; pages =
        budget / page_bytes (crates/fellm-runtime/src/kv_fabric/fabric.rs:40-61)."""
        from ..parts.base import PagedKV
        esize = 2 if cache_dtype == torch.bfloat16 else 4
        per_token = {}
        for need in needs:
            if isinstance(need, PagedKV):
                per_token[need] = per_token.get(need, 0) + 2 * need.kv_heads * need.head_dim * esize
        total = sum(per_token.values())
        if total == 0:
            return self.options.page_tokens
        free, _ = torch.cuda.mem_get_info(self.device)
        budget = int(max(free - (2 << 30), 0) * self.options.kv_memory_fraction)
        tokens = budget // total
        cap = self.options.max_requests * self.n_ctx
        tokens = max(min(tokens, cap), self.options.page_tokens)
        return tokens - tokens % self.options.page_tokens

    # ---- the step function and request bookkeeping around it
    def add_request(self, req):
        return self.cache.add_request(req)

    def release(self, req):
        self.cache.release(req)

    def step(self, items: List[StepItem]) -> torch.Tensor:
        return self.stepper.step(items)

    def check_status(self):
        self.stepper.check_status()
