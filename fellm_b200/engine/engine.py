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
from ..sampling.params import GenParams, GenStats
from ..sampling.sampler import Sampler
from .scheduler import Scheduler
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
        if options.ctx_past_model and options.n_ctx > 0:
            n_ctx = options.n_ctx          # positions past max_position_embeddings rotate like any other: nothing is learned per position
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
        for part in self.model.all_parts():
            part.reserve(self.device, options.max_requests, n_ctx)
        from .. import ops
        ops.register_weight_chain(self.model.weight_chain())
        self.stepper = Stepper(self.model, self.cache, max_rows=max_rows, max_items=options.max_requests,
                               device=self.device, cuda_graphs=options.cuda_graphs)
        self._sampler: Optional[Sampler] = None
        # sampled tokens (and the status word behind them) come back through a few pinned buffers in
        # turn: a launch may be in flight while the one before it is read
        self._tok_ring = [(torch.zeros(options.max_requests + 1, dtype=torch.int32, pin_memory=True), torch.cuda.Event())
                          for _ in range(4)]
        self._tok_count = [0] * len(self._tok_ring)
        self._launch_no = 0
        self._scheduler: Optional[Scheduler] = None

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
        """FeLLM: usable = free - reserves; budget = usable * kv_memory_fraction, or the explicit
        device budget; pages = budget / page_bytes (crates/fellm-runtime/src/kv_fabric/fabric.rs:40-61)."""
        esize = 2 if cache_dtype == torch.bfloat16 else 4
        pt = self.options.page_tokens
        cap = self.options.max_requests * (-(-self.n_ctx // pt) * pt)
        if self.options.kv_device_budget > 0:
            budget = self.options.kv_device_budget
            if CacheManager.tokens_for_budget(needs, esize, budget, 1, cap) < pt:
                raise ConfigError(f"kv_device_budget of {budget} bytes does not hold one page of {pt} tokens")
        else:
            free, _ = torch.cuda.mem_get_info(self.device)
            budget = int(max(free - (2 << 30), 0) * self.options.kv_memory_fraction)
        return CacheManager.tokens_for_budget(needs, esize, budget, pt, cap)

    @property
    def sampler(self) -> Sampler:
        """Made on first use: replaying a trace samples nothing and need not build the sampling kernels."""
        if self._sampler is None:
            self._sampler = Sampler(self.spec.vocab_size, self.options.max_requests, self.options.max_requests,
                                    self.device)
        return self._sampler

    # ---- the step function and request bookkeeping around it
    def add_request(self, req):
        return self.cache.add_request(req)

    def release(self, req):
        self.cache.release(req)

    def step(self, items: List[StepItem], device_tokens=None) -> torch.Tensor:
        """The step function (Stepper.step).  The logits are the caller's own: with CUDA graphs on,
        the step's graph keeps writing into its own output, so a copy is handed out."""
        logits = self.stepper.step(items, device_tokens)
        return logits.clone() if self.stepper.cuda_graphs else logits

    def check_status(self):
        self.stepper.check_status()

    # ---- what the scheduler drives (its `backend`)
    def start_request(self, slot: int, prompt, params: GenParams):
        self.sampler.start_request(slot, prompt, params)

    def launch(self, items: List[StepItem], sample_rows, chain: bool = False) -> int:
        """One step and one sampling launch, not waited for; returns a handle for collect().
        chain: the items (one token each, in the order of the last launch's sample rows) take the
        last launch's sampled tokens as they lie on the device.  The tokens and the kernels'
        status word are copied to one of a few pinned host buffers behind the launch."""
        n = len(sample_rows)
        # plain greedy rows: the head may pick the tokens itself and leave the logits unwritten
        greedy = self.sampler.out_tokens if n and self.sampler.plain_greedy(sample_rows) else None
        logits = self.stepper.step(items, device_tokens=self.sampler.out_tokens if chain else None, greedy_tokens=greedy)
        k = self._launch_no % len(self._tok_ring)
        self._launch_no += 1
        host, done = self._tok_ring[k]
        if n:
            toks = self.sampler.out_tokens[:n] if logits is None else self.sampler.sample(logits, sample_rows)
            host[:n].copy_(toks, non_blocking=True)
        host[-1:].copy_(self.stepper.buffers.status, non_blocking=True)
        done.record()
        self._tok_count[k] = n
        return k

    def collect(self, handle: int) -> List[int]:
        """Waits for a launch and returns its sampled tokens on the host."""
        host, done = self._tok_ring[handle]
        done.synchronize()
        if int(host[-1]):
            self.stepper.check_status()
        return host[:self._tok_count[handle]].tolist()

    def run(self, items: List[StepItem], sample_rows) -> List[int]:
        """launch() and collect() in one: the tokens and the status word come back in one
        synchronisation."""
        return self.collect(self.launch(items, sample_rows))

    # ---- generation
    def scheduler(self) -> Scheduler:
        """The engine's scheduler (made on first use): enqueue_ids / poll_event / step."""
        if self._scheduler is None:
            self._scheduler = Scheduler(self, self.options.n_batch, self.options.n_ubatch)
        return self._scheduler

    def generate(self, ids, params: Optional[GenParams] = None) -> "TokenStream":
        """Token ids in, an iterator of generated token ids out (FeLLM: Engine::generate ->
        TokenStream, engine.rs:947,3343-3538; text and tokenizer are outside this engine)."""
        return TokenStream(self, [list(ids)], params or GenParams())

    def generate_batch(self, prompts, params: Optional[GenParams] = None):
        """Runs several prompts together; returns (list of generated id lists, list of GenStats)."""
        sched = self.scheduler()
        params = params or GenParams()
        plist = params if isinstance(params, (list, tuple)) else [params] * len(prompts)
        rids = [sched.enqueue_ids(p, q) for p, q in zip(prompts, plist)]
        out = {r: [] for r in rids}
        stats = {}
        while len(stats) < len(rids):
            ev = sched.poll_event(rids)          # other callers' events stay queued for them
            if ev is None:
                break
            if ev.kind == "token":
                out[ev.req].append(ev.token)
            elif ev.kind == "done":
                stats[ev.req] = ev.stats
            elif ev.kind == "error":
                raise KernelError(f"request {ev.req} failed: {ev.message}")
        return [out[r] for r in rids], [stats.get(r) for r in rids]


class TokenStream:
    """Iterator over one request's generated tokens; finish_stats() after the last one."""

    def __init__(self, engine: Engine, prompts, params: GenParams):
        self.engine, self.sched = engine, engine.scheduler()
        self.rid = self.sched.enqueue_ids(prompts[0], params)
        self.stats: Optional[GenStats] = None
        self._done = False

    def __iter__(self):
        return self

    def __next__(self) -> int:
        while not self._done:
            ev = self.sched.poll_event(self.rid)     # other streams' events stay queued for them
            if ev is None:
                break
            if ev.kind == "token":
                return ev.token
            self.stats, self._done = ev.stats, True
            if ev.kind == "error":
                raise KernelError(f"generation failed: {ev.message}")
        raise StopIteration

    def finish_stats(self) -> GenStats:
        for _ in self:
            pass
        return self.stats
