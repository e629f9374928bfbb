"""The step function: one batch of (request, its next tokens) through the model, from the cache.

FeLLM's `Engine::step_batch(sequences, conv_states, rows: [BatchToken{sequence, token, position,
compute_logits}])` takes one entry per token row and, for the hybrid model, at most one row per
sequence (crates/fellm-runtime/src/engine.rs:461-470,1805-1818,2801-2996;
crates/fellm-runtime/src/scheduler.rs:423-427).  Here an item is a request with n >= 1 next
tokens: a portion of its prompt, cut anywhere, or one decoded token; all items of a step run as
one batch.  Positions are absolute and continue the request's length in the cache
(engine.rs:2848-2873: position = RoPE position = cache row; visible length = position + 1).

Per step, the host fills ONE pinned int32 buffer with every index array the kernels need and
copies it once; the logits come back for the wanted rows only.
"""
from __future__ import annotations

import gc
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..config.errors import CacheError, FellmError, KernelError


@dataclass
class StepItem:
    """`want`: indices into `tokens` whose logits are asked for (may be empty)."""
    req: object
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=list)


class StepContext:
    """Who is in the batch and where: device int32 arrays, all views of one buffer.

    tokens[T], positions[T] (absolute), row_item[T] (index of the row's item), row_slot[T] (its
    request's slot: the row of block tables and state arrays), item_start[n_items+1] (row offsets),
    item_slot[n_items], item_len[n_items] (request length after this step), logit_rows[W].
    """
    __slots__ = ("tokens", "positions", "row_item", "row_slot", "item_start", "item_slot", "item_len",
                 "logit_rows", "n_rows", "n_items", "n_logit_rows", "all_single", "max_item_rows",
                 "max_len", "status", "host", "logits_all", "fixed_addresses")


class StepBuffers:
    """Pinned host staging and its device twin, sized for the largest step."""

    def __init__(self, max_rows: int, max_items: int, device):
        self.max_rows, self.max_items = max_rows, max_items
        self.capacity = 5 * max_rows + 3 * max_items + 16
        self.on_gpu = torch.cuda.is_available() and str(device).startswith("cuda")
        # The copy engine reads a pinned buffer when the copy runs, not when it is queued: a ring
        # of staging buffers, each guarded by an event, keeps a later step from overwriting what an
        # earlier, still queued copy has yet to read.
        self.ring = [torch.zeros(self.capacity, dtype=torch.int32, pin_memory=self.on_gpu) for _ in range(4)]
        self.ring_np = [b.numpy() for b in self.ring]
        self.ring_events = [torch.cuda.Event() if self.on_gpu else None for _ in self.ring]
        self.ring_used = [False] * len(self.ring)
        self.ring_next = 0
        self.ring_sig = [None] * len(self.ring)
        self._decode_ctx = {}
        self.dev = torch.zeros(self.capacity, dtype=torch.int32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)

    def fill(self, tokens, positions, row_item, row_slot, item_start, item_slot, item_len, logit_rows,
             max_item_rows, max_len) -> StepContext:
        T, n, W = len(tokens), len(item_slot), len(logit_rows)
        if T > self.max_rows or n > self.max_items:
            raise FellmError(f"a step of {T} rows / {n} items exceeds the engine's buffers "
                             f"({self.max_rows} rows / {self.max_items} items)")
        ctx = StepContext()
        off = 0
        k = self.ring_next
        self.ring_next = (k + 1) % len(self.ring)
        if self.on_gpu and self.ring_used[k]:
            self.ring_events[k].synchronize()
        h, d = self.ring_np[k], self.dev
        self.ring_sig[k] = None

        def put(name, arr, count):
            nonlocal off
            h[off:off + count] = arr
            setattr(ctx, name, d[off:off + count])
            off += count
        put("tokens", tokens, T)
        put("positions", positions, T)
        put("row_item", row_item, T)
        put("row_slot", row_slot, T)
        put("item_start", item_start, n + 1)
        put("item_slot", item_slot, n)
        put("item_len", item_len, n)
        put("logit_rows", logit_rows, W)
        d[:off].copy_(self.ring[k][:off], non_blocking=True)
        if self.on_gpu:
            self.ring_events[k].record()
            self.ring_used[k] = True
        ctx.n_rows, ctx.n_items, ctx.n_logit_rows = T, n, W
        ctx.all_single = (T == n)
        ctx.logits_all = (W == T and list(logit_rows) == list(range(T)))
        ctx.max_item_rows, ctx.max_len = max_item_rows, max_len
        ctx.status = self.status
        ctx.host = None
        ctx.fixed_addresses = False
        return ctx


def _fill_decode(self, plan, wants, toks, lens) -> StepContext:
    """The decode form of fill(): n items of one row each.  The layout of the buffer is the one
    fill() makes for T = n; the parts that only depend on the composition are written once per
    staging buffer."""
    n = len(lens)
    if n > self.max_items or n > self.max_rows:
        raise FellmError(f"a step of {n} items exceeds the engine's buffers")
    k = self.ring_next
    self.ring_next = (k + 1) % len(self.ring)
    if self.on_gpu and self.ring_used[k]:
        self.ring_events[k].synchronize()
    h, d = self.ring_np[k], self.dev
    logit_rows = [i for i, w in enumerate(wants) if w]
    W = len(logit_rows)
    o_tok, o_pos, o_ri, o_rs = 0, n, 2 * n, 3 * n
    o_is, o_slot, o_len, o_lr = 4 * n, 5 * n + 1, 6 * n + 1, 7 * n + 1
    total = o_lr + W
    sig = (plan["serial"], wants)
    if plan["ring"][k] != sig or self.ring_sig[k] != sig:
        h[o_ri:o_ri + n] = plan["arange"][:n]
        h[o_rs:o_rs + n] = plan["slots"]
        h[o_is:o_is + n + 1] = plan["arange"]
        h[o_slot:o_slot + n] = plan["slots"]
        h[o_lr:o_lr + W] = logit_rows
        plan["ring"][k] = sig
        self.ring_sig[k] = sig
    if toks is not None:
        h[o_tok:o_tok + n] = toks
    h[o_pos:o_pos + n] = lens
    h[o_len:o_len + n] = lens + 1
    d[:total].copy_(self.ring[k][:total], non_blocking=True)
    if self.on_gpu:
        self.ring_events[k].record()
        self.ring_used[k] = True
    ctx = self._decode_ctx.get((n, W))
    if ctx is None:
        ctx = StepContext()
        ctx.tokens, ctx.positions, ctx.row_item, ctx.row_slot = d[o_tok:o_tok + n], d[o_pos:o_pos + n], d[o_ri:o_ri + n], d[o_rs:o_rs + n]
        ctx.item_start, ctx.item_slot, ctx.item_len = d[o_is:o_is + n + 1], d[o_slot:o_slot + n], d[o_len:o_len + n]
        ctx.logit_rows = d[o_lr:o_lr + W]
        ctx.n_rows, ctx.n_items, ctx.n_logit_rows = n, n, W
        ctx.all_single, ctx.max_item_rows = True, 1
        ctx.status, ctx.host = self.status, None
        ctx.fixed_addresses = True
        self._decode_ctx[(n, W)] = ctx
    ctx.logits_all = (W == n)
    ctx.max_len = int(lens.max()) + 1
    return ctx


StepBuffers.fill_decode = _fill_decode


_NOT_TAKEN = object()       # _step_decode's answer when the general path has to run the step (None is a result: tokens without logits)
MAX_ROW_GRAPHS = 8          # captured graphs of steps that are not pure decode (each keeps its activations)
DECODE_ROWS_STEP = 8        # decode steps of more than 16 rows run with a multiple of this many rows (the last ones padding)
MAX_DECODE_GRAPHS = 48      # captured decode steps (each keeps its logits [wanted, vocab]); the least recently used goes


class Stepper:
    """Owns the model, the cache manager and the step buffers; `step()` is the step function.

    Steps are replayed from CUDA graphs when `cuda_graphs` is on (decode steps, and the shapes of
    other steps that come again, e.g. prompts cut into equal portions: 121 direct launches of a
    2,048-token portion cost the host as long as they cost the device): FeLLM captures one decode step the same way
    (crates/backend-cuda/src/graph.rs:39-160, crates/fellm-runtime/src/engine.rs:3195-3233).  A
    graph is keyed by the number of items, the number of wanted rows and the longest context
    rounded up to 1024 (the key-range split of decode attention follows it); the first step with a
    new key runs directly (kernels get loaded), the second is captured, later ones are replayed.
    Index arrays and block tables live at fixed device addresses and are refreshed by copies before
    the replay."""

    def __init__(self, model, cache, *, max_rows: int, max_items: int, device, cuda_graphs: bool = False):
        self.model, self.cache, self.device = model, cache, device
        self.buffers = StepBuffers(max_rows, max_items, device)
        self.vocab = model.spec.vocab_size
        self.steps_run = 0
        self.cuda_graphs = bool(cuda_graphs)
        self.graphs = {}
        self.graph_seen = {}
        self.graph_pool = None
        self.row_graph_keys = []
        self.decode_graph_keys = []            # least recently used first
        self.launches = 0                      # kernels of ours launched, replays included
        self._decode_plans = {}
        self._plan_serial = 0

    def step(self, items: List[StepItem], device_tokens: Optional[torch.Tensor] = None,
             greedy_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Runs exactly the given tokens as one batch and returns float32 logits
        [sum(len(want)), vocab] on the device, in the order of the items and of each `want`.
        Nothing is changed when the step cannot be placed (unknown request, no pages).
        With cuda_graphs on, the tensor returned belongs to the step's graph and is written again
        by the next step of the same shape: read it, or copy it, before the next call
        (Engine.step hands out a copy).

        device_tokens: int32 [rows] on the device to use instead of the items' token ids (which
        are then placeholders): lets a decode loop feed sampled tokens back without the host.
        greedy_tokens: int32 [>= wanted rows] on the device: the caller only wants the greedy token of
        every wanted row.  Where the model's head can pick them without storing the logits, they are
        written there and None is returned; else the logits come back as usual."""
        if not items:
            raise FellmError("a step needs at least one item")
        if all(len(it.tokens) == 1 for it in items):
            fast = self._step_decode(items, device_tokens, greedy_tokens)
            if fast is not _NOT_TAKEN:
                return fast
        cache = self.cache
        seen = set()
        for it in items:
            if it.req in seen:
                raise FellmError(f"request {it.req!r} appears twice in one step")
            seen.add(it.req)
            if not cache.has(it.req):
                raise CacheError(f"unknown request {it.req!r}")
            if len(it.tokens) < 1:
                raise FellmError(f"request {it.req!r} brings no tokens")
            for w in it.want:
                if not 0 <= w < len(it.tokens):
                    raise FellmError(f"request {it.req!r}: wanted place {w} is outside its {len(it.tokens)} tokens")
        asks = [(it.req, len(it.tokens)) for it in items]
        for req, n in asks:
            if cache.length(req) + n > cache.n_ctx:
                raise CacheError(f"request {req!r} would reach {cache.length(req) + n} tokens; "
                                 f"the context holds {cache.n_ctx}")
        if not cache.can_reserve(asks):
            raise CacheError("out of cache pages for this step")

        tok_parts, pos_parts, ri_parts, rs_parts, logit_rows = [], [], [], [], []
        item_start, item_slot, item_len = [0], [], []
        max_rows, max_len = 0, 0
        for i, it in enumerate(items):
            n = len(it.tokens)
            t = np.asarray(it.tokens, dtype=np.int64)
            if t.min() < 0 or t.max() >= self.vocab:
                raise FellmError(f"request {it.req!r}: token id outside the vocabulary of {self.vocab}")
            p0, slot = cache.length(it.req), cache.slot(it.req)
            tok_parts.append(t)
            pos_parts.append(np.arange(p0, p0 + n))
            ri_parts.append(np.full(n, i))
            rs_parts.append(np.full(n, slot))
            base = item_start[-1]
            logit_rows += [base + w for w in it.want]
            item_start.append(base + n)
            item_slot.append(slot)
            item_len.append(p0 + n)
            max_rows, max_len = max(max_rows, n), max(max_len, p0 + n)
        for req, n in asks:
            cache.reserve(req, n)
        ctx = self.buffers.fill(np.concatenate(tok_parts), np.concatenate(pos_parts), np.concatenate(ri_parts),
                                np.concatenate(rs_parts), item_start, item_slot, item_len, logit_rows,
                                max_rows, max_len)
        if device_tokens is not None:
            ctx.tokens.copy_(device_tokens[:ctx.n_rows])
        cache.flush()
        logits = self._run(ctx, greedy_tokens)
        for req, n in asks:
            cache.advance(req, n)
        self.steps_run += 1
        return logits

    def _step_decode(self, items: List[StepItem], device_tokens, greedy_tokens=None):
        """Every item brings one token: the host work is a handful of numpy writes.  What does
        not change while the same requests decode together (slots, offsets, the wanted rows) is
        kept per composition; positions and lengths come from the cache's own counters.  Returns
        _NOT_TAKEN when the general path has to look at the step (unknown request, page or context
        limits, windows to trim)."""
        cache = self.cache
        reqs = tuple(it.req for it in items)
        n = len(items)
        lens_d, slot_d = cache.req_len, cache.req_slot
        try:
            lens = np.fromiter((lens_d[r] for r in reqs), dtype=np.int64, count=n)
            # a request's name may come again later in another slot: the slots are part of the key
            key = (reqs, tuple(slot_d[r] for r in reqs))
        except KeyError:
            return _NOT_TAKEN
        wants = tuple(bool(it.want) for it in items)
        # A graph is captured for every count of rows a decode step has; from 17 rows on the count is filled up
        # to a multiple of 8 with rows that belong to nobody (the cache's pad slot: position 0 of a page of its
        # own, a state row of its own), so that a batch that grows or drains by one request at a time meets a
        # new graph every eighth count, not at every one.  Up to 16 rows each count has kernels of its own cost.
        n_pad = n
        if self.cuda_graphs and n > 16 and all(wants):
            n_pad = -(-n // DECODE_ROWS_STEP) * DECODE_ROWS_STEP
            if n_pad > self.buffers.max_items:
                n_pad = n
        key = key + (n_pad,)
        plan = self._decode_plans.get(key)
        if plan is None:
            if len(set(reqs)) != n:
                return _NOT_TAKEN
            if len(self._decode_plans) > 64:
                self._decode_plans.clear()
            self._plan_serial += 1                         # never reused, unlike id(): names what a staging buffer holds
            plan = {"slots": np.array(key[1] + (cache.pad_slot,) * (n_pad - n), dtype=np.int64), "arange": np.arange(n_pad + 1),
                    "ring": [None] * len(self.buffers.ring), "serial": self._plan_serial}
            self._decode_plans[key] = plan
        if int(lens.max()) + 1 > cache.n_ctx:
            return _NOT_TAKEN
        if cache.has_windows:
            return _NOT_TAKEN
        if device_tokens is None:
            toks = np.fromiter((it.tokens[0] for it in items), dtype=np.int64, count=n)
            if toks.min() < 0 or toks.max() >= self.vocab:
                raise FellmError(f"token id outside the vocabulary of {self.vocab}")
        else:
            toks = None
        pt = cache.page_tokens
        if (lens % pt == 0).any():                          # somebody starts a page
            asks = [(r, 1) for r in reqs]
            if not cache.can_reserve(asks):
                raise CacheError("out of cache pages for this step")
            for r, l in zip(reqs, lens):
                if l % pt == 0:
                    cache.reserve(r, 1)
        if n_pad > n:
            wants = wants + (True,) * (n_pad - n)
            fill = np.zeros(n_pad - n, dtype=np.int64)
            lens = np.concatenate([lens, fill])
            # (token 0 for the padding rows, also where the real rows' tokens come from the device)
            toks = np.zeros(n_pad, dtype=np.int64) if toks is None else np.concatenate([toks, fill])
        ctx = self.buffers.fill_decode(plan, wants, toks, lens)
        if device_tokens is not None:
            ctx.tokens[:n].copy_(device_tokens[:n])
        cache.flush()
        logits = self._run(ctx, greedy_tokens)
        for r in reqs:
            lens_d[r] += 1
        self.steps_run += 1
        return logits if (logits is None or n_pad == n) else logits[:n]

    def _run(self, ctx, greedy_tokens=None) -> torch.Tensor:
        from .. import ops
        views = self.cache.views(ctx.item_slot)
        greedy_key = None if greedy_tokens is None else greedy_tokens.data_ptr()
        if not self.cuda_graphs:
            before = ops.launch_count()
            logits = self.model.forward(ctx, views, greedy_tokens)
            self.launches += ops.launch_count() - before
            return logits
        # what the launches of a step depend on besides the device arrays: the counts that size the
        # grids and pick the kernels.  Decode steps: the longest context rounded up to 1024 (the
        # key-range split of decode attention).  Other steps (portions of prompts, mixed batches)
        # repeat their shape when prompts are cut into equal portions: a few of their graphs are kept.
        if ctx.all_single:
            key = (ctx.n_items, ctx.n_logit_rows, -(-ctx.max_len // 1024), greedy_key)
        else:
            key = ("rows", ctx.n_rows, ctx.n_items, ctx.n_logit_rows, ctx.max_item_rows, ctx.logits_all, greedy_key)
        entry = self.graphs.get(key)
        if entry is None:
            n_seen = self.graph_seen.get(key, 0)
            if len(self.graph_seen) > 4096:                  # shapes seen once and never again
                self.graph_seen = {k: v for k, v in self.graph_seen.items() if k in self.graphs}
            self.graph_seen[key] = n_seen + 1
            # a shape of prompt portions is captured when it comes a second time (most never do); a decode step's
            # count of requests comes again almost surely, and a direct run costs as much as a capture
            if n_seen == 0 and not ctx.all_single:
                before = ops.launch_count()
                logits = self.model.forward(ctx, views, greedy_tokens)
                self.launches += ops.launch_count() - before
                return logits
            graph = torch.cuda.CUDAGraph()
            before = ops.launch_count()
            # The garbage collector must not run inside a capture: if it finds an engine that was dropped
            # earlier, that engine's graphs are destroyed then and there, which the capturing stream does not
            # permit (the capture is invalidated and the next launch fails).  It waits until the capture is over.
            gc_was_on = gc.isenabled()
            gc.disable()
            try:
                with torch.cuda.graph(graph, pool=self.graph_pool):
                    logits = self.model.forward(ctx, views, greedy_tokens)
            finally:
                if gc_was_on:
                    gc.enable()
            if self.graph_pool is None:
                self.graph_pool = graph.pool()
            entry = (graph, logits, ops.launch_count() - before)
            self.graphs[key] = entry
            if not ctx.all_single:
                self.row_graph_keys.append(key)
                if len(self.row_graph_keys) > MAX_ROW_GRAPHS:            # the oldest goes; its buffers return to the pool
                    old = self.row_graph_keys.pop(0)
                    self.graphs.pop(old, None)
                    self.graph_seen.pop(old, None)
            else:
                self.decode_graph_keys.append(key)
                if len(self.decode_graph_keys) > MAX_DECODE_GRAPHS:
                    old = self.decode_graph_keys.pop(0)
                    self.graphs.pop(old, None)
                    self.graph_seen.pop(old, None)
        elif ctx.all_single and self.decode_graph_keys[-1] != key:
            self.decode_graph_keys.remove(key)
            self.decode_graph_keys.append(key)
        graph, logits, n_launches = entry
        graph.replay()
        self.launches += n_launches
        return logits

    def check_status(self):
        """Reads the device status word (synchronises).  Kernels set it instead of faulting:
        1 = a token id outside the embedding table, 2 = a cache write with no page mapped."""
        from .. import ops
        ops.check_umma_status(self.device)
        code = int(self.buffers.status.item())
        if code:
            self.buffers.status.zero_()
            what = {1: "a token id outside the embedding table",
                    2: "a cache write to a position with no page"}.get(code, f"code {code}")
            raise KernelError(f"a kernel reported: {what}")
