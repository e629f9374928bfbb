"""The device sampler: one launch samples every row of a step's logits, each row with its own
request's parameters.  What FeLLM keeps per request on the host - the token history for the
penalties (SamplerState.history, crates/fellm-runtime/src/sampling.rs:97-191) - is a count table
[slot, vocab] on the device here, updated by the sampling kernel itself and primed with the
prompt at admission (scheduler.rs:319-372 primes the history with the prompt ids)."""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence

import numpy as np
import torch

from .. import ops
from ..config.errors import KernelError
from .params import GenParams

ROW_PARAMS = np.dtype([("temperature", "<f4"), ("top_p", "<f4"), ("min_p", "<f4"), ("rep_pen", "<f4"),
                       ("freq_pen", "<f4"), ("pres_pen", "<f4"), ("top_k", "<i4"), ("slot", "<i4"),
                       ("bias_begin", "<i4"), ("bias_end", "<i4"), ("seed", "<u8")])


class Sampler:
    def __init__(self, vocab: int, n_slots: int, max_rows: int, device):
        self.vocab, self.n_slots, self.max_rows, self.device = vocab, n_slots, max_rows, device
        size = ops.sample_params_size()
        if size != ROW_PARAMS.itemsize:
            raise KernelError(f"sampling parameter record is {size} bytes in the kernel, {ROW_PARAMS.itemsize} here")
        # a few pinned parameter buffers in turn: the host may fill the next launch's records while
        # the copy of the last launch's still waits in the stream behind that launch's kernels
        self._params_ring = []
        for _ in range(4):
            host = torch.zeros(max_rows * size, dtype=torch.uint8, pin_memory=True)
            self._params_ring.append([host, host.numpy().view(ROW_PARAMS), torch.cuda.Event(), False])
        self._params_no = 0
        self.params_dev = torch.zeros(max_rows * size, dtype=torch.uint8, device=device)
        self.out_tokens = torch.zeros(max_rows, dtype=torch.int32, device=device)
        self.out_host = torch.zeros(max_rows, dtype=torch.int32, pin_memory=True)
        self.arg_val = torch.zeros(max_rows * 64, dtype=torch.float32, device=device)
        self.arg_idx = torch.zeros(max_rows * 64, dtype=torch.int32, device=device)
        self.counts: Optional[torch.Tensor] = None

    # ---- history for the penalties
    def _ensure_counts(self):
        if self.counts is None:
            self.counts = torch.zeros((self.n_slots, self.vocab), dtype=torch.int32, device=self.device)

    def start_request(self, slot: int, prompt: Sequence[int], params: GenParams):
        if self.counts is not None:
            self.counts[slot].zero_()
        if params.uses_history():
            self._ensure_counts()
            toks = torch.tensor(list(prompt), dtype=torch.int32).to(self.device)
            slots = torch.full_like(toks, slot)
            ops.count_tokens(self.counts, slots, toks)

    @staticmethod
    def plain_greedy(rows: List[tuple]) -> bool:
        """Every row is argmax of its logits as they are (no penalties, no bias): such a step can ask the model
        for the tokens themselves (Stepper.step(greedy_tokens=...)) and skip the logits."""
        return all(p.is_greedy() and not p.uses_history() and not p.logit_bias for _, p, _ in rows)

    # ---- one launch per step
    def sample(self, logits: torch.Tensor, rows: List[tuple], return_probs: bool = False):
        """rows[i] = (slot, GenParams, draw_index) for logits[i].  Returns int32 tokens on the device
        (a view of a buffer the next call overwrites), and the processed distributions if asked."""
        n = len(rows)
        assert logits.shape[0] == n and logits.dtype == torch.float32 and logits.is_contiguous()
        if n > self.max_rows:
            raise KernelError(f"{n} rows to sample exceed the sampler's {self.max_rows}")
        if not return_probs and self.plain_greedy(rows):
            # plain argmax: no per-row parameters to ship, the row is reduced by 64 blocks at once
            ops.argmax_rows(logits, self.arg_val, self.arg_idx, self.out_tokens)
            return self.out_tokens[:n]
        entry = self._params_ring[self._params_no % len(self._params_ring)]
        self._params_no += 1
        params_host, rec, copy_done, pending = entry
        if pending:
            copy_done.synchronize()
        bias_tok, bias_val = [], []
        need_counts = False
        for i, (slot, p, draw) in enumerate(rows):
            b0 = len(bias_tok)
            for t, b in p.logit_bias.items():
                bias_tok.append(int(t)), bias_val.append(float(b))
            rec[i] = (p.temperature, p.top_p, p.min_p, p.repetition_penalty, p.frequency_penalty,
                      p.presence_penalty, p.top_k, slot, b0, len(bias_tok), (p.seed + draw) & 0xFFFFFFFFFFFFFFFF)
            need_counts |= p.uses_history()
        if need_counts:
            self._ensure_counts()
        nbytes = n * ROW_PARAMS.itemsize
        self.params_dev[:nbytes].copy_(params_host[:nbytes], non_blocking=True)
        copy_done.record()
        entry[3] = True
        bt = bv = None
        if bias_tok:
            bt = torch.tensor(bias_tok, dtype=torch.int32).to(self.device)
            bv = torch.tensor(bias_val, dtype=torch.float32).to(self.device)
        probs = torch.empty_like(logits) if return_probs else None
        ops.sample(logits, self.params_dev, self.counts, bt, bv, self.out_tokens, probs)
        toks = self.out_tokens[:n]
        return (toks, probs) if return_probs else toks
