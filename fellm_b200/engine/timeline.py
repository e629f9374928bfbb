"""Kernel timeline of a step: when each launch of this package's kernels began, when it stopped
waiting for the kernel before it, and when its last CTA left.

Built only when FELLM_B200_TRACE=1 is set before the kernels are loaded (the modules are then
compiled with -DFELLM_TRACE=1 into libraries of their own).  Thread 0 of every CTA records the
GPU's global timer three times; `Timeline.launches()` groups the records into launches.  The
records cost an atomic and three stores per CTA, so a traced step is a little slower than a plain
one: read the shares and the gaps, not the total.

FeLLM times its decode phases on the host (crates/fellm-runtime/src/profiler.rs); a timeline of
the device's kernels has no counterpart there.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List

import torch

from ..config.errors import KernelError
from ..csrc import jit

KERNEL_NAMES = {1: "embed_rows", 2: "rmsnorm", 3: "rmsnorm_vec", 4: "silu_mul", 5: "gemm_simt", 6: "gemm_tiled",
                7: "gemm_umma", 8: "shortconv", 9: "qk_rope_write", 10: "qk_rope_write_vec", 11: "attention_simt",
                12: "attention_prefill", 13: "attention_decode", 14: "sample", 15: "count_tokens",
                16: "argmax_partial", 17: "argmax_final"}
SKINNY_EPILOGUES = {0: "store", 1: "accumulate", 2: "swiglu", 3: "float32"}


def kernel_name(ident: int) -> str:
    if ident >= 32:
        return f"gemm_skinny[{SKINNY_EPILOGUES.get(ident // 32 - 1, ident // 32 - 1)}]"
    return KERNEL_NAMES.get(ident, f"kernel{ident}")


@dataclass
class Launch:
    name: str
    blocks: int
    begin_us: float          # first CTA's entry, from the first record of the trace
    waited_us: float         # first CTA past its wait for the kernel before it
    end_us: float            # last CTA's exit
    marks_us: tuple = (0.0, 0.0, 0.0, 0.0)   # latest time any CTA passed each of the kernel's own marks (0: none did)
    ctas: list = field(default_factory=list)     # with detail=True: (begin, waited, end, marks...) of every CTA


def group_records(records, detail: bool = False) -> List[Launch]:
    """records: one [tag, entry, after wait, exit, mark0..3] (nanoseconds of the global timer; tag =
    kernel id | CTAs of the launch << 16) per CTA, in any order.  CTAs of one launch share a tag and
    lie together in time: a launch is closed when as many records as it has CTAs have come, so two
    launches of the same kernel and grid that overlap (programmatic dependents) still come apart."""
    if not records:
        return []
    records = sorted(records, key=lambda r: r[1])
    t0 = int(records[0][1])
    out: List[Launch] = []
    open_groups = {}                     # tag -> [records still expected, Launch]
    for tag, begin, waited, end, *marks in records:
        ident, blocks = tag & 0xFFFF, tag >> 16
        b, w, e = (begin - t0) / 1e3, ((waited or begin) - t0) / 1e3, ((end or begin) - t0) / 1e3
        mk = tuple((m - t0) / 1e3 if m else 0.0 for m in marks)
        g = open_groups.get(tag)
        if g is None:
            g = [blocks, Launch(kernel_name(ident), blocks, b, w, e, mk)]
            open_groups[tag] = g
            out.append(g[1])
        else:
            g[1].waited_us = min(g[1].waited_us, w)
            g[1].end_us = max(g[1].end_us, e)
            g[1].marks_us = tuple(max(x, y) for x, y in zip(g[1].marks_us, mk))
        if detail:
            g[1].ctas.append((b, w, e) + mk)
        g[0] -= 1
        if g[0] == 0:
            del open_groups[tag]
    return out


class Timeline:
    def __init__(self, device="cuda:0", capacity: int = 1 << 17):
        if not jit.tracing():
            raise KernelError("the kernel timeline needs FELLM_B200_TRACE=1 in the environment before the kernels load")
        self.capacity = capacity
        self.records = torch.zeros(capacity, 8, dtype=torch.int64, device=device)
        self.count = torch.zeros(1, dtype=torch.int32, device=device)
        self._point(self.records.data_ptr(), self.count.data_ptr(), capacity)

    @staticmethod
    def _point(buf: int, count: int, capacity: int):
        import ctypes
        for lib in jit.loaded_libraries():
            fn = getattr(lib, "fellm_set_trace", None)
            if fn is None:
                continue
            fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint]
            fn.restype = ctypes.c_int
            code = fn(buf, count, capacity)
            if code != 0:
                raise KernelError(f"fellm_set_trace: CUDA error {code}")

    def reset(self):
        """Forgets the records so far; libraries loaded since the last call start recording."""
        torch.cuda.synchronize()
        self.count.zero_()
        self._point(self.records.data_ptr(), self.count.data_ptr(), self.capacity)
        torch.cuda.synchronize()

    def close(self):
        torch.cuda.synchronize()
        self._point(0, 0, 0)

    def launches(self, detail: bool = False) -> List[Launch]:
        torch.cuda.synchronize()
        n = min(int(self.count.item()), self.capacity)
        return group_records(self.records[:n].cpu().tolist(), detail)

    @staticmethod
    def phases(launches: List[Launch]) -> str:
        """For launches made with detail=True: what a CTA spends between its own wait and its exit, cut at the
        kernel's marks (medians over the CTAs of all launches of a kernel and grid; marks a CTA did not pass
        are left out).  Which place of a kernel a mark is, the kernel's source says (FELLM_TRACE_MARK)."""
        groups = {}
        for l in launches:
            for c in l.ctas:
                begin, waited, end, marks = c[0], c[1], c[2], c[3:]
                if not any(marks):
                    continue
                g = groups.setdefault((l.name, l.blocks), {})
                prev, label = waited, "wait"
                for k, m in enumerate(marks):
                    if m:
                        g.setdefault(f"{label} -> mark {k}", []).append(m - prev)
                        prev, label = m, f"mark {k}"
                g.setdefault(f"{label} -> exit", []).append(end - prev)
                g.setdefault("wait -> exit", []).append(end - waited)
                g.setdefault("entry -> wait", []).append(waited - begin)
        lines = ["| kernel | CTAs | phase | median us | 90% us | max us |", "|---|---|---|---|---|---|"]
        for (name, blocks), g in groups.items():
            for phase, v in g.items():
                v = sorted(v)
                lines.append(f"| {name} | {blocks} | {phase} | {v[len(v) // 2]:.2f} | {v[int(len(v) * 0.9)]:.2f} | {v[-1]:.2f} |")
        return "\n".join(lines)

    @staticmethod
    def table(launches: List[Launch]) -> str:
        lines = ["| # | kernel | CTAs | begin us | wait us | run us | gap to the one before us |", "|---|---|---|---|---|---|---|"]
        prev_end = None
        for i, l in enumerate(launches):
            gap = "" if prev_end is None else f"{l.begin_us - prev_end:.2f}"
            lines.append(f"| {i} | {l.name} | {l.blocks} | {l.begin_us:.2f} | {l.waited_us - l.begin_us:.2f} | "
                         f"{l.end_us - l.waited_us:.2f} | {gap} |")
            prev_end = l.end_us
        return "\n".join(lines)
