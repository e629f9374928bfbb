"""Drives bin/trace_run as a user would: a subprocess, steps on standard input, logits from files."""
from __future__ import annotations

import json
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent


def run_trace(folder, dtype, max_tokens, steps, vocab, page_tokens=None, timeout=600):
    """steps: list of dicts {"entries": [...], "end": [...]} (numbered here).  Returns
    {step: float32 tensor [wanted, vocab]}."""
    out = tempfile.mkdtemp(prefix="fellm_trace_")
    cmd = [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
           "--out", out, "--max-tokens", str(max_tokens)]
    if page_tokens:
        cmd += ["--page-tokens", str(page_tokens)]
    lines = []
    for i, st in enumerate(steps):
        lines.append(json.dumps({"step": i, "entries": st.get("entries", []), "end": st.get("end", [])}))
    proc = subprocess.run(cmd, input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=timeout)
    assert proc.returncode == 0, f"trace_run failed ({proc.returncode}):\n{proc.stderr[-3000:]}"
    done = [l for l in proc.stdout.splitlines() if l.startswith("done ")]
    assert done == [f"done {i}" for i in range(len(steps))], proc.stdout[-2000:]
    res = {}
    for i, st in enumerate(steps):
        wanted = sum(len(e.get("want", [])) for e in st.get("entries", []))
        f = Path(out) / f"{i}.f32"
        if wanted:
            a = np.fromfile(f, dtype="<f4")
            assert a.size == wanted * vocab, (i, a.size, wanted, vocab)
            res[i] = torch.from_numpy(a.reshape(wanted, vocab).copy())
        else:
            assert not f.exists()
    return res


def collect(steps, results):
    """{request id: {position: logits row}} from a trace and its results."""
    pos = {}
    out = {}
    for i, st in enumerate(steps):
        row = 0
        for e in st.get("entries", []):
            p0 = pos.get(e["id"], 0)
            for w in e.get("want", []):
                out.setdefault(e["id"], {})[p0 + w] = results[i][row]
                row += 1
            pos[e["id"]] = p0 + len(e["tokens"])
        for rid in st.get("end", []):
            pos.pop(rid, None)
    return out
