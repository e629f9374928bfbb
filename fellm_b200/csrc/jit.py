"""Compiles the CUDA modules of this folder for sm_100a with nvcc and loads them with ctypes.

Each `<name>.cu` is one shared library with `extern "C"` launchers that take raw device pointers
and a stream.  A module is compiled the first time something needs it (a model asks for the
modules of its own parts, with its own specialisations as -D defines), into `_build/` beside the
sources, keyed by a hash of the sources, the defines and the flags.  While nvcc runs, a line is
printed to stderr every few seconds.  There is no fallback: a missing compiler or a failed build
raises KernelError.

FeLLM loads its kernels as a prebuilt plugin library through a C ABI
(crates/fellm-plugin-host, plugins/cuda_kernels/src/lib.rs:246-261 picks the sm target).
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import re
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import Dict, Iterable, Optional, Tuple

from ..config.errors import KernelError

CSRC = Path(__file__).resolve().parent
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "--shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]

_loaded: Dict[Tuple[str, Tuple], ctypes.CDLL] = {}
_lock = threading.Lock()
_print_lock = threading.Lock()
_dir_lock = threading.Lock()


def _say(msg: str):
    with _print_lock:
        print(f"[fellm_b200] {msg}", file=sys.stderr, flush=True)


def _nvcc() -> str:
    for cand in (os.environ.get("FELLM_B200_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise KernelError("nvcc not found: the CUDA kernels cannot be built (set FELLM_B200_NVCC)")


_build_dir: Optional[Path] = None


def build_dir() -> Path:
    """`_build/` beside the sources when it can be written, else a per-user folder under the
    system's temporary directory (FELLM_B200_BUILD_DIR overrides both).  Chosen once."""
    global _build_dir
    if _build_dir is None:
        with _dir_lock:
            if _build_dir is None:
                _build_dir = _choose_build_dir()
    return _build_dir


def _choose_build_dir() -> Path:
    env = os.environ.get("FELLM_B200_BUILD_DIR")
    cands = [Path(env)] if env else []
    cands += [CSRC / "_build", Path(tempfile.gettempdir()) / f"fellm_b200_build_{os.getuid()}"]
    for d in cands:
        try:
            d.mkdir(parents=True, exist_ok=True)
            probe = d / f".w{os.getpid()}_{threading.get_ident()}"
            probe.write_text("")
            probe.unlink()
            return d
        except OSError:
            continue
    raise KernelError(f"no writable folder for built kernels (tried {', '.join(map(str, cands))})")


def tracing() -> bool:
    """FELLM_B200_TRACE=1 builds every module with the kernel timeline compiled in (separate
    libraries, tagged by the define)."""
    return os.environ.get("FELLM_B200_TRACE", "") == "1"


def _defines_key(defines: Optional[dict]) -> Tuple:
    d = dict(defines or {})
    if tracing():
        d["FELLM_TRACE"] = 1
    for item in filter(None, os.environ.get("FELLM_B200_DEFINES", "").split(",")):      # experiments: NAME=VALUE,...
        k, _, v = item.partition("=")
        d[k] = v or "1"
    return tuple(sorted((str(k), str(v)) for k, v in d.items()))


def loaded_libraries():
    return list(_loaded.values())


def _source_hash(name: str, dkey: Tuple) -> str:
    h = hashlib.sha1()
    src = CSRC / f"{name}.cu"
    if not src.exists():
        raise KernelError(f"no kernel source {src}")
    text = src.read_bytes()
    h.update(text)
    for inc in sorted(set(re.findall(rb'#include\s+"([^"]+\.(?:cu|h))"', text))):      # sources a module pulls in
        f = CSRC / inc.decode()
        if f.exists():
            h.update(inc)
            h.update(f.read_bytes())
    for hdr in sorted(CSRC.glob("*.cuh")):
        h.update(hdr.name.encode())
        h.update(hdr.read_bytes())
    h.update(repr(dkey).encode())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _stem(name: str, dkey: Tuple) -> str:
    tag = "".join(f"_{k}{v}" for k, v in dkey)
    return f"fellm_{name}{re.sub(r'[^A-Za-z0-9_]', '', tag)}"


def library_path(name: str, defines: Optional[dict] = None) -> Path:
    dkey = _defines_key(defines)
    return build_dir() / f"{_stem(name, dkey)}-{_source_hash(name, dkey)}.so"


def compile_module(name: str, defines: Optional[dict] = None, verbose_ptxas: bool = False) -> Path:
    """Builds the module if its library is not there yet; returns the library's path."""
    dkey = _defines_key(defines)
    out = library_path(name, defines)
    if out.exists():
        return out
    tmp = out.with_suffix(f".tmp{os.getpid()}_{threading.get_ident()}.so")
    cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(CSRC)]
    cmd += [f"-D{k}={v}" for k, v in dkey]
    if verbose_ptxas:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", str(tmp), str(CSRC / f"{name}.cu")]
    label = name + ("" if not dkey else " [" + " ".join(f"{k}={v}" for k, v in dkey) + "]")
    _say(f"compiling {label} for sm_100a ...")
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def ticker():
        while not done.wait(10.0):
            _say(f"  still compiling {label} ({time.time() - t0:.0f} s)")
    th = threading.Thread(target=ticker, daemon=True)
    th.start()
    try:
        log, _ = proc.communicate()
    finally:
        done.set()
    if proc.returncode != 0 or not tmp.exists():
        try:
            tmp.unlink()
        except OSError:
            pass
        raise KernelError(f"nvcc failed for {label} (exit {proc.returncode}):\n{log}")
    os.replace(tmp, out)
    for old in out.parent.glob(f"{_stem(name, dkey)}-*.so"):      # libraries of earlier versions of these sources
        if old != out and re.fullmatch(rf"{re.escape(_stem(name, dkey))}-[0-9a-f]{{16}}\.so", old.name):
            try:
                old.unlink()
            except OSError:
                pass
    _say(f"compiled {label} in {time.time() - t0:.1f} s")
    if verbose_ptxas:
        _say(log)
    return out


def load_module(name: str, defines: Optional[dict] = None) -> ctypes.CDLL:
    key = (name, _defines_key(defines))
    lib = _loaded.get(key)
    if lib is not None:
        return lib
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            path = compile_module(name, defines)
            try:
                lib = ctypes.CDLL(str(path))
            except OSError as e:
                raise KernelError(f"cannot load {path}: {e}") from None
            _loaded[key] = lib
    return lib


def compile_many(mods: Iterable[Tuple[str, Optional[dict]]], jobs: Optional[int] = None):
    """Compiles several modules side by side (nvcc is single-threaded per file)."""
    todo, seen = [], set()
    for name, defines in mods:
        key = (name, _defines_key(defines))
        if key in seen or key in _loaded:
            continue
        seen.add(key)
        if not library_path(name, defines).exists():
            todo.append((name, defines))
    if not todo:
        return
    jobs = jobs or min(len(todo), os.cpu_count() or 2, 8)
    with ThreadPoolExecutor(max_workers=jobs) as pool:
        for f in [pool.submit(compile_module, n, d) for n, d in todo]:
            f.result()


def all_modules():
    return sorted(p.stem for p in CSRC.glob("*.cu"))
