"""Compiles the CUDA sources of this package for sm_100a and loads them.

Kernels are grouped in *modules*, each a shared library with a plain C ABI
that Python calls through ctypes.  A module is compiled the first time it is
asked for (so a model only pays for the kernels and head sizes it uses) into
``infernum_b200/csrc/_build/`` - or, when the package folder is not writable,
into a per-user folder under the temporary directory.  The file name carries a
hash of the sources and flags, so an edited source is rebuilt and a stale
library is never loaded.  While nvcc runs, a line is printed every few seconds.
"""

from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, List, Sequence, Tuple

from ..errors import KernelError

CSRC_DIR = os.path.dirname(os.path.abspath(__file__))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler",
              "-fvisibility=hidden", "--expt-relaxed-constexpr"]

# More nvcc flags for every module, e.g. "-DNAME=1 -Xptxas -v" (they are part of a library's name)
EXTRA_FLAGS = os.environ.get("INFERNUM_NVCC_FLAGS", "").split()

_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


def _log(msg: str) -> None:
    print(f"[infernum_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("INFERNUM_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise KernelError(
        "nvcc was not found (looked at $INFERNUM_NVCC, PATH, $CUDA_HOME/bin and "
        "/usr/local/cuda/bin); the CUDA kernels of infernum_b200 cannot be built"
    )


def build_dir() -> str:
    """Where libraries go: in the source tree when it can be written."""
    override = os.environ.get("INFERNUM_BUILD_DIR")
    candidates = [override] if override else []
    candidates.append(os.path.join(CSRC_DIR, "_build"))
    candidates.append(os.path.join(tempfile.gettempdir(), f"infernum_b200_build_{os.getuid()}"))
    for cand in candidates:
        try:
            os.makedirs(cand, exist_ok=True)
            # a name of its own for every caller: modules are built from several threads
            fd, probe = tempfile.mkstemp(prefix=".probe_", dir=cand)
            os.close(fd)
            os.remove(probe)
            return cand
        except OSError:
            continue
    raise KernelError("no writable folder for the compiled kernels: tried " + ", ".join(candidates))


def _hash_module(sources: Sequence[str], defines: Sequence[str], nvcc: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS + list(defines) + EXTRA_FLAGS).encode())
    try:
        h.update(subprocess.run([nvcc, "--version"], capture_output=True, check=True).stdout)
    except (OSError, subprocess.CalledProcessError):
        pass
    headers = sorted(f for f in os.listdir(CSRC_DIR) if f.endswith((".cuh", ".h")))
    for name in list(sources) + headers:
        with open(os.path.join(CSRC_DIR, name), "rb") as fh:
            h.update(name.encode())
            h.update(fh.read())
    return h.hexdigest()[:16]


def _run_with_heartbeat(cmds: List[Tuple[str, List[str]]], what: str) -> None:
    """Run commands in parallel, print a line every few seconds meanwhile."""
    start = time.time()
    errors: List[str] = []

    def run(item):
        label, cmd = item
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            errors.append(f"{label}: {' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")

    workers = max(1, min(len(cmds), os.cpu_count() or 1))
    with ThreadPoolExecutor(max_workers=workers) as pool:
        futures = [pool.submit(run, c) for c in cmds]
        last_print = start
        while True:
            pending = [f for f in futures if not f.done()]
            if not pending:
                break
            time.sleep(0.2)
            if time.time() - last_print >= 5:
                last_print = time.time()
                _log(f"{what}: still compiling, {len(pending)} of {len(cmds)} file(s) left, "
                     f"{time.time() - start:.0f} s")
        for f in futures:
            f.result()
    if errors:
        raise KernelError("nvcc failed:\n" + "\n".join(errors))


def compile_module(name: str, sources: Sequence[str], defines: Sequence[str] = (),
                   verbose: bool = True) -> str:
    """Build (if needed) the shared library of a module and return its path."""
    nvcc = find_nvcc()
    out_dir = build_dir()
    tag = _hash_module(sources, defines, nvcc)
    lib_path = os.path.join(out_dir, f"libib200_{name}_{tag}.so")
    if os.path.isfile(lib_path):
        return lib_path
    if verbose:
        _log(f"compiling kernel module '{name}' for sm_100a ({len(sources)} file(s)) -> {lib_path}")
    start = time.time()
    work = tempfile.mkdtemp(prefix=f"{name}_", dir=out_dir)
    try:
        objs, cmds = [], []
        for src in sources:
            obj = os.path.join(work, os.path.splitext(src)[0] + ".o")
            objs.append(obj)
            cmds.append((src, [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, *defines, *EXTRA_FLAGS, "-I", CSRC_DIR, "-c",
                               os.path.join(CSRC_DIR, src), "-o", obj]))
        _run_with_heartbeat(cmds, name)
        tmp_lib = os.path.join(work, "lib.so")
        _run_with_heartbeat(
            [("link", [nvcc, *ARCH_FLAGS, "-shared", "-o", tmp_lib, *objs, "-lcudart_static",
                       "-lpthread", "-ldl", "-lrt"])], name)
        os.replace(tmp_lib, lib_path)
    finally:
        shutil.rmtree(work, ignore_errors=True)
    if verbose:
        _log(f"module '{name}' built in {time.time() - start:.1f} s")
    return lib_path


def load_module(name: str, sources: Sequence[str], defines: Sequence[str] = ()) -> ctypes.CDLL:
    key = name + "|" + " ".join(defines)
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            path = compile_module(name, sources, defines)
            try:
                lib = ctypes.CDLL(path)
            except OSError as exc:
                raise KernelError(f"cannot load {path}: {exc}") from exc
            lib._ib_path = path
            serial = os.environ.get("INFERNUM_PDL", "1") == "0" or os.environ.get("INFERNUM_PROFILE", "0") not in ("", "0")
            if serial and hasattr(lib, "ib_set_pdl"):
                lib.ib_set_pdl(0)  # launch every kernel strictly after its predecessor
            _loaded[key] = lib
        return lib


def loaded_libraries() -> List[str]:
    return [lib._ib_path for lib in _loaded.values()]
