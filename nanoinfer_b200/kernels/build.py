"""Building the native code: one shared library per .cu file (CUDA kernels, nvcc) and per .cpp
file (host-side runtime, the C++ compiler) of ``csrc``.

Each CUDA library is compiled for sm_100a with nvcc at its first use (or ahead of time by
``build_all``) into ``csrc/_build`` inside the package, or, when that folder cannot be
written, into ``$NANOINFER_B200_BUILD_DIR`` or a per-user folder under the system's
temporary directory.  A library is rebuilt when its source, a shared header or the
flags change.  While nvcc runs, a line is printed every few seconds.

There is no fallback: a missing library that cannot be built is an error.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from typing import Dict, Iterable, List, Optional

CSRC_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")

NVCC_FLAGS = ["-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "-Xcompiler", "-fPIC", "-shared"]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-Wall"]

_lock = threading.Lock()


class KernelBuildError(RuntimeError):
    pass


def module_names() -> List[str]:
    return sorted(os.path.splitext(f)[0] for f in os.listdir(CSRC_DIR) if f.endswith((".cu", ".cpp")))


def _source_file(module: str) -> str:
    """``module``.cu (a CUDA library) or ``module``.cpp (host code)."""
    for ext in (".cu", ".cpp"):
        if os.path.isfile(os.path.join(CSRC_DIR, module + ext)):
            return module + ext
    raise KernelBuildError(f"no source '{module}.cu' or '{module}.cpp' in {CSRC_DIR}")


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f".probe_{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return True
    except OSError:
        return False


_build_dir_cache: Optional[str] = None


def build_dir() -> str:
    global _build_dir_cache
    if _build_dir_cache:
        return _build_dir_cache
    candidates = []
    if os.environ.get("NANOINFER_B200_BUILD_DIR"):
        candidates.append(os.environ["NANOINFER_B200_BUILD_DIR"])
    candidates.append(os.path.join(CSRC_DIR, "_build"))
    candidates.append(os.path.join(tempfile.gettempdir(), f"nanoinfer_b200_build_{os.getuid()}"))
    for c in candidates:
        if _writable_dir(c):
            _build_dir_cache = c
            return c
    raise KernelBuildError("no writable folder for the compiled kernels; tried " + ", ".join(candidates))


def _find_cxx() -> Optional[str]:
    for c in (os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++"), shutil.which("clang++")):
        if c and os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    return None


def _find_nvcc() -> Optional[str]:
    for c in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if c and os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    return None


def _source_hash(module: str) -> str:
    h = hashlib.sha256()
    src = _source_file(module)
    h.update(" ".join(NVCC_FLAGS if src.endswith(".cu") else CXX_FLAGS).encode())
    names = [src] + sorted(f for f in os.listdir(CSRC_DIR) if f.endswith((".cuh", ".h")))
    for n in names:
        with open(os.path.join(CSRC_DIR, n), "rb") as f:
            h.update(n.encode())
            h.update(f.read())
    return h.hexdigest()


def library_path(module: str) -> str:
    return os.path.join(build_dir(), f"libni_{module}.so")


def _is_current(module: str) -> bool:
    lib = library_path(module)
    stamp = lib + ".hash"
    if not (os.path.isfile(lib) and os.path.isfile(stamp)):
        return False
    with open(stamp, "r") as f:
        return f.read().strip() == _source_hash(module)


def _compile(module: str, log) -> None:
    src = _source_file(module)
    lib = library_path(module)
    tmp = f"{lib}.tmp{os.getpid()}_{threading.get_ident()}"
    if src.endswith(".cu"):
        nvcc = _find_nvcc()
        if nvcc is None:
            raise KernelBuildError(f"the CUDA library for '{module}' is not built and nvcc was not found "
                                   f"(set NVCC or put nvcc on PATH); there is no fallback path")
        cmd = [nvcc] + NVCC_FLAGS + ["-I", CSRC_DIR, "-o", tmp, os.path.join(CSRC_DIR, src)]
    else:
        cxx = _find_cxx()
        if cxx is None:
            raise KernelBuildError(f"the host library for '{module}' is not built and no C++ compiler was found "
                                   f"(set CXX or put g++ on PATH); there is no fallback path")
        cmd = [cxx] + CXX_FLAGS + ["-I", CSRC_DIR, "-o", tmp, os.path.join(CSRC_DIR, src)]
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, cwd=build_dir())
    last = t0
    while True:
        try:
            out, _ = proc.communicate(timeout=1.0)
            break
        except subprocess.TimeoutExpired:
            if time.time() - last >= 5.0:
                last = time.time()
                log(f"[nanoinfer_b200] compiling {src} ... {last - t0:.0f} s")
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise KernelBuildError(f"{cmd[0]} failed on {src}:\n{out.decode(errors='replace')}")
    os.replace(tmp, lib)
    with open(lib + ".hash", "w") as f:
        f.write(_source_hash(module))
    log(f"[nanoinfer_b200] compiled {src} in {time.time() - t0:.1f} s")


def _log(msg: str) -> None:
    print(msg, file=sys.stderr, flush=True)


def ensure_built(modules: Iterable[str], log=_log) -> Dict[str, str]:
    """Compile what is missing or stale among ``modules`` (in parallel); return their paths."""
    modules = list(dict.fromkeys(modules))
    known = set(module_names())
    for m in modules:
        if m not in known:
            raise KernelBuildError(f"no source '{m}.cu' or '{m}.cpp' in {CSRC_DIR}")
    with _lock:
        todo = [m for m in modules if not _is_current(m)]
        if todo:
            log(f"[nanoinfer_b200] compiling {len(todo)} file(s) (CUDA for sm_100a, host C++): {', '.join(todo)}")
            errors: List[BaseException] = []

            def work(m):
                try:
                    _compile(m, log)
                except BaseException as e:  # noqa: BLE001 (re-raised below)
                    errors.append(e)

            threads = [threading.Thread(target=work, args=(m,)) for m in todo]
            for i in range(0, len(threads), max(1, os.cpu_count() or 1)):
                batch = threads[i:i + max(1, os.cpu_count() or 1)]
                for t in batch:
                    t.start()
                for t in batch:
                    t.join()
            if errors:
                raise errors[0]
    return {m: library_path(m) for m in modules}


def build_all(log=_log) -> Dict[str, str]:
    return ensure_built(module_names(), log)
