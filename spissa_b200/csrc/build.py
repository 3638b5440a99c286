"""Compiles the CUDA sources of this folder for sm_100a into shared libraries.

One library per source file, named after a hash of the source, the shared headers
and the flags, so a changed file is rebuilt and an unchanged one is reused. The
libraries land in ``csrc/_build`` inside the package (or, when that is not
writable, in ``$SPISSA_B200_BUILD_DIR`` or a per-user folder under the system's
temporary directory). Only ``nvcc`` is needed: the libraries export plain C
functions and are loaded with ``ctypes``.
"""
from __future__ import annotations

import atexit
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

CSRC = Path(__file__).resolve().parent
HEADERS = ["common.cuh", "async_copy.cuh", "tcgen05.cuh", "flash_common.cuh", "attention_noalloc.h"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo", "--shared",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]
# The debug build: every kernel that takes an index from a table the host packed checks it against the bounds the
# host declares, records a code in the status word and leaves the access out (see common.cuh). It is a separate set
# of libraries (the flag is part of their names' hash), chosen for a whole process by SPISSA_B200_RANGE_CHECK=1.
RANGE_CHECK_FLAG = "-DSP_RANGE_CHECK"


def range_check_enabled() -> bool:
    return os.environ.get("SPISSA_B200_RANGE_CHECK", "") not in ("", "0")


def flags(range_check=None) -> list:
    on = range_check_enabled() if range_check is None else bool(range_check)
    return NVCC_FLAGS + ([RANGE_CHECK_FLAG] if on else [])


# module name -> source file
MODULES = {
    "generic": "generic_kernels.cu",
    "sampling": "sampling_kernels.cu",
    "tc_gemm": "tc_gemm.cu",
    "attention": "attention_kernels.cu",
    "gemv": "gemv_kernels.cu",
    "flash_tc": "flash_tc.cu",
    "decode_layers": "decode_layers.cu",
    "tc_stream": "tc_stream.cu",
    "host_step": "host_step.cu",
}


class BuildError(RuntimeError):
    pass


_say_lock = threading.Lock()


def _say(msg: str) -> None:
    with _say_lock:                                    # builds run side by side: one line at a time
        sys.stderr.write(f"[spissa_b200] {msg}\n")
        sys.stderr.flush()


def find_nvcc() -> str:
    cand = [os.environ.get("SPISSA_B200_NVCC"), shutil.which("nvcc"),
            os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
            "/usr/local/cuda/bin/nvcc"]
    for c in cand:
        if c and os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    raise BuildError("nvcc was not found (looked at $SPISSA_B200_NVCC, PATH, $CUDA_HOME/bin, "
                     "/usr/local/cuda/bin); the CUDA kernels cannot be built")


def _writable_dir(p: Path) -> bool:
    try:
        p.mkdir(parents=True, exist_ok=True)
        probe = p / f".probe_{os.getpid()}"
        probe.write_bytes(b"")
        probe.unlink()
        return True
    except OSError:
        return False


def build_dir() -> Path:
    env = os.environ.get("SPISSA_B200_BUILD_DIR")
    if env and _writable_dir(Path(env)):
        return Path(env)
    local = CSRC / "_build"
    if _writable_dir(local):
        return local
    fallback = Path(tempfile.gettempdir()) / f"spissa_b200_build_{os.getuid()}"
    if _writable_dir(fallback):
        return fallback
    raise BuildError(f"no writable folder for built kernels (tried {local} and {fallback})")


def _digest(source: str, range_check=None) -> str:
    h = hashlib.sha256()
    for name in [source] + HEADERS:
        h.update(name.encode())
        h.update((CSRC / name).read_bytes())
    h.update(" ".join(flags(range_check)).encode())
    return h.hexdigest()[:16]


def _stem(module: str, range_check=None) -> str:
    on = range_check_enabled() if range_check is None else bool(range_check)
    return f"libspissa_{module}_" + ("checked_" if on else "")


def library_path(module: str, folder: Path | None = None, range_check=None) -> Path:
    source = MODULES[module]
    return (folder or build_dir()) / f"{_stem(module, range_check)}{_digest(source, range_check)}.so"


def find_built(module: str, range_check=None) -> Path | None:
    """An up-to-date library of ``module`` in any of the known folders, if there is one."""
    name = f"{_stem(module, range_check)}{_digest(MODULES[module], range_check)}.so"
    folders = [CSRC / "_build", Path(tempfile.gettempdir()) / f"spissa_b200_build_{os.getuid()}"]
    env = os.environ.get("SPISSA_B200_BUILD_DIR")
    if env:
        folders.insert(0, Path(env))
    for f in folders:
        if (f / name).is_file():
            return f / name
    return None


# Builds started ahead of their first use (``prefetch``): a model's first step needs several libraries one after the
# other, each ten seconds or more of nvcc; started together they take as long as the slowest.
_background: dict = {}             # (module, debug build?) -> the thread that builds it
_background_lock = threading.Lock()
_compilers: list = []              # nvcc processes in flight (ended with this process, should it leave first)


def _end_compilers() -> None:
    for proc in list(_compilers):
        if proc.poll() is None:
            proc.kill()


atexit.register(_end_compilers)


def prefetch(modules, verbose: bool = True, range_check=None) -> None:
    """Start building, in the background, those of ``modules`` that have no up-to-date library yet. ``build_module``
    waits for a build in flight instead of starting a second one; a build that fails here fails again, loudly, there."""
    on = range_check_enabled() if range_check is None else bool(range_check)
    for module in modules:
        if module not in MODULES:
            continue
        with _background_lock:
            if (module, on) in _background or find_built(module, on) is not None:
                continue

            def work(m=module):
                try:
                    build_module(m, verbose, range_check=on)
                except Exception:
                    pass

            t = threading.Thread(target=work, name=f"spissa-build-{module}", daemon=True)
            _background[(module, on)] = t
            t.start()


def build_module(module: str, verbose: bool = True, extra_flags=(), range_check=None) -> Path:
    """Compile ``module`` if no up-to-date library exists; return the library's path. ``range_check`` None: as the
    environment says (the regular build unless SPISSA_B200_RANGE_CHECK=1)."""
    if module not in MODULES:
        raise BuildError(f"unknown kernel module {module!r}; known: {sorted(MODULES)}")
    on = range_check_enabled() if range_check is None else bool(range_check)
    ahead = _background.get((module, on))
    if ahead is not None and ahead is not threading.current_thread():
        ahead.join()                                   # started ahead of its use: wait for it rather than build twice
    have = find_built(module, range_check)
    if have is not None:
        return have
    out = library_path(module, None, range_check)
    nvcc = find_nvcc()
    tmp = out.with_suffix(f".tmp{os.getpid()}_{threading.get_ident()}.so")
    cmd = [nvcc] + flags(range_check) + list(extra_flags) + ["-I", str(CSRC), "-o", str(tmp), str(CSRC / MODULES[module])]
    if verbose:
        kind = " (debug build with range checks)" if RANGE_CHECK_FLAG in cmd else ""
        _say(f"compiling {MODULES[module]} for sm_100a{kind} (first use) ...")
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                            env=dict(os.environ, TMPDIR=str(out.parent)))
    _compilers.append(proc)
    last = t0
    while True:
        try:
            log, _ = proc.communicate(timeout=5)
            break
        except subprocess.TimeoutExpired:
            if verbose and time.time() - last >= 10:
                _say(f"  still compiling {MODULES[module]} ({time.time() - t0:.0f} s)")
                last = time.time()
    _compilers.remove(proc)
    if proc.returncode != 0:
        try:
            tmp.unlink()
        except OSError:
            pass
        raise BuildError(f"nvcc failed on {MODULES[module]}:\n{log}")
    os.replace(tmp, out)
    checked = "_checked_" in out.name
    for old in out.parent.glob(f"libspissa_{module}_*.so"):
        if old != out and ("_checked_" in old.name) == checked:
            try:
                old.unlink()
            except OSError:
                pass
    if verbose:
        _say(f"built {out.name} in {time.time() - t0:.1f} s")
    return out


def build_all(verbose: bool = True, range_check=None) -> dict:
    prefetch(MODULES, verbose, range_check)            # side by side
    return {m: build_module(m, verbose, range_check=range_check) for m in MODULES}


if __name__ == "__main__":
    for m, p in build_all().items():
        print(m, p)
