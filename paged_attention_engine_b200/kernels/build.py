"""Builds the CUDA libraries of `csrc/` for sm_100a with nvcc, on first use.

Each kernel family is one `.cu` file and becomes one shared library that `ops.py`
loads with ctypes (the entry points are `extern "C"` and take raw pointers, so no
Python or torch headers are compiled). A library's file name carries a hash of its
sources and flags; it is built when no file of that name exists, in the package's own
`_build/` folder, or under the system's temporary folder when the package cannot be
written to. Only the families that a model asks for are built. Progress lines go to
stderr while nvcc runs.
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
from pathlib import Path

CSRC = Path(__file__).resolve().parent.parent / "csrc"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-shared",
]
# PAE_SPLIT_COMPILE=1 lets nvcc optimise a file's kernels on all cores (the few-token products build in
# 18 s instead of 35). Off by default: the kernels it made were slower on the same GPU in the same
# call (prefill of 2,048 tokens 6.73 to 6.95 ms against 6.52 to 6.53, a decode step 1.046 against 1.018 ms).
if os.environ.get("PAE_SPLIT_COMPILE", "0") == "1":
    NVCC_FLAGS += ["--split-compile", "0"]

# family -> sources (the first is compiled, the others are headers it includes)
FAMILIES: dict[str, list[str]] = {
    "elementwise": ["elementwise.cu", "common.cuh"],
    "gemm_simt": ["gemm_simt.cu", "common.cuh"],
    "attention_simt": ["attention_simt.cu", "common.cuh"],
    "sampling": ["sampling.cu", "common.cuh"],
    "gemm_tcgen05": ["gemm_tcgen05.cu", "tcgen05.cuh", "common.cuh"],
    "gemv_mma": ["gemv_mma.cu", "tcgen05.cuh", "common.cuh"],
    "attention_mma": ["attention_mma.cu", "attention_mma.cuh", "common.cuh"],
    "fused_decode": ["fused_decode.cu", "common.cuh"],
    "attention_tcgen05": ["attention_tcgen05.cu", "common.cuh"],
    "attention_decode_noalloc": [
        "attention_decode_noalloc.cu", "attention_decode_noalloc.h", "attention_mma.cuh", "common.cuh",
    ],
}

# The checked build: `PAE_BOUNDS=1` in the environment compiles every family with -DPAE_BOUNDS
# (slots, block-table indices and page ids are range-checked on the device before they become
# addresses; see csrc/common.cuh). Its libraries carry `checked` in their names and live beside
# the ordinary ones.
BOUNDS = os.environ.get("PAE_BOUNDS", "0") not in ("", "0")

_lock = threading.Lock()


def say(message: str) -> None:
    print(f"[paged_attention_engine_b200] {message}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for candidate in (
        os.environ.get("PAE_NVCC"),
        shutil.which("nvcc"),
        os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
        "/usr/local/cuda/bin/nvcc",
    ):
        if candidate and os.path.isfile(candidate) and os.access(candidate, os.X_OK):
            return candidate
    raise RuntimeError(
        "nvcc was not found (PATH, CUDA_HOME, /usr/local/cuda): the CUDA kernels cannot be built, "
        "and this engine has no other path"
    )


def build_dir() -> Path:
    """The package's own `_build/` when it can be written to, else a per-user temporary folder."""
    own = Path(__file__).resolve().parent.parent / "_build"
    try:
        own.mkdir(exist_ok=True)
        probe = own / f".write_probe_{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return own
    except OSError:
        fallback = Path(tempfile.gettempdir()) / f"paged_attention_engine_b200_build_{os.getuid()}"
        fallback.mkdir(parents=True, exist_ok=True)
        return fallback


def nvcc_flags(bounds: bool | None = None) -> list[str]:
    bounds = BOUNDS if bounds is None else bounds
    return NVCC_FLAGS + (["-DPAE_BOUNDS"] if bounds else [])


def family_hash(name: str, bounds: bool | None = None) -> str:
    digest = hashlib.sha256()
    for source in FAMILIES[name]:
        digest.update(source.encode())
        digest.update((CSRC / source).read_bytes())
    digest.update(" ".join(nvcc_flags(bounds)).encode())
    return digest.hexdigest()[:12]


def _stem(name: str, bounds: bool | None = None) -> str:
    bounds = BOUNDS if bounds is None else bounds
    return f"libpae_{name}_checked" if bounds else f"libpae_{name}"


def library_path(name: str, folder: Path | None = None, bounds: bool | None = None) -> Path:
    return (folder or build_dir()) / f"{_stem(name, bounds)}_{family_hash(name, bounds)}.so"


def _compile(name: str, target: Path, bounds: bool | None = None) -> None:
    nvcc = find_nvcc()
    source = CSRC / FAMILIES[name][0]
    partial = target.with_suffix(f".tmp{os.getpid()}.so")
    command = [nvcc, *nvcc_flags(bounds), "-I", str(CSRC), "-o", str(partial), str(source)]
    say(f"compiling {source.name} for sm_100a ...")
    started = time.time()
    process = subprocess.Popen(command, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    while True:
        try:
            output, _ = process.communicate(timeout=15)
            break
        except subprocess.TimeoutExpired:
            say(f"... still compiling {source.name} ({int(time.time() - started)} s)")
    if process.returncode != 0:
        partial.unlink(missing_ok=True)
        raise RuntimeError(f"nvcc failed on {source.name}:\n{output}")
    os.replace(partial, target)
    for stale in target.parent.glob(f"{_stem(name, bounds)}_????????????.so"):
        if stale != target:
            stale.unlink(missing_ok=True)      # an older build of the same family
    say(f"built {target.name} in {time.time() - started:.0f} s")


def ensure_built(names: list[str], bounds: bool | None = None) -> dict[str, Path]:
    """Paths of the libraries of the given families, compiling those that are missing."""
    with _lock:
        folder = build_dir()
        paths = {n: library_path(n, folder, bounds) for n in names}
        missing = [n for n in names if not paths[n].is_file()]
        if missing:
            errors: list[BaseException] = []

            def work(n: str) -> None:
                try:
                    _compile(n, paths[n], bounds)
                except BaseException as exc:  # noqa: BLE001  (reported below)
                    errors.append(exc)

            threads = [threading.Thread(target=work, args=(n,)) for n in missing]
            for t in threads:
                t.start()
            for t in threads:
                t.join()
            if errors:
                raise errors[0]
        return paths


def build_all(bounds: bool | None = None) -> dict[str, Path]:
    return ensure_built(list(FAMILIES), bounds)
