"""Builds the CUDA sources of this folder into one shared library for sm_100a.

The library has a plain C interface and is loaded with ``ctypes``; nothing here
needs the PyTorch C++ headers, so a cold build takes seconds per file.  Objects
and the library live in ``_build/`` beside the sources; if that folder cannot be
written the build goes to ``$TOKAMAK_B200_BUILD_DIR`` or to a per-user folder
under the system's temporary directory.  A stamp of the sources' hashes decides
whether anything has to be compiled again.
"""

from __future__ import annotations

import hashlib
import json
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

SOURCE_DIR = Path(__file__).resolve().parent
LIB_NAME = "libtokamak_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


# extra compiler flags, e.g. -DTK_TIMELINE (see timeline.cuh); they are part of the stamp
EXTRA_FLAGS = os.environ.get("TOKAMAK_B200_NVCC_FLAGS", "").split()


class BuildError(RuntimeError):
    """The CUDA extension could not be compiled."""


def _log(msg: str) -> None:
    print(f"[tokamak_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("TOKAMAK_B200_NVCC"), shutil.which("nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc was not found (set TOKAMAK_B200_NVCC or put it on PATH); "
                     "the engine has no path without its CUDA kernels")


def sources() -> list[Path]:
    return sorted(SOURCE_DIR.glob("*.cu"))


def _source_stamp() -> str:
    h = hashlib.sha256()
    for path in sorted(list(SOURCE_DIR.glob("*.cu")) + list(SOURCE_DIR.glob("*.cuh")) + list(SOURCE_DIR.glob("*.h"))):
        h.update(path.name.encode())
        h.update(path.read_bytes())
    h.update(" ".join(NVCC_FLAGS + EXTRA_FLAGS).encode())
    return h.hexdigest()


def _writable_dir(path: Path) -> bool:
    try:
        path.mkdir(parents=True, exist_ok=True)
        probe = path / f".probe_{os.getpid()}"
        probe.write_text("x")
        probe.unlink()
        return True
    except OSError:
        return False


def build_dir() -> Path:
    env = os.environ.get("TOKAMAK_B200_BUILD_DIR")
    candidates = [Path(env)] if env else []
    candidates.append(SOURCE_DIR / "_build")
    candidates.append(Path(tempfile.gettempdir()) / f"tokamak_b200_build_{os.getuid()}")
    for cand in candidates:
        if _writable_dir(cand):
            return cand
    raise BuildError(f"no writable build folder among {[str(c) for c in candidates]}")


def _up_to_date(folder: Path, stamp: str) -> bool:
    stamp_file = folder / "stamp.json"
    lib = folder / LIB_NAME
    if not (stamp_file.is_file() and lib.is_file()):
        return False
    try:
        return json.loads(stamp_file.read_text()).get("sources") == stamp
    except (OSError, ValueError):
        return False


def _compile_one(nvcc: str, src: Path, obj: Path, verbose_ptxas: bool) -> str:
    cmd = [nvcc, *NVCC_FLAGS, *EXTRA_FLAGS, "-I", str(SOURCE_DIR), "-c", str(src), "-o", str(obj)]
    if verbose_ptxas:
        cmd[1:1] = ["-Xptxas", "-v"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError(f"nvcc failed on {src.name}:\n{proc.stdout}\n{proc.stderr}")
    return proc.stderr


def ensure_built(force: bool = False, verbose_ptxas: bool = False) -> Path:
    """Compile what is stale and return the path of the shared library."""
    stamp = _source_stamp()
    in_tree = SOURCE_DIR / "_build"
    if not force and _up_to_date(in_tree, stamp):
        return in_tree / LIB_NAME
    folder = build_dir()
    if not force and _up_to_date(folder, stamp):
        return folder / LIB_NAME

    nvcc = find_nvcc()
    srcs = sources()
    _log(f"compiling {len(srcs)} CUDA sources for sm_100a into {folder} (first call only)")
    t0 = time.time()
    objs = [folder / (s.stem + ".o") for s in srcs]
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        futures = {pool.submit(_compile_one, nvcc, s, o, verbose_ptxas): s for s, o in zip(srcs, objs)}
        pending = set(futures)
        while pending:
            finished = {f for f in pending if f.done()}
            for f in finished:
                out = f.result()
                _log(f"  compiled {futures[f].name} ({time.time() - t0:.0f}s)")
                if verbose_ptxas and out:
                    print(out, file=sys.stderr)
            pending -= finished
            if pending:
                time.sleep(0.5)
                if int(time.time() - t0) % 10 == 0 and not finished:
                    _log(f"  still compiling {len(pending)} file(s) ({time.time() - t0:.0f}s)")
                    time.sleep(1.0)
    tmp_lib = folder / (LIB_NAME + f".tmp{os.getpid()}")
    link = [nvcc, "-shared", "-o", str(tmp_lib), *[str(o) for o in objs]]
    proc = subprocess.run(link, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    os.replace(tmp_lib, folder / LIB_NAME)
    (folder / "stamp.json").write_text(json.dumps({"sources": stamp}))
    _log(f"built {LIB_NAME} in {time.time() - t0:.0f}s")
    return folder / LIB_NAME


if __name__ == "__main__":
    print(ensure_built(force="--force" in sys.argv, verbose_ptxas="--ptxas" in sys.argv))
