"""Builds the kernel library (``libtokenomos_b200.so``) from the ``.cu`` files beside this file.

The library is compiled with ``nvcc`` for sm_100a only, one object per source in parallel, and
kept in ``_build/<hash of the sources and flags>/`` beside the sources (or, when that folder
cannot be written, under the system's temporary folder, per user). A fresh checkout compiles at
its first use and says so on stderr now and then; after that the hash finds the finished
library. Nothing here falls back to another implementation: no compiler, no library.
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
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB_NAME = "libtokenomos_b200.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC"]


class BuildError(RuntimeError):
    pass


def sources() -> list[Path]:
    return sorted(HERE.glob("*.cu"))


def _headers() -> list[Path]:
    return sorted(list(HERE.glob("*.cuh")) + list(HERE.glob("*.h")))


def find_nvcc() -> str:
    for root in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if root and (Path(root) / "bin" / "nvcc").exists():
            return str(Path(root) / "bin" / "nvcc")
    found = shutil.which("nvcc")
    if found:
        return found
    raise BuildError(
        "nvcc not found (looked in $CUDA_HOME, /usr/local/cuda and PATH): the CUDA kernels of "
        "tokenomos_b200 cannot be compiled, and there is no other implementation to fall back to"
    )


def source_hash() -> str:
    h = hashlib.sha256()
    for p in sources() + _headers():
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _writable(folder: Path) -> bool:
    try:
        folder.mkdir(parents=True, exist_ok=True)
        probe = folder / f".probe-{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return True
    except OSError:
        return False


def build_root() -> Path:
    """Where built libraries live: beside the sources if possible, else a per-user temp folder."""
    override = os.environ.get("TOKENOMOS_B200_BUILD_DIR")
    if override:
        return Path(override)
    local = HERE / "_build"
    if _writable(local):
        return local
    return Path(tempfile.gettempdir()) / f"tokenomos_b200-build-{os.getuid()}"


def checks_wanted() -> bool:
    """``TOKENOMOS_B200_CHECKS=1``: the debug build whose kernels check every index they follow
    into a pool (checks.cuh)."""
    return os.environ.get("TOKENOMOS_B200_CHECKS", "0") == "1"


def library_path(checks: bool | None = None) -> Path:
    """Path of the library for the current sources (it may not exist yet); the build with
    index checks lives beside the plain one."""
    checks = checks_wanted() if checks is None else checks
    tag = source_hash() + ("-checks" if checks else "")
    local = HERE / "_build" / tag / LIB_NAME
    if local.exists():
        return local
    return build_root() / tag / LIB_NAME


def _say(msg: str) -> None:
    print(f"[tokenomos_b200] {msg}", file=sys.stderr, flush=True)


def _compile(nvcc: str, src: Path, obj: Path, verbose: bool, checks: bool = False) -> None:
    cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, *(["-DTK_CHECKS"] if checks else []), "-I", str(HERE), "-c",
           str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError(f"nvcc failed on {src.name}:\n{proc.stderr[-4000:]}")
    if verbose and proc.stderr:
        _say(f"{src.name}:\n{proc.stderr}")


def build(force: bool = False, verbose: bool = False, checks: bool | None = None) -> Path:
    """Compile if needed and return the library's path. ``checks``: the debug build with index
    checks (default: what ``TOKENOMOS_B200_CHECKS`` says)."""
    checks = checks_wanted() if checks is None else checks
    target = library_path(checks)
    if target.exists() and not force:
        return target
    nvcc = find_nvcc()
    srcs = sources()
    target.parent.mkdir(parents=True, exist_ok=True)
    work = Path(tempfile.mkdtemp(prefix="obj-", dir=str(target.parent)))
    _say(f"compiling {len(srcs)} CUDA sources for sm_100a into {target.parent} (first use only)")
    t0 = time.time()
    done = threading.Event()

    def heartbeat():
        while not done.wait(15.0):
            _say(f"still compiling ... {time.time() - t0:.0f} s")

    beat = threading.Thread(target=heartbeat, daemon=True)
    beat.start()
    try:
        objs = [work / (s.stem + ".o") for s in srcs]
        with ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 4)) as pool:
            futs = [pool.submit(_compile, nvcc, s, o, verbose, checks) for s, o in zip(srcs, objs)]
            for s, f in zip(srcs, futs):
                f.result()
                _say(f"  compiled {s.name} ({time.time() - t0:.0f} s)")
        tmp_lib = work / LIB_NAME
        link = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp_lib), *map(str, objs)]
        proc = subprocess.run(link, capture_output=True, text=True)
        if proc.returncode != 0:
            raise BuildError(f"linking {LIB_NAME} failed:\n{proc.stderr[-4000:]}")
        os.replace(tmp_lib, target)
        # libraries of earlier source states are dead weight (each is a few MB)
        current = source_hash()
        for old in target.parent.parent.iterdir():
            if old.is_dir() and not old.name.startswith(current) and (old / LIB_NAME).exists():
                shutil.rmtree(old, ignore_errors=True)
    finally:
        done.set()
        shutil.rmtree(work, ignore_errors=True)
    _say(f"built {target} in {time.time() - t0:.0f} s")
    return target


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv,
                checks=True if "--checks" in sys.argv else None))
