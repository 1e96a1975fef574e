"""Compiles the CUDA sources under ``delta_b200/csrc`` into one shared library.

The library has a C interface only (no torch headers), so a fresh checkout
builds it with plain ``nvcc`` for sm_100a in about a minute at its first use.
Object files and the library live in ``csrc/_build/<hash of sources and flags>``;
when the package folder cannot be written to, in a per-user folder under the
system's temporary directory.  There is no fallback to other code: if ``nvcc``
is missing or a file does not compile, the error is raised.
"""
from __future__ import annotations

import concurrent.futures
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from pathlib import Path

CSRC = Path(__file__).resolve().parent.parent / "csrc"
LIB_NAME = "libdelta_b200.so"
# fast-math is never switched on: softmax, norms and the rotation are kept exact.
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
              "-Xcompiler", "-fPIC"] + os.environ.get("DELTA_B200_NVCC_EXTRA", "").split()


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[delta_b200 build] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("DELTA_B200_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).is_file():
            return cand
    raise BuildError("nvcc was not found (looked at $DELTA_B200_NVCC, PATH and /usr/local/cuda/bin): "
                     "the CUDA kernels of delta_b200 cannot be built, and there is no other code path")


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _digest() -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _build_root() -> Path:
    root = CSRC / "_build"
    try:
        root.mkdir(exist_ok=True)
        probe = root / f".w{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return root
    except OSError:
        alt = Path(tempfile.gettempdir()) / f"delta_b200_build_{os.getuid()}"
        alt.mkdir(parents=True, exist_ok=True)
        return alt


def _compile_one(nvcc: str, src: Path, obj: Path, extra: list[str]) -> tuple[str, float]:
    t0 = time.time()
    cmd = [nvcc, *NVCC_FLAGS, *extra, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise BuildError(f"nvcc failed on {src.name}:\n{' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    return src.name, time.time() - t0


def build(verbose: bool = True, ptxas_info: bool = False) -> Path:
    """Returns the path of the built library, compiling what is missing."""
    root = _build_root()
    out_dir = root / _digest()
    lib = out_dir / LIB_NAME
    if lib.is_file():
        return lib
    nvcc = find_nvcc()
    out_dir.mkdir(parents=True, exist_ok=True)
    with open(root / ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if lib.is_file():
            return lib
        srcs = sources()
        if not srcs:
            raise BuildError(f"no CUDA sources in {CSRC}")
        if verbose:
            _say(f"compiling {len(srcs)} CUDA files for sm_100a into {out_dir} (first use; about a minute)")
        extra = ["-Xptxas", "-v"] if ptxas_info else []
        t0 = time.time()
        objs = [out_dir / (s.stem + ".o") for s in srcs]
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(srcs), os.cpu_count() or 1)) as ex:
            futs = [ex.submit(_compile_one, nvcc, s, o, extra) for s, o in zip(srcs, objs)]
            for f in concurrent.futures.as_completed(futs):
                name, dt = f.result()
                if verbose:
                    _say(f"  {name} done in {dt:.0f} s ({time.time() - t0:.0f} s since start)")
        tmp = out_dir / (LIB_NAME + f".tmp{os.getpid()}")
        cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(tmp), *map(str, objs)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise BuildError(f"linking failed:\n{' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, lib)
        for o in objs:
            o.unlink(missing_ok=True)
        # older builds of other source versions are dropped so the folder stays small
        for d in root.iterdir():
            if d.is_dir() and d != out_dir:
                shutil.rmtree(d, ignore_errors=True)
        if verbose:
            _say(f"built {lib.name} in {time.time() - t0:.0f} s")
    return lib


if __name__ == "__main__":
    print(build(ptxas_info="-v" in sys.argv))
