"""Build libfba_b200.so in-tree with nvcc, for sm_100a only.

Takes the place of the reference's setup.py / config.py (reference setup.py:29-45 selects
``-arch=sm_90a`` and the ThunderKittens include paths; config.py:2-15 selects the target).  Here
there is one target and no third-party headers: every ``csrc/*.cu`` is compiled with
``-gencode arch=compute_100a,code=sm_100a`` and linked into one shared library next to this file.

Run ``python -m flex_block_attn_b200.build`` (add ``--force`` to rebuild, ``--verbose`` for the
ptxas register / shared-memory report).  ``FBA_NVCC_EXTRA`` in the environment appends flags to
every compile, e.g. ``FBA_NVCC_EXTRA="-DFBA_RED_SLEEP_NS=16" python -m flex_block_attn_b200.build
--force`` for an A/B of one of the kernels' compile-time tuning constants (``FBA_RED_SLEEP_NS``,
``FBA_BWD_PREFETCH``, ``FBA_FWD_POLY_PAIRS``, ``FBA_TRACE``).
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
OBJ_DIR = PKG_DIR / "csrc" / "build"
LIB_PATH = PKG_DIR / "libfba_b200.so"

NVCC_FLAGS = [
    "-O3",
    "-std=c++17",
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-Xcompiler",
    "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC or put it on PATH")
    return cand


def _sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _deps() -> list[Path]:
    return _sources() + sorted(CSRC.glob("*.cuh")) + [PKG_DIR.parent / "include" / "fba.h"]


def is_stale() -> bool:
    if not LIB_PATH.exists():
        return True
    t = LIB_PATH.stat().st_mtime
    return any(d.stat().st_mtime > t for d in _deps() if d.exists())


def _compile_one(nvcc: str, src: Path, verbose: bool) -> tuple[Path, str]:
    obj = OBJ_DIR / (src.stem + ".o")
    cmd = [nvcc, *NVCC_FLAGS, *os.environ.get("FBA_NVCC_EXTRA", "").split(), "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
    return obj, r.stderr


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compile and link the library if it is missing or older than its sources."""
    if not force and not is_stale():
        return LIB_PATH
    nvcc = _nvcc()
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    srcs = _sources()
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        results = list(ex.map(lambda s: _compile_one(nvcc, s, verbose), srcs))
    if verbose:
        for _, log in results:
            sys.stderr.write(log)
    objs = [str(o) for o, _ in results]
    cmd = [nvcc, "-shared", "-o", str(LIB_PATH), *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-ldl"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB_PATH


if __name__ == "__main__":
    path = build_library(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
