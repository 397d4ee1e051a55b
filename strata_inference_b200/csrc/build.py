"""Compile the CUDA sources of this folder into one shared library for sm_100a.

``ensure_built()`` compiles what is missing or stale (a hash of the sources
and flags is kept beside the objects) and returns the library's path.  The
objects and the library live in ``csrc/_build`` of the checkout; when that
folder cannot be written, a per-user folder under the system's temporary
directory is used instead.  A line is printed per compiled file, so a first
call in a fresh checkout shows that it is working.
"""

from __future__ import annotations

import hashlib
import json
import os
import shutil
import subprocess
import sys
import tempfile
from concurrent.futures import ThreadPoolExecutor
from typing import List, Optional

CSRC = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libstrata_b200.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-DSIB_ARCH=100",
              "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr"]


class BuildError(RuntimeError):
    pass


def sources() -> List[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers() -> List[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))


def find_nvcc() -> str:
    for base in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if base and os.path.isfile(os.path.join(base, "bin", "nvcc")):
            return os.path.join(base, "bin", "nvcc")
    found = shutil.which("nvcc")
    if found:
        return found
    raise BuildError("nvcc not found (looked in $CUDA_HOME, /usr/local/cuda and $PATH); "
                     "the sm_100a kernels cannot be compiled")


def _digest(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        h.update(f.read())
    return h.hexdigest()


def _stamp() -> dict:
    heads = {h: _digest(os.path.join(CSRC, h)) for h in _headers()}
    return {"flags": ARCH_FLAGS + NVCC_FLAGS, "headers": heads,
            "sources": {s: _digest(os.path.join(CSRC, s)) for s in sources()}}


def _build_dir() -> str:
    local = os.path.join(CSRC, "_build")
    try:
        os.makedirs(local, exist_ok=True)
        probe = os.path.join(local, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return local
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"strata_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _log(msg: str, quiet: bool) -> None:
    if not quiet:
        print(f"[strata_inference_b200 build] {msg}", file=sys.stderr, flush=True)


def ensure_built(quiet: bool = False, force: bool = False, ptxas_verbose: bool = False) -> str:
    """Return the path of an up-to-date library, compiling as needed."""
    out = _build_dir()
    lib = os.path.join(out, LIB_NAME)
    stamp_path = os.path.join(out, "stamp.json")
    want = _stamp()
    have = None
    if os.path.isfile(stamp_path):
        try:
            with open(stamp_path) as f:
                have = json.load(f)
        except (OSError, json.JSONDecodeError):
            have = None
    if not force and have == want and os.path.isfile(lib):
        return lib

    nvcc = find_nvcc()
    all_stale = force or have is None or have.get("flags") != want["flags"] \
        or have.get("headers") != want["headers"]
    todo = []
    for s in sources():
        obj = os.path.join(out, s[:-3] + ".o")
        stale = all_stale or not os.path.isfile(obj) \
            or have["sources"].get(s) != want["sources"][s]
        if stale:
            todo.append((s, obj))
    _log(f"compiling {len(todo)} of {len(sources())} CUDA files for sm_100a "
         f"into {out} (a minute or so the first time)", quiet)

    def compile_one(item):
        src, obj = item
        cmd = [nvcc] + ARCH_FLAGS + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_verbose else []) + \
            ["-I", CSRC, "-c", os.path.join(CSRC, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise BuildError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        _log(f"compiled {src}", quiet)
        return r.stderr

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        logs = list(pool.map(compile_one, todo))
    if ptxas_verbose:
        for (src, _), text in zip(todo, logs):
            print(f"==== {src}\n{text}")
    objs = [os.path.join(out, s[:-3] + ".o") for s in sources()]
    tmp_lib = lib + f".{os.getpid()}.tmp"
    cmd = [nvcc] + ARCH_FLAGS + ["-shared", "-o", tmp_lib] + objs + ["-lcudart"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise BuildError(f"linking {LIB_NAME} failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp_lib, lib)
    with open(stamp_path, "w") as f:
        json.dump(want, f)
    _log(f"built {lib}", quiet)
    return lib


if __name__ == "__main__":
    ensure_built(force="--force" in sys.argv, ptxas_verbose="-v" in sys.argv)
