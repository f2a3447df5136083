"""Builds the package's CUDA kernels into one shared library for sm_100a.

nvcc is called directly (no torch headers are involved, so a file compiles in a
couple of seconds) and the result is loaded through ctypes. The library is
rebuilt when the hash of the sources and flags changes. It is written into the
package (``openinfer_b200/_lib``) when that folder can be written, else into a
per-user folder under the system's temporary directory, so a read-only checkout
and a user without a home directory both work. Progress lines go to stderr.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor, as_completed
from typing import List, Optional

CSRC = os.path.dirname(os.path.abspath(__file__))
PACKAGE = os.path.dirname(CSRC)
LIB_NAME = "liboi_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


class BuildError(RuntimeError):
    pass


def sources() -> List[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers() -> List[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))


def find_nvcc() -> str:
    cands = []
    for env in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(env):
            cands.append(os.path.join(os.environ[env], "bin", "nvcc"))
    cands.append("/usr/local/cuda/bin/nvcc")
    which = shutil.which("nvcc")
    if which:
        cands.append(which)
    for c in cands:
        if os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    raise BuildError("nvcc not found (looked at $CUDA_HOME/bin, /usr/local/cuda/bin and PATH)")


def source_hash() -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for name in sources() + _headers():
        h.update(name.encode())
        with open(os.path.join(CSRC, name), "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f".probe-{os.getpid()}")
        with open(probe, "w"):
            pass
        os.unlink(probe)
        return True
    except OSError:
        return False


def lib_dir() -> str:
    override = os.environ.get("OPENINFER_B200_LIB_DIR")
    if override:
        os.makedirs(override, exist_ok=True)
        return override
    in_tree = os.path.join(PACKAGE, "_lib")
    if _writable_dir(in_tree):
        return in_tree
    fallback = os.path.join(tempfile.gettempdir(), f"openinfer_b200-{os.getuid()}")
    if not _writable_dir(fallback):
        raise BuildError(f"neither {in_tree} nor {fallback} can be written")
    return fallback


def _say(msg: str, verbose: bool) -> None:
    if verbose:
        print(f"[openinfer_b200 build] {msg}", file=sys.stderr, flush=True)


def _up_to_date(folder: str, want: str) -> bool:
    lib = os.path.join(folder, LIB_NAME)
    stamp = lib + ".hash"
    if not (os.path.isfile(lib) and os.path.isfile(stamp)):
        return False
    with open(stamp) as fh:
        return fh.read().strip() == want


def ensure_built(verbose: bool = True, force: bool = False) -> str:
    """Return the path of an up-to-date library, compiling it first if needed."""
    want = source_hash()
    # a library that already matches (in the tree or in the fallback folder) is used as it is
    in_tree = os.path.join(PACKAGE, "_lib")
    if not force:
        for folder in (os.environ.get("OPENINFER_B200_LIB_DIR"), in_tree,
                       os.path.join(tempfile.gettempdir(), f"openinfer_b200-{os.getuid()}")):
            if folder and _up_to_date(folder, want):
                return os.path.join(folder, LIB_NAME)
    folder = lib_dir()
    nvcc = find_nvcc()
    obj_dir = os.path.join(folder, "obj")
    os.makedirs(obj_dir, exist_ok=True)
    srcs = sources()
    _say(f"compiling {len(srcs)} CUDA files for sm_100a with {nvcc} into {folder}", verbose)
    t0 = time.time()

    def compile_one(name: str) -> str:
        obj = os.path.join(obj_dir, name[:-3] + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", CSRC, "-c", os.path.join(CSRC, name), "-o", obj]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise BuildError(f"nvcc failed on {name}:\n{proc.stdout}\n{proc.stderr}")
        return obj

    objs: List[str] = []
    workers = max(1, min(len(srcs), os.cpu_count() or 1, 8))
    with ThreadPoolExecutor(max_workers=workers) as pool:
        futs = {pool.submit(compile_one, s): s for s in srcs}
        done = 0
        for fut in as_completed(futs):
            objs.append(fut.result())
            done += 1
            _say(f"  [{done}/{len(srcs)}] {futs[fut]} ({time.time() - t0:.0f}s)", verbose)
    tmp_lib = os.path.join(folder, f".{LIB_NAME}.{os.getpid()}")
    cmd = [nvcc, "-shared", "-o", tmp_lib, *sorted(objs), "-Xcompiler", "-fPIC"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    lib = os.path.join(folder, LIB_NAME)
    os.replace(tmp_lib, lib)
    with open(lib + ".hash", "w") as fh:
        fh.write(want)
    _say(f"built {lib} in {time.time() - t0:.0f}s", verbose)
    return lib


def main(argv: Optional[List[str]] = None) -> int:
    import argparse

    ap = argparse.ArgumentParser(description="build the openinfer_b200 CUDA library")
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--quiet", action="store_true")
    args = ap.parse_args(argv)
    print(ensure_built(verbose=not args.quiet, force=args.force))
    return 0


if __name__ == "__main__":
    sys.exit(main())
