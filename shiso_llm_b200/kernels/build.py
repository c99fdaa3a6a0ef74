"""Builds the CUDA kernels into one shared library, in the tree, on first use.

Every ``*.cu`` under ``csrc/`` is compiled with nvcc for sm_100a only
(``-gencode arch=compute_100a,code=sm_100a``) and linked into ``libshiso_b200.so``.
The sources include no PyTorch headers: they export plain C launchers that take device
pointers and a stream, which Python calls through ctypes.  A hash of the sources and
flags is stored beside the library; a library whose hash does not match is rebuilt.
The build directory is ``csrc/_build`` when that is writable, else a per-user folder
under the system's temporary directory, so a read-only checkout or another user still
works.  A line is printed when compilation starts, per file, and at the end.
"""

from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
LIB_NAME = "libshiso_b200.so"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
]


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[shiso_llm_b200 build] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("SHISO_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found (looked at $SHISO_NVCC, PATH and /usr/local/cuda/bin): the CUDA kernels cannot be built")


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))


def source_hash() -> str:
    h = hashlib.sha256()
    for path in sources() + _headers():
        h.update(os.path.basename(path).encode())
        with open(path, "rb") as f:
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()[:20]


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f".probe{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return True
    except OSError:
        return False


def build_dir() -> str:
    override = os.environ.get("SHISO_BUILD_DIR")
    if override:
        if not _writable_dir(override):
            raise BuildError(f"SHISO_BUILD_DIR={override} is not writable")
        return override
    in_tree = os.path.join(CSRC, "_build")
    if _writable_dir(in_tree):
        return in_tree
    fallback = os.path.join(tempfile.gettempdir(), f"shiso_llm_b200_build_{os.getuid()}")
    if _writable_dir(fallback):
        return fallback
    raise BuildError(f"neither {in_tree} nor {fallback} is writable: nowhere to build the CUDA kernels")


def library_path(create: bool = True) -> str:
    """Path of an up-to-date library, building it first if needed."""
    want = source_hash()
    # An up-to-date library in the tree wins even when the tree is read-only.
    for d in (os.path.join(CSRC, "_build"),):
        lib, stamp = os.path.join(d, LIB_NAME), os.path.join(d, "source_hash")
        if os.path.isfile(lib) and os.path.isfile(stamp) and open(stamp).read().strip() == want:
            return lib
    d = build_dir()
    lib, stamp = os.path.join(d, LIB_NAME), os.path.join(d, "source_hash")
    if os.path.isfile(lib) and os.path.isfile(stamp) and open(stamp).read().strip() == want:
        return lib
    if not create:
        raise BuildError("the CUDA kernel library is not built")
    return build(d)


def _compile_one(nvcc: str, src: str, obj: str, verbose: bool) -> str:
    cmd = [nvcc, *NVCC_FLAGS, "-I", CSRC, "-c", src, "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError(f"nvcc failed on {os.path.basename(src)}:\n{proc.stdout}\n{proc.stderr}")
    return proc.stderr


def build(directory: str | None = None, verbose: bool = False) -> str:
    nvcc = find_nvcc()
    d = directory or build_dir()
    srcs = sources()
    if not srcs:
        raise BuildError(f"no .cu sources under {CSRC}")
    started = time.time()
    _say(f"compiling {len(srcs)} CUDA files for sm_100a into {d} (first use; this takes a minute or two)")
    objs = [os.path.join(d, os.path.basename(s)[:-3] + ".o") for s in srcs]
    log = []
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        futures = {pool.submit(_compile_one, nvcc, s, o, verbose): s for s, o in zip(srcs, objs)}
        for fut in concurrent.futures.as_completed(futures):
            log.append(fut.result())
            _say(f"  compiled {os.path.basename(futures[fut])} ({time.time() - started:.0f} s)")
    tmp_lib = os.path.join(d, f".{LIB_NAME}.{os.getpid()}")
    link = [nvcc, "-shared", "-o", tmp_lib, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
    proc = subprocess.run(link, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError(f"linking {LIB_NAME} failed:\n{proc.stdout}\n{proc.stderr}")
    lib = os.path.join(d, LIB_NAME)
    os.replace(tmp_lib, lib)
    with open(os.path.join(d, "source_hash"), "w") as f:
        f.write(source_hash() + "\n")
    if verbose:
        with open(os.path.join(d, "ptxas.log"), "w") as f:
            f.write("\n".join(log))
    _say(f"built {lib} in {time.time() - started:.0f} s")
    return lib
