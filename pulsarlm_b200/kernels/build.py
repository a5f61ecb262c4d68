"""Builds the CUDA kernel library for sm_100a with nvcc, in the tree.

Sources are pulsarlm_b200/csrc/*.cu. Each is compiled to an object in a build
folder (pulsarlm_b200/csrc/_build, or $PULSARLM_B200_BUILD_DIR, or a per-user
folder under the temporary directory when the tree cannot be written) and the
objects are linked into libpulsarlm_kernels.so. An object is rebuilt when its
source, any header or the flags change. While nvcc runs, a line is printed now
and then so a first call does not look hung.
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

CSRC = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "csrc"))
LIB_NAME = "libpulsarlm_kernels.so"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


class BuildError(RuntimeError):
    pass


def _say(message: str) -> None:
    print(f"[pulsarlm_b200] {message}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    candidates = []
    for var in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(var):
            candidates.append(os.path.join(os.environ[var], "bin", "nvcc"))
    candidates.append("/usr/local/cuda/bin/nvcc")
    found = shutil.which("nvcc")
    if found:
        candidates.append(found)
    for c in candidates:
        if os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    raise BuildError("nvcc not found (looked at $CUDA_HOME/bin, /usr/local/cuda/bin and PATH); "
                     "the CUDA kernels cannot be built and there is no fallback")


def _writable(folder: str) -> bool:
    try:
        os.makedirs(folder, exist_ok=True)
        probe = os.path.join(folder, f".probe{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return True
    except OSError:
        return False


def build_dir() -> str:
    env = os.environ.get("PULSARLM_B200_BUILD_DIR")
    if env:
        if not _writable(env):
            raise BuildError(f"PULSARLM_B200_BUILD_DIR={env} cannot be written")
        return env
    in_tree = os.path.join(CSRC, "_build")
    if _writable(in_tree):
        return in_tree
    fallback = os.path.join(tempfile.gettempdir(), f"pulsarlm_b200_build_{os.getuid()}")
    if _writable(fallback):
        return fallback
    raise BuildError(f"neither {in_tree} nor {fallback} can be written")


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, n) for n in os.listdir(CSRC) if n.endswith(".cu"))


def _headers_digest() -> str:
    h = hashlib.sha256()
    for n in sorted(os.listdir(CSRC)):
        if n.endswith((".cuh", ".h", ".hpp")):
            with open(os.path.join(CSRC, n), "rb") as f:
                h.update(n.encode())
                h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _source_digest(path: str, headers: str) -> str:
    h = hashlib.sha256(headers.encode())
    with open(path, "rb") as f:
        h.update(f.read())
    return h.hexdigest()


def _run(cmd: list[str], what: str) -> None:
    """Runs a tool, printing a heartbeat every 10 s."""
    done = threading.Event()

    def heartbeat():
        start = time.time()
        while not done.wait(10.0):
            _say(f"still {what} ({int(time.time() - start)} s)")

    thread = threading.Thread(target=heartbeat, daemon=True)
    thread.start()
    try:
        result = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    finally:
        done.set()
    if result.returncode != 0:
        raise BuildError(f"{what} failed:\n{' '.join(cmd)}\n{result.stdout}")


def library_path(build: bool = True, verbose: bool = True) -> str:
    """Path of an up-to-date library; builds what is stale when `build`."""
    folder = build_dir()
    lib = os.path.join(folder, LIB_NAME)
    headers = _headers_digest()
    stale: list[tuple[str, str, str]] = []
    objects = []
    for src in sources():
        name = os.path.splitext(os.path.basename(src))[0]
        obj = os.path.join(folder, name + ".o")
        stamp = os.path.join(folder, name + ".hash")
        digest = _source_digest(src, headers)
        objects.append(obj)
        current = None
        if os.path.isfile(obj) and os.path.isfile(stamp):
            with open(stamp) as f:
                current = f.read().strip()
        if current != digest:
            stale.append((src, obj, digest))
    lib_stamp = os.path.join(folder, LIB_NAME + ".hash")
    all_digest = hashlib.sha256(
        "".join(_source_digest(s, headers) for s in sources()).encode()).hexdigest()
    lib_current = None
    if os.path.isfile(lib) and os.path.isfile(lib_stamp):
        with open(lib_stamp) as f:
            lib_current = f.read().strip()
    if not stale and lib_current == all_digest:
        return lib
    if not build:
        raise BuildError(f"{lib} is missing or stale")
    nvcc = find_nvcc()
    if verbose and stale:
        _say(f"compiling {len(stale)} CUDA source file(s) for sm_100a into {folder} (first call only)")
    threads = []
    errors: list[BaseException] = []

    def compile_one(src: str, obj: str, digest: str) -> None:
        try:
            _run([nvcc, *NVCC_FLAGS, "-I", CSRC, "-c", src, "-o", obj], f"compiling {os.path.basename(src)}")
            with open(os.path.splitext(obj)[0] + ".hash", "w") as f:
                f.write(digest)
            if verbose:
                _say(f"compiled {os.path.basename(src)}")
        except BaseException as error:  # noqa: BLE001 - reported after the join
            errors.append(error)

    limit = max(1, min(8, (os.cpu_count() or 2)))
    pending = list(stale)
    while pending or threads:
        while pending and len(threads) < limit:
            t = threading.Thread(target=compile_one, args=pending.pop(0))
            t.start()
            threads.append(t)
        threads[0].join()
        threads.pop(0)
    if errors:
        raise errors[0]
    tmp = lib + f".tmp{os.getpid()}"
    _run([nvcc, "-shared", "-o", tmp, *objects, "-lcudart_static", "-ldl", "-lrt", "-lpthread"], "linking")
    os.replace(tmp, lib)
    with open(lib_stamp, "w") as f:
        f.write(all_digest)
    if verbose:
        _say(f"built {lib}")
    return lib


HOST_SRC = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "csrc_host"))
HOST_LIB_NAME = "libpulsarlm_host.so"
HOST_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-Wall", "-ffp-contract=off"]
HOST_SHARED_HEADERS = ["random_values.h"]  # headers of the kernel tree that the host core includes too


def host_library_path(build: bool = True, verbose: bool = True) -> str:
    """Path of the host core (C++, no CUDA: page pools, block tables, scheduler),
    built with g++ next to the kernel library when stale."""
    folder = build_dir()
    lib = os.path.join(folder, HOST_LIB_NAME)
    stamp = os.path.join(folder, HOST_LIB_NAME + ".hash")
    digest = hashlib.sha256(" ".join(HOST_FLAGS).encode())
    files = sorted(n for n in os.listdir(HOST_SRC) if n.endswith((".cpp", ".hpp", ".h")))
    for n in files:
        with open(os.path.join(HOST_SRC, n), "rb") as f:
            digest.update(n.encode())
            digest.update(f.read())
    for n in HOST_SHARED_HEADERS:
        with open(os.path.join(CSRC, n), "rb") as f:
            digest.update(n.encode())
            digest.update(f.read())
    current = None
    if os.path.isfile(lib) and os.path.isfile(stamp):
        with open(stamp) as f:
            current = f.read().strip()
    if current == digest.hexdigest():
        return lib
    if not build:
        raise BuildError(f"{lib} is missing or stale")
    compiler = shutil.which("g++") or shutil.which("c++")
    if compiler is None:
        raise BuildError("no C++ compiler (g++) found: the host core cannot be built")
    if verbose:
        _say(f"compiling the host core into {folder} (first call only)")
    tmp = lib + f".tmp{os.getpid()}"
    sources = [os.path.join(HOST_SRC, n) for n in files if n.endswith(".cpp")]
    _run([compiler, *HOST_FLAGS, "-I", HOST_SRC, *sources, "-o", tmp], "compiling the host core")
    os.replace(tmp, lib)
    with open(stamp, "w") as f:
        f.write(digest.hexdigest())
    return lib


if __name__ == "__main__":
    print(host_library_path())
    print(library_path())
