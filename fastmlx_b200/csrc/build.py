"""Builds the CUDA libraries for sm_100a with nvcc, in-tree, the first time they are needed.

The kernels are plain `extern "C"` entry points that take device pointers and a stream;
they include no PyTorch header, so a library compiles in seconds and is loaded with
ctypes.  Each group of sources becomes one shared library, and only the groups a run
needs are built: the 32-bit path compiles none of the bfloat16 tensor-core kernels.
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

HERE = os.path.dirname(os.path.abspath(__file__))

GROUPS = {
    # name: directory of its sources.  A name like "attn_hd64" is the group "attn" compiled
    # with -DFMX_HD=64: one library per head size, built when a model of that size is met.
    "common": "common",
    "bf16": "bf16",
    "attn": "attn",
    "tc": "tc",
    # host code: the native step executor (no kernel of its own)
    "host": "host",
    # the tensor-core product built for one test: a wait limit of 100,000 clocks and a producer that
    # leaves out its last block, so that the path a wait takes when it runs out is executed
    "tc_expiry": "tc",
}
EXTRA_FLAGS = {"tc_expiry": ["-DFMX_WAIT_CYCLES=100000LL", "-DFMX_SKIP_LAST_STAGE=1"]}
HEAD_DIMS = tuple(range(16, 257, 16))


def _split(group: str) -> tuple[str, list[str]]:
    """'attn_hd64' -> ('attn', ['-DFMX_HD=64']); other names stand for themselves."""
    if group.startswith("attn_hd"):
        hd = int(group[len("attn_hd"):])
        if hd not in HEAD_DIMS:
            raise BuildError(f"the tiled attention kernels take head sizes in steps of 16 up to 256, not {hd}")
        return "attn", [f"-DFMX_HD={hd}"]
    if group not in GROUPS:
        raise BuildError(f"unknown kernel group {group!r}")
    return group, list(EXTRA_FLAGS.get(group, ()))

NVCC_FLAGS = ["-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
              "-I", os.path.join(HERE, "common")]


class BuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    for cand in (os.environ.get("FASTMLX_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise BuildError("nvcc not found (set FASTMLX_NVCC or CUDA_HOME): the CUDA kernels cannot be built, "
                     "and there is no other path")


def sources(group: str) -> list[str]:
    d = os.path.join(HERE, GROUPS[_split(group)[0]])
    if not os.path.isdir(d):
        return []
    srcs = sorted(os.path.join(d, f) for f in os.listdir(d) if f.endswith(".cu"))
    if srcs and _split(group)[0] != "common":
        srcs.append(os.path.join(HERE, "common", "error.cu"))     # every library carries its own error text
    return srcs


def _digest(group: str) -> str:
    h = hashlib.sha256(" ".join(NVCC_FLAGS + _split(group)[1]).replace(HERE, ".").encode())
    files = sources(group)
    for d in {os.path.dirname(f) for f in files} | {os.path.join(HERE, "common")}:
        files += [os.path.join(d, f) for f in os.listdir(d) if f.endswith((".cuh", ".h"))]
    for f in sorted(set(files)):
        h.update(os.path.relpath(f, HERE).encode())        # the same tree elsewhere needs no rebuild
        with open(f, "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()[:16]


def build_dir() -> str:
    """In-tree `_build/` beside the sources; a private temporary folder when the tree is
    read-only."""
    d = os.environ.get("FASTMLX_BUILD_DIR") or os.path.join(HERE, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        # one probe file per thread: groups are built side by side, and two threads that shared a
        # name took each other's file away and mistook that for a read-only tree
        probe = os.path.join(d, f".w{os.getpid()}_{threading.get_ident()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"fastmlx_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def library_path(group: str) -> str:
    return os.path.join(build_dir(), f"libfmx_{group}.so")


def _say(msg: str) -> None:
    print(f"[fastmlx_b200 build] {msg}", file=sys.stderr, flush=True)


def _run_with_heartbeat(cmd: list[str], what: str) -> None:
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def beat():
        t0 = time.time()
        while not done.wait(10.0):
            _say(f"still compiling {what} ({time.time() - t0:.0f} s)")

    th = threading.Thread(target=beat, daemon=True)
    th.start()
    out, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        raise BuildError(f"nvcc failed on {what}:\n{' '.join(cmd)}\n{out}")


def build(group: str, force: bool = False, verbose: bool = False) -> str:
    """Compile one group if its library is missing or older than its sources."""
    lib = library_path(group)
    stamp = lib + ".digest"
    digest = _digest(group)
    if not force and os.path.exists(lib) and os.path.exists(stamp):
        with open(stamp) as f:
            if f.read().strip() == digest:
                return lib
    nvcc = find_nvcc()
    srcs = sources(group)
    if not srcs:
        raise BuildError(f"group {group!r} has no sources")
    bdir = build_dir()
    _say(f"compiling {len(srcs)} CUDA files of group '{group}' for sm_100a (first use; a minute or so)")
    t0 = time.time()
    objs = []
    extra = ["-Xptxas", "-v"] if verbose else []

    def compile_one(src):
        obj = os.path.join(bdir, f"{group}_{os.path.basename(src)[:-3]}.o")
        _run_with_heartbeat([nvcc, *NVCC_FLAGS, *_split(group)[1], *extra, "-c", src, "-o", obj],
                            os.path.basename(src))
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(srcs), os.cpu_count() or 1)) as ex:
        objs = list(ex.map(compile_one, srcs))
    tmp = f"{lib}.{os.getpid()}.tmp"
    _run_with_heartbeat([nvcc, "-shared", "-o", tmp, *objs, "-gencode",
                         "arch=compute_100a,code=sm_100a"], f"libfmx_{group}.so")
    os.replace(tmp, lib)
    with open(stamp, "w") as f:
        f.write(digest)
    _say(f"built {os.path.basename(lib)} in {time.time() - t0:.1f} s")
    return lib


def build_all(force: bool = False, verbose: bool = False, head_dims=HEAD_DIMS) -> list[str]:
    """Every library: the plain groups and the attention kernels of every head size."""
    groups = [g for g in GROUPS if g != "attn" and sources(g)] + [f"attn_hd{hd}" for hd in head_dims]
    with ThreadPoolExecutor(max_workers=max(1, (os.cpu_count() or 2) // 2)) as ex:
        return list(ex.map(lambda g: build(g, force, verbose), groups))


if __name__ == "__main__":
    for p in build_all(force="--force" in sys.argv, verbose="-v" in sys.argv):
        print(p)
