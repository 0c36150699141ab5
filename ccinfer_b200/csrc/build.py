"""Builds the CUDA extension in-tree with nvcc for sm_100a and returns the path of the shared object.

Each ``.cu`` file is compiled to an object file on its own (in parallel) and the
objects are linked into one ``libccinfer_b200_<group>.so`` under
``ccinfer_b200/csrc/_build``.  A stamp made of the sources' contents and the
flags decides whether a build is current, so a library built on one machine is
taken as it is on another with the same sources.  If the package folder cannot
be written (a read-only install) the build goes to a per-user folder under the
system's temporary directory.  There is no fallback to anything but these
kernels: if nvcc is missing or a file does not compile, ExtensionMissing says
so.
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time

from ..errors import ExtensionMissing

CSRC = os.path.dirname(os.path.abspath(__file__))

# group -> source files.  "core" is every kernel a model step needs; "host" is the C++ host core (cache manager,
# request slots, the arrays of a step) behind the C interface of host/ccinfer.h: no device code in it.
GROUPS = {
    "core": [
        "elementwise.cu",
        "norm.cu",
        "rope_kv.cu",
        "attention_generic.cu",
        "attention_split.cu",
        "attention_decode_mma.cu",
        "attention_decode_tma.cu",
        "attention_prefill_mma.cu",
        "attention_prefill_tc.cu",
        "gemm_f32.cu",
        "gemm_cublas.cu",
        "gemm_skinny.cu",
        "gemm_tcgen05.cu",
        "gemm_tc_pair.cu",
        "gemm_fewrows.cu",
        "sampling.cu",
        "random_init.cu",
    ],
    "host": [
        "host/host_core.cpp",
        "host/scheduler.cpp",
    ],
}
GROUP_LIBS = {"core": ["-lcublas"]}
GROUP_HEADERS = {"host": ["host/ccinfer.h"]}   # default: every header beside the kernels

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
]


def find_nvcc() -> str:
    for cand in (os.environ.get("CCINFER_NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 shutil.which("nvcc")):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise ExtensionMissing("nvcc was not found (looked at $CCINFER_NVCC, $CUDA_HOME/bin, /usr/local/cuda/bin "
                           "and PATH); the CUDA kernels cannot be built and there is no other path")


def _stamp(group: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS + GROUP_LIBS.get(group, [])).encode())
    headers = GROUP_HEADERS.get(group) or sorted(f for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))
    for name in headers + GROUPS[group]:
        h.update(name.encode())
        with open(os.path.join(CSRC, name), "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def _build_dir() -> str:
    d = os.path.join(CSRC, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.unlink(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"ccinfer_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _say(msg: str) -> None:
    print(f"[ccinfer_b200 build] {msg}", file=sys.stderr, flush=True)


def _compile_one(nvcc: str, src: str, obj: str) -> None:
    cmd = [nvcc] + NVCC_FLAGS + ["-I", CSRC, "-c", os.path.join(CSRC, src), "-o", obj]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise ExtensionMissing(f"nvcc failed on {src}:\n{' '.join(cmd)}\n{r.stdout}")


def library_path(group: str = "core", verbose: bool = True) -> str:
    """Path of the up-to-date shared object of a group, building it if needed."""
    if group not in GROUPS:
        raise ExtensionMissing(f"unknown kernel group {group!r}")
    bdir = _build_dir()
    stamp = _stamp(group)
    lib = os.path.join(bdir, f"libccinfer_b200_{group}.so")
    stamp_file = lib + ".stamp"
    if os.path.isfile(lib) and os.path.isfile(stamp_file):
        with open(stamp_file) as f:
            if f.read().strip() == stamp:
                return lib
    nvcc = find_nvcc()
    srcs = GROUPS[group]
    if verbose:
        _say(f"compiling {len(srcs)} files of group '{group}'" + (" for sm_100a" if group != "host" else "") + f" into {bdir}")
    t0 = time.time()
    done = threading.Event()

    def ticker():
        while not done.wait(10.0):
            _say(f"still compiling ... {time.time() - t0:.0f} s")

    th = threading.Thread(target=ticker, daemon=True)
    if verbose:
        th.start()
    objs = [os.path.join(bdir, f"{group}_{os.path.splitext(os.path.basename(s))[0]}.{os.getpid()}.o") for s in srcs]
    try:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
            futs = {ex.submit(_compile_one, nvcc, s, o): s for s, o in zip(srcs, objs)}
            for fut in concurrent.futures.as_completed(futs):
                fut.result()
                if verbose:
                    _say(f"compiled {futs[fut]} ({time.time() - t0:.0f} s)")
        tmp = lib + f".{os.getpid()}.tmp"
        cmd = [nvcc, "-shared", "-o", tmp] + objs + GROUP_LIBS.get(group, [])
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            raise ExtensionMissing(f"linking {lib} failed:\n{' '.join(cmd)}\n{r.stdout}")
        os.replace(tmp, lib)
        with open(stamp_file + f".{os.getpid()}", "w") as f:
            f.write(stamp)
        os.replace(stamp_file + f".{os.getpid()}", stamp_file)
    finally:
        done.set()
        for o in objs:   # also after a failed build: no object files are left behind
            try:
                os.unlink(o)
            except OSError:
                pass
    if verbose:
        _say(f"built {os.path.basename(lib)} in {time.time() - t0:.0f} s")
    return lib


def build_all(verbose: bool = True) -> list:
    return [library_path(g, verbose) for g in GROUPS]


if __name__ == "__main__":
    for p in build_all():
        print(p)
