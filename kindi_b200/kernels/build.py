"""Building the kernel library for sm_100a with nvcc, in-tree, at first use.

Each ``csrc/*.cu`` is compiled to an object file (in parallel) and the objects are linked into
``libkindi_b200.so``; a stamp with the hash of the sources and flags makes later imports skip the build. The
library lives under the package (``kindi_b200/_build``) when that folder can be written, else under the system's
temporary folder. While nvcc runs, a progress line is printed every few seconds.

(The reference compiles its kernels at start too, through NVRTC: ``kindi/nanbeige.py:54-65``.)
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
from typing import List, Optional

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(os.path.dirname(HERE), "csrc")
LIB_NAME = "libkindi_b200.so"

NVCC_FLAGS = ["-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v"]
LINK_LIBS = ["-lcuda"]


def _say(msg: str) -> None:
    sys.stderr.write("[kindi_b200 build] %s\n" % msg)
    sys.stderr.flush()


def find_nvcc() -> Optional[str]:
    for c in (os.environ.get("CUDACXX"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if c and os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    return None


def sources() -> List[str]:
    return sorted(os.path.join(CSRC, n) for n in os.listdir(CSRC) if n.endswith(".cu"))


def _headers() -> List[str]:
    return sorted(os.path.join(CSRC, n) for n in os.listdir(CSRC) if n.endswith((".cuh", ".h")))


def source_hash() -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS + LINK_LIBS).encode())
    for p in sources() + _headers():
        h.update(os.path.basename(p).encode())
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:20]


def build_dir() -> str:
    d = os.path.join(os.path.dirname(HERE), "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, ".w%d" % os.getpid())
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), "kindi_b200_build_%d" % os.getuid())
        os.makedirs(d, exist_ok=True)
        return d


def library_path(build: bool = True, verbose: bool = True) -> str:
    """the path of the built library; builds it first when it is missing or older than the sources"""
    d = build_dir()
    lib, stamp = os.path.join(d, LIB_NAME), os.path.join(d, "stamp.json")
    want = source_hash()
    if os.path.isfile(lib) and os.path.isfile(stamp):
        try:
            with open(stamp) as f:
                if json.load(f).get("hash") == want:
                    return lib
        except (OSError, ValueError):
            pass
    if not build:
        raise RuntimeError("kindi_b200: the kernel library is not built (%s)" % lib)
    _build(d, lib, stamp, want, verbose)
    return lib


def _build(d: str, lib: str, stamp: str, want: str, verbose: bool) -> None:
    nvcc = find_nvcc()
    if nvcc is None:
        raise RuntimeError("kindi_b200: nvcc not found; the CUDA kernels cannot be built (set CUDACXX or PATH)")
    srcs = sources()
    t0 = time.time()
    if verbose:
        _say("compiling %d CUDA files for sm_100a with %s into %s" % (len(srcs), nvcc, d))
    jobs = []
    max_par = max(1, min(len(srcs), (os.cpu_count() or 2)))
    pending = list(srcs)
    logs = {}
    objs = []
    running = []
    last = time.time()
    while pending or running:
        while pending and len(running) < max_par:
            s = pending.pop(0)
            o = os.path.join(d, os.path.basename(s)[:-3] + ".o")
            objs.append(o)
            log = open(os.path.join(d, os.path.basename(s) + ".log"), "w")
            p = subprocess.Popen([nvcc] + NVCC_FLAGS + ["-I", CSRC, "-c", s, "-o", o], stdout=log,
                                 stderr=subprocess.STDOUT)
            running.append((p, s, log))
        time.sleep(0.2)
        for item in list(running):
            p, s, log = item
            rc = p.poll()
            if rc is None:
                continue
            running.remove(item)
            log.close()
            if rc != 0:
                for q, _, lg in running:
                    q.kill()
                    lg.close()
                with open(os.path.join(d, os.path.basename(s) + ".log")) as f:
                    out = f.read()
                raise RuntimeError("kindi_b200: nvcc failed on %s:\n%s" % (os.path.basename(s), out[-6000:]))
            if verbose:
                _say("compiled %s (%.0f s)" % (os.path.basename(s), time.time() - t0))
        if verbose and time.time() - last > 5.0 and running:
            _say("still compiling: %s (%.0f s)" % (", ".join(os.path.basename(s) for _, s, _ in running),
                                                    time.time() - t0))
            last = time.time()
    tmp = lib + ".%d.tmp" % os.getpid()
    r = subprocess.run([nvcc, "-shared", "-o", tmp] + objs + LINK_LIBS, stdout=subprocess.PIPE,
                       stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("kindi_b200: linking the kernel library failed:\n%s" % r.stdout[-4000:])
    os.replace(tmp, lib)
    with open(stamp, "w") as f:
        json.dump({"hash": want, "built": time.strftime("%Y-%m-%d %H:%M:%S"), "sources": [os.path.basename(s) for s in srcs]}, f)
    if verbose:
        _say("built %s in %.0f s" % (lib, time.time() - t0))


if __name__ == "__main__":
    print(library_path())
