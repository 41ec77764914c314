"""Builds ``libmni_b200.so`` in-tree with nvcc for sm_100a (cross-compiles without a GPU)."""
from __future__ import annotations

import glob
import os
import subprocess
import sys

_PKG = os.path.dirname(os.path.abspath(__file__))
_ROOT = os.path.dirname(_PKG)
CSRC = os.path.join(_PKG, "csrc")
LIB_PATH = os.path.join(_PKG, "lib", "libmni_b200.so")

NVCC_FLAGS = [
    "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-shared",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def sources() -> list:
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def is_stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(d) > t for d in sources() + _headers())


def source_hash() -> str:
    """sha256 over the names and contents of every file the library is built from."""
    import hashlib
    h = hashlib.sha256()
    for path in sorted(sources() + _headers()):
        h.update(os.path.basename(path).encode() + b"\0")
        with open(path, "rb") as f:
            h.update(f.read())
        h.update(b"\0")
    return h.hexdigest()


def _headers() -> list:
    return glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(_ROOT, "include", "*.h"))


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compile every .cu under csrc/ (one nvcc per file, side by side; objects whose source and headers
    are unchanged are kept) and link them into lib/libmni_b200.so; returns its path."""
    if not force and not is_stale():
        return LIB_PATH
    os.makedirs(os.path.dirname(LIB_PATH), exist_ok=True)
    obj_dir = os.path.join(_PKG, "lib", "obj")
    os.makedirs(obj_dir, exist_ok=True)
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)
    compile_flags = [f for f in NVCC_FLAGS if f != "-shared"]
    newest_header = max((os.path.getmtime(h) for h in _headers()), default=0.0)
    jobs, objects = [], []
    for src in sources():
        obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + ".o")
        objects.append(obj)
        fresh = (not force and os.path.exists(obj)
                 and os.path.getmtime(obj) >= max(os.path.getmtime(src), newest_header))
        if fresh:
            continue
        cmd = [_nvcc(), *compile_flags, "-I", os.path.join(_ROOT, "include"), "-I", CSRC]
        if verbose:
            cmd += ["-Xptxas", "-v"]
        cmd += ["-c", "-o", obj, src]
        jobs.append((src, subprocess.Popen(cmd, env=env)))
    # The hash of the sources is linked in, so that a loader can tell a library built from other sources.
    id_src, id_obj = os.path.join(obj_dir, "build_id.c"), os.path.join(obj_dir, "build_id.o")
    with open(id_src, "w") as f:
        f.write('__attribute__((visibility("default"))) const char *mni_b200_build_id(void) '
                '{ return "%s"; }\n' % source_hash())
    subprocess.check_call(["gcc", "-O1", "-fPIC", "-c", "-o", id_obj, id_src], env=env)
    failed = [src for src, proc in jobs if proc.wait() != 0]
    if failed:
        raise subprocess.CalledProcessError(1, f"nvcc -c {' '.join(failed)}")
    arch = NVCC_FLAGS[NVCC_FLAGS.index("-gencode"):NVCC_FLAGS.index("-gencode") + 2]
    subprocess.check_call([_nvcc(), *arch, "-shared", "-o", LIB_PATH, *objects, id_obj], env=env)
    return LIB_PATH


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
