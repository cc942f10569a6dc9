"""Builds the device library (libendia_b200.so) in-tree with nvcc for sm_100a.

Usage: python -m endia_b200.build [--force]
The library lands in endia_b200/lib/ so that it travels with the source tree.
"""
import hashlib
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
LIBPATH = os.path.join(LIBDIR, "libendia_b200.so")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Wno-deprecated-gpu-targets",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-O3",
]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _digest():
    h = hashlib.sha256()
    files = sources() + sorted(
        os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cuh"))
    files.append(os.path.join(INCLUDE, "endia_b200.h"))
    for f in files:
        h.update(os.path.basename(f).encode())  # not the absolute path: the tree may be relocated
        with open(f, "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def build(force=False, verbose=False):
    """Compile every .cu under csrc/ and link the shared library. Returns its path."""
    os.makedirs(LIBDIR, exist_ok=True)
    stamp = os.path.join(LIBDIR, "build.stamp")
    digest = _digest()

    def fresh():
        if not force and os.path.exists(LIBPATH) and os.path.exists(stamp):
            with open(stamp) as fh:
                return fh.read().strip() == digest
        return False
    if fresh():
        return LIBPATH
    # Several ranks may import the package at once: only one of them compiles.
    import fcntl
    lock = open(os.path.join(LIBDIR, "build.lock"), "w")
    fcntl.flock(lock, fcntl.LOCK_EX)
    try:
        if fresh():
            return LIBPATH
        return _compile(digest, stamp, verbose)
    finally:
        fcntl.flock(lock, fcntl.LOCK_UN)
        lock.close()


def _compile(digest, stamp, verbose):
    nvcc = _nvcc()
    objs = []
    procs = []
    for src in sources():
        obj = os.path.join(LIBDIR, os.path.basename(src)[:-3] + ".o")
        cmd = [nvcc] + NVCC_FLAGS + ["-I", INCLUDE, "-c", src, "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)))
        objs.append(obj)
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode != 0:
            sys.stderr.write(out.decode(errors="replace"))
        if p.returncode != 0:
            failed = True
            sys.stderr.write("nvcc failed on %s\n" % src)
    if failed:
        raise RuntimeError("building libendia_b200.so failed")
    link = [nvcc, "-Wno-deprecated-gpu-targets", "-shared", "-o", LIBPATH] + objs + ["-lcudart", "-ldl"]
    subprocess.check_call(link)
    with open(stamp, "w") as fh:
        fh.write(digest)
    return LIBPATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
