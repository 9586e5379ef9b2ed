"""Builds libguffin_b200.so in-tree with nvcc for sm_100a (no JIT cache, no CPU fallback)."""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libguffin_b200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr", "-Xptxas", "-v"]


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cpp")))


TESTING_LIB = os.path.join(HERE, "libguffin_b200_testing.so")


def stale(lib: str = LIB) -> bool:
    if not os.path.exists(lib):
        return True
    built = os.path.getmtime(lib)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(HERE, "..", "include", "guffin_b200.h")]
    return any(os.path.getmtime(d) > built for d in deps)


def build(force: bool = False, verbose: bool = False, testing: bool = False) -> str:
    """Compiles every source and links the library.  `testing` builds the variant with the host-side
    fault seam (-DGF_TESTING, libguffin_b200_testing.so) that only the give-up tests load."""
    lib = TESTING_LIB if testing else LIB
    if not force and not stale(lib):
        return lib
    objects = []
    out_dir = os.path.join(HERE, "build", "testing" if testing else "")
    os.makedirs(out_dir, exist_ok=True)
    procs = []
    for src in sources():
        obj = os.path.join(out_dir, os.path.basename(src) + ".o")
        objects.append(obj)
        cmd = [NVCC, *FLAGS, *(["-DGF_TESTING"] if testing else []), "-x", "cu", "-c", src, "-o", obj]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, proc in procs:
        out, _ = proc.communicate()
        if verbose or proc.returncode != 0:
            sys.stderr.write(out)
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}")
        with open(os.path.join(out_dir, os.path.basename(src) + ".ptxas.txt"), "w") as f:
            f.write(out)
    subprocess.run([NVCC, "-shared", "-o", lib, *objects, "-lcudart"], check=True)
    return lib


TP_LIB = os.path.join(HERE, "libguffin_tp.so")


def build_tp(force: bool = False) -> str | None:
    """The NCCL reduction hook of the optional tensor-parallel mode (libguffin_tp.so); None where NCCL's
    header or library is not installed."""
    src = os.path.join(HERE, "csrc_tp", "tp_nccl.cpp")
    if not force and os.path.exists(TP_LIB) and os.path.getmtime(TP_LIB) >= os.path.getmtime(src):
        return TP_LIB
    cuda = os.path.dirname(os.path.dirname(NVCC))
    cmd = [os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", f"-I{cuda}/include", src,
           "-o", TP_LIB, f"-L{cuda}/lib64", "-lnccl", "-lcudart"]
    done = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if done.returncode != 0:
        sys.stderr.write("libguffin_tp.so not built (NCCL absent?):\n" + done.stdout[-600:])
        return None
    return TP_LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, testing=True))
    print(build_tp(force="--force" in sys.argv))
