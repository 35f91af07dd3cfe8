"""Build the CUDA kernels of this package into one in-tree shared library.

``python -m dttt_b200.build`` compiles every ``csrc/*.cu`` for sm_100a with nvcc (object files in
``dttt_b200/lib/obj``) and links ``dttt_b200/lib/libdttt_b200.so``.  The library exposes a plain C ABI
(``extern "C"`` launchers that take device pointers and a stream) and is loaded with ``ctypes`` by
``dttt_b200.ops._lib``; it has no link-time dependency on libtorch or libcuda (the one driver call it
needs, the tensor-map encoder, is looked up through the runtime at first use), so it also loads on a
machine without a GPU.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
OBJDIR = os.path.join(LIBDIR, "obj")
LIBPATH = os.path.join(LIBDIR, "libdttt_b200.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v"]


def nvcc_path() -> str | None:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    return None


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _digest(path: str) -> str:
    h = hashlib.sha256()
    for p in [path] + sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))):
        with open(p, "rb") as f:
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _compile_one(nvcc: str, src: str, verbose: bool) -> tuple[str, str]:
    base = os.path.splitext(os.path.basename(src))[0]
    obj = os.path.join(OBJDIR, base + ".o")
    stamp = obj + ".sha"
    dig = _digest(src)
    if os.path.exists(obj) and os.path.exists(stamp) and open(stamp).read() == dig:
        return obj, ""
    cmd = [nvcc, *NVCC_FLAGS, "-c", src, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
    with open(stamp, "w") as f:
        f.write(dig)
    log = r.stderr if verbose else ""
    return obj, log


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile and link; returns the library path.  Unchanged sources are not recompiled."""
    nvcc = nvcc_path()
    if nvcc is None:
        raise RuntimeError("nvcc not found: the CUDA kernels cannot be built")
    os.makedirs(OBJDIR, exist_ok=True)
    if force:
        for f in os.listdir(OBJDIR):
            os.remove(os.path.join(OBJDIR, f))
    srcs = sources()
    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        results = list(ex.map(lambda s: _compile_one(nvcc, s, verbose), srcs))
    objs = [o for o, _ in results]
    for _, log in results:
        if log:
            print(log, file=sys.stderr)
    newest = max(os.path.getmtime(o) for o in objs)
    if force or not os.path.exists(LIBPATH) or os.path.getmtime(LIBPATH) < newest:
        tmp = LIBPATH + f".{os.getpid()}.tmp"             # link beside the target, then rename: a reader never sees half a library
        cmd = [nvcc, "-shared", "-o", tmp, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            if os.path.exists(tmp):
                os.remove(tmp)
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, LIBPATH)
    return LIBPATH


def is_built() -> bool:
    return os.path.exists(LIBPATH)


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
