"""Builds libcachegen_b200.so in-tree with nvcc for sm_100a (no torch headers: a few seconds per file).

    python -m cachegen_b200.build [--force] [--verbose]
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "libcachegen_b200.so")
SOURCES = ["cg_api.cu", "cg_quant.cu", "cg_tables.cu", "cg_encode.cu", "cg_decode.cu"]
HEADERS = [os.path.join(CSRC, "cg_common.cuh"), os.path.join(CSRC, "cg_coder.cuh"), os.path.join(PKG, "..", "include", "cachegen_b200.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC"]


def _nvcc():
    home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    return os.path.join(home, "bin", "nvcc")


def needs_build():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, s) for s in SOURCES] + HEADERS
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False, extra_flags=(), out=None):
    """Compiles the library and returns its path.  `out` builds a second copy elsewhere (with
    `extra_flags`, e.g. -D switches) without touching the in-tree one; CACHEGEN_B200_LIB selects it."""
    target = out or LIB
    if not out and not force and not needs_build():
        return target
    flags = NVCC_FLAGS + list(extra_flags)
    if verbose:
        flags = flags + ["-Xptxas", "-v"]
    obj_prefix = (out + ".") if out else (CSRC + os.sep)

    def one(src):
        obj = obj_prefix + src.replace(".cu", ".o")
        cmd = [_nvcc(), "-c", os.path.join(CSRC, src), "-o", obj] + flags
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            sys.stderr.write(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as ex:
        objs = list(ex.map(one, SOURCES))
    cmd = [_nvcc(), "-shared", "-o", target] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-lcudart"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return target


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
