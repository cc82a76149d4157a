"""Build the reference's own `torchac_cuda` extension, unmodified, into oracle/_ref/.

TEST INFRASTRUCTURE ONLY.  The sources are compiled where they lie in the
reference checkout (LMCache/third_party/torchac_cuda: main.cpp, cal_cdf.cu,
torchac_kernel_enc_new.cu, torchac_kernel_dec_new.cu -- the list in the
reference's setup.py:7-14); nothing is copied.  Only object files and the final
shared object are written, and only under oracle/_ref/ (git-ignored).

The result is a CUDA extension: it cannot run without a GPU.  The GPU tests and
tests/golden/make_golden_gpu.py use it, when it is present, as the bit-exact
authority for CDF tables, encoded streams and decoded symbols.

Usage:  python oracle/build_ref.py [--ref /path/to/reference] [--force]
"""
import argparse
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
SRC_REL = "LMCache/third_party/torchac_cuda"
SOURCES = ["main.cpp", "cal_cdf.cu", "torchac_kernel_enc_new.cu", "torchac_kernel_dec_new.cu"]


def target_path():
    return os.path.join(OUT, "torchac_cuda" + sysconfig.get_config_var("EXT_SUFFIX"))


def build(ref_root, force=False, verbose=True):
    src_dir = os.path.join(ref_root, SRC_REL)
    if not os.path.isdir(src_dir):
        raise FileNotFoundError(src_dir)
    target = target_path()
    srcs = [os.path.join(src_dir, s) for s in SOURCES]
    if (not force and os.path.exists(target)
            and all(os.path.getmtime(target) >= os.path.getmtime(s) for s in srcs)):
        return target
    import torch  # noqa: F401  (only for its header / library locations)
    from torch.utils import cpp_extension as ce
    os.makedirs(OUT, exist_ok=True)
    inc = []
    for p in ce.include_paths("cuda") + [sysconfig.get_paths()["include"], os.path.join(src_dir, "include")]:
        inc += ["-I", p]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    defs = ["-DTORCH_EXTENSION_NAME=torchac_cuda", "-DTORCH_API_INCLUDE_EXTENSION_H",
            f"-D_GLIBCXX_USE_CXX11_ABI={abi}"]
    nvcc = os.path.join(ce.CUDA_HOME or "/usr/local/cuda", "bin", "nvcc")

    def compile_one(src):
        obj = os.path.join(OUT, os.path.basename(src) + ".o")
        if src.endswith(".cu"):
            cmd = [nvcc, "-c", src, "-o", obj, "-O3", "-std=c++17", "--expt-relaxed-constexpr",
                   "-gencode", "arch=compute_100,code=sm_100", "-Xcompiler", "-fPIC",
                   "-D__CUDA_NO_HALF_OPERATORS__", "-D__CUDA_NO_HALF_CONVERSIONS__",
                   "-D__CUDA_NO_HALF2_OPERATORS__", "-w"] + defs + inc
        else:
            cmd = ["g++", "-c", src, "-o", obj, "-O2", "-std=c++17", "-fPIC", "-w"] + defs + inc
        if verbose:
            print("[build_ref]", os.path.basename(src), flush=True)
        subprocess.check_call(cmd)
        return obj

    with ThreadPoolExecutor(max_workers=4) as ex:
        objs = list(ex.map(compile_one, srcs))
    libs = []
    for p in ce.library_paths("cuda"):
        libs += ["-L", p, f"-Wl,-rpath,{p}"]
    link = ["g++", "-shared", "-o", target] + objs + libs + [
        "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"]
    subprocess.check_call(link)
    for o in objs:
        os.remove(o)
    if verbose:
        print("[build_ref] wrote", target, flush=True)
    return target


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("CACHEGEN_REFERENCE_ROOT", "/root/reference"))
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    try:
        build(a.ref, a.force)
    except FileNotFoundError as e:
        print("reference sources not found:", e, file=sys.stderr)
        sys.exit(1)
