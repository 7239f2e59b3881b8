"""Build libssconv_b200.so (the C-ABI CUDA library) in-tree for sm_100a with nvcc.

Usage: python ss-conv_b200/build.py [--force] [--verbose]
The shared library is written next to the Python package (ss_conv/libssconv_b200.so) so that
it travels with the source tree; no JIT cache is involved.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "ss_conv", "libssconv_b200.so")
SOURCES = ["ssc_error.cu", "ssc_rulebook.cu", "ssc_conv.cu", "ssc_conv_tc.cu", "ssc_conv_stage.cu", "ssc_conv_pairs.cu", "ssc_backward.cu", "ssc_order.cu", "ssc_wgrad_tc.cu", "ssc_pool.cu", "ssc_voxel.cu",
           "ssc_bnact.cu", "ssc_ceiling.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC"]


def _nvcc():
    home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cand = os.path.join(home, "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def _newest_input():
    files = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(HERE, "..", "include", "ssconv_b200.h")]
    return max(os.path.getmtime(f) for f in files if os.path.exists(f))


def build(force=False, verbose=False):
    sources = [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    if os.path.exists(LIB) and not force and os.path.getmtime(LIB) >= _newest_input():
        return LIB
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    nvcc = _nvcc()
    flags = list(NVCC_FLAGS)

    def compile_one(src):
        obj = os.path.join(objdir, src + ".o")
        cmd = [nvcc, "-c", os.path.join(CSRC, src), "-o", obj] + flags + (["-Xptxas", "-v"] if verbose else [])
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed on %s:\n%s" % (src, r.stderr[-6000:]))
        if verbose:
            print(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(compile_one, sources))
    r = subprocess.run([nvcc, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static"],
                       capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed:\n" + r.stderr[-4000:])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
