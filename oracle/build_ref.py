"""Build the UNMODIFIED reference extension (SS_Conv_lib/src) into oracle/_ref/_ext*.so.

Test infrastructure only.  The reference sources are compiled where they lie (nothing is
copied); two stand-in headers under oracle/ref_shims/ replace headers that no longer exist
(THC/THC.h, google/dense_hash_map) and one stand-in source defines the `state` global.
The resulting module exports the reference's own 32 pybind functions
(SS_Conv_lib/src/ss_conv_ops_api.cpp:15-55) and is used as the parity checker and as the
timed CPU baseline.  Usage: python oracle/build_ref.py [reference_root]
"""
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from glob import glob

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")


def ref_ext_path():
    return os.path.join(OUT, "_ext" + sysconfig.get_config_var("EXT_SUFFIX"))


def build(ref_root=None, force=False, verbose=True):
    if ref_root is None:
        sys.path.insert(0, HERE)
        from ref_loader import reference_root
        ref_root = reference_root() or ""
    src = os.path.join(ref_root, "SS_Conv_lib", "src")
    target = ref_ext_path()
    if not os.path.isdir(src):
        return target if os.path.exists(target) else None
    if os.path.exists(target) and not force:
        return target
    from torch.utils import cpp_extension as ce
    import torch
    os.makedirs(os.path.join(OUT, "obj"), exist_ok=True)
    subdirs = sorted(d for d in glob(os.path.join(src, "*")) if os.path.isdir(d))
    sources = []
    for d in subdirs:
        sources += sorted(glob(os.path.join(d, "*.cpp"))) + sorted(glob(os.path.join(d, "*.cu")))
    sources += [os.path.join(src, "ss_conv_ops_api.cpp"), os.path.join(src, "ss_conv_ops.cu"),
                os.path.join(HERE, "ref_shims", "thc_state.cpp")]
    incs = [os.path.join(HERE, "ref_shims"), src] + subdirs + ce.include_paths("cuda") + \
        [sysconfig.get_path("include")]
    inc_flags = [f for i in incs for f in ("-I", i)]
    common = ["-DTORCH_EXTENSION_NAME=_ext", "-DTORCH_API_INCLUDE_EXTENSION_H",
              "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)]
    cuda_home = ce.CUDA_HOME or "/usr/local/cuda"
    nvcc = os.path.join(cuda_home, "bin", "nvcc")

    def compile_one(path):
        obj = os.path.join(OUT, "obj", os.path.basename(path) + ".o")
        if os.path.exists(obj) and os.path.getmtime(obj) >= os.path.getmtime(path) and not force:
            return obj
        if path.endswith(".cu"):
            cmd = [nvcc, "-c", path, "-o", obj, "-O2", "-std=c++17", "--expt-relaxed-constexpr",
                   "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC", "-w",
                   "-D__CUDA_NO_HALF_OPERATORS__", "-D__CUDA_NO_HALF_CONVERSIONS__",
                   "-D__CUDA_NO_BFLOAT16_CONVERSIONS__", "-D__CUDA_NO_HALF2_OPERATORS__"] + common + inc_flags
        else:
            cmd = ["g++", "-c", path, "-o", obj, "-O2", "-std=c++17", "-fPIC", "-w"] + common + inc_flags
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("reference build failed on %s:\n%s" % (path, r.stderr[-4000:]))
        if verbose:
            print("compiled", os.path.relpath(path, ref_root) if path.startswith(ref_root) else path, flush=True)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(compile_one, sources))
    libdirs = ce.library_paths("cuda")
    link = ["g++", "-shared", "-o", target] + objs + [f for l in libdirs for f in ("-L", l)] + \
        ["-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python", "-lc10_cuda", "-ltorch_cuda", "-lcudart"] + \
        ["-Wl,-rpath," + l for l in libdirs]
    r = subprocess.run(link, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("reference link failed:\n" + r.stderr[-4000:])
    return target


if __name__ == "__main__":
    p = build(*(sys.argv[1:2]), force="--force" in sys.argv)
    print("reference extension:", p)
