"""Compile the CUDA sources in csrc/ for sm_100a into lib/libmc_b200.so (in-tree).

    python -m mappedconvolutions_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU.  Objects are rebuilt only when a source or header is newer.
"""
import concurrent.futures as cf
import glob
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIBDIR = os.path.join(PKG, "lib")
LIB = os.path.join(LIBDIR, "libmc_b200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC", "-I", os.path.join(ROOT, "include"), "-I", CSRC]


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    os.makedirs(LIBDIR, exist_ok=True)
    objdir = os.path.join(PKG, "build")
    os.makedirs(objdir, exist_ok=True)
    srcs = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    hdrs = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(ROOT, "include", "*.h"))
    jobs = []
    for s in srcs:
        o = os.path.join(objdir, os.path.basename(s)[:-3] + ".o")
        if force or _newer(o, [s] + hdrs):
            cmd = [NVCC] + FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", s, "-o", o]
            jobs.append((s, cmd))

    def run(job):
        s, cmd = job
        r = subprocess.run(cmd, capture_output=True, text=True)
        return s, r

    with cf.ThreadPoolExecutor(max(1, min(8, len(jobs)))) as ex:
        for s, r in ex.map(run, jobs):
            if verbose or r.returncode:
                sys.stderr.write(r.stdout + r.stderr)
            if r.returncode:
                raise RuntimeError("nvcc failed on " + s)
    objs = [os.path.join(objdir, os.path.basename(s)[:-3] + ".o") for s in srcs]
    if force or jobs or _newer(LIB, objs):
        cmd = [NVCC, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return LIB


TORCH_EXT_SRC = os.path.join(PKG, "csrc_torch", "mc_torch_ext.cpp")
TORCH_EXT_NAME = "_mc_torch_ext"


def torch_ext_path():
    import sysconfig
    return os.path.join(PKG, TORCH_EXT_NAME + sysconfig.get_config_var("EXT_SUFFIX"))


def build_torch_ext(force=False):
    """Compiles the PyTorch C++ extension (the reference's pybind surface on top of the C ABI)
    in-tree with the host compiler; it links against libmc_b200.so through an $ORIGIN rpath."""
    import sysconfig
    import torch
    from torch.utils import cpp_extension as ce
    out = torch_ext_path()
    hdrs = glob.glob(os.path.join(ROOT, "include", "*.h"))
    if not force and not _newer(out, [TORCH_EXT_SRC, LIB] + hdrs):
        return out
    # The plain system compiler.  ($CXX is deliberately not consulted: a compiler wrapper that
    # reorders the system include directories produced an extension whose error messages crashed
    # while formatting integers; MC_CXX overrides.)
    cxx = os.environ.get("MC_CXX", "g++")
    cuda_inc = os.path.join(os.path.dirname(os.path.dirname(NVCC)), "include")
    cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-Wno-deprecated-declarations",
           "-DTORCH_EXTENSION_NAME=" + TORCH_EXT_NAME, "-DTORCH_API_INCLUDE_EXTENSION_H",
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch.compiled_with_cxx11_abi())]
    for inc in ce.include_paths() + [sysconfig.get_paths()["include"], cuda_inc,
                                     os.path.join(ROOT, "include")]:
        cmd += ["-I", inc]
    cmd += [TORCH_EXT_SRC, "-o", out]
    for lp in ce.library_paths():
        cmd += ["-L", lp, "-Wl,-rpath," + lp]
    cmd += ["-lc10", "-ltorch", "-ltorch_cpu", "-ltorch_python", "-lc10_cuda",
            "-L", LIBDIR, "-lmc_b200", "-Wl,-rpath,$ORIGIN/lib"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("compiling the torch extension failed")
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    print(build_torch_ext(force="--force" in sys.argv))
