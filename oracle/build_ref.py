"""Build the reference's own CPU extensions into oracle/_ref/ (test infrastructure only).

The sources are compiled where they lie in the reference checkout (never copied):
package/ext_modules/src/nn/cpp/*.cpp and src/util/cpp/sphere.cpp, with the reference's own
flags from package/setup.py:36-44 (-fopenmp -O3 -D__NO_CUDA__).  Outputs are the pybind
modules `_mapped_convolution_ext.<name>` as .so files under oracle/_ref/_mapped_convolution_ext/.

This directory is the *checker* and the timed CPU baseline.  Nothing in the product package may
import it.

Usage:  python oracle/build_ref.py [--ref /path/to/reference] [--jobs N] [module ...]
"""
import argparse
import concurrent.futures as cf
import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref", "_mapped_convolution_ext")

# module name -> source file relative to package/ext_modules (package/setup.py:56-95)
MODULES = {
    "_mapped_convolution": "src/nn/cpp/mapped_convolution_layer.cpp",
    "_mapped_transposed_convolution": "src/nn/cpp/mapped_transposed_convolution_layer.cpp",
    "_mapped_max_pooling": "src/nn/cpp/mapped_max_pooling_layer.cpp",
    "_mapped_avg_pooling": "src/nn/cpp/mapped_avg_pooling_layer.cpp",
    "_resample": "src/nn/cpp/resample_layer.cpp",
    "_weighted_mapped_convolution": "src/nn/cpp/weighted_mapped_convolution_layer.cpp",
    "_weighted_mapped_transposed_convolution":
        "src/nn/cpp/weighted_mapped_transposed_convolution_layer.cpp",
    "_weighted_mapped_max_pooling": "src/nn/cpp/weighted_mapped_max_pooling_layer.cpp",
    "_weighted_mapped_avg_pooling": "src/nn/cpp/weighted_mapped_avg_pooling_layer.cpp",
    "_weighted_resample": "src/nn/cpp/weighted_resample_layer.cpp",
    "_sphere": "src/util/cpp/sphere.cpp",
    # not on the hot path; only needed so that the reference's `mapped_convolution.nn` package,
    # which imports every layer module, can be imported when the golden vectors are generated
    "_voting_resample": "src/nn/cpp/voting_resample_layer.cpp",
    "_convolution": "src/nn/cpp/convolution_layer.cpp",
    "_transposed_convolution": "src/nn/cpp/transposed_convolution_layer.cpp",
}


def _gomp_dir():
    for d in sorted(glob.glob("/usr/lib/gcc/x86_64-linux-gnu/*"), reverse=True):
        if glob.glob(os.path.join(d, "libgomp.so*")):
            return d
    return None


def build_one(name, ref_root):
    import sysconfig
    import torch
    from torch.utils import cpp_extension as ce

    ext = os.path.join(ref_root, "package", "ext_modules")
    src = os.path.join(ext, MODULES[name])
    os.makedirs(OUT, exist_ok=True)
    so = os.path.join(OUT, name + ".so")
    if os.path.exists(so) and os.path.getmtime(so) >= os.path.getmtime(src):
        return name, "cached"
    inc = [os.path.join(ext, "include")] + ce.include_paths() + [sysconfig.get_paths()["include"]]
    cmd = ["g++", "-shared", "-fPIC", "-O3", "-fopenmp", "-std=c++17", "-w",
           "-DTORCH_EXTENSION_NAME=" + name, "-DTORCH_API_INCLUDE_EXTENSION_H",
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)]
    if name != "_sphere":
        cmd.append("-D__NO_CUDA__")
    for i in inc:
        cmd += ["-isystem", i]
    cmd += [src, "-o", so]
    libdir = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd += ["-L" + libdir, "-Wl,-rpath," + libdir,
            "-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python"]
    g = _gomp_dir()
    if g:
        cmd += ["-L" + g]
    cmd += ["-lgomp"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        if os.path.exists(so):
            os.remove(so)
        return name, "FAILED\n" + r.stderr[-3000:]
    return name, "built"


# CUDA-only utility modules of the reference: name -> (kernel source, binding source)
CUDA_MODULES = {
    "_knn": ("src/util/cuda/knn_layer.cu", "src/util/cpp/knn_layer.cpp"),
    "_cube2rect": ("src/util/cuda/cube2rect_layer.cu", "src/util/cpp/cube2rect_layer.cpp"),
}


def build_cuda_module(ref_root, name):
    """One of the reference's CUDA-only utility modules, compiled for sm_100a with nvcc from the
    sources where they lie (kernel source + the .cpp that holds the pybind binding).

    _knn: src/util/cuda/knn_layer.cu + include/util/cuda/knn.cuh.  The reference gives its kernels a
    (k, N) buffer but indexes it as an (M, N) distance matrix (knn_layer.cu:20-23 against
    knn.cuh:111-112, :144-187), so it is only ever run with M == k, where every access stays inside
    the buffers; tests/golden/make_golden_knn.py enforces that.
    _cube2rect: src/util/cuda/cube2rect_layer.cu + include/util/cuda/cube2rect.cuh.  Its bilinear
    branch can read one element past the cube map (the right neighbour of the last face's last
    pixel, weight zero); tests/golden/make_golden_cube2rect.py hands it a view into a larger zeroed
    buffer so that this read stays inside an allocation."""
    import sysconfig
    import torch
    from torch.utils import cpp_extension as ce
    ext = os.path.join(ref_root, "package", "ext_modules")
    cu = os.path.join(ext, CUDA_MODULES[name][0])
    cpp = os.path.join(ext, CUDA_MODULES[name][1])
    os.makedirs(OUT, exist_ok=True)
    so = os.path.join(OUT, name + ".so")
    if os.path.exists(so) and os.path.getmtime(so) >= os.path.getmtime(cu):
        return name, "cached"
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    inc = [os.path.join(ext, "include")] + ce.include_paths() + [sysconfig.get_paths()["include"],
                                                                 os.path.join(os.path.dirname(os.path.dirname(nvcc)), "include")]
    defs = ["-DTORCH_EXTENSION_NAME=" + name, "-DTORCH_API_INCLUDE_EXTENSION_H",
            "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)]
    obj_cu, obj_cpp = so + ".cu.o", so + ".cpp.o"
    cmd1 = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-w", "-Xcompiler",
            "-fPIC"] + defs + sum((["-isystem", i] for i in inc), []) + ["-c", cu, "-o", obj_cu]
    cmd2 = ["g++", "-fPIC", "-O2", "-std=c++17", "-w"] + defs + sum((["-isystem", i] for i in inc), []) + \
           ["-c", cpp, "-o", obj_cpp]
    libdir = os.path.join(os.path.dirname(torch.__file__), "lib")
    cudalib = os.path.join(os.path.dirname(os.path.dirname(nvcc)), "lib64")
    cmd3 = ["g++", "-shared", obj_cu, obj_cpp, "-o", so, "-L" + libdir, "-Wl,-rpath," + libdir, "-lc10",
            "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-L" + cudalib,
            "-lcudart"]
    for cmd in (cmd1, cmd2, cmd3):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            return name, "FAILED\n" + r.stderr[-3000:]
    for o in (obj_cu, obj_cpp):
        os.remove(o)
    return name, "built"


def build_knn(ref_root):
    return build_cuda_module(ref_root, "_knn")


def default_reference_root():
    """$MC_REFERENCE_ROOT, else a checkout named `reference` beside this repository."""
    return os.environ.get("MC_REFERENCE_ROOT",
                          os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=default_reference_root())
    ap.add_argument("--knn", action="store_true", help="also build the reference's CUDA k-NN module")
    ap.add_argument("--cube2rect", action="store_true", help="also build the reference's CUDA cube2rect module")
    ap.add_argument("--jobs", type=int, default=min(8, os.cpu_count() or 1))
    ap.add_argument("modules", nargs="*")
    a = ap.parse_args()
    if not os.path.isdir(os.path.join(a.ref, "package", "ext_modules")):
        print("reference checkout not found at", a.ref, "- nothing built")
        return 0
    names = a.modules or list(MODULES)
    ok = True
    with cf.ThreadPoolExecutor(a.jobs) as ex:
        for name, status in ex.map(lambda n: build_one(n, a.ref), names):
            print(name, status, flush=True)
            ok &= not status.startswith("FAILED")
    for flag, cuda_name in ((a.knn, "_knn"), (a.cube2rect, "_cube2rect")):
        if flag:
            name, status = build_cuda_module(a.ref, cuda_name)
            print(name, status, flush=True)
            ok &= not status.startswith("FAILED")
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
