"""In-tree build of the native runtime ``horovod_b200/_C.so``.

The C++ core and transport compile with g++, the kernels with nvcc for
sm_100a only, and everything links into one pybind11 module next to the
Python sources (no JIT cache, no site-packages install). A ninja file is
generated under ``build/`` so rebuilds are incremental and parallel.

Run ``python horovod_b200/build_ext.py`` (add ``-v`` for the command lines).

Parity: the reference drives CMake from setup.py (setup.py:30-98,
CMakeLists.txt:103-265); this build has one target and no feature switches.
"""
import os
import subprocess
import sys
import sysconfig

PKG = os.path.dirname(os.path.abspath(__file__))
# When run as a script the package directory lands on sys.path, where its
# "torch" subpackage would shadow PyTorch.
sys.path[:] = [p for p in sys.path if os.path.abspath(p or ".") != PKG]
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
BUILD = os.path.join(ROOT, "build")
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")

NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _sources():
    cxx, cu = [], []
    for base, _dirs, files in os.walk(CSRC):
        for f in sorted(files):
            p = os.path.join(base, f)
            if f.endswith((".cc", ".cpp")):
                cxx.append(p)
            elif f.endswith(".cu"):
                cu.append(p)
    return sorted(cxx), sorted(cu)


def _torch_paths():
    import torch
    from torch.utils import cpp_extension
    inc = cpp_extension.include_paths()
    lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    return inc, lib, abi


def _nccl_include():
    try:
        import nvidia.nccl
        p = os.path.join(os.path.dirname(nvidia.nccl.__path__[0] + "/x"), "include")
        if os.path.exists(os.path.join(p, "nccl.h")):
            return p
    except Exception:
        pass
    return "/usr/include"


def rule_for(src):
    return "nvcc" if src.endswith(".cu") else "cxx"


def write_ninja():
    import pybind11
    os.makedirs(BUILD, exist_ok=True)
    torch_inc, torch_lib, abi = _torch_paths()
    cxx_srcs, cu_srcs = _sources()
    includes = [CSRC, os.path.join(CUDA_HOME, "include"),
                sysconfig.get_paths()["include"], pybind11.get_include(),
                _nccl_include()] + torch_inc
    inc_flags = " ".join("-I" + p for p in includes)
    common = ("-O2 -std=c++17 -fPIC -fvisibility=hidden -Wall -Wno-sign-compare "
              "-Wno-unused-function -D_GLIBCXX_USE_CXX11_ABI=%d "
              "-DTORCH_EXTENSION_NAME=_C -DTORCH_API_INCLUDE_EXTENSION_H" % abi)
    nvcc_flags = (" ".join(NVCC_ARCH) + " -lineinfo -O3 -std=c++17 "
                  "--expt-relaxed-constexpr -Xcompiler -fPIC "
                  "-Xcompiler -fvisibility=hidden "
                  "-D_GLIBCXX_USE_CXX11_ABI=%d" % abi)
    # HOROVOD_B200_SANITIZE=address|undefined|thread instruments the host code
    # (objects go to their own directory; the module is linked in place, so
    # rebuild without the variable afterwards). Run the CPU tests with the
    # matching runtime preloaded, e.g.
    #   LD_PRELOAD=$(g++ -print-file-name=libasan.so) ASAN_OPTIONS=detect_leaks=0 pytest ...
    sanitize = os.environ.get("HOROVOD_B200_SANITIZE", "")
    link_extra = ""
    if sanitize:
        common = common.replace("-O2", "-O1 -g -fno-omit-frame-pointer") + \
            " -fsanitize=%s" % sanitize
        link_extra = " -fsanitize=%s" % sanitize
    if os.environ.get("HVD_PTXAS_VERBOSE"):
        nvcc_flags += " -Xptxas -v"
    out = os.path.join(PKG, "_C.so")
    lines = [
        "ninja_required_version = 1.3",
        "cxx = g++",
        "nvcc = %s" % os.path.join(CUDA_HOME, "bin", "nvcc"),
        "rule cxx",
        "  command = $cxx -MMD -MF $out.d %s %s -c $in -o $out" % (common, inc_flags),
        "  depfile = $out.d",
        "  deps = gcc",
        "rule nvcc",
        "  command = $nvcc %s -I%s -I%s -MD -MF $out.d -c $in -o $out"
        % (nvcc_flags, CSRC, os.path.join(CUDA_HOME, "include")),
        "  depfile = $out.d",
        "  deps = gcc",
        "rule link",
        "  command = $cxx -shared $in -o $out -L%s -ltorch -ltorch_cpu "
        "-ltorch_python -lc10 -ltorch_cuda -lc10_cuda -L%s -lcudart -lpthread -ldl "
        "-Wl,-rpath,%s -Wl,--no-undefined-version%s"
        % (torch_lib, os.path.join(CUDA_HOME, "lib64"), torch_lib, link_extra),
    ]
    objs = []
    for src in cxx_srcs + cu_srcs:
        rel = os.path.relpath(src, CSRC).replace(os.sep, "_")
        obj = os.path.join(BUILD, ("san_" + sanitize + "_" if sanitize and rule_for(src) == "cxx"
                                   else "") + rel + ".o")
        objs.append(obj)
        rule = "nvcc" if src.endswith(".cu") else "cxx"
        lines.append("build %s: %s %s" % (obj, rule, src))
    lines.append("build %s: link %s" % (out, " ".join(objs)))
    lines.append("default %s" % out)
    path = os.path.join(BUILD, "build.ninja")
    text = "\n".join(lines) + "\n"
    old = open(path).read() if os.path.exists(path) else None
    if old != text:
        with open(path, "w") as f:
            f.write(text)
    return path, out


def build(verbose=False):
    """Compiles whatever is out of date and returns the path of the module."""
    path, out = write_ninja()
    cmd = ["ninja", "-C", BUILD, "-f", path]
    if verbose:
        cmd.append("-v")
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                         text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout)
    if res.returncode != 0:
        raise RuntimeError("building horovod_b200._C failed (see output above)")
    return out


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv))
