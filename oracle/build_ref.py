"""Build the UNMODIFIED reference CUDA extension for sm_100a into oracle/_ref/ (test infrastructure only).

The three reference sources (extension/csrc/K_cache.cu, V_cache.cu, KV_cache_ops.cpp) are compiled where they
lie in the reference checkout; nothing is copied into this repository and the only output is
``oracle/_ref/kv_cache_cuda.so`` (git-ignored).  The reference's own loader
(extension/KV_cache_cpp_extention.py:6-9) cannot be used because it hard-codes ``-ccbin=/usr/bin/gcc-10``.

The resulting module is the bit-exact checker that the ``-m gpu`` parity tests and the golden-vector generator
(tests/golden/make_golden_gpu.py) load when it is present.  It is never imported by the product package.

Usage:  python oracle/build_ref.py [/path/to/reference]
"""
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")


def build(ref_root: str = "/root/reference", verbose: bool = True) -> str | None:
    src_dir = os.path.join(ref_root, "extension", "csrc")
    srcs = [os.path.join(src_dir, f) for f in ("K_cache.cu", "V_cache.cu", "KV_cache_ops.cpp")]
    if not all(os.path.exists(s) for s in srcs):
        return None
    so = os.path.join(OUT, "kv_cache_cuda.so")
    if os.path.exists(so) and all(os.path.getmtime(so) >= os.path.getmtime(s) for s in srcs):
        return so
    import torch
    from torch.utils import cpp_extension as ce

    os.makedirs(OUT, exist_ok=True)
    incs = [f"-I{p}" for p in ce.include_paths("cuda")] + [f"-I{sysconfig.get_paths()['include']}"]
    common = incs + ["-DTORCH_EXTENSION_NAME=kv_cache_cuda", "-DTORCH_API_INCLUDE_EXTENSION_H",
                     f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}", "-std=c++17", "-O3"]
    jobs = []
    objs = []
    for s in srcs:
        o = os.path.join(OUT, os.path.basename(s) + ".o")
        objs.append(o)
        if s.endswith(".cu"):
            cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "--expt-relaxed-constexpr",
                   "-Xcompiler", "-fPIC", "-c", s, "-o", o] + common
        else:
            cmd = ["g++", "-fPIC", "-c", s, "-o", o] + common
        jobs.append(cmd)

    def run(cmd):
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.run(cmd, check=True)

    with ThreadPoolExecutor(max_workers=3) as ex:
        list(ex.map(run, jobs))
    libdirs = ce.library_paths("cuda")
    link = ["g++", "-shared", "-o", so] + objs + [f"-L{d}" for d in libdirs] + \
           ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"]
    run(link)
    return so


if __name__ == "__main__":
    r = build(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
    print("built:", r)
