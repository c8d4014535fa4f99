"""Build the UNMODIFIED reference CUDA extension for sm_100a into oracle/_ref/ (test infrastructure only).

The three reference sources (extension/csrc/K_cache.cu, V_cache.cu, KV_cache_ops.cpp) are compiled where they
lie in the reference checkout; nothing is copied into this repository and the only output is
``oracle/_ref/kv_cache_cuda.so`` (git-ignored).  The reference's own loader
(extension/KV_cache_cpp_extention.py:6-9) cannot be used because it hard-codes ``-ccbin=/usr/bin/gcc-10``.

The resulting module is the bit-exact checker that the ``-m gpu`` parity tests and the golden-vector generator
(tests/golden/make_golden_gpu.py) load when it is present.  It is never imported by the product package.

`vendor()` additionally copies the reference checkout (a dozen small files) to ``baseline/_ref/`` (git-ignored), so that
the GPU tests can import the reference's own model/KVCache_AlignedKV.py unchanged on a machine that has no checkout.

Usage:  python oracle/build_ref.py [/path/to/reference]      (default: $AKV_REFERENCE_ROOT, else ../reference)
"""
import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
OUT = os.path.join(HERE, "_ref")
VENDOR = os.path.join(ROOT, "baseline", "_ref")


def default_reference_root() -> str | None:
    """$AKV_REFERENCE_ROOT, else a directory `reference` next to this repository; None when neither exists."""
    for cand in (os.environ.get("AKV_REFERENCE_ROOT"), os.path.join(os.path.dirname(ROOT), "reference")):
        if cand and os.path.isdir(os.path.join(cand, "extension", "csrc")):
            return cand
    return None


def vendor(ref_root: str) -> str:
    """Copy the reference checkout to baseline/_ref (git-ignored; it travels to the GPU box with the working tree)."""
    def ignore(_dir, names):
        return [n for n in names if n in (".git", "__pycache__")]
    if os.path.isdir(VENDOR):
        shutil.rmtree(VENDOR)
    shutil.copytree(ref_root, VENDOR, ignore=ignore)
    return VENDOR


def build(ref_root: str, verbose: bool = True) -> str | None:
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
    root = sys.argv[1] if len(sys.argv) > 1 else default_reference_root()
    if root is None:
        raise SystemExit("no reference checkout: pass its path or set AKV_REFERENCE_ROOT")
    print("built:", build(root))
    print("vendored:", vendor(root))
