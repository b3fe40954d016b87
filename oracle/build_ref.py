"""Recipe that stages the REFERENCE itself as a checker.  TEST INFRASTRUCTURE ONLY.

    python oracle/build_ref.py [/path/to/MorphServe-checkout]

Writes, into the git-ignored ``oracle/_ref/`` and nowhere else:

* ``MorphServe/``: the reference's Python package tree (its Triton kernels,
  worker, block manager, layers, server bookkeeping), staged unmodified.  The
  kernels are Triton source, so "building" them means letting Triton JIT-compile
  them for whatever GPU the tests run on; nothing is interpreted or patched.
* ``swiftllm_c*.so``: the reference's native extension, compiled with g++ from
  the three C++ files where they lie in the checkout (csrc/src/*.cpp: host-only
  C++ over the CUDA runtime and libtorch; the reference's own setup.py never
  invokes nvcc either).

Nothing under ``oracle/_ref/`` is committed and nothing in ``morphserve_b200/``
may import it: ``tests/`` use it to hold the CUDA path to the reference's own
output at full size, and ``bench.py`` times it as a comparison column.  Without
a checkout (or when the directory has not been staged) those tests skip and the
bench column says so.
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
DEFAULT_CHECKOUT = "/root/reference"


def _make_writable(tree: str) -> None:
    for root, dirs, files in os.walk(tree):
        for n in dirs + files:
            p = os.path.join(root, n)
            os.chmod(p, os.stat(p).st_mode | 0o200)
    os.chmod(tree, os.stat(tree).st_mode | 0o200)


def stage_python(checkout: str) -> str:
    src = os.path.join(checkout, "MorphServe")
    dst = os.path.join(OUT, "MorphServe")
    if os.path.isdir(dst):
        _make_writable(dst)
        shutil.rmtree(dst)
    shutil.copytree(src, dst, ignore=shutil.ignore_patterns("__pycache__", "*.pyc", "*.png"))
    _make_writable(dst)      # a read-only checkout would otherwise leave a tree that cannot be restaged
    return dst


def ext_path() -> str:
    return os.path.join(OUT, "swiftllm_c" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))


def build_ext(checkout: str, verbose: bool = False) -> str:
    """g++ on csrc/src/*.cpp in place; the only output is oracle/_ref/swiftllm_c<abi>.so."""
    import torch
    from torch.utils import cpp_extension as CE

    srcdir = os.path.join(checkout, "csrc", "src")
    sources = sorted(glob.glob(os.path.join(srcdir, "*.cpp")))
    if not sources:
        raise RuntimeError(f"no C++ sources under {srcdir}")
    out = ext_path()
    newest = max(os.path.getmtime(s) for s in sources + glob.glob(os.path.join(srcdir, "*.h")))
    if os.path.exists(out) and os.path.getmtime(out) > newest:
        return out
    inc = CE.include_paths("cuda") if "device_type" in CE.include_paths.__code__.co_varnames else CE.include_paths(True)
    inc += [sysconfig.get_paths()["include"], srcdir]
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cuda_home = CE.CUDA_HOME or "/usr/local/cuda"
    cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-w",
           "-DTORCH_EXTENSION_NAME=swiftllm_c", "-DTORCH_API_INCLUDE_EXTENSION_H",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    for i in inc:
        cmd += ["-isystem", i]
    cmd += sources
    cmd += ["-o", out, f"-L{torch_lib}", f"-Wl,-rpath,{torch_lib}", "-lc10", "-lc10_cuda", "-ltorch_cpu",
            "-ltorch_cuda", "-ltorch", "-ltorch_python", f"-L{os.path.join(cuda_home, 'lib64')}", "-lcudart"]
    if verbose:
        print(" ".join(cmd))
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("g++ failed on the reference's csrc:\n" + r.stdout + r.stderr[-4000:])
    return out


def build(checkout: str = DEFAULT_CHECKOUT, verbose: bool = False) -> dict:
    if not os.path.isdir(os.path.join(checkout, "MorphServe")):
        raise FileNotFoundError(f"{checkout} is not a MorphServe checkout")
    os.makedirs(OUT, exist_ok=True)
    res = {"python": stage_python(checkout)}
    try:
        res["ext"] = build_ext(checkout, verbose)
    except Exception as e:       # the Python half is still usable without the extension
        res["ext_error"] = str(e)
    return res


if __name__ == "__main__":
    args = [a for a in sys.argv[1:] if not a.startswith("-")]
    print(build(args[0] if args else DEFAULT_CHECKOUT, verbose="-v" in sys.argv))
