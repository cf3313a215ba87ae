"""Build recipe for the checker-side native code (test infrastructure, not product).

Two artefacts, both written under ``oracle/``:

* ``oracle/liblrqk_oracle.so`` -- the plain-C restatement in ``lrqk_oracle.c``
  (gcc, OpenMP).
* ``oracle/_ref/take_along_dim_grouped*.so`` -- the reference project's own CPU
  row-gather extension (``cpp_kernel/take_along_dim_grouped.cpp``), compiled
  from the sources where they lie in the reference checkout with ``g++``
  against the torch headers.  Nothing is copied from the reference; only the
  built object lands in ``oracle/_ref/`` (git-ignored).  When the reference
  checkout is absent the step is skipped and a previously built file is used.

Run: ``python oracle/build_ref.py [--reference /path/to/reference]``.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
# a checkout of the reference project: LRQK_REFERENCE_DIR, else a directory "reference" beside this repository
DEFAULT_REFERENCE = os.environ.get("LRQK_REFERENCE_DIR",
                                   os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))


def build_c_oracle(verbose: bool = False) -> str:
    src = os.path.join(HERE, "lrqk_oracle.c")
    out = os.path.join(HERE, "liblrqk_oracle.so")
    if os.path.exists(out) and os.path.getmtime(out) >= os.path.getmtime(src):
        return out
    cmd = ["gcc", "-O3", "-march=x86-64-v2", "-fopenmp", "-fPIC", "-shared",
           "-std=c11", "-Wall", "-o", out, src, "-lm"]
    if verbose:
        print(" ".join(cmd))
    subprocess.check_call(cmd)
    return out


def ref_ext_path() -> str:
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return os.path.join(HERE, "_ref", "take_along_dim_grouped" + suffix)


def build_reference_ext(reference_dir: str = DEFAULT_REFERENCE, verbose: bool = False):
    """Compile the reference's pybind11/ATen gather extension into oracle/_ref/."""
    src = os.path.join(reference_dir, "cpp_kernel", "take_along_dim_grouped.cpp")
    out = ref_ext_path()
    if not os.path.exists(src):
        return out if os.path.exists(out) else None
    if os.path.exists(out) and os.path.getmtime(out) >= os.path.getmtime(src):
        return out
    os.makedirs(os.path.dirname(out), exist_ok=True)
    import torch
    from torch.utils import cpp_extension as ce

    inc = []
    for p in ce.include_paths():
        inc += ["-isystem", p]
    inc += ["-isystem", sysconfig.get_paths()["include"]]
    libdir = os.path.join(os.path.dirname(torch.__file__), "lib")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = ["g++", "-O3", "-march=x86-64-v3", "-funroll-loops", "-fopenmp", "-DNDEBUG",
           "-std=c++17", "-fPIC", "-shared",
           "-DTORCH_EXTENSION_NAME=take_along_dim_grouped",
           "-DTORCH_API_INCLUDE_EXTENSION_H",
           f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
           *inc, src, "-o", out,
           f"-L{libdir}", "-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python",
           f"-Wl,-rpath,{libdir}"]
    if verbose:
        print(" ".join(cmd))
    subprocess.check_call(cmd)
    return out


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=DEFAULT_REFERENCE)
    ap.add_argument("-v", "--verbose", action="store_true")
    a = ap.parse_args()
    print("oracle C :", build_c_oracle(a.verbose))
    print("oracle/_ref:", build_reference_ext(a.reference, a.verbose))
    return 0


if __name__ == "__main__":
    sys.exit(main())
