"""Compile the reference's own host-side wave buffer into ``oracle/_ref``.
TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).

The single translation unit
``library/retroinfer/retroinfer_kernels/src/wave_buffer_cpu.cpp`` (with its header
``thread_pool.hpp``) is compiled where it lies in the reference checkout with one
``g++`` command; nothing is copied.  The result is a CPython extension module
``oracle/_ref/WaveBuffer*.so`` exposing ``WaveBufferCPU`` and ``ThreadPool`` exactly
as the reference's ``retroinfer_kernels`` package does.  ``-fopenmp`` is passed for
``<omp.h>`` at compile time only (this image has no ``libgomp.spec`` to link with,
and the file uses no OpenMP construct).

Run:  python -m oracle.build_ref [reference_root]
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
SRC_REL = "library/retroinfer/retroinfer_kernels/src/wave_buffer_cpu.cpp"


def default_reference_root() -> str:
    """``RI_REFERENCE_ROOT`` if set, else a checkout named ``reference`` beside this repository."""
    return os.environ.get("RI_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def module_path() -> str:
    return os.path.join(OUT_DIR, "WaveBuffer" + sysconfig.get_config_var("EXT_SUFFIX"))


def build(reference_root: str | None = None, force: bool = False) -> str | None:
    """Returns the path of the built module, or None when the reference checkout is
    not present (then a previously built module, if any, keeps being used)."""
    reference_root = reference_root or default_reference_root()
    out = module_path()
    src = os.path.join(reference_root, SRC_REL)
    if not os.path.exists(src):
        return out if os.path.exists(out) else None
    if os.path.exists(out) and not force and os.path.getmtime(out) >= os.path.getmtime(src):
        return out
    import torch
    from torch.utils import cpp_extension

    os.makedirs(OUT_DIR, exist_ok=True)
    inc = [f"-I{p}" for p in cpp_extension.include_paths()] + [f"-I{sysconfig.get_paths()['include']}"]
    lib_dir = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-O3", "-std=c++17", "-fPIC", "-shared", "-w",
           "-DTORCH_EXTENSION_NAME=WaveBuffer", "-DTORCH_API_INCLUDE_EXTENSION_H",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           *inc, src, "-o", out,
           f"-L{lib_dir}", f"-Wl,-rpath,{lib_dir}", "-lc10", "-ltorch", "-ltorch_cpu", "-ltorch_python"]
    subprocess.run(cmd, check=True)
    return out


def load():
    """Import the built module (None if it was never built)."""
    path = module_path()
    if not os.path.exists(path):
        return None
    import importlib.util
    import torch  # noqa: F401  (the module links against libtorch)

    spec = importlib.util.spec_from_file_location("WaveBuffer", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else None, force=True))
