"""Compile the reference's own native modules into ``oracle/_ref``.
TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).

Three translation units of ``library/retroinfer/retroinfer_kernels/src`` are compiled where they lie in the
reference checkout, one compiler command each; nothing is copied.  The results are CPython extension modules
with the names the reference's ``retroinfer_kernels`` package gives them:

* ``WaveBuffer``    ``wave_buffer_cpu.cpp`` (+ ``thread_pool.hpp``), ``g++``: ``WaveBufferCPU`` and ``ThreadPool``.
  ``-fopenmp`` is left out (this image has no ``libgomp.spec`` to link with, and the file uses no OpenMP
  construct).
* ``Copy``          ``gather_copy.cu`` (+ ``copy_kernel.cuh``), ``nvcc`` for sm_100a: ``gather_copy_vectors``,
  ``gather_copy_and_concat``, ``gather_copy_and_scatter``.
* ``gemm_softmax``  ``batch_gemm_softmax.cu`` (+ its two headers), ``nvcc`` for sm_100a against the header-only
  CUTLASS tree that ships inside the ``flashinfer`` package of this image (the reference expects a CUTLASS
  checkout beside it, README.md:33, unpinned) and ``oracle/shim/helper.h``, a stand-in for the one macro the
  file takes from CUTLASS's examples folder.

The two CUDA modules need a GPU to run: they are built here, travel with the repository to the GPU machine
and serve there as bit-level oracles of the score/softmax and copy operators and as the reference-side GPU
baseline.  Each nvcc command takes several minutes (torch headers).

Run:  python -m oracle.build_ref [reference_root]
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
SRC_DIR_REL = "library/retroinfer/retroinfer_kernels/src"
MODULES = {
    # name: (source, other files whose change forces a rebuild, compiler)
    "WaveBuffer": ("wave_buffer_cpu.cpp", ("thread_pool.hpp",), "g++"),
    "Copy": ("gather_copy.cu", ("copy_kernel.cuh",), "nvcc"),
    "gemm_softmax": ("batch_gemm_softmax.cu", ("batch_gemm_softmax.h", "batch_gemm_with_epilogue_visitor.h"), "nvcc"),
}


def default_reference_root() -> str:
    """``RI_REFERENCE_ROOT`` if set, else a checkout named ``reference`` beside this repository."""
    return os.environ.get("RI_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def module_path(name: str = "WaveBuffer") -> str:
    return os.path.join(OUT_DIR, name + sysconfig.get_config_var("EXT_SUFFIX"))


def cutlass_root() -> str | None:
    """The header-only CUTLASS tree inside the flashinfer package (include/ and tools/util/include/)."""
    try:
        import importlib.util
        spec = importlib.util.find_spec("flashinfer")
    except (ImportError, ValueError):
        return None
    if spec is None or not spec.submodule_search_locations:
        return None
    root = os.path.join(list(spec.submodule_search_locations)[0], "data", "cutlass")
    return root if os.path.isdir(os.path.join(root, "include", "cutlass")) else None


def _build_one(name: str, src_dir: str, force: bool) -> str | None:
    source, deps, compiler = MODULES[name]
    src = os.path.join(src_dir, source)
    out = module_path(name)
    if not os.path.exists(src):
        return out if os.path.exists(out) else None
    newest = max(os.path.getmtime(os.path.join(src_dir, f)) for f in (source, *deps) if os.path.exists(os.path.join(src_dir, f)))
    if os.path.exists(out) and not force and os.path.getmtime(out) >= newest:
        return out
    import torch
    from torch.utils import cpp_extension

    os.makedirs(OUT_DIR, exist_ok=True)
    inc = [f"-I{p}" for p in cpp_extension.include_paths()] + [f"-I{sysconfig.get_paths()['include']}"]
    lib_dir = os.path.join(os.path.dirname(torch.__file__), "lib")
    defs = [f"-DTORCH_EXTENSION_NAME={name}", "-DTORCH_API_INCLUDE_EXTENSION_H",
            f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    libs = [f"-L{lib_dir}", "-lc10", "-ltorch", "-ltorch_cpu", "-ltorch_python"]
    if compiler == "g++":
        cmd = ["g++", "-O3", "-std=c++17", "-fPIC", "-shared", "-w", *defs, *inc, src, "-o", out,
               f"-Wl,-rpath,{lib_dir}", *libs]
    else:
        if name == "gemm_softmax":
            cut = cutlass_root()
            if cut is None:
                return out if os.path.exists(out) else None
            inc += [f"-I{cut}/include", f"-I{cut}/tools/util/include", f"-I{os.path.join(HERE, 'shim')}"]
        cmd = ["nvcc", "-O3", "-std=c++17", "--expt-relaxed-constexpr", "-gencode", "arch=compute_100a,code=sm_100a",
               "-shared", "-Xcompiler", "-fPIC", "-w", *defs, *inc, src, "-o", out,
               "-Xlinker", "-rpath", "-Xlinker", lib_dir, *libs, "-lc10_cuda", "-ltorch_cuda"]
    subprocess.run(cmd, check=True)
    return out


def build(reference_root: str | None = None, force: bool = False, names=None) -> dict:
    """Builds what is missing or older than its sources.  Returns {module name: path or None}; None where the
    reference checkout (or, for ``gemm_softmax``, the CUTLASS headers) is not present and no earlier build exists."""
    src_dir = os.path.join(reference_root or default_reference_root(), SRC_DIR_REL)
    names = list(names or MODULES)
    with ThreadPoolExecutor(max_workers=len(names)) as pool:
        paths = list(pool.map(lambda n: _build_one(n, src_dir, force), names))
    return dict(zip(names, paths))


def load(name: str = "WaveBuffer"):
    """Import a built module (None if it was never built)."""
    path = module_path(name)
    if not os.path.exists(path):
        return None
    import importlib.util
    import torch  # noqa: F401  (the module links against libtorch)

    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else None, force="--force" in sys.argv))
