"""Compiles the reference project's own CUDA extension, from its sources where they lie, into
``oracle/_ref/`` (git-ignored build output; test infrastructure, never part of the product).

    python oracle/build_ref.py [--ref /path/to/PCEngine] [--force]

What it produces:

* ``oracle/_ref/PCEngine/backend.so`` -- the reference's pybind module (``backend/pybind_cuda.cpp``,
  ``backend/hash.cu``, ``backend/spconv.cu``), compiled unmodified with plain ``nvcc``/``g++`` calls
  for ``sm_100`` against this interpreter's torch headers (the reference's ``setup.py`` is not run).
* ``oracle/_ref/script/*.code`` -- byte-compiled images (marshalled code objects of this interpreter)
  of the reference's Python operator layer (``script/*.py``), so the drop-in test can run the
  reference's own ``conv3d`` on this library's ``PCEngine.backend`` replacement on a machine that does
  not hold the reference tree (``load_reference_script`` below imports them).

Only ``tests/golden/make_ref_golden.py`` (fixture generation on a GPU), the GPU tests that compare
against the reference and ``bench.py``'s reference-on-GPU comparator load these files. Without the
reference tree this script does nothing and says so.
"""
from __future__ import annotations

import marshal
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
DEFAULT_REF = os.environ.get("PCE_REFERENCE_TREE", "/root/reference")
SOURCES = ["pybind_cuda.cpp", "hash.cu", "spconv.cu"]
SCRIPTS = ["__init__", "activation", "batchnorm", "spconv", "sptensor", "utils"]


def ref_module_path() -> str:
    return os.path.join(OUT, "PCEngine", "backend.so")


def _nvcc() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(ref: str = DEFAULT_REF, force: bool = False) -> str | None:
    backend = os.path.join(ref, "backend")
    if not os.path.isdir(backend):
        print(f"reference tree not found at {ref}: nothing built")
        return ref_module_path() if os.path.exists(ref_module_path()) else None
    import torch  # headers and libraries only
    from torch.utils import cpp_extension as ce

    objdir = os.path.join(OUT, "build")
    os.makedirs(objdir, exist_ok=True)
    os.makedirs(os.path.join(OUT, "PCEngine"), exist_ok=True)
    inc = []
    for p in ce.include_paths("cuda") + [sysconfig.get_paths()["include"], backend]:
        inc += ["-I", p]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    common = inc + ["-DTORCH_EXTENSION_NAME=backend", "-DTORCH_API_INCLUDE_EXTENSION_H",
                    f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-std=c++17", "-O3"]
    headers = [os.path.join(backend, f) for f in os.listdir(backend) if f.endswith((".h", ".cuh"))]
    procs, objs = [], []
    for s in SOURCES:
        src = os.path.join(backend, s)
        obj = os.path.join(objdir, s.rsplit(".", 1)[0] + ".o")
        objs.append(obj)
        if not (force or _stale(obj, [src] + headers)):
            continue
        if s.endswith(".cu"):
            cmd = [_nvcc(), "-gencode", "arch=compute_100,code=sm_100", "--expt-relaxed-constexpr",
                   "-Xcompiler", "-fPIC", "-w"] + common + ["-c", src, "-o", obj]
        else:
            cmd = ["g++", "-fPIC", "-w"] + common + ["-c", src, "-o", obj]
        procs.append((s, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for s, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError(f"compiling the reference's {s} failed:\n{out[-4000:]}")
    lib = ref_module_path()
    if force or procs or _stale(lib, objs):
        ld = []
        for p in ce.library_paths("cuda"):
            ld += ["-L", p, f"-Wl,-rpath,{p}"]
        cmd = ["g++", "-shared", "-o", lib] + objs + ld + [
            "-lc10", "-ltorch", "-ltorch_cpu", "-ltorch_python", "-lc10_cuda", "-ltorch_cuda", "-lcudart", "-lcublas"]
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"linking the reference's extension failed:\n{r.stdout[-4000:]}")
    # byte-compiled operator layer: one marshalled code object per module
    sdir = os.path.join(OUT, "script")
    os.makedirs(sdir, exist_ok=True)
    for name in SCRIPTS:
        src = os.path.join(ref, "script", name + ".py")
        dst = os.path.join(sdir, name + ".code")
        text = open(src).read() if os.path.exists(src) else ""
        if not os.path.exists(src) and name != "__init__":
            continue
        if force or not os.path.exists(dst) or (os.path.exists(src) and _stale(dst, [src])):
            with open(dst, "wb") as f:
                marshal.dump(compile(text, f"script/{name}.py", "exec"), f)
    return lib


def load_reference_script(root: str = OUT):
    """Imports the reference's ``script`` package from the marshalled images under ``root``/script
    (``sys.modules`` must already hold whatever it imports: ``PCEngine.backend``, ``open3d``).  Returns
    the package; its modules are ``script.spconv``, ``script.sptensor``, ``script.utils`` ..."""
    import importlib.abc
    import importlib.util
    import sys

    sdir = os.path.join(root, "script")

    class _Loader(importlib.abc.Loader):
        def __init__(self, path, is_pkg):
            self.path, self.is_pkg = path, is_pkg

        def create_module(self, spec):
            return None

        def exec_module(self, module):
            with open(self.path, "rb") as f:
                exec(marshal.load(f), module.__dict__)

    class _Finder(importlib.abc.MetaPathFinder):
        def find_spec(self, fullname, path=None, target=None):
            if fullname == "script":
                p = os.path.join(sdir, "__init__.code")
                return importlib.util.spec_from_loader(fullname, _Loader(p, True), is_package=True) if os.path.exists(p) else None
            if fullname.startswith("script."):
                p = os.path.join(sdir, fullname.split(".", 1)[1] + ".code")
                return importlib.util.spec_from_loader(fullname, _Loader(p, False)) if os.path.exists(p) else None
            return None

    finder = _Finder()
    sys.meta_path.insert(0, finder)
    try:
        import importlib
        pkg = importlib.import_module("script")
        for name in ("utils", "sptensor", "spconv"):
            importlib.import_module("script." + name)
        return pkg
    finally:
        sys.meta_path.remove(finder)


if __name__ == "__main__":
    ref = DEFAULT_REF
    if "--ref" in sys.argv:
        ref = sys.argv[sys.argv.index("--ref") + 1]
    print(build(ref, force="--force" in sys.argv))
