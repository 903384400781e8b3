"""Build the reference's own CPU extensions, unchanged, as parity anchors.

TEST INFRASTRUCTURE ONLY.  Nothing under oracle/ is part of the product; only
tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / reference arm may
load what this script builds.

The sources are compiled from where they lie in the reference checkout
(torch_c/sc-extension/{sc.cpp,sc_conv.cpp,sc_matmul.cpp} -> module
``sc_extension_ref``; torch_c/sc-extension/fixed.cpp -> ``fixed_extension_ref``)
with plain g++ and libtorch's headers; no reference source is copied and the
only outputs are the two shared objects under oracle/_ref/.  If the reference
checkout is not present (for example on a GPU box that received prebuilt
files) the script does nothing.

Usage:  python oracle/build_ref.py [reference_root]
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")


def default_reference_root() -> str:
    """Where the reference checkout lies: REXSC_REFERENCE_ROOT, else the ``reference_path`` entry of the BASELINE.json
    next to this directory, else nothing (an empty string: no sources, nothing is built)."""
    env = os.environ.get("REXSC_REFERENCE_ROOT")
    if env:
        return env
    try:
        import json

        with open(os.path.join(os.path.dirname(HERE), "BASELINE.json")) as fh:
            return json.load(fh).get("reference_path") or ""
    except Exception:
        return ""

MODULES = {
    "sc_extension_ref": ["sc.cpp", "sc_conv.cpp", "sc_matmul.cpp"],
    "fixed_extension_ref": ["fixed.cpp"],
}


def _cxx() -> str:
    # a g++ that ships libgomp; the first g++ on PATH may not
    for cand in (os.environ.get("REXSC_REF_CXX"), "/usr/bin/g++", "g++"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "g++"


def build(reference_root: str | None = None, force: bool = False) -> bool:
    """Return True when both modules exist under oracle/_ref after the call."""
    root = reference_root or default_reference_root()
    src_dir = os.path.join(root, "torch_c", "sc-extension")
    have_src = os.path.isdir(src_dir)
    os.makedirs(OUT, exist_ok=True)
    ok = True
    for name, files in MODULES.items():
        so = os.path.join(OUT, name + ".so")
        if os.path.exists(so) and not force:
            continue
        if not have_src:
            ok = False
            continue
        import torch
        from torch.utils import cpp_extension

        inc = []
        for p in cpp_extension.include_paths():
            inc += ["-isystem", p]
        inc += ["-isystem", sysconfig.get_paths()["include"]]
        libdir = os.path.join(os.path.dirname(torch.__file__), "lib")
        objs = []
        for f in files:
            obj = os.path.join(OUT, f"{name}_{os.path.splitext(f)[0]}.o")
            cmd = [
                _cxx(), "-c", os.path.join(src_dir, f), "-o", obj,
                "-O2", "-march=native", "-fopenmp", "-fPIC", "-std=c++17", "-w",
                f"-DTORCH_EXTENSION_NAME={name}", "-DTORCH_API_INCLUDE_EXTENSION_H",
                f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
            ] + inc
            subprocess.check_call(cmd)
            objs.append(obj)
        cmd = [
            _cxx(), "-shared", "-o", so, *objs, "-fopenmp",
            f"-L{libdir}", f"-Wl,-rpath,{libdir}",
            "-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python",
        ]
        subprocess.check_call(cmd)
        for obj in objs:
            os.remove(obj)
    return ok and all(os.path.exists(os.path.join(OUT, n + ".so")) for n in MODULES)


GPU_MODULES = {
    # the reference's CUDA extensions (torch_c/sc-extension/setup_cuda.py, setup_cuda_fixed.py), compiled for
    # sm_100 instead of the sm_75 / sm_86 its own setup scripts name; sources unchanged
    "sc_extension_cuda_ref": (["sc_cuda.cpp", "sc_cuda_kernel.cu", "sc_cuda_matmul.cu", "sc_cuda_pw.cu", "sc_device.cu",
                               "sc_cuda_conv.cu"], ["-t=0"]),
    "fixed_extension_cuda_ref": (["fixed_cuda.cpp", "fixed_cuda_kernel.cu"], ["-maxrregcount=64"]),
}


def build_gpu(reference_root: str | None = None, force: bool = False) -> bool:
    """Cross-compile the reference's GPU extensions (no GPU needed) into oracle/_ref; used on a GPU box as a
    second parity anchor (the reference's own kernels, XNOR generator included) and as the kernel to beat."""
    root = reference_root or default_reference_root()
    src_dir = os.path.join(root, "torch_c", "sc-extension")
    have_src = os.path.isdir(src_dir)
    os.makedirs(OUT, exist_ok=True)
    import shutil

    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    for name, (files, nvcc_extra) in GPU_MODULES.items():
        so = os.path.join(OUT, name + ".so")
        if os.path.exists(so) and not force:
            continue
        if not have_src or not os.path.exists(nvcc):
            return False
        import torch
        from torch.utils import cpp_extension

        inc = []
        for p in cpp_extension.include_paths(device_type="cuda"):
            inc += ["-isystem", p]
        inc += ["-isystem", sysconfig.get_paths()["include"]]
        libdir = os.path.join(os.path.dirname(torch.__file__), "lib")
        common = [f"-DTORCH_EXTENSION_NAME={name}", "-DTORCH_API_INCLUDE_EXTENSION_H",
                  f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
        objs = []
        for f in files:
            obj = os.path.join(OUT, f"{name}_{os.path.splitext(f)[0]}.o")
            if f.endswith(".cu"):
                cmd = [nvcc, "-c", os.path.join(src_dir, f), "-o", obj, "-O2", "-std=c++17", "-w",
                       "-gencode", "arch=compute_100,code=sm_100", "-Xcompiler", "-fPIC",
                       "-ccbin", _cxx(), "--expt-relaxed-constexpr", *nvcc_extra, *common, *inc]
            else:
                cmd = [_cxx(), "-c", os.path.join(src_dir, f), "-o", obj, "-O2", "-fPIC", "-std=c++17", "-w",
                       *common, *inc]
            subprocess.check_call(cmd)
            objs.append(obj)
        cuda_lib = os.path.join(os.path.dirname(os.path.dirname(nvcc)), "lib64")
        cmd = [_cxx(), "-shared", "-o", so, *objs, f"-L{libdir}", f"-Wl,-rpath,{libdir}", f"-L{cuda_lib}",
               "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"]
        subprocess.check_call(cmd)
        for obj in objs:
            os.remove(obj)
    return all(os.path.exists(os.path.join(OUT, n + ".so")) for n in GPU_MODULES)


def load_gpu():
    """Import (sc_extension_cuda_ref, fixed_extension_cuda_ref) from oracle/_ref or return None."""
    import importlib.util

    import torch  # noqa: F401

    mods = []
    for name in GPU_MODULES:
        so = os.path.join(OUT, name + ".so")
        if not os.path.exists(so):
            return None
        if name in sys.modules:
            mods.append(sys.modules[name])
            continue
        spec = importlib.util.spec_from_file_location(name, so)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        sys.modules[name] = mod
        mods.append(mod)
    return tuple(mods)


def load():
    """Import (sc_extension_ref, fixed_extension_ref) from oracle/_ref or return None."""
    import importlib.util

    mods = []
    import torch  # noqa: F401  (the modules link against libtorch)

    for name in MODULES:
        so = os.path.join(OUT, name + ".so")
        if not os.path.exists(so):
            return None
        if name in sys.modules:
            mods.append(sys.modules[name])
            continue
        spec = importlib.util.spec_from_file_location(name, so)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        sys.modules[name] = mod
        mods.append(mod)
    return tuple(mods)


if __name__ == "__main__":
    args = [a for a in sys.argv[1:] if not a.startswith("--")]
    good = build(args[0] if args else None, force="--force" in sys.argv)
    print("oracle/_ref (CPU extensions):", "built" if good else "reference sources not available; nothing built")
    if "--gpu" in sys.argv:
        good = build_gpu(args[0] if args else None, force="--force" in sys.argv)
        print("oracle/_ref (GPU extensions, sm_100):", "built" if good else "not built")
