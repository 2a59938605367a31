"""Compiles the reference's own CUDA extensions into ``oracle/_ref/`` (TEST INFRASTRUCTURE, not product).

    python -m oracle.build_ref [--ref /path/to/reference/checkout] [--force]

The sources are compiled where they lie in the reference checkout (nothing is copied into this
repository); only the two resulting python extension modules land in ``oracle/_ref/``:

  * ``mustafar_package_quant``  from ``kernel_quant/kernel_wrapper/{pybind_quant.cpp,mustafar_wrapper_quant.cu}``
    and ``kernel_quant/csrc/SpMM_API_Quant.cu`` (the sources its ``setup.py:22-26`` lists);
  * ``mustafar_package``        from ``kernel/kernel_wrapper/{pybind.cpp,mustafar_wrapper.cu}`` and
    ``kernel/csrc/SpMM_API.cu`` (its ``setup.py:35`` links a prebuilt ``../build/SpMM_API.o`` whose Makefile
    is not in the tree, so the object is compiled here by hand).

``stage_model_files()`` copies the two reference model files that the drop-in must run unchanged
(``models/llama_mustafar_kernel.py``, ``models/llama_mustafar_quant_kernel.py``) into the git-ignored
``baseline/_ref/models/`` so that a GPU box without the reference checkout can import them in the tests.

The reference selects its architecture from the local GPU (``setup.py:9-15``); here the kernels
(``mma.sync`` / ``ldmatrix`` / ``cp.async``, Ampere-class code) are compiled for sm_100.  Only
``tests/`` may import the result, as a second opinion beside the CPU restatement in this package.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
STAGE = os.path.join(os.path.dirname(HERE), "baseline", "_ref")
MODEL_FILES = ("models/llama_mustafar_kernel.py", "models/llama_mustafar_quant_kernel.py")
DEFAULT_REF = os.environ.get("MUSTAFAR_REFERENCE", "/root/reference")

MODULES = {
    "mustafar_package_quant": {
        "dir": "kernel_quant/kernel_wrapper",
        "sources": ["pybind_quant.cpp", "mustafar_wrapper_quant.cu", "../csrc/SpMM_API_Quant.cu"],
        "include": ["../csrc"],
    },
    "mustafar_package": {
        "dir": "kernel/kernel_wrapper",
        "sources": ["pybind.cpp", "mustafar_wrapper.cu", "../csrc/SpMM_API.cu"],
        "include": ["../csrc"],
    },
}


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def build(ref: str = DEFAULT_REF, force: bool = False, verbose: bool = False) -> dict:
    """Returns {module name: path of the built .so, or an error string}."""
    from torch.utils import cpp_extension as ce
    import torch

    os.makedirs(OUT, exist_ok=True)
    nvcc = _nvcc()
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    inc = [f"-I{p}" for p in ce.include_paths()] + [f"-I{sysconfig.get_paths()['include']}"]
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    result = {}
    for name, m in MODULES.items():
        src_dir = os.path.join(ref, m["dir"])
        target = os.path.join(OUT, name + suffix)
        if not os.path.isdir(src_dir):
            result[name] = f"unavailable: {src_dir} not found"
            continue
        if os.path.exists(target) and not force:
            result[name] = target
            continue
        obj_dir = os.path.join(OUT, "obj_" + name)
        os.makedirs(obj_dir, exist_ok=True)
        def compile_one(src_rel):
            src = os.path.normpath(os.path.join(src_dir, src_rel))
            obj = os.path.join(obj_dir, os.path.basename(src_rel) + ".o")
            cmd = [nvcc, "-gencode", "arch=compute_100,code=sm_100", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
                   "--expt-relaxed-constexpr", "-lineinfo", f"-DTORCH_EXTENSION_NAME={name}",
                   "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
                   *inc, *[f"-I{os.path.normpath(os.path.join(src_dir, i))}" for i in m["include"]],
                   "-x", "cu", "-c", src, "-o", obj]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if verbose or r.returncode != 0:
                sys.stderr.write(" ".join(cmd) + "\n" + r.stdout[-4000:] + r.stderr[-4000:] + "\n")
            if r.returncode != 0:
                return None, f"unavailable: nvcc failed on {src_rel}: " + (r.stderr.strip().splitlines() or ["?"])[-1]
            return obj, None

        with ThreadPoolExecutor(max_workers=len(m["sources"])) as ex:
            done = list(ex.map(compile_one, m["sources"]))
        objs = [o for o, _ in done if o]
        failed = next((e for _, e in done if e), None)
        if failed:
            result[name] = failed
            continue
        cmd = [nvcc, "-shared", "-o", target, *objs, f"-L{torch_lib}", "-lc10", "-ltorch", "-ltorch_cpu",
               "-ltorch_python", "-lc10_cuda", "-ltorch_cuda", "-lcudart", "-Xlinker", f"-rpath={torch_lib}"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr + "\n")
            result[name] = "unavailable: link failed"
            continue
        result[name] = target
    return result


def stage_model_files(ref: str = DEFAULT_REF) -> list:
    """Copies the two reference model files into baseline/_ref/models/ (git-ignored); returns what was staged."""
    staged = []
    for rel in MODEL_FILES:
        src = os.path.join(ref, rel)
        if not os.path.exists(src):
            continue
        dst = os.path.join(STAGE, rel)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        if not os.path.exists(dst) or os.path.getmtime(dst) < os.path.getmtime(src):
            shutil.copyfile(src, dst)
        staged.append(dst)
    return staged


def load(name: str):
    """Imports a built reference extension from ``oracle/_ref`` or returns None when it was not built."""
    import importlib.util
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    path = os.path.join(OUT, name + suffix)
    if not os.path.exists(path):
        return None
    import torch  # noqa: F401  (the extension links against libtorch)
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=DEFAULT_REF)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    for k, v in build(a.ref, a.force, a.verbose).items():
        print(k, "->", v)
    for f in stage_model_files(a.ref):
        print("staged", f)
