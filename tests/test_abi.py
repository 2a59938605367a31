"""CPU-side checks of the boundary: the shared library builds/loads and exports every
symbol that include/mustafar_b200.h declares; host-side argument validation."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from mustafar_b200 import build, _lib
    build.build()
    return _lib.lib()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "mustafar_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mfar_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(lib):
    names = declared_symbols()
    assert len(names) >= 9
    for n in names:
        assert hasattr(lib, n), n


def test_binding_covers_header(lib):
    from mustafar_b200 import _lib
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_version_and_strings(lib):
    assert lib.mfar_version() >= 100
    assert lib.mfar_status_string(0) == b"ok"
    assert b"align" in lib.mfar_status_string(2)


def test_scratch_and_plan_sizes(lib):
    assert lib.mfar_compress_scratch_bytes(64, 8192) == 16 + 8 * 64 * 128
    ns, nbytes = ctypes.c_int(), ctypes.c_size_t()
    assert lib.mfar_decode_plan(8, 4096, 128, 0, ctypes.byref(ns), ctypes.byref(nbytes), 4) == 0
    assert 1 <= ns.value <= 64 and nbytes.value >= 8 * (ns.value + 1) * 4 * 132 * 4
    assert lib.mfar_decode_plan(8, 4097, 128, 0, ctypes.byref(ns), ctypes.byref(nbytes), 4) != 0
    # long sequences are never split into more than 256 blocks per CTA
    assert lib.mfar_decode_plan(512, 64 * 1024, 0, 1, ctypes.byref(ns), ctypes.byref(nbytes), 4) == 0
    assert ns.value >= 4


def test_host_argument_validation_needs_no_gpu(lib):
    # null pointers / bad sizes are rejected before any CUDA call
    assert lib.mfar_compress_fp16(None, 0, 0, 0, 0, 1, 64, 0, 0, None, 0, None, 0, 0, None, None, 0, 0, None, 0,
                                  None, None, None) == 1
    assert lib.mfar_compress_fp16(None, 0, 0, 0, 0, 1, 65, 0, 0, None, 0, None, 0, 0, None, None, 0, 0, None, 0,
                                  None, None, None) == 1
    assert lib.mfar_prune_fp16(None, None, 4, 128, 200, None) == 1
    assert lib.mfar_prune_fp16(None, None, 0, 128, 89, None) == 0          # empty input is fine


def test_cpu_tensors_are_refused():
    import torch
    from mustafar_b200 import compression
    with pytest.raises(RuntimeError):
        compression.convert_key_batched(torch.zeros(1, 64, 128, dtype=torch.float16))
    with pytest.raises(RuntimeError):
        compression.prune(torch.zeros(4, 128, dtype=torch.float16), 0.7)


def test_header_is_plain_c_and_links_from_c(lib, tmp_path):
    """The boundary is a C ABI: the header compiles as C99 (no C++ in it) and a C program links against the library
    and calls entry points that need no GPU - what a cgo / JNI / FFI binding of the reference's host language would do."""
    import shutil
    import subprocess
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    src = tmp_path / "abi.c"
    src.write_text('#include <stdio.h>\n#include "mustafar_b200.h"\n'
                   'int main(void) {\n'
                   '    int ns = 0; size_t bytes = 0;\n'
                   '    if (mfar_version() < 100) return 1;\n'
                   '    if (mfar_decode_plan(8, 4096, 128, 0, &ns, &bytes, 4) != MFAR_OK) return 2;\n'
                   '    if (mfar_prune_fp16(NULL, NULL, 4, 128, 200, NULL) != MFAR_ERR_ARG) return 3;\n'
                   '    printf("%s %d %zu\\n", mfar_status_string(MFAR_ERR_ALIGN), ns, bytes);\n'
                   '    return 0;\n}\n')
    inc = os.path.join(ROOT, "include")
    libdir = os.path.join(ROOT, "mustafar_b200")
    exe = tmp_path / "abi"
    r = subprocess.run([gcc, "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-I", inc, str(src), "-o", str(exe),
                        "-L", libdir, "-lmustafar_b200", f"-Wl,-rpath,{libdir}"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    assert r.returncode == 0 and "align" in r.stdout, (r.returncode, r.stdout, r.stderr)
