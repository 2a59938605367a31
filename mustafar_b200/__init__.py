"""mustafar_b200: B200 (sm_100a) kernels for Mustafar's sparse KV-cache hot path.

Host side of the C ABI in ``include/mustafar_b200.h``:

* ``mustafar_b200.compression``        convert_key_batched / convert_value_batched
  (reference ``kernel/compression.py``) + fused prune+compress and the cache arena;
* ``mustafar_b200.ops``                mustafar_key_formulation / mustafar_value_formulation
  (reference ``mustafar_package``) + the fused decode-attention entry;
* ``mustafar_b200.compat.install()``   registers those under the reference's module
  names so ``models/llama_mustafar_kernel.py`` imports them unchanged.

CUDA only.  Nothing here computes on the CPU.
"""
from ._lib import LIB_PATH, MustafarError, lib  # noqa: F401

__all__ = ["LIB_PATH", "MustafarError", "lib"]
