"""Registers the package under the module names the reference model files import, so that
``models/llama_mustafar_kernel.py`` and ``models/llama_mustafar_quant_kernel.py`` run unchanged:

    import mustafar_b200.compat as compat
    compat.install()
    # now, as in the reference (models/llama_mustafar_kernel.py:15-20,
    # models/llama_mustafar_quant_kernel.py:15-20):
    import mustafar_package, mustafar_package_quant
    import kernel.compression as compression
    import kernel_quant.compression_quant as compression_quant

The model files append their own parent directory to ``sys.path``; modules already present
in ``sys.modules`` win, which is what ``install()`` relies on.
"""
from __future__ import annotations

import sys
import types

_NAMES = ("mustafar_package", "mustafar_package_quant", "kernel", "kernel.compression", "kernel_quant",
          "kernel_quant.compression_quant")


def install(force: bool = True) -> None:
    from . import compression, compression_quant, ops, ops_quant

    def module(name, doc, members):
        m = types.ModuleType(name, doc)
        for k, v in members.items():
            setattr(m, k, v)
        if force or name not in sys.modules:
            sys.modules[name] = m
        return sys.modules[name]

    module("mustafar_package", "mustafar_b200 drop-in for the reference torch extension mustafar_package", {
        "mustafar_key_formulation": ops.mustafar_key_formulation,
        "mustafar_value_formulation": ops.mustafar_value_formulation,
    })
    module("mustafar_package_quant", "mustafar_b200 drop-in for the reference torch extension mustafar_package_quant", {
        n: getattr(ops_quant, n) for n in (
            "mustafar_key_formulation_quant", "mustafar_key_formulation_quant_meta",
            "mustafar_value_formulation_quant", "mustafar_value_formulation_quant_decode_n1",
            "mustafar_quant_sparse_forward", "mustafar_quant_sparse_forward_meta",
            "mustafar_quant_sparse_value_forward", "mustafar_quant_sparse_value_forward_decode_n1")
    })
    k = module("kernel", "namespace package stand-in", {"__path__": []})
    k.compression = module("kernel.compression", "mustafar_b200 drop-in for kernel/compression.py", {
        "convert_key_batched": compression.convert_key_batched,
        "convert_value_batched": compression.convert_value_batched,
    })
    kq = module("kernel_quant", "namespace package stand-in", {"__path__": []})
    kq.compression_quant = module("kernel_quant.compression_quant",
                                  "mustafar_b200 drop-in for kernel_quant/compression_quant.py", {
        "convert_key_batched_quant": compression_quant.convert_key_batched_quant,
        "convert_value_batched_quant": compression_quant.convert_value_batched_quant,
    })


def uninstall() -> None:
    for n in _NAMES:
        sys.modules.pop(n, None)
