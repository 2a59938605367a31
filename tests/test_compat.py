"""The drop-in module names and signatures the reference model files rely on (CPU: no kernel runs)."""
import inspect
import sys

import pytest


@pytest.fixture()
def installed():
    from mustafar_b200 import compat
    compat.install()
    yield
    compat.uninstall()


def test_modules_and_names(installed):
    import mustafar_package
    import mustafar_package_quant
    import kernel.compression as compression
    import kernel_quant.compression_quant as compression_quant
    assert callable(mustafar_package.mustafar_key_formulation)
    assert callable(mustafar_package.mustafar_value_formulation)
    for n in ("mustafar_key_formulation_quant", "mustafar_key_formulation_quant_meta",
              "mustafar_value_formulation_quant", "mustafar_value_formulation_quant_decode_n1",
              "mustafar_quant_sparse_forward", "mustafar_quant_sparse_forward_meta",
              "mustafar_quant_sparse_value_forward", "mustafar_quant_sparse_value_forward_decode_n1"):
        assert callable(getattr(mustafar_package_quant, n)), n
    assert callable(compression.convert_key_batched) and callable(compression.convert_value_batched)
    assert callable(compression_quant.convert_key_batched_quant)
    assert callable(compression_quant.convert_value_batched_quant)
    assert "kernel.compression" in sys.modules


def test_positional_signatures_match_the_reference(installed):
    """Positional order is the contract (kernel/kernel_wrapper/mustafar_wrapper.h:7-37,
    kernel_quant/kernel_wrapper/pybind_quant.cpp:10-92)."""
    import mustafar_package as p
    import mustafar_package_quant as pq

    def names(f):
        return list(inspect.signature(f).parameters)

    assert names(p.mustafar_key_formulation) == [
        "bmp", "NZ", "idx", "NZ_Offset", "B", "M_Global", "K_Global", "Batch_Size", "num_key_value_groups"]
    assert names(p.mustafar_value_formulation) == [
        "bmp", "NZ", "idx", "NZ_Offset", "B", "Reduction_Workspace", "M_Global", "K_Global", "Batch_Size",
        "num_key_value_groups"]
    assert names(pq.mustafar_key_formulation_quant) == [
        "bmp", "NZ_quant", "tile_offsets", "scales", "zeros", "B", "M_Global", "K_Global", "Batch_Size",
        "num_key_value_groups", "bit", "capacity", "dequant_mode"]
    assert names(pq.mustafar_key_formulation_quant_meta) == [
        "bmp", "NZ_quant", "tile_offsets", "tile_counts", "tile_units", "scales", "zeros", "B", "M_Global",
        "K_Global", "Batch_Size", "num_key_value_groups", "bit", "capacity", "dequant_mode"]
    assert names(pq.mustafar_value_formulation_quant) == [
        "bmp", "NZ_quant", "tile_offsets", "tile_counts", "tile_units", "scales", "zeros", "B",
        "Reduction_Workspace", "M_Global", "K_Global", "Batch_Size", "num_key_value_groups", "bit", "capacity",
        "dequant_mode", "split_k", "value_tile_config"]
    assert names(pq.mustafar_value_formulation_quant_decode_n1) == [
        "bmp", "NZ_quant", "tile_offsets", "tile_counts", "tile_units", "scales", "zeros", "score",
        "Reduction_Workspace", "M_Global", "K_Global", "Batch_Size", "num_key_value_groups", "bit", "capacity",
        "dequant_mode", "split_k"]
    sig = inspect.signature(pq.mustafar_value_formulation_quant)
    assert sig.parameters["dequant_mode"].default == 0 and sig.parameters["split_k"].default == 1
    assert sig.parameters["value_tile_config"].default == 0
