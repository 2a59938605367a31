"""Lets the reference model files import under a current ``transformers``.

``models/llama_mustafar_kernel.py`` and ``models/llama_mustafar_quant_kernel.py`` were written against
transformers 4.43: they star-import ``transformers.models.llama.modeling_llama`` (``:11-12``) and use
names that newer releases no longer define or no longer export through ``__all__``.  ``install()``
puts those names back into that module *before* the model file is imported; the model file itself is
not edited.  What is restored:

* ``__all__`` is widened to every public name of the module (newer releases export six classes only,
  so ``LlamaRotaryEmbedding``, ``LlamaRMSNorm``, ``LlamaMLP``, ``repeat_kv``, ``logger`` ... would be missing);
* the docstring decorators ``add_start_docstrings_to_model_forward`` / ``replace_return_docstrings``
  (used at ``:818``, ``:969-970``) as pass-through decorators, ``LLAMA_INPUTS_DOCSTRING`` as an empty string;
* ``_get_unpad_data`` and the flash-attn padding helpers ``index_first_axis`` / ``pad_input`` / ``unpad_input``
  (used by ``_upad_input``, ``:657-693``);
* ``CrossEntropyLoss``, ``math``, ``F`` and the ``typing`` names the annotations use;
* ``apply_rotary_pos_emb`` accepting the old fifth positional argument ``position_ids`` (call at ``:374``).

``llama_config(**kw)`` builds a ``LlamaConfig`` carrying the attributes the reference's drivers set on it
(``benchmark/mem_spd_test.py:71-81``) plus ``rope_theta``, which the attention module reads directly (``:162``)
and newer configs keep under ``rope_parameters``.
"""
from __future__ import annotations

import math
import typing


def install() -> None:
    import torch
    import torch.nn.functional as F
    import transformers.models.llama.modeling_llama as ml

    if getattr(ml, "_mustafar_b200_shim", False):
        return

    def passthrough_decorator(*_a, **_k):
        def wrap(fn):
            return fn
        return wrap

    def _get_unpad_data(attention_mask):
        seqlens = attention_mask.sum(dim=-1, dtype=torch.int32)
        indices = torch.nonzero(attention_mask.flatten(), as_tuple=False).flatten()
        max_len = int(seqlens.max().item())
        cu = F.pad(torch.cumsum(seqlens, dim=0, dtype=torch.int32), (1, 0))
        return indices, cu, max_len

    missing = {
        "add_start_docstrings_to_model_forward": passthrough_decorator,
        "replace_return_docstrings": passthrough_decorator,
        "add_start_docstrings": passthrough_decorator,
        "LLAMA_INPUTS_DOCSTRING": "",
        "LLAMA_START_DOCSTRING": "",
        "_get_unpad_data": _get_unpad_data,
        "CrossEntropyLoss": torch.nn.CrossEntropyLoss,
        "BCEWithLogitsLoss": torch.nn.BCEWithLogitsLoss,
        "MSELoss": torch.nn.MSELoss,
        "math": math,
        "F": F,
        "List": typing.List, "Tuple": typing.Tuple, "Union": typing.Union, "Optional": typing.Optional,
    }
    try:
        from flash_attn.bert_padding import index_first_axis, pad_input, unpad_input
        missing.update(index_first_axis=index_first_axis, pad_input=pad_input, unpad_input=unpad_input)
    except Exception:       # only the padded-batch prefill path needs them
        pass
    for name, obj in missing.items():
        if not hasattr(ml, name):
            setattr(ml, name, obj)

    new_rope = ml.apply_rotary_pos_emb

    def apply_rotary_pos_emb(q, k, cos, sin, position_ids=None, unsqueeze_dim=1):
        return new_rope(q, k, cos, sin, unsqueeze_dim=unsqueeze_dim)

    ml.apply_rotary_pos_emb = apply_rotary_pos_emb
    ml.__all__ = sorted({n for n in vars(ml) if not n.startswith("__")} | {"_get_unpad_data"})
    ml._mustafar_b200_shim = True


def llama_config(k_sparsity: float = 0.7, v_sparsity: float = 0.7, residual_length: int = 128, **kw):
    """A ``LlamaConfig`` with the attributes the reference model reads
    (``models/llama_mustafar_kernel.py:151-166,670``; driver: ``benchmark/mem_spd_test.py:71-81``)."""
    from transformers import LlamaConfig
    theta = kw.pop("rope_theta", 500000.0)
    cfg = LlamaConfig(**kw)
    try:
        cfg.rope_theta = theta
    except Exception:
        object.__setattr__(cfg, "rope_theta", theta)
    if getattr(cfg, "rope_parameters", None) is not None:
        cfg.rope_parameters["rope_theta"] = theta
    cfg.k_sparsity, cfg.v_sparsity = k_sparsity, v_sparsity
    cfg.group_size = cfg.residual_length = residual_length
    cfg.use_flash = True
    cfg.use_cache = True
    return cfg
