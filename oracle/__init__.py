"""CPU oracle for the sparse KV-cache hot path (TEST INFRASTRUCTURE, not product).

This package restates, on the CPU with numpy / torch, what the reference
(Haozon/mustafar) computes on the path

    prune (per-token magnitude)  ->  bitmap + packed-nonzero compression
    ->  decode q.K^T / softmax / P.V over the compressed cache
    (+ the 2-bit per-tile quantised variant)

Every function cites the reference file:line it follows.  It exists so the
CUDA kernels can be checked against something that is *not* themselves:

  * only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline /
    ``--impl reference`` leg may import it;
  * the product package never imports it and has no CPU fallback.

Parity status: the fp16 and 2-bit formats are pinned bit-for-bit against the
reference's own Triton kernels executed under ``TRITON_INTERPRET=1`` (fixtures
in ``tests/golden``, generator ``tests/golden/make_golden.py``).  The 4-bit
and group-of-32 quantised extensions have no reference implementation:
**parity unpinned** for those two (restatement of the same formulas only).
"""

from .prune import prune_ref, keep_count  # noqa: F401
from .fp16_format import (  # noqa: F401
    key_tiles, value_tiles, pack_tiles, compress_key_ref, compress_value_ref,
    decompress_key_ref, decompress_value_ref, nz_offsets_ref,
)
from .quant_format import (  # noqa: F401
    quant_compress_key_ref, quant_compress_value_ref,
    dequant_key_ref, dequant_value_ref,
)
from .attention import (  # noqa: F401
    key_formulation_ref, value_formulation_ref, decode_attention_ref,
    decode_attention_model_order_ref, rel_l2,
)
from .synth import make_kv, make_query  # noqa: F401
