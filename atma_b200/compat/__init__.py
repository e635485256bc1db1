"""Import-path shim: with this directory at the front of ``sys.path`` (``atma_b200.compat.install()``),
the reference's own import statements - ``from kernel.polar_triton import ...``,
``from kernel.gated_delta_triton import ...``, ``from kernel.causal_conv1d_triton import ...``,
``from kernel.inference_ops_triton import ...`` (inference/models/atma.py:31-80) and
``from fla.ops.gated_delta_rule import chunk_gated_delta_rule`` (inference/models/atma.py:53;
model/blocks.py:24) - resolve to this library, so the reference runs on it without an edit.
``store_kvcache`` lives inside the reference's own ``inference.layers.attention`` module; it is
replaced by assignment: ``inference.layers.attention.store_kvcache = atma_b200.store_kvcache``."""

import os
import sys


def install():
    """Put the shim packages ``kernel`` and ``fla`` ahead of everything else on ``sys.path``."""
    here = os.path.dirname(os.path.abspath(__file__))
    if here not in sys.path:
        sys.path.insert(0, here)
    return here
