"""kernel/gated_delta_triton.py of the reference, by name (kernel/gated_delta_triton.py:79-117)."""
from atma_b200.gated_delta import HAS_TRITON, gated_delta_decode_step  # noqa: F401
