"""kernel/causal_conv1d_triton.py of the reference, by name (kernel/causal_conv1d_triton.py:46-63)."""
from atma_b200.causal_conv1d import causal_conv1d_decode_step  # noqa: F401
from atma_b200.polar import HAS_TRITON  # noqa: F401
