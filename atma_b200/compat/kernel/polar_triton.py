"""kernel/polar_triton.py of the reference, by name (kernel/polar_triton.py:594-609,613-669,796-858)."""
from atma_b200.polar import HAS_TRITON, polar_attention_decode, polar_attention_fwd, polar_attention_packed_fwd  # noqa: F401
