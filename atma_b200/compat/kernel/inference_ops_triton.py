"""kernel/inference_ops_triton.py of the reference, by name (kernel/inference_ops_triton.py:124-223)."""
from atma_b200.inference_ops import linear_head_rms, packed_causal_conv1d, softcap_logits, squared_relu_gate  # noqa: F401
from atma_b200.polar import HAS_TRITON  # noqa: F401
