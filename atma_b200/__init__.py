"""atma_b200: hand-written sm_100a kernels for ATMA's global-mixing hot path.

Polar Attention prefill / paged decode, the gated-delta memory chunked scan and decode
step, the depthwise causal convolutions and the small decode fusions, behind the call
signatures of the reference's kernel modules.  Host code is Python/PyTorch (device memory,
streams, torch.distributed); all device work goes through the C ABI of libatma_b200.so.
There is no CPU or PyTorch fallback: a missing library raises on first use.
"""

from .polar import (polar_attention_fwd, polar_attention_packed_fwd, polar_attention_decode,
                    polar_prefill_raw, invalidate_param_cache)
from .gated_delta import (gated_delta_decode_step, gated_delta_decode_step_fused, chunk_gated_delta_rule,
                          packed_gated_delta_prefill)
from .causal_conv1d import causal_conv1d_decode_step, causal_conv1d_fn
from .inference_ops import squared_relu_gate, packed_causal_conv1d, softcap_logits, linear_head_rms, qkv_prep_prefill, sigmoid_gate_mul, rms_sigmoid_gate, lfm2_conv_decode_step, lfm2_conv_packed, qkv_prep_decode, add_rms_norm, decode_linear
from .kvcache import store_kvcache
from ._lib import device_status

__all__ = [
    "polar_attention_fwd", "polar_attention_packed_fwd", "polar_attention_decode", "polar_prefill_raw",
    "gated_delta_decode_step", "chunk_gated_delta_rule", "packed_gated_delta_prefill",
    "causal_conv1d_decode_step", "causal_conv1d_fn",
    "device_status", "squared_relu_gate", "packed_causal_conv1d", "softcap_logits", "linear_head_rms", "qkv_prep_prefill", "sigmoid_gate_mul", "rms_sigmoid_gate", "lfm2_conv_decode_step", "lfm2_conv_packed", "qkv_prep_decode", "add_rms_norm", "decode_linear",
    "gated_delta_decode_step_fused", "invalidate_param_cache",
    "store_kvcache",
]
