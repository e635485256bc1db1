"""CPU restatement of ATMA's global-mixing hot path.  TEST INFRASTRUCTURE ONLY.

Every function here is an independent torch-CPU (fp32 / fp64) restatement of one
function on the reference's Polar + gated-delta path, citing the reference
file:line it follows.  It is the checker for the CUDA kernels: only the test
suite, the smoke check and the benchmark's CPU-baseline leg may import it.  The
product package never does - it fails loudly when its CUDA library is missing.

Parity pin: the restatement is checked against golden vectors produced by
importing the reference's own pure-PyTorch oracle (model/blocks.py,
model/reference.py, scripts/titans_proto.py, inference/models/atma.py CPU
branches); the generating script and the vectors live in tests/golden/.
"""

from .polar import (polar_params_host, polar_materialized, polar_streaming,
                    polar_prefill_oracle, polar_decode_oracle)
from .gated_delta import (gated_delta_sequential, gated_delta_chunked,
                          gated_delta_step, chunk_gated_delta_rule_oracle)
from .conv import (causal_conv1d_prefill, causal_conv1d_step,
                   packed_causal_conv1d_oracle, store_kvcache_oracle, qkv_prep_prefill_oracle,
                   lfm2_conv_step_oracle, lfm2_conv_packed_oracle)
from .elementwise import (squared_relu_gate_oracle, softcap_logits_oracle, linear_head_rms_oracle,
                          sigmoid_gate_mul_oracle, rms_sigmoid_gate_oracle)
from .model import (block_oracle, model_oracle, lfm2_mix_oracle, memory_readout_oracle, polar_mix_oracle,
                    mlp_oracle)

__all__ = [
    "polar_params_host", "polar_materialized", "polar_streaming",
    "polar_prefill_oracle", "polar_decode_oracle",
    "gated_delta_sequential", "gated_delta_chunked", "gated_delta_step",
    "chunk_gated_delta_rule_oracle",
    "causal_conv1d_prefill", "causal_conv1d_step", "packed_causal_conv1d_oracle", "qkv_prep_prefill_oracle",
    "lfm2_conv_step_oracle", "lfm2_conv_packed_oracle",
    "store_kvcache_oracle",
    "squared_relu_gate_oracle", "softcap_logits_oracle", "linear_head_rms_oracle",
    "sigmoid_gate_mul_oracle", "rms_sigmoid_gate_oracle",
    "block_oracle", "model_oracle", "lfm2_mix_oracle", "memory_readout_oracle", "polar_mix_oracle", "mlp_oracle",
]
