"""Small decode fusions on the CPU - checkers for the bit-exact elementwise kernels.

TEST INFRASTRUCTURE: see the package docstring.

The reference's fused kernels reproduce what eager PyTorch computes for a bf16
tensor, i.e. every eager op rounds its result to bf16 before the next one
(kernel/inference_ops_triton.py:112-120, 198-211).  The restatements below make
those roundings explicit in fp32 arithmetic.
"""

import torch
import torch.nn.functional as F


def _round_like(x_f32, dtype):
    return x_f32.to(dtype).float() if dtype != torch.float32 else x_f32


def squared_relu_gate_oracle(x, gate):
    """gate * relu(x)^2 (model/layers.py:27-31).  For bf16 the square is rounded
    before the gate multiply (kernel/inference_ops_triton.py:117-119)."""
    pos = x.float().clamp_min(0.0)
    sq = _round_like(pos * pos, x.dtype if x.dtype == torch.bfloat16 else torch.float32)
    return (gate.float() * sq).to(x.dtype)


def softcap_logits_oracle(logits):
    """15 x / sqrt(x^2 + 225) (model/reference.py:267-268), with eager-bf16 rounding
    after each op for bf16 input (kernel/inference_ops_triton.py:200-210)."""
    dt = logits.dtype if logits.dtype == torch.bfloat16 else torch.float32
    x = logits.float()
    left = _round_like(15.0 * x, dt)
    sq = _round_like(x * x, dt)
    den = _round_like(sq + 225.0, dt)
    inv = _round_like(torch.rsqrt(den), dt)
    return (left * inv).to(logits.dtype)


def linear_head_rms_oracle(x, weight, bias, *, num_heads, head_dim=128, gated=False, eps=1e-6):
    """x W^T + b, then affine-free RMSNorm over each head's first ``head_dim`` columns;
    with ``gated`` each head is [q | gate] and the gate half passes through
    (kernel/inference_ops_triton.py:65-100,164-189).  fp32 result."""
    width = head_dim * (2 if gated else 1)
    y = F.linear(x.float(), weight.float(), None if bias is None else bias.float())
    y = y.view(x.shape[0], num_heads, width)
    qh = y[..., :head_dim]
    qn = qh * torch.rsqrt(qh.square().mean(-1, keepdim=True) + eps)
    out = torch.cat([qn, y[..., head_dim:]], dim=-1) if gated else qn
    return out.reshape(x.shape[0], num_heads * width)


def sigmoid_gate_mul_oracle(x, gate):
    """x * torch.sigmoid(gate) as eager runs it (inference/models/atma.py:555-556)."""
    return x * torch.sigmoid(gate)


def rms_sigmoid_gate_oracle(r, gate):
    """F.rms_norm(r, (dk,)) flattened over heads, times torch.sigmoid(gate)
    (inference/models/atma.py:373-375).  r (tokens, H, dk); gate (tokens, H*dk)."""
    import torch.nn.functional as F
    rows, H, dk = r.shape
    return F.rms_norm(r, (dk,)).reshape(rows, H * dk) * torch.sigmoid(gate)
