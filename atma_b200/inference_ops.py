"""Small forward-only fusions of the paged inference model, with the reference's signatures
(kernel/inference_ops_triton.py:124-223)."""

import torch

from . import _lib

HAS_TRITON = torch.cuda.is_available()


@torch.no_grad()
def squared_relu_gate(x, gate):
    """gate * relu(x)^2, preserving eager bf16's rounding of the square.  x, gate (rows,
    width), typically the two strided halves of one (rows, 2*width) tensor."""
    _lib.require_cuda(x, "squared_relu_gate")
    lib = _lib.load()
    rows, width = x.shape
    if x.stride(1) != 1:
        x = x.contiguous()
    if gate.stride(1) != 1 or gate.dtype != x.dtype:
        gate = gate.to(x.dtype).contiguous()
    out = torch.empty((rows, width), device=x.device, dtype=x.dtype)
    _lib.check(lib.atma_squared_relu_gate(_lib.ptr(x), x.stride(0), _lib.ptr(gate), gate.stride(0),
                                          _lib.ptr(out), rows, width, _lib.dtype_code(x),
                                          _lib.stream_ptr()))
    return out


def _packed_conv(x, weight, state_table, starts, ends, slots, init_state=None, residual=False):
    lib = _lib.load()
    total, C = x.shape
    K = weight.shape[1]
    if x.stride(1) != 1:
        x = x.contiguous()
    weight = weight.to(x.dtype).contiguous()
    if state_table.dtype != x.dtype or state_table.stride(2) != 1 or state_table.stride(1) != K - 1:
        raise ValueError("state_table must be (max_seqs, C, K-1) with dense rows in x's dtype")
    maps = [t.to(device=x.device, dtype=torch.int32).contiguous() for t in (starts, ends, slots)]
    out = torch.empty((total, C), device=x.device, dtype=x.dtype)
    _lib.check(lib.atma_packed_causal_conv1d(
        _lib.ptr(x), x.stride(0), _lib.ptr(weight), _lib.ptr(out), out.stride(0),
        _lib.ptr(state_table), _lib.ptr(init_state), state_table.stride(0),
        _lib.ptr(maps[0]), _lib.ptr(maps[1]), _lib.ptr(maps[2]), total, C, K,
        _lib.dtype_code(x), 1 if residual else 0, _lib.stream_ptr()))
    return out


@torch.no_grad()
def packed_causal_conv1d(x, weight, state_table, token_seq_starts, token_seq_ends, token_seq_slots):
    """Fresh causal depthwise convolution over packed variable-length sequences; writes each
    sequence's last K-1 inputs into ``state_table[slot]``."""
    if not x.is_cuda:
        raise RuntimeError("packed_causal_conv1d requires CUDA")
    if x.ndim != 2 or weight.ndim != 2 or weight.shape[0] != x.shape[1]:
        raise ValueError("expected x [tokens, channels], weight [channels, kernel]")
    if weight.shape[1] not in (3, 4):
        raise ValueError("packed convolution supports ATMA kernel sizes 3 and 4")
    return _packed_conv(x, weight, state_table, token_seq_starts, token_seq_ends, token_seq_slots)


@torch.no_grad()
def softcap_logits(logits):
    """15 x / sqrt(x^2 + 225) with eager bf16's per-op rounding."""
    _lib.require_cuda(logits, "softcap_logits")
    lib = _lib.load()
    x = logits.contiguous()
    out = torch.empty_like(x)
    _lib.check(lib.atma_softcap_logits(_lib.ptr(x), _lib.ptr(out), x.numel(), _lib.dtype_code(x),
                                       _lib.stream_ptr()))
    return out


@torch.no_grad()
def linear_head_rms(x, weight, bias, *, num_heads, head_dim=128, gated=False, eps=1e-6):
    """Projection followed by affine-free per-head RMSNorm of each head's first ``head_dim``
    columns (with ``gated`` each head stores Q then its untouched gate)."""
    if not x.is_cuda:
        raise RuntimeError("linear_head_rms requires CUDA")
    width = head_dim * (2 if gated else 1)
    if x.ndim != 2 or weight.shape != (num_heads * width, x.shape[1]):
        raise ValueError("incompatible x/weight shape for head projection")
    if head_dim != 128:
        raise ValueError("the prototype is shape-dispatched only for head_dim=128")
    lib = _lib.load()
    x, weight = x.contiguous(), weight.to(x.dtype).contiguous()
    bias = None if bias is None else bias.to(x.dtype).contiguous()
    out = torch.empty((x.shape[0], weight.shape[0]), device=x.device, dtype=x.dtype)
    _lib.check(lib.atma_linear_head_rms(_lib.ptr(x), _lib.ptr(weight), _lib.ptr(bias), _lib.ptr(out),
                                        x.shape[0], x.shape[1], num_heads, head_dim, 1 if gated else 0,
                                        float(eps), _lib.dtype_code(x), _lib.stream_ptr()))
    return out
