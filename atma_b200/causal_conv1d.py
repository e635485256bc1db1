"""Depthwise causal convolution entry points with the reference's call signatures.

``causal_conv1d_decode_step`` is a drop-in for kernel/causal_conv1d_triton.py:46-63.
``causal_conv1d_fn`` has the call shape of the kernels-community/causal-conv1d function
the reference uses for fresh prefill (inference/models/atma.py:123-126), extended with an
``initial_states`` argument for a continuation chunk (:128-137).
"""

import torch

from . import _lib

HAS_TRITON = torch.cuda.is_available()


@torch.no_grad()
def causal_conv1d_decode_step(x, weight, slots, state_table):
    """Apply one depthwise convolution step and update the slot-indexed state in place.
    x (B,D); weight (D,K); slots (B,) integer; state_table (max_seqs,D,K-1).  Returns (B,D)."""
    _lib.require_cuda(x, "causal_conv1d_decode_step")
    lib = _lib.load()
    B, D = x.shape
    K = weight.shape[1]
    if K < 2:
        return x * weight[:, 0]
    if x.stride(1) != 1:
        x = x.contiguous()
    weight = weight.to(x.dtype).contiguous()
    if state_table.dtype != x.dtype or state_table.stride(2) != 1 or state_table.stride(1) != K - 1:
        raise ValueError("state_table must be (max_seqs, D, K-1) with dense rows in x's dtype")
    slots = slots.to(torch.int64).contiguous()
    out = torch.empty((B, D), device=x.device, dtype=x.dtype)
    _lib.check(lib.atma_causal_conv1d_decode_step(
        _lib.ptr(x), x.stride(0), _lib.ptr(weight), _lib.ptr(slots), _lib.ptr(state_table),
        state_table.stride(0), _lib.ptr(out), out.stride(0), B, D, K, _lib.dtype_code(x),
        _lib.stream_ptr()))
    return out


@torch.no_grad()
def causal_conv1d_fn(x, weight, bias=None, return_final_states=False, initial_states=None):
    """x (1 or B, C, T) channel-major as the third-party kernel takes it; weight (C,K).
    Returns out (B,C,T) and, if asked, final_states (B,C,K-1) = last K-1 inputs."""
    from .inference_ops import _packed_conv
    if bias is not None:
        raise ValueError("ATMA's depthwise convs have no bias")
    Bn, C, T = x.shape
    K = weight.shape[1]
    xt = x.transpose(1, 2).reshape(Bn * T, C).contiguous()                  # packed (tokens, C)
    ar = torch.arange(Bn, device=x.device, dtype=torch.int32)
    starts = (ar * T).repeat_interleave(T)
    ends = starts + T
    slots = ar.repeat_interleave(T)
    state = torch.zeros((Bn, C, K - 1), device=x.device, dtype=x.dtype)
    init = None if initial_states is None else initial_states.to(x.dtype).contiguous()
    out = _packed_conv(xt, weight, state, starts, ends, slots, init_state=init, residual=False)
    out = out.view(Bn, T, C).transpose(1, 2)
    return (out, state) if return_final_states else out
