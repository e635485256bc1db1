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


@torch.no_grad()
def qkv_prep_prefill(q_gate, k, v, w_q, w_k, w_v, state_q, state_k, state_v, token_seq_starts, token_seq_ends,
                     token_seq_slots, k_cache=None, v_cache=None, slot_mapping=None, initial_states=None, eps=None):
    """One launch for what the reference's packed global-layer prefill does in nine
    (inference/models/atma.py:391-399,431-441,468-471): per-head RMSNorm of q and k, the three
    Canon convolutions in residual form with their conv-state rows, and the K/V cache scatter.

    q_gate (tokens, H, 2*dk) as the q projection produces it (the gate half is left alone);
    k, v (tokens, Hkv, dk); w_* (C, K); state_* (rows, C, K-1) updated IN PLACE (None = not
    kept); token_seq_* per-token int32 maps as for ``packed_causal_conv1d``; k_cache, v_cache
    with ``slot_mapping`` (tokens,) int64 updated IN PLACE; ``initial_states`` = (iq, ik, iv)
    tables read as every sequence's left context (must not be the tables being written), None =
    fresh prompts.  Returns q (tokens, H, dk), k, v (tokens, Hkv, dk), ready for
    ``polar_attention_packed_fwd`` / the scan with un-expanded KV heads."""
    _lib.require_cuda(q_gate, "qkv_prep_prefill")
    lib = _lib.load()
    total, H, two_dk = q_gate.shape
    dk = two_dk // 2
    Hkv = k.shape[1]
    K = w_q.shape[1]
    dt = q_gate.dtype
    if q_gate.stride(2) != 1:
        q_gate = q_gate.contiguous()
    k, v = k.to(dt).contiguous(), v.to(dt).contiguous()
    w_q, w_k, w_v = (w.to(dt).contiguous() for w in (w_q, w_k, w_v))
    if eps is None:
        eps = torch.finfo(torch.float32).eps            # what F.rms_norm uses when eps is None (also for 16-bit inputs)
    for st in (state_q, state_k, state_v):
        if st is not None and (st.dtype != dt or st.stride(2) != 1 or st.stride(1) != K - 1):
            raise ValueError("conv-state tables must be in the activation dtype with dense [C, K-1] rows")
    iq, ik, iv = initial_states if initial_states is not None else (None, None, None)
    for a, b in ((iq, state_q), (ik, state_k), (iv, state_v)):
        if a is not None and (b is None or a.shape[1:] != b.shape[1:] or a.stride() != b.stride() or a.dtype != dt):
            raise ValueError("an initial-state table must have the layout of the table that is written")
    i32 = lambda t: t.to(device=q_gate.device, dtype=torch.int32).contiguous()
    s0, e0, sl = i32(token_seq_starts), i32(token_seq_ends), i32(token_seq_slots)
    if k_cache is not None:
        if k_cache.dtype != dt or not k_cache.is_contiguous() or not v_cache.is_contiguous():
            raise ValueError("the caches must be contiguous and in the activation dtype")
        slot_mapping = slot_mapping.to(device=q_gate.device, dtype=torch.int64).contiguous()
    q_out = torch.empty((total, H, dk), device=q_gate.device, dtype=dt)
    k_out = torch.empty((total, Hkv, dk), device=q_gate.device, dtype=dt)
    v_out = torch.empty((total, Hkv, dk), device=q_gate.device, dtype=dt)
    ss = lambda t: 0 if t is None else t.stride(0)
    _lib.check(lib.atma_qkv_prep_prefill(
        _lib.ptr(q_gate), q_gate.stride(0), q_gate.stride(1), _lib.ptr(k), k.stride(0), _lib.ptr(v), v.stride(0),
        _lib.ptr(w_q), _lib.ptr(w_k), _lib.ptr(w_v), _lib.ptr(state_q), _lib.ptr(state_k), _lib.ptr(state_v),
        _lib.ptr(iq), _lib.ptr(ik), _lib.ptr(iv), ss(state_q), ss(state_k), ss(state_v),
        _lib.ptr(s0), _lib.ptr(e0), _lib.ptr(sl), _lib.ptr(q_out), _lib.ptr(k_out), _lib.ptr(v_out),
        _lib.ptr(k_cache), _lib.ptr(v_cache), _lib.ptr(slot_mapping) if k_cache is not None else None,
        total, H, Hkv, dk, K, float(eps), _lib.dtype_code(q_gate), _lib.stream_ptr()))
    return q_out, k_out, v_out


@torch.no_grad()
def sigmoid_gate_mul(x, gate):
    """x * sigmoid(gate) for (tokens, H, dk) operands with arbitrary (row, head) strides and a
    contiguous last dim - e.g. x = the Polar content c and gate = the gate half of the q|gate
    projection, read in place (inference/models/atma.py:552-558).  Returns (tokens, H, dk) dense."""
    _lib.require_cuda(x, "sigmoid_gate_mul")
    lib = _lib.load()
    if x.shape != gate.shape or x.ndim != 3:
        raise ValueError("x and gate must both be (tokens, H, dk)")
    if x.stride(2) != 1:
        x = x.contiguous()
    if gate.stride(2) != 1 or gate.dtype != x.dtype:
        gate = gate.to(x.dtype).contiguous()
    rows, H, dk = x.shape
    out = torch.empty((rows, H, dk), device=x.device, dtype=x.dtype)
    _lib.check(lib.atma_sigmoid_gate_mul(_lib.ptr(x), x.stride(0), x.stride(1), _lib.ptr(gate), gate.stride(0),
                                         gate.stride(1), _lib.ptr(out), rows, H, dk, _lib.dtype_code(x), _lib.stream_ptr()))
    return out


@torch.no_grad()
def rms_sigmoid_gate(r, gate, eps=None):
    """RMSNorm(r) over the head dim (affine-free) times sigmoid(gate): r (tokens, H, dk),
    gate (tokens, H*dk); the memory read-out before ``mem.proj``
    (inference/models/atma.py:373-375).  Returns (tokens, H*dk)."""
    _lib.require_cuda(r, "rms_sigmoid_gate")
    lib = _lib.load()
    rows, H, dk = r.shape
    if gate.shape != (rows, H * dk):
        raise ValueError("gate must be (tokens, H*dk)")
    r = r.contiguous()
    if gate.stride(1) != 1 or gate.dtype != r.dtype:
        gate = gate.to(r.dtype).contiguous()
    if eps is None:
        eps = torch.finfo(torch.float32).eps
    out = torch.empty((rows, H * dk), device=r.device, dtype=r.dtype)
    _lib.check(lib.atma_rms_sigmoid_gate(_lib.ptr(r), _lib.ptr(gate), gate.stride(0), _lib.ptr(out), rows, H, dk,
                                         float(eps), _lib.dtype_code(r), _lib.stream_ptr()))
    return out


def _check_conv_state(state_table, dt, K):
    if state_table.dtype != dt or state_table.stride(2) != 1 or state_table.stride(1) != K - 1:
        raise ValueError("state_table must be (max_seqs, D, K-1) with dense rows in the activation dtype")


@torch.no_grad()
def lfm2_conv_decode_step(projected, weight, slots, state_table):
    """One decode step of the local layers' gated short conv: projected (B, 3*D) = [B | C | x'] as
    ``in_proj`` returns it, weight (D, K), slots (B,), state_table (max_seqs, D, K-1) updated IN
    PLACE.  Returns C * conv(B * x') (B, D) - what inference/models/atma.py:633-636,668-673 feed
    to ``out_proj``."""
    _lib.require_cuda(projected, "lfm2_conv_decode_step")
    lib = _lib.load()
    Bn, D3 = projected.shape
    D, K = weight.shape
    if D3 != 3 * D:
        raise ValueError("projected must be (B, 3*D)")
    if projected.stride(1) != 1:
        projected = projected.contiguous()
    weight = weight.to(projected.dtype).contiguous()
    _check_conv_state(state_table, projected.dtype, K)
    slots = slots.to(torch.int64).contiguous()
    out = torch.empty((Bn, D), device=projected.device, dtype=projected.dtype)
    _lib.check(lib.atma_lfm2_conv_decode_step(_lib.ptr(projected), projected.stride(0), _lib.ptr(weight), _lib.ptr(slots),
                                              _lib.ptr(state_table), state_table.stride(0), _lib.ptr(out), out.stride(0),
                                              Bn, D, K, _lib.dtype_code(projected), _lib.stream_ptr()))
    return out


@torch.no_grad()
def lfm2_conv_packed(projected, weight, state_table, token_seq_starts, token_seq_ends, token_seq_slots,
                     initial_state=None):
    """The same block over packed ragged prompts (inference/models/atma.py:648-653): projected
    (tokens, 3*D); each sequence's row of ``state_table`` receives its last K-1 gated inputs.
    ``initial_state`` (a table of the same layout, not the one being written) continues cached
    prefixes; None = fresh prompts.  Returns C * conv(B * x') (tokens, D)."""
    _lib.require_cuda(projected, "lfm2_conv_packed")
    lib = _lib.load()
    total, D3 = projected.shape
    D, K = weight.shape
    if D3 != 3 * D:
        raise ValueError("projected must be (tokens, 3*D)")
    if projected.stride(1) != 1:
        projected = projected.contiguous()
    weight = weight.to(projected.dtype).contiguous()
    _check_conv_state(state_table, projected.dtype, K)
    if initial_state is not None and (initial_state.stride() != state_table.stride() or initial_state.dtype != state_table.dtype):
        raise ValueError("initial_state must have the layout of state_table")
    i32 = lambda t: t.to(device=projected.device, dtype=torch.int32).contiguous()
    s0, e0, sl = i32(token_seq_starts), i32(token_seq_ends), i32(token_seq_slots)
    out = torch.empty((total, D), device=projected.device, dtype=projected.dtype)
    _lib.check(lib.atma_lfm2_conv_packed(_lib.ptr(projected), projected.stride(0), _lib.ptr(weight), _lib.ptr(out),
                                         out.stride(0), _lib.ptr(state_table), _lib.ptr(initial_state), state_table.stride(0),
                                         _lib.ptr(s0), _lib.ptr(e0), _lib.ptr(sl), total, D, K,
                                         _lib.dtype_code(projected), _lib.stream_ptr()))
    return out


@torch.no_grad()
def qkv_prep_decode(q_gate, k, v, w_q, w_k, w_v, state_q, state_k, state_v, slots, k_cache=None, v_cache=None,
                    slot_mapping=None, eps=None):
    """One launch for the decode-side glue of a global layer (inference/models/atma.py:557-572): per-head
    RMSNorm of q and k, the three Canon conv steps in residual form on the slot-indexed state tables
    (updated IN PLACE), and the scatter of the new K/V row into the paged cache.

    q_gate (B, H, 2*dk) as the q projection produces it, any (row, head) strides (the gate half is left
    alone); k, v (B, Hkv, dk), any row stride; w_* (C, K); state_* (rows, C, K-1); slots (B,) int64
    (negative = padded row); k_cache / v_cache (..., Hkv, dk) contiguous with slot_mapping (B,) int32
    (-1 = skip).  Returns q (B, H, dk), k, v (B, Hkv, dk)."""
    _lib.require_cuda(q_gate, "qkv_prep_decode")
    lib = _lib.load()
    B, H, two_dk = q_gate.shape
    dk, Hkv, K, dt = two_dk // 2, k.shape[1], w_q.shape[1], q_gate.dtype
    if q_gate.stride(2) != 1:
        q_gate = q_gate.contiguous()
    if k.stride(2) != 1 or k.stride(1) != dk or k.dtype != dt:
        k = k.to(dt).contiguous()
    if v.stride(2) != 1 or v.stride(1) != dk or v.dtype != dt:
        v = v.to(dt).contiguous()
    w_q, w_k, w_v = (w.to(dt).contiguous() for w in (w_q, w_k, w_v))
    for st in (state_q, state_k, state_v):
        _check_conv_state(st, dt, K)
    if eps is None:
        eps = torch.finfo(torch.float32).eps
    slots = slots.to(torch.int64).contiguous()
    if k_cache is not None:
        if k_cache.dtype != dt or not k_cache.is_contiguous() or not v_cache.is_contiguous():
            raise ValueError("the caches must be contiguous and in the activation dtype")
        slot_mapping = slot_mapping.to(torch.int32).contiguous()
    q_out = torch.empty((B, H, dk), device=q_gate.device, dtype=dt)
    k_out = torch.empty((B, Hkv, dk), device=q_gate.device, dtype=dt)
    v_out = torch.empty((B, Hkv, dk), device=q_gate.device, dtype=dt)
    _lib.check(lib.atma_qkv_prep_decode(
        _lib.ptr(q_gate), q_gate.stride(0), q_gate.stride(1), _lib.ptr(k), k.stride(0), _lib.ptr(v), v.stride(0),
        _lib.ptr(w_q), _lib.ptr(w_k), _lib.ptr(w_v), _lib.ptr(state_q), _lib.ptr(state_k), _lib.ptr(state_v),
        state_q.stride(0), state_k.stride(0), state_v.stride(0), _lib.ptr(slots), _lib.ptr(q_out), _lib.ptr(k_out),
        _lib.ptr(v_out), _lib.ptr(k_cache), _lib.ptr(v_cache), _lib.ptr(slot_mapping) if k_cache is not None else None,
        B, H, Hkv, dk, K, float(eps), _lib.dtype_code(q_gate), _lib.stream_ptr()))
    return q_out, k_out, v_out


@torch.no_grad()
def add_rms_norm(x, y, weight, eps=1e-6):
    """(x + y, RMSNorm(x + y) * weight) in one pass over rows of up to 4096 values; y None = no add
    (then the first result is x itself).  The residual add of one sub-layer fused with the norm in
    front of the next (inference/models/atma.py:709-712)."""
    _lib.require_cuda(x, "add_rms_norm")
    lib = _lib.load()
    D = x.shape[-1]
    x2 = x.reshape(-1, D)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    y2 = None
    if y is not None:
        y2 = y.reshape(-1, D).to(x.dtype)
        if not y2.is_contiguous():
            y2 = y2.contiguous()
    w = None if weight is None else weight.to(x.dtype).contiguous()
    x_out = torch.empty_like(x2) if y is not None else None
    h = torch.empty_like(x2)
    _lib.check(lib.atma_add_rms_norm(_lib.ptr(x2), _lib.ptr(y2), _lib.ptr(w), _lib.ptr(x_out), _lib.ptr(h), x2.shape[0], D,
                                     float(eps), _lib.dtype_code(x), _lib.stream_ptr()))
    return (x if y is None else x_out.view(x.shape)), h.view(x.shape)



DECODE_LINEAR_MAX_ROWS = 16


def decode_linear_supported(x, weight, gated=False):
    """Whether ``decode_linear`` serves this product: CUDA, 16-bit, 1..16 rows, K a multiple of 32, N a multiple of 16
    (32 for the gated form), 16-byte aligned rows."""
    return (x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and weight.dtype == x.dtype and x.ndim == 2 and
            0 < x.shape[0] <= DECODE_LINEAR_MAX_ROWS and x.shape[1] % 32 == 0 and weight.shape[0] % (32 if gated else 16) == 0 and
            weight.is_contiguous() and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0)


@torch.no_grad()
def decode_linear(x, weight, bias=None, gated=False):
    """x @ weight.T + bias for a decode batch of up to 16 rows, the weights streamed once from HBM
    (``F.linear`` at these sizes); ``gated``: weight is the MLP's fc projection (2F, K) and the result is
    second_half * relu(first_half)^2, (rows, F) - the fc GEMM and ``squared_relu_gate`` of
    inference/models/atma.py:87-97 in one launch.  x (rows, K), weight (N, K) contiguous, 16-bit."""
    _lib.require_cuda(x, "decode_linear")
    lib = _lib.load()
    B, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K or weight.dtype != x.dtype or not weight.is_contiguous():
        raise ValueError("weight must be a contiguous (N, K) tensor in x's dtype")
    if x.stride(1) != 1:
        x = x.contiguous()
    if bias is not None:
        bias = bias.to(x.dtype).contiguous()
    out = torch.empty((B, N // 2 if gated else N), device=x.device, dtype=x.dtype)
    _lib.check(lib.atma_decode_linear(_lib.ptr(x), x.stride(0), _lib.ptr(weight), _lib.ptr(bias), _lib.ptr(out), out.stride(0),
                                      B, N, K, 1 if gated else 0, _lib.dtype_code(x), _lib.stream_ptr()))
    return out
