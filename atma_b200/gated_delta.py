"""Gated-delta ("Titans MAG") memory entry points with the reference's call signatures.

``gated_delta_decode_step`` is a drop-in for kernel/gated_delta_triton.py:79-117.
``chunk_gated_delta_rule`` takes the keyword call the reference makes into
flash-linear-attention (inference/models/atma.py:285-287,318-322; model/blocks.py:48-49)
and implements the recurrence of model/blocks.py:375-423 with the [K,V] fp32 state.
"""

import torch

from . import _lib

HAS_TRITON = torch.cuda.is_available()


def _inner_contiguous(t):
    return t if t.stride(-1) == 1 else t.contiguous()


@torch.no_grad()
def gated_delta_decode_step(q, k, v, gamma, beta, state_table, slots, eps=1e-12, block_v=None):
    """One batched gated-delta step, in place on the slot-indexed state table.

    q, k, v (B,H,dk) current-token tensors (KV heads expanded to H, any strides with a
    contiguous last dim); gamma, beta (B,H); state_table (max_seqs,H,dk,dv) fp32, [K,V]
    layout, updated IN PLACE; slots (B,) integer rows of the table.  Returns r (B,H,dv)
    fp32.  ``block_v`` is the reference's tile knob, accepted and ignored."""
    _lib.require_cuda(q, "gated_delta_decode_step")
    lib = _lib.load()
    B, H, dk = q.shape
    dv = state_table.shape[3]
    if state_table.dtype != torch.float32:
        raise ValueError("state_table must be float32")
    if state_table.stride(3) != 1 or state_table.stride(2) != dv:
        raise ValueError("state_table's [dk, dv] planes must be dense")
    q, k, v = _inner_contiguous(q), _inner_contiguous(k), _inner_contiguous(v)
    if k.dtype != q.dtype or v.dtype != q.dtype:
        k, v = k.to(q.dtype), v.to(q.dtype)
    gamma = gamma.float().contiguous()
    beta = beta.float().contiguous()
    slots = slots.to(torch.int64).contiguous()
    r = torch.empty((B, H, dv), device=q.device, dtype=torch.float32)
    _lib.check(lib.atma_gated_delta_decode_step(
        _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), q.stride(0), q.stride(1), k.stride(0), k.stride(1),
        v.stride(0), v.stride(1), _lib.dtype_code(q), _lib.ptr(gamma), _lib.ptr(beta),
        _lib.ptr(state_table), state_table.stride(0), state_table.stride(1), _lib.ptr(slots),
        _lib.ptr(r), B, H, dk, dv, float(eps), _lib.stream_ptr()))
    return r


_scratch_cache = {}


def _scan_scratch(device, nbytes):
    key = (device.type, device.index)
    buf = _scratch_cache.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(int(nbytes), device=device, dtype=torch.uint8)
        _scratch_cache[key] = buf
    return buf


@torch.no_grad()
def chunk_gated_delta_rule(q=None, k=None, v=None, g=None, beta=None, scale=None,
                           initial_state=None, output_final_state=False,
                           use_qk_l2norm_in_kernel=False, **unused):
    """Chunked gated-delta scan.  q (B,T,H,dk); k (B,T,H or Hkv,dk), v (B,T,H or Hkv,dv) - the
    un-expanded KV heads are accepted, head h then reads KV head h // (H // Hkv); g (B,T,H) log-decay (<= 0);
    beta (B,T,H); initial_state (B,H,dk,dv) fp32 or None.  Returns (o (B,T,H,dv) in q's dtype,
    final_state (B,H,dk,dv) fp32 or None).  ``scale`` defaults to dk**-0.5 as in
    flash-linear-attention; the reference always passes 1.0."""
    _lib.require_cuda(q, "chunk_gated_delta_rule")
    lib = _lib.load()
    B, T, H, dk = q.shape
    dv = v.shape[-1]
    Hkv = k.shape[2]
    if v.shape[2] != Hkv or H % Hkv != 0:
        raise ValueError("k and v must share a head count that divides q's")
    if scale is None:
        scale = dk ** -0.5
    q, k, v = q.contiguous(), k.to(q.dtype).contiguous(), v.to(q.dtype).contiguous()
    g = g.float().contiguous()
    beta = beta.float().contiguous()
    if initial_state is not None:
        initial_state = initial_state.float().contiguous()
    o = torch.empty((B, T, H, dv), device=q.device, dtype=q.dtype)
    final = torch.empty((B, H, dk, dv), device=q.device, dtype=torch.float32) if output_final_state else None
    scratch = _scan_scratch(q.device, max(16, lib.atma_gated_delta_scan_scratch_bytes(B, T, H, dk, dv)))
    _lib.check(lib.atma_gated_delta_scan(
        _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.dtype_code(q), _lib.ptr(g), _lib.ptr(beta),
        _lib.ptr(initial_state), _lib.ptr(o), _lib.ptr(final), _lib.ptr(scratch),
        B, T, H, Hkv, dk, dv, 1 if use_qk_l2norm_in_kernel else 0, float(scale), _lib.stream_ptr()))
    return o, final


class ScanFactors:
    """Handle on the per-chunk factors of B sequences (see ``scan_factors``)."""

    def __init__(self, scratch, B, T, H, dk, dv, dtype, device):
        self.scratch, self.B, self.T, self.H, self.dk, self.dv, self.dtype, self.device = scratch, B, T, H, dk, dv, dtype, device


@torch.no_grad()
def scan_factors(q, k, v, g, beta, scale=1.0, use_qk_l2norm_in_kernel=True):
    """First half of ``chunk_gated_delta_rule`` for a sequence that is split across GPUs: the
    state-independent per-chunk factors (16-bit inputs, dk = dv = 128).  The returned handle owns
    its scratch memory; pass it to ``scan_recur`` any number of times."""
    _lib.require_cuda(q, "scan_factors")
    lib = _lib.load()
    B, T, H, dk = q.shape
    dv, Hkv = v.shape[-1], k.shape[2]
    q, k, v = q.contiguous(), k.to(q.dtype).contiguous(), v.to(q.dtype).contiguous()
    g, beta = g.float().contiguous(), beta.float().contiguous()
    scratch = torch.empty(int(lib.atma_gated_delta_scan_scratch_bytes(B, T, H, dk, dv)), device=q.device, dtype=torch.uint8)
    _lib.check(lib.atma_gated_delta_scan_factors(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.dtype_code(q), _lib.ptr(g),
                                                 _lib.ptr(beta), _lib.ptr(scratch), B, T, H, Hkv, dk, dv,
                                                 1 if use_qk_l2norm_in_kernel else 0, float(scale), _lib.stream_ptr()))
    return ScanFactors(scratch, B, T, H, dk, dv, q.dtype, q.device)


@torch.no_grad()
def scan_recur(factors, rec_of, initial_state=None, zero_value=None, want_output=True):
    """Second half: run ``len(rec_of)`` (<= 16) recurrences over ``factors``.  Recurrence i walks
    the factors of sequence ``rec_of[i]`` from ``initial_state[i]`` ((n,H,dk,dv) fp32 or None).
    ``zero_value[i]`` true runs it with v = 0 (started from the identity it yields the
    state-transfer matrix of the segment).  Returns (o (n,T,H,dv) or None, final_state (n,H,dk,dv))."""
    import ctypes
    lib = _lib.load()
    f = factors
    n = len(rec_of)
    rec_arr = (ctypes.c_int * n)(*[int(x) for x in rec_of])
    zero_arr = (ctypes.c_int * n)(*[1 if (zero_value is not None and zero_value[i]) else 0 for i in range(n)])
    if initial_state is not None:
        initial_state = initial_state.float().contiguous()
    o = torch.empty((n, f.T, f.H, f.dv), device=f.device, dtype=f.dtype) if want_output else None
    final = torch.empty((n, f.H, f.dk, f.dv), device=f.device, dtype=torch.float32)
    _lib.check(lib.atma_gated_delta_scan_recur(_lib.ptr(f.scratch), _lib.DTYPE_CODE[f.dtype], f.B, f.T, f.H, f.dk, f.dv, n,
                                               rec_arr, zero_arr, _lib.ptr(initial_state), _lib.ptr(o), _lib.ptr(final),
                                               _lib.stream_ptr()))
    return o, final
