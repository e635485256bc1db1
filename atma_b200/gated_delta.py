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


@torch.no_grad()
def gated_delta_decode_step_fused(q, k, v, state_table, slots, *, gamma=None, beta=None, gate_logits=None,
                                  gamma_bias=3.9, beta_bias=0.0, gate=None, out=None, eps=1e-12):
    """The decode step of the memory with the ops around it folded in (dk = dv = 128): q (B,H,dk); k, v
    (B,Hkv,d) UN-expanded KV heads; gamma/beta (B,H) fp32, or ``gate_logits`` = (g_logit, b_logit), the
    (B,H) outputs of the two gate projections in q's dtype (gamma = sigmoid(g + gamma_bias), ...);
    ``gate`` (B,H*dv) with ``out`` (B,H*dv) view -> out = RMSNorm(r) * sigmoid(gate) in q's dtype (the
    operand of mem.proj, inference/models/atma.py:373-375) and ``out`` is returned; else r (B,H,dv) fp32."""
    _lib.require_cuda(q, "gated_delta_decode_step_fused")
    lib = _lib.load()
    B, H, dk = q.shape
    Hkv, dv = k.shape[1], state_table.shape[3]
    if state_table.dtype != torch.float32 or state_table.stride(3) != 1 or state_table.stride(2) != dv:
        raise ValueError("state_table must be float32 with dense [dk, dv] planes")
    q, k, v = _inner_contiguous(q), _inner_contiguous(k).to(q.dtype), _inner_contiguous(v).to(q.dtype)
    slots = slots.to(torch.int64).contiguous()
    g_l = b_l = None
    logit_sb = 0
    if gate_logits is not None:
        g_l, b_l = gate_logits
        if g_l.dtype != q.dtype or b_l.dtype != q.dtype or g_l.stride(1) != 1 or b_l.stride(1) != 1 or g_l.stride(0) != b_l.stride(0):
            raise ValueError("gate_logits must be two (B,H) tensors in q's dtype with equal row strides")
        logit_sb = g_l.stride(0)
    else:
        gamma, beta = gamma.float().contiguous(), beta.float().contiguous()
    r = None
    if gate is None:
        r = torch.empty((B, H, dv), device=q.device, dtype=torch.float32)
    else:
        if out is None:
            out = torch.empty((B, H * dv), device=q.device, dtype=q.dtype)
        if gate.dtype != q.dtype or gate.stride(1) != 1 or out.dtype != q.dtype or out.stride(1) != 1:
            raise ValueError("gate and out must be (B,H*dv) in q's dtype with contiguous rows")
    _lib.check(lib.atma_gated_delta_decode_step_fused(
        _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), q.stride(0), q.stride(1), k.stride(0), k.stride(1), v.stride(0), v.stride(1),
        _lib.dtype_code(q), Hkv, _lib.ptr(gamma) if g_l is None else None, _lib.ptr(beta) if g_l is None else None,
        _lib.ptr(g_l), _lib.ptr(b_l), logit_sb, float(gamma_bias), float(beta_bias),
        _lib.ptr(state_table), state_table.stride(0), state_table.stride(1), _lib.ptr(slots), _lib.ptr(r),
        _lib.ptr(gate), 0 if gate is None else gate.stride(0), _lib.ptr(out), 0 if out is None else out.stride(0),
        B, H, dk, dv, float(eps), float(torch.finfo(torch.float32).eps), _lib.stream_ptr()))
    return r if gate is None else out


_scratch_cache = {}
_scratch_retired = []


def _scan_scratch(device, nbytes):
    """Scratch for the chunk records: one buffer per (device, stream), grown on demand; an outgrown
    buffer is kept alive (a CUDA graph captured earlier may still point at it), and while a capture
    is in progress the buffer comes from the graph's own pool."""
    if torch.cuda.is_current_stream_capturing():
        return torch.empty(int(nbytes), device=device, dtype=torch.uint8)
    key = (device.type, device.index, torch.cuda.current_stream(device).cuda_stream)
    buf = _scratch_cache.get(key)
    if buf is None or buf.numel() < nbytes:
        if buf is not None:
            _scratch_retired.append(buf)
        buf = torch.empty(int(nbytes), device=device, dtype=torch.uint8)
        _scratch_cache[key] = buf
    return buf


def _varlen_supported(q, dk, dv):
    return q.dtype in (torch.bfloat16, torch.float16) and dk == 128 and dv == 128


@torch.no_grad()
def _scan_varlen(q, k, v, g, beta, cu_seqlens, scale, use_qk_l2norm_in_kernel, *, initial_state=None,
                 want_final=False, state_table=None, slots=None, has_initial=None, snapshots=None,
                 snapshot_offsets=None, snapshot_every=0):
    """Packed batch through one factor launch and one recurrence launch (16-bit, dk = dv = 128)."""
    lib = _lib.load()
    total, H, dk = q.shape
    Hkv, dv = k.shape[1], v.shape[-1]
    n_seqs = cu_seqlens.numel() - 1
    q, k, v = q.contiguous(), k.to(q.dtype).contiguous(), v.to(q.dtype).contiguous()
    g, beta = g.float().contiguous(), beta.float().contiguous()
    cu = cu_seqlens.to(device=q.device, dtype=torch.int32).contiguous()
    o = torch.empty((total, H, dv), device=q.device, dtype=q.dtype)
    final = None
    if state_table is None:
        if initial_state is not None:
            initial_state = initial_state.float().contiguous()
        if want_final:
            final = torch.empty((n_seqs, H, dk, dv), device=q.device, dtype=torch.float32)
        slot_stride = 0
    else:
        if state_table.dtype != torch.float32 or state_table.stride(3) != 1 or state_table.stride(2) != dv \
                or state_table.stride(1) != dk * dv:
            raise ValueError("state_table must be float32 with dense [H, dk, dv] rows")
        slots = slots.to(device=q.device, dtype=torch.int64).contiguous()
        if has_initial is not None:
            has_initial = has_initial.to(device=q.device, dtype=torch.int32).contiguous()
        slot_stride = state_table.stride(0)
    scratch = _scan_scratch(q.device, max(256, lib.atma_gated_delta_scan_varlen_scratch_bytes(total, n_seqs, H, dk, dv)))
    if snapshots is not None:
        off = snapshot_offsets.to(device=q.device, dtype=torch.int32).contiguous()
        _lib.check(lib.atma_gated_delta_scan_varlen_snapshots(
            _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.dtype_code(q), _lib.ptr(g), _lib.ptr(beta), _lib.ptr(cu), n_seqs,
            total, _lib.ptr(state_table), slot_stride, _lib.ptr(slots), _lib.ptr(has_initial), _lib.ptr(o),
            _lib.ptr(scratch), H, Hkv, dk, dv, 1 if use_qk_l2norm_in_kernel else 0, float(scale), _lib.ptr(snapshots),
            _lib.ptr(off), int(snapshot_every), _lib.stream_ptr()))
        return o, None
    _lib.check(lib.atma_gated_delta_scan_varlen(
        _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.dtype_code(q), _lib.ptr(g), _lib.ptr(beta), _lib.ptr(cu), n_seqs,
        total, _lib.ptr(initial_state), _lib.ptr(final), _lib.ptr(state_table), slot_stride, _lib.ptr(slots),
        _lib.ptr(has_initial), _lib.ptr(o), _lib.ptr(scratch), H, Hkv, dk, dv, 1 if use_qk_l2norm_in_kernel else 0,
        float(scale), _lib.stream_ptr()))
    return o, final


def _packed_prefill_snapshots_by_page(q, k, v, g, beta, seqlens, state_table, slots, has_initial, scale, l2norm, page):
    """fp32 inputs / other head sizes: every sequence is scanned page by page through the dense entry, the state
    after each full page is kept.  Same return value as the one-pass form."""
    counts = [int(n) // page for n in seqlens]
    offsets = [0]
    for c in counts:
        offsets.append(offsets[-1] + c)
    H, dk, dv = q.shape[1], q.shape[-1], v.shape[-1]
    snaps = torch.empty((max(offsets[-1], 1), H, dk, dv), device=q.device, dtype=torch.float32)
    o = torch.empty((q.shape[0], H, dv), device=q.device, dtype=q.dtype)
    slot_l = slots.tolist()
    init_l = None if has_initial is None else has_initial.tolist()
    pos = 0
    for i, n in enumerate(seqlens):
        n = int(n)
        S = state_table[slot_l[i]].unsqueeze(0).clone() if (init_l is None or init_l[i]) else None
        for j, a in enumerate(range(0, n, page)):
            b = min(a + page, n)
            sl = slice(pos + a, pos + b)
            oi, S = chunk_gated_delta_rule(q=q[sl].unsqueeze(0), k=k[sl].unsqueeze(0), v=v[sl].unsqueeze(0), g=g[sl].unsqueeze(0),
                                           beta=beta[sl].unsqueeze(0), scale=scale, initial_state=S, output_final_state=True,
                                           use_qk_l2norm_in_kernel=l2norm)
            o[sl] = oi[0]
            if b - a == page:
                snaps[offsets[i] + j] = S[0]
        if n > 0:
            state_table[slot_l[i]] = S[0]
        pos += n
    return o, snaps[:offsets[-1]], offsets[:-1]


@torch.no_grad()
def packed_gated_delta_prefill(q, k, v, g, beta, cu_seqlens, state_table, slots, has_initial=None, scale=1.0,
                               use_qk_l2norm_in_kernel=True, snapshot_every=None, seqlens=None):
    """The memory branch of a packed (several sequences, one token axis) prefill in one call.

    The reference loops over the sequences, calls the scan once per sequence with that
    sequence's table row as ``initial_state`` when it continues a cached prefix, and copies
    the final state back (inference/models/atma.py:494-503).  Here the rows are read and
    written by the recurrence kernel itself.

    q (total,H,dk); k, v (total,H or Hkv,d); g, beta (total,H); cu_seqlens (n+1,) int, on the
    host or the device; state_table (rows,H,dk,dv) fp32, updated IN PLACE at rows ``slots``
    (n,); has_initial (n,) bool/int or None (= every sequence continues from its row).
    Returns o (total,H,dv) in q's dtype.

    ``snapshot_every`` (tokens, a multiple of 64 - e.g. the KV page size) with ``seqlens`` (host
    list of the sequence lengths) also returns the memory state after every full page of each
    sequence: (o, snapshots (n_pages_total, H, dk, dv) fp32, page_offsets list) where sequence
    i's j-th page boundary is row page_offsets[i] + j.  With these a request that reuses cached
    K/V pages can start its memory from the matching state instead of from zero
    (one kernel pass for 16-bit inputs with dk = dv = 128; other inputs are scanned page by page)."""
    _lib.require_cuda(q, "packed_gated_delta_prefill")
    dk, dv = q.shape[-1], v.shape[-1]
    if snapshot_every is not None:
        if seqlens is None or snapshot_every % 64 != 0:
            raise ValueError("state snapshots need the host-side seqlens and a spacing that is a multiple of 64 tokens")
        if not _varlen_supported(q, dk, dv):
            return _packed_prefill_snapshots_by_page(q, k, v, g, beta, seqlens, state_table, slots, has_initial, scale,
                                                     use_qk_l2norm_in_kernel, snapshot_every)
        counts = [int(n) // snapshot_every for n in seqlens]
        offsets = [0]
        for cnt in counts:
            offsets.append(offsets[-1] + cnt)
        snaps = torch.empty((max(offsets[-1], 1), q.shape[1], dk, dv), device=q.device, dtype=torch.float32)
        o, _ = _scan_varlen(q, k, v, g, beta, cu_seqlens, scale, use_qk_l2norm_in_kernel, state_table=state_table,
                            slots=slots, has_initial=has_initial, snapshots=snaps,
                            snapshot_offsets=torch.tensor(offsets[:-1], dtype=torch.int32), snapshot_every=snapshot_every)
        return o, snaps[:offsets[-1]], offsets[:-1]
    if _varlen_supported(q, dk, dv):
        o, _ = _scan_varlen(q, k, v, g, beta, cu_seqlens, scale, use_qk_l2norm_in_kernel, state_table=state_table,
                            slots=slots, has_initial=has_initial)
        return o
    # fp32 inputs or other head sizes: the dense entry once per sequence (lengths read on the host)
    cu = cu_seqlens.tolist()
    slot_l = slots.tolist()
    init_l = None if has_initial is None else has_initial.tolist()
    o = torch.empty((q.shape[0], q.shape[1], dv), device=q.device, dtype=q.dtype)
    for i in range(len(cu) - 1):
        a, b = cu[i], cu[i + 1]
        if b <= a:
            continue
        s0 = state_table[slot_l[i]].unsqueeze(0) if (init_l is None or init_l[i]) else None
        oi, Si = chunk_gated_delta_rule(q=q[a:b].unsqueeze(0), k=k[a:b].unsqueeze(0), v=v[a:b].unsqueeze(0),
                                        g=g[a:b].unsqueeze(0), beta=beta[a:b].unsqueeze(0), scale=scale,
                                        initial_state=s0, output_final_state=True,
                                        use_qk_l2norm_in_kernel=use_qk_l2norm_in_kernel)
        o[a:b] = oi[0]
        state_table[slot_l[i]] = Si[0]
    return o


@torch.no_grad()
def chunk_gated_delta_rule(q=None, k=None, v=None, g=None, beta=None, scale=None,
                           initial_state=None, output_final_state=False,
                           use_qk_l2norm_in_kernel=False, cu_seqlens=None, segments=None, **unused):
    """Chunked gated-delta scan.  q (B,T,H,dk); k (B,T,H or Hkv,dk), v (B,T,H or Hkv,dv) - the
    un-expanded KV heads are accepted, head h then reads KV head h // (H // Hkv); g (B,T,H) log-decay (<= 0);
    beta (B,T,H); initial_state (B,H,dk,dv) fp32 or None.  Returns (o (B,T,H,dv) in q's dtype,
    final_state (B,H,dk,dv) fp32 or None).  ``scale`` defaults to dk**-0.5 as in
    flash-linear-attention; the reference always passes 1.0.

    ``cu_seqlens`` (n+1,) as in flash-linear-attention: the batch axis must be 1 and the token
    axis holds n sequences back to back; initial_state / final_state are then (n,H,dk,dv).

    ``segments`` (not in the reference's call): how many pieces each sequence is cut into along T so
    that a batch of few sequences still fills the GPU (None = chosen from the shapes, 1 = single pass,
    which is the least total work and what a caller running the scan beside other kernels wants)."""
    _lib.require_cuda(q, "chunk_gated_delta_rule")
    lib = _lib.load()
    B, T, H, dk = q.shape
    dv = v.shape[-1]
    Hkv = k.shape[2]
    if v.shape[2] != Hkv or H % Hkv != 0:
        raise ValueError("k and v must share a head count that divides q's")
    if scale is None:
        scale = dk ** -0.5
    if cu_seqlens is not None:
        if B != 1:
            raise ValueError("with cu_seqlens the batch axis must be 1 (sequences are packed on the token axis)")
        n = cu_seqlens.numel() - 1
        if _varlen_supported(q, dk, dv):
            o, final = _scan_varlen(q[0], k[0], v[0], g[0], beta[0], cu_seqlens, scale, use_qk_l2norm_in_kernel,
                                    initial_state=initial_state, want_final=output_final_state)
            return o.unsqueeze(0), final
        cu = cu_seqlens.tolist()
        o = torch.empty((1, T, H, dv), device=q.device, dtype=q.dtype)
        finals = []
        for i in range(n):
            a, b = cu[i], cu[i + 1]
            s0 = None if initial_state is None else initial_state[i:i + 1]
            oi, Si = chunk_gated_delta_rule(q=q[:, a:b], k=k[:, a:b], v=v[:, a:b], g=g[:, a:b], beta=beta[:, a:b],
                                            scale=scale, initial_state=s0, output_final_state=True,
                                            use_qk_l2norm_in_kernel=use_qk_l2norm_in_kernel)
            o[:, a:b] = oi
            finals.append(Si)
        return o, (torch.cat(finals) if output_final_state else None)
    q, k, v = q.contiguous(), k.to(q.dtype).contiguous(), v.to(q.dtype).contiguous()
    g = g.float().contiguous()
    beta = beta.float().contiguous()
    if initial_state is not None:
        initial_state = initial_state.float().contiguous()
    o = torch.empty((B, T, H, dv), device=q.device, dtype=q.dtype)
    final = torch.empty((B, H, dk, dv), device=q.device, dtype=torch.float32) if output_final_state else None
    scratch = _scan_scratch(q.device, max(16, lib.atma_gated_delta_scan_scratch_bytes(B, T, H, dk, dv)))
    _lib.check(lib.atma_gated_delta_scan_segmented(
        _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.dtype_code(q), _lib.ptr(g), _lib.ptr(beta),
        _lib.ptr(initial_state), _lib.ptr(o), _lib.ptr(final), _lib.ptr(scratch),
        B, T, H, Hkv, dk, dv, 1 if use_qk_l2norm_in_kernel else 0, float(scale),
        0 if segments is None else int(segments), _lib.stream_ptr()))
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
    """Second half: run ``len(rec_of)`` (<= 64) recurrences over ``factors``.  Recurrence i walks
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
