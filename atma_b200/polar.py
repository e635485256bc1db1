"""Polar Attention entry points with the reference's call signatures.

Drop-in for the forward-only functions of the reference's ``kernel/polar_triton.py``:
``polar_attention_fwd`` (:594-609), ``polar_attention_packed_fwd`` (:613-669) and
``polar_attention_decode`` (:796-858).  Same argument names, meaning, return values and
error behaviour; the work is done by hand-written sm_100a kernels behind the C ABI.

One extension that is not a signature change: ``k`` and ``v`` may carry the un-expanded
``Hkv`` KV heads (``Hkv`` dividing ``H``); the reference always expands them to ``H`` first
(inference/models/atma.py:417-420), which quadruples K/V traffic.
"""

import math
from ctypes import byref

import torch
import torch.nn.functional as F

from . import _lib

HAS_TRITON = torch.cuda.is_available()     # the flag the reference's callers gate on
HAS_CUDA_EXT = HAS_TRITON


_param_cache = {}


def invalidate_param_cache():
    """Forget the prepared Polar parameters.  The cache is keyed on each raw tensor's storage address and
    version counter; a write that bypasses the counter (``param.data.copy_``, ``set_``, a loader that
    assigns ``.data``) leaves a stale entry behind - call this after such a write."""
    _param_cache.clear()


def _params(v_null, null_base, null_slope_raw, len_gain_raw, mag_beta_raw, device):
    """softplus on the host, as kernel/polar_triton.py:540-544 does.  The five small tensors are
    prepared once per (storage, version) of the raw parameters and reused, so a decode step
    launches nothing but its own kernels.  Writes through ``.data`` do not bump the version:
    see ``invalidate_param_cache``."""
    raw = (v_null, null_base, null_slope_raw, len_gain_raw, mag_beta_raw)
    key = tuple((t.data_ptr(), t._version, t.dtype, str(t.device)) for t in raw) + (str(device),)
    hit = _param_cache.get(key)
    if hit is not None:
        return hit
    if len(_param_cache) > 256:
        _param_cache.clear()
    out = _params_uncached(v_null, null_base, null_slope_raw, len_gain_raw, mag_beta_raw, device)
    out["_raw"] = raw                       # keeps the storages alive, so the key cannot be recycled
    _param_cache[key] = out
    return out


def _params_uncached(v_null, null_base, null_slope_raw, len_gain_raw, mag_beta_raw, device):
    return dict(
        spg=F.softplus(len_gain_raw.detach().float()).contiguous().to(device),
        sps=F.softplus(null_slope_raw.detach().float()).contiguous().to(device),
        beta=F.softplus(mag_beta_raw.detach().float()).contiguous().to(device),
        null_base=null_base.detach().float().contiguous().to(device),
        v_null=v_null.detach().float().contiguous().to(device),
    )


def _inner_contiguous(t):
    return t if t.stride(-1) == 1 else t.contiguous()


def _fill_common(a, p, eps, window, dtype_code):
    a.v_null, a.spg, a.null_base = _lib.ptr(p["v_null"]), _lib.ptr(p["spg"]), _lib.ptr(p["null_base"])
    a.sps, a.beta = _lib.ptr(p["sps"]), _lib.ptr(p["beta"])
    a.eps = float(eps)
    a.window = 0 if window is None else int(window)
    a.dtype = dtype_code


def polar_prefill_raw(q, k, v, n_keys, params, *, eps=1e-6, window=None, key_offset=0,
                      stats_in=None, finalize=True, n_base=None):
    """Lower-level form used by ``polar_attention_fwd`` and by the ring (context-parallel)
    prefill: q (B,H,Tq,dk) and k, v (B,Hkv,Tk,dk) as strided views with a contiguous last
    dimension.  ``stats_in`` = (m, L, Q2, S) fp32 from earlier key blocks; with
    ``finalize=False`` the updated statistics are returned instead of (c, mag)."""
    _lib.require_cuda(q, "polar_attention_fwd")
    lib = _lib.load()
    B, H, Tq, dk = q.shape
    Hkv, Tk = k.shape[1], k.shape[2]
    q, k, v = _inner_contiguous(q), _inner_contiguous(k), _inner_contiguous(v)
    a = _lib.PolarPrefillArgs()
    a.q, a.k, a.v = _lib.ptr(q), _lib.ptr(k), _lib.ptr(v)
    a.q_sb, a.q_sh, a.q_st = q.stride(0), q.stride(1), q.stride(2)
    a.k_sb, a.k_sh, a.k_st = k.stride(0), k.stride(1), k.stride(2)
    a.v_sb, a.v_sh, a.v_st = v.stride(0), v.stride(1), v.stride(2)
    a.B, a.H, a.Hkv, a.Tq, a.Tk, a.dk = B, H, Hkv, Tq, Tk, dk
    a.key_offset = int(key_offset)
    if n_keys is not None:
        n_keys = n_keys.to(device=q.device, dtype=torch.float32).contiguous()
        a.n_keys = _lib.ptr(n_keys)
    else:
        a.n_keys, a.n_base = None, float(n_base)
    _fill_common(a, params, eps, window, _lib.dtype_code(q))
    keep = [q, k, v, n_keys, params]
    if stats_in is not None:
        m, L, Q2, S = (t.contiguous() for t in stats_in)
        a.stats_in_m, a.stats_in_l, a.stats_in_q2, a.stats_in_s = map(_lib.ptr, (m, L, Q2, S))
        keep += [m, L, Q2, S]
    a.finalize = 1 if finalize else 0
    a.n_tiles = 0
    if finalize:
        c = torch.empty((B, H, Tq, dk), device=q.device, dtype=q.dtype)
        mag = torch.empty((B, H, Tq), device=q.device, dtype=q.dtype)
        a.c, a.c_sb, a.c_sh, a.c_st = _lib.ptr(c), c.stride(0), c.stride(1), c.stride(2)
        a.mag, a.mag_sb, a.mag_sh, a.mag_st = _lib.ptr(mag), mag.stride(0), mag.stride(1), mag.stride(2)
        _lib.check(lib.atma_polar_prefill(byref(a), _lib.stream_ptr()))
        return c, mag
    om = torch.empty((B, H, Tq), device=q.device, dtype=torch.float32)
    ol, oq2 = torch.empty_like(om), torch.empty_like(om)
    os_ = torch.empty((B, H, Tq, dk), device=q.device, dtype=torch.float32)
    a.stats_out_m, a.stats_out_l, a.stats_out_q2, a.stats_out_s = map(_lib.ptr, (om, ol, oq2, os_))
    _lib.check(lib.atma_polar_prefill(byref(a), _lib.stream_ptr()))
    return om, ol, oq2, os_


@torch.no_grad()
def polar_attention_fwd(q, k, v, n_keys, *, v_null, null_base, null_slope_raw,
                        len_gain_raw, mag_beta_raw, eps=1e-6, is_causal=True,
                        input_precision="ieee", window=None):
    """Forward-only Polar attention.  q (B,H,Tq,dk); k, v (B,H or Hkv,Tk,dk); n_keys (Tq,)
    valid-key count per query.  Returns (c (B,H,Tq,dk), mag (B,H,Tq)) in q's dtype.

    ``is_causal`` only asserts the standard self-attention layout (Tq == Tk), as in the
    reference; masking always comes from ``n_keys`` and key tiles no query can see are
    skipped either way.  ``input_precision`` is accepted for signature parity: fp32 inputs
    are always multiplied in full fp32."""
    B, H, Tq, dk = q.shape
    Tk = k.shape[2]
    if is_causal and Tq != Tk:
        raise ValueError(
            f"is_causal=True requires Tq == Tk (standard causal self-attention); got "
            f"Tq={Tq}, Tk={Tk}. Use is_causal=False with an explicit n_keys for "
            f"decode / offset-prefill layouts.")
    if dk & (dk - 1) != 0:
        raise ValueError(f"head_dim (dk={dk}) must be a power of two.")
    params = _params(v_null, null_base, null_slope_raw, len_gain_raw, mag_beta_raw, q.device)
    return polar_prefill_raw(q, k, v, n_keys, params, eps=eps, window=window)


@torch.no_grad()
def polar_attention_packed_fwd(q, k, v, tile_seq_starts, tile_q_starts, tile_seq_lens, *,
                               v_null, null_base, null_slope_raw, len_gain_raw, mag_beta_raw,
                               eps=1e-6, input_precision="ieee", window=None):
    """Fresh causal Polar attention over a packed ragged batch.  q (tokens,H,dk); k, v
    (tokens,H or Hkv,dk); one tile-map entry per 128-row query tile.  Returns c like q and
    mag (tokens,H)."""
    if not q.is_cuda:
        raise RuntimeError("packed Polar attention requires CUDA")
    if q.ndim != 3 or k.ndim != 3 or k.shape != v.shape or k.shape[0] != q.shape[0] or k.shape[2] != q.shape[2]:
        raise ValueError("q, k, and v must have [tokens, heads, dim] shapes with equal tokens and dim")
    total, heads, dk = q.shape
    if heads % k.shape[1] != 0:
        raise ValueError("the number of query heads must be a multiple of the KV heads")
    if q.dtype not in (torch.bfloat16, torch.float16):
        raise ValueError("packed Polar route is enabled only for 16-bit inference")
    if dk & (dk - 1):
        raise ValueError(f"head_dim (dk={dk}) must be a power of two")
    if not (tile_seq_starts.numel() == tile_q_starts.numel() == tile_seq_lens.numel()):
        raise ValueError("packed Polar tile-map tensors must have equal lengths")
    lib = _lib.load()
    params = _params(v_null, null_base, null_slope_raw, len_gain_raw, mag_beta_raw, q.device)
    q, k, v = _inner_contiguous(q), _inner_contiguous(k), _inner_contiguous(v)
    maps = [t.to(device=q.device, dtype=torch.int32).contiguous()
            for t in (tile_seq_starts, tile_q_starts, tile_seq_lens)]
    c = torch.empty_like(q, memory_format=torch.contiguous_format)
    mag = torch.empty((total, heads), device=q.device, dtype=q.dtype)
    a = _lib.PolarPrefillArgs()
    a.q, a.k, a.v = _lib.ptr(q), _lib.ptr(k), _lib.ptr(v)
    a.q_sb, a.q_sh, a.q_st = 0, q.stride(1), q.stride(0)
    a.k_sb, a.k_sh, a.k_st = 0, k.stride(1), k.stride(0)
    a.v_sb, a.v_sh, a.v_st = 0, v.stride(1), v.stride(0)
    a.c, a.c_sb, a.c_sh, a.c_st = _lib.ptr(c), 0, c.stride(1), c.stride(0)
    a.mag, a.mag_sb, a.mag_sh, a.mag_st = _lib.ptr(mag), 0, mag.stride(1), mag.stride(0)
    a.B, a.H, a.Hkv, a.Tq, a.Tk, a.dk = 1, heads, k.shape[1], total, total, dk
    a.n_keys, a.n_base, a.key_offset, a.finalize = None, 0.0, 0, 1
    a.tile_seq_start, a.tile_q_start, a.tile_seq_len = map(_lib.ptr, maps)
    a.n_tiles = maps[0].numel()
    _fill_common(a, params, eps, window, _lib.dtype_code(q))
    if a.n_tiles:
        _lib.check(lib.atma_polar_prefill(byref(a), _lib.stream_ptr()))
    return c, mag


_sm_counts = {}


def _sm_count(device=None):
    idx = torch.cuda.current_device() if device is None or device.index is None else device.index
    if idx not in _sm_counts:
        _sm_counts[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _sm_counts[idx]


def decode_num_splits(B, Hkv, max_context, sm_count=None, ctas_per_sm=2):
    """Key ranges per (sequence, KV head).  The split kernel keeps ``ctas_per_sm`` CTAs resident
    per SM, so the grid B*Hkv*n runs in ceil(B*Hkv*n / (sm_count*ctas_per_sm)) waves; pick the n
    (at least 1024 keys per range, at most 64 ranges) whose last wave is fullest, preferring
    more ranges on a tie-ish.  Depends only on launch-time shapes (CUDA-graph safe)."""
    if sm_count is None:
        sm_count = _sm_count() if torch.cuda.is_available() else 148
    slots = sm_count * ctas_per_sm
    n_max = int(max(1, min(64, max_context // 1024)))
    best_n, best_eff = 1, -1.0
    for n in range(1, n_max + 1):
        ctas = B * Hkv * n
        waves = -(-ctas // slots)
        eff = ctas / (waves * slots)
        if ctas < slots:                       # under one wave: more ranges always help
            eff = ctas / slots
        if eff > best_eff + 0.02:              # a larger n must buy at least 2% to be preferred
            best_n, best_eff = n, eff
    return best_n


_scratch_cache = {}
_scratch_retired = []


def _decode_scratch(device, nfloats):
    """Scratch for the split partials: one buffer per (device, stream), so calls on different streams
    never share it; grown on demand and reused across calls (stable address once warm).  A buffer
    that is outgrown is kept alive, not freed: a CUDA graph captured earlier may still point at it.
    While a capture is in progress the buffer comes from the graph's own pool instead."""
    if torch.cuda.is_current_stream_capturing():
        return torch.empty(int(nfloats), device=device, dtype=torch.float32)     # owned by the graph being captured
    key = (device.type, device.index, torch.cuda.current_stream(device).cuda_stream)
    buf = _scratch_cache.get(key)
    if buf is None or buf.numel() < nfloats:
        if buf is not None:
            _scratch_retired.append(buf)
        buf = torch.empty(int(nfloats), device=device, dtype=torch.float32)
        _scratch_cache[key] = buf
    return buf


@torch.no_grad()
def polar_attention_decode(q, k_cache, v_cache, block_tables, context_lens, *,
                           v_null, null_base, null_slope_raw, len_gain_raw, mag_beta_raw,
                           eps=1e-6, block_n=None, num_warps=None, num_stages=None, window=None,
                           num_splits=None, gate=None, out=None, append=None, beside=None):
    """Paged Polar decode.  q (B,H,dk); caches (num_blocks, block_size, Hkv, dk) contiguous;
    block_tables (B,max_blocks) int32; context_lens (B,) int32 including the current token.
    Returns c (B,H,dk), mag (B,H) in q's dtype.  ``block_n``, ``num_warps``, ``num_stages``
    are the reference's Triton launch knobs, accepted and ignored.

    Two extensions that are not in the reference's signature: ``gate`` (B,H,dk), any (row, head)
    strides - c comes back as c * sigmoid(gate), the operand of the output projection
    (inference/models/atma.py:246-252), from the merge kernel itself; ``out`` = (c_view, mag_view),
    preallocated views with a dense last dimension (e.g. two column ranges of one activation
    buffer) that receive the results instead of fresh tensors; ``append`` = (k_new (B,Hkv,dk), v_new, slot_mapping
    (B,) int32): the K/V rows of the token being decoded and their cache rows - the call stores them before it
    reads the cache, i.e. it replaces the ``store_kvcache`` that precedes the decode call in the reference's
    attention layer (inference/layers/attention.py:85-97); one launch less per step.

    ``beside`` = a callable that launches work which neither reads nor writes anything this call touches (the
    memory branch of the layer).  It is run on a side stream between the key-range kernel and the merge kernel, so
    that it shares the machine with the small merge launch instead of the bandwidth-bound key-range launch; the
    call then returns (c, mag, beside()) and has joined the side stream."""
    _lib.require_cuda(q, "polar_attention_decode")
    lib = _lib.load()
    B, H, dk = q.shape
    num_blocks, block_size, Hkv, _ = k_cache.shape
    if not (k_cache.is_contiguous() and v_cache.is_contiguous()):
        raise ValueError("k_cache and v_cache must be contiguous")
    if k_cache.dtype != q.dtype or v_cache.dtype != q.dtype:
        raise ValueError("q and the KV cache must share a dtype")
    max_blocks = block_tables.shape[1]
    q = q.contiguous()
    if block_tables.dtype != torch.int32 or block_tables.stride(1) != 1:
        block_tables = block_tables.to(torch.int32).contiguous()
    if context_lens.dtype != torch.int32 or not context_lens.is_contiguous():
        context_lens = context_lens.to(torch.int32).contiguous()
    params = _params(v_null, null_base, null_slope_raw, len_gain_raw, mag_beta_raw, q.device)
    n_splits = num_splits or decode_num_splits(B, Hkv, max_blocks * block_size)
    scratch = _decode_scratch(q.device, lib.atma_polar_decode_scratch_floats(B, H, dk, n_splits))
    a = _lib.PolarDecodeArgs()
    if out is None:
        c = torch.empty((B, H, dk), device=q.device, dtype=q.dtype)
        mag = torch.empty((B, H), device=q.device, dtype=q.dtype)
    else:
        c, mag = out
        if c.shape != (B, H, dk) or mag.shape != (B, H) or c.dtype != q.dtype or mag.dtype != q.dtype or \
                c.stride(2) != 1 or c.stride(1) != dk or mag.stride(1) != 1:
            raise ValueError("out = (c (B,H,dk), mag (B,H)) views in q's dtype with dense rows")
        a.c_sb, a.mag_sb = c.stride(0), mag.stride(0)
    if gate is not None:
        if gate.shape != (B, H, dk) or gate.dtype != q.dtype or gate.stride(2) != 1:
            raise ValueError("gate must be (B,H,dk) in q's dtype with a contiguous last dimension")
        a.gate, a.gate_sb, a.gate_sh = _lib.ptr(gate), gate.stride(0), gate.stride(1)
    a.q, a.k_cache, a.v_cache = _lib.ptr(q), _lib.ptr(k_cache), _lib.ptr(v_cache)
    a.block_tables, a.bt_stride, a.context_lens = _lib.ptr(block_tables), block_tables.stride(0), _lib.ptr(context_lens)
    a.v_null, a.spg, a.null_base = _lib.ptr(params["v_null"]), _lib.ptr(params["spg"]), _lib.ptr(params["null_base"])
    a.sps, a.beta = _lib.ptr(params["sps"]), _lib.ptr(params["beta"])
    a.c, a.mag, a.scratch = _lib.ptr(c), _lib.ptr(mag), _lib.ptr(scratch)
    a.B, a.H, a.Hkv, a.dk, a.block_size = B, H, Hkv, dk, block_size
    a.max_blocks, a.num_blocks, a.n_splits = max_blocks, num_blocks, n_splits
    a.dtype, a.window, a.eps = _lib.dtype_code(q), (0 if window is None else int(window)), float(eps)
    if append is not None:
        k_new, v_new, slot_mapping = append
        if k_new.shape != (B, Hkv, dk) or v_new.shape != (B, Hkv, dk) or k_new.dtype != q.dtype or v_new.dtype != q.dtype:
            raise ValueError("append = (k_new (B,Hkv,dk), v_new (B,Hkv,dk), slot_mapping (B,)) in q's dtype")
        if k_new.stride(2) != 1 or k_new.stride(1) != dk:
            k_new = k_new.contiguous()
        if v_new.stride(2) != 1 or v_new.stride(1) != dk:
            v_new = v_new.contiguous()
        slot_mapping = slot_mapping.to(torch.int32).contiguous()
        a.append_k, a.append_v = _lib.ptr(k_new), _lib.ptr(v_new)
        a.append_k_stride, a.append_v_stride = k_new.stride(0), v_new.stride(0)
        a.append_slots = _lib.ptr(slot_mapping)
        if not lib.atma_polar_decode_appends(byref(a)):          # this shape is not served in-kernel: the separate scatter
            from .kvcache import store_kvcache
            store_kvcache(k_new, v_new, k_cache, v_cache, slot_mapping)
            a.append_k = a.append_v = a.append_slots = None
    if beside is None:
        _lib.check(lib.atma_polar_decode(byref(a), _lib.stream_ptr()))
        return c, mag
    a.skip_merge = 1
    _lib.check(lib.atma_polar_decode(byref(a), _lib.stream_ptr()))          # the key-range kernel alone
    cur = torch.cuda.current_stream(q.device)
    side = _beside_stream(q.device)
    side.wait_stream(cur)
    with torch.cuda.stream(side):
        extra = beside()
    a.skip_merge = 0
    _lib.check(lib.atma_polar_decode_merge(byref(a), _lib.stream_ptr()))
    cur.wait_stream(side)
    return c, mag, extra


# Up to this many sequences a caller's side work (the memory step) is better placed beside the merge launch
# (``beside=``) than beside the key-range launch (a fork before the call): 51.6 against 55.9 us per step at 8
# sequences of 32K context, 90.3 against 98.3 at 16, a tie at 32; at 64 the fork is ahead, 324.9 against 329.2.
DECODE_BESIDE_MAX_ROWS = 32

_beside_streams = {}


def _beside_stream(device):
    s = _beside_streams.get(device.index)
    if s is None:
        s = _beside_streams[device.index] = torch.cuda.Stream(device=device)
    return s


@torch.no_grad()
def polar_decode_partials(q, k_cache, v_cache, block_tables, local_lens, total_lens, params, *, eps=1e-6, num_splits=None):
    """Key-range pass of the paged decode over the keys of THIS cache only, for a context whose keys are spread
    over several caches (a sequence prefilled context-parallel over several GPUs).  ``local_lens`` (B,) int32 =
    keys in this cache, ``total_lens`` (B,) int32 = the whole context (it sets the temperature); ``params`` as
    returned by ``_params``.  Returns the un-merged statistics (stats (B,H,n,4) = {m, L, Q2, 0}, sums (B,H,n,dk)),
    fp32; ``polar_decode_merge`` folds any number of them."""
    _lib.require_cuda(q, "polar_decode_partials")
    lib = _lib.load()
    B, H, dk = q.shape
    num_blocks, block_size, Hkv, _ = k_cache.shape
    q = q.contiguous()
    block_tables = block_tables.to(torch.int32).contiguous()
    local_lens = local_lens.to(torch.int32).contiguous()
    total_lens = total_lens.to(torch.int32).contiguous()
    n = num_splits or decode_num_splits(B, Hkv, block_tables.shape[1] * block_size)
    scratch = torch.empty(int(lib.atma_polar_decode_scratch_floats(B, H, dk, n)), device=q.device, dtype=torch.float32)
    a = _lib.PolarDecodeArgs()
    a.q, a.k_cache, a.v_cache = _lib.ptr(q), _lib.ptr(k_cache), _lib.ptr(v_cache)
    a.block_tables, a.bt_stride, a.context_lens = _lib.ptr(block_tables), block_tables.stride(0), _lib.ptr(local_lens)
    a.temp_lens, a.skip_merge = _lib.ptr(total_lens), 1
    a.v_null, a.spg, a.null_base = _lib.ptr(params["v_null"]), _lib.ptr(params["spg"]), _lib.ptr(params["null_base"])
    a.sps, a.beta, a.scratch = _lib.ptr(params["sps"]), _lib.ptr(params["beta"]), _lib.ptr(scratch)
    a.B, a.H, a.Hkv, a.dk, a.block_size = B, H, Hkv, dk, block_size
    a.max_blocks, a.num_blocks, a.n_splits = block_tables.shape[1], num_blocks, n
    a.dtype, a.window, a.eps = _lib.dtype_code(q), 0, float(eps)
    _lib.check(lib.atma_polar_decode(byref(a), _lib.stream_ptr()))
    cut = B * H * n * 4
    return scratch[:cut].view(B, H, n, 4), scratch[cut:].view(B, H, n, dk)


@torch.no_grad()
def polar_decode_merge(stats, sums, total_lens, params, dtype, *, eps=1e-6):
    """Merge partial statistics (stats (B,H,P,4), sums (B,H,P,dk)) of one context from any number of caches, fold
    the null sink for a context of ``total_lens`` keys and emit c (B,H,dk), mag (B,H) in ``dtype``."""
    lib = _lib.load()
    B, H, P, dk = sums.shape
    scratch = torch.cat([stats.reshape(-1), sums.reshape(-1)]).contiguous()
    total_lens = total_lens.to(torch.int32).contiguous()
    c = torch.empty((B, H, dk), device=sums.device, dtype=dtype)
    mag = torch.empty((B, H), device=sums.device, dtype=dtype)
    a = _lib.PolarDecodeArgs()
    a.context_lens, a.scratch = _lib.ptr(total_lens), _lib.ptr(scratch)
    a.v_null, a.spg, a.null_base = _lib.ptr(params["v_null"]), _lib.ptr(params["spg"]), _lib.ptr(params["null_base"])
    a.sps, a.beta = _lib.ptr(params["sps"]), _lib.ptr(params["beta"])
    a.c, a.mag = _lib.ptr(c), _lib.ptr(mag)
    a.B, a.H, a.dk, a.n_splits = B, H, dk, P
    a.dtype, a.window, a.eps = _lib.DTYPE_CODE[dtype], 0, float(eps)
    _lib.check(lib.atma_polar_decode_merge(byref(a), _lib.stream_ptr()))
    return c, mag
