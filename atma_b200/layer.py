"""Packed prefill of one global attention layer, composed from this package's kernels.

Host-side mirror of the packed ("grouped") prefill branch of the reference's
``AtmaGlobalAttention.forward`` (inference/models/atma.py:389-399,429-441,466-510) together with
the per-token maps its model runner builds (inference/engine/model_runner.py:395-404):

    q|gate, k, v projections      cuBLAS (F.linear)
    RMSNorm + Canon convs + cache  qkv_prep_prefill            one launch, conv-state rows and K/V pages written
    Polar attention                polar_attention_packed_fwd  un-expanded KV heads, one launch for all sequences
    memory branch                  packed_gated_delta_prefill  one call for all sequences, state rows in place,
                                                               on a side stream beside the attention
    gate epilogues                 sigmoid_gate_mul, rms_sigmoid_gate   one pass each
    combine                        W_o(c * sigmoid(gate)) + W_mu(mag) + mem.proj(RMSNorm(r) * sigmoid(mem.gate x))

The reference expands K/V to H heads, loops over the sequences for the memory branch and runs
the q/k/v preparation as nine separate ops; the results are the same.
"""

import torch
import torch.nn.functional as F

from .gated_delta import packed_gated_delta_prefill
from .inference_ops import qkv_prep_prefill, rms_sigmoid_gate, sigmoid_gate_mul
from .mixing import _side_stream
from .polar import polar_attention_fwd, polar_attention_packed_fwd


class PackedMaps:
    """Device-side index tensors of a packed batch (sequences back to back on the token axis)."""

    def __init__(self, seqlens, seq_slots, device, tile=128):
        lens = torch.tensor([int(n) for n in seqlens], dtype=torch.int64)
        slots = torch.tensor([int(s) for s in seq_slots], dtype=torch.int64)
        cu = torch.zeros(lens.numel() + 1, dtype=torch.int64)
        cu[1:] = lens.cumsum(0)
        self.total = int(cu[-1])
        starts = cu[:-1].repeat_interleave(lens)                    # per token: its sequence's first / past-the-end token, slot
        ends = cu[1:].repeat_interleave(lens)
        tslots = slots.repeat_interleave(lens)
        n_tiles = (lens + tile - 1) // tile                         # per 128-row query tile: sequence start, row offset, length
        t_seq = cu[:-1].repeat_interleave(n_tiles)
        t_len = lens.repeat_interleave(n_tiles)
        first = torch.zeros(n_tiles.numel() + 1, dtype=torch.int64)
        first[1:] = n_tiles.cumsum(0)
        t_q = (torch.arange(int(first[-1])) - first[:-1].repeat_interleave(n_tiles)) * tile
        i32 = lambda v: v.to(device=device, dtype=torch.int32)
        self.token_seq_starts, self.token_seq_ends, self.token_seq_slots = i32(starts), i32(ends), i32(tslots)
        self.tile_seq_starts, self.tile_q_starts, self.tile_seq_lens = i32(t_seq), i32(t_q), i32(t_len)
        self.cu_seqlens = i32(cu)
        self.seq_slots = slots.to(device)


def _linear(x, sd, name):
    b = sd.get(name + ".bias")
    return F.linear(x, sd[name + ".weight"].to(x.dtype), None if b is None else b.to(x.dtype))


@torch.no_grad()
def global_attention_prefill_packed(x, sd, maps, *, num_heads, num_kv_heads, head_dim, conv_states, mem_state_table,
                                    k_cache=None, v_cache=None, slot_mapping=None, window=None, mem_gamma_bias=3.9,
                                    mem_beta_bias=0.0, prefix="attn.", overlap=True, has_initial=None, snapshots=None):
    """x (tokens, D) packed fresh prompts; ``sd`` the attention module's tensors (reference names
    under ``prefix``: q, k, v, proj, mu_proj, canon_q/k/v, the five Polar parameters, and mem.*
    when the layer has a memory); ``maps`` a ``PackedMaps``; ``conv_states`` = (q, k, v) conv-state
    tables and ``mem_state_table`` (rows, H, dk, dk) fp32, all updated IN PLACE at the sequences'
    slots; ``k_cache``/``v_cache`` with ``slot_mapping`` receive the post-conv K/V rows.
    ``has_initial``: per sequence, whether its memory continues from its state row (None = all do;
    False = fresh prompts: every memory starts from zero, as the reference's fresh prefill does,
    inference/models/atma.py:272-279).  ``snapshots`` = (PrefixSnapshots, layer index, seqlens): also record the
    memory state and the three convs' last K-1 inputs at every page boundary.  Returns the layer's mixing
    output (tokens, D)."""
    P = prefix
    H, Hkv, dk = num_heads, num_kv_heads, head_dim
    total = x.shape[0]
    q_gate = _linear(x, sd, P + "q").view(total, H, 2 * dk)
    k = _linear(x, sd, P + "k").view(total, Hkv, dk)
    v = _linear(x, sd, P + "v").view(total, Hkv, dk)
    w = [sd[P + f"canon_{n}.weight"].squeeze(1) for n in ("q", "k", "v")]
    k_raw, v_raw = k, v
    q, k, v = qkv_prep_prefill(q_gate, k, v, *w, *conv_states, maps.token_seq_starts, maps.token_seq_ends,
                               maps.token_seq_slots, k_cache, v_cache, slot_mapping)

    if snapshots is not None:                            # the convs' inputs (normalised q, k; v) before each page boundary
        snaps, layer, _ = snapshots
        Kc = w[0].shape[1]
        rows = snaps.rows(Kc - 1)
        eps32 = torch.finfo(torch.float32).eps
        tails = {"q": F.rms_norm(q_gate[rows, :, :dk], (dk,), eps=eps32), "k": F.rms_norm(k_raw[rows], (dk,), eps=eps32),
                 "v": v_raw[rows]}
        for n, t in tails.items():
            snaps.conv[f"attn_{layer}_{n}"] = t.reshape(-1, Kc - 1, t.shape[-2] * t.shape[-1]).transpose(1, 2).contiguous()
    has_mem = (P + "mem.proj.weight") in sd
    cur = torch.cuda.current_stream(x.device)
    side = _side_stream(x.device) if (overlap and has_mem) else cur
    r = None
    if has_mem:
        if side is not cur:
            side.wait_stream(cur)
        with torch.cuda.stream(side):
            g = F.logsigmoid(_linear(x, sd, P + "mem.w_gamma").float() + mem_gamma_bias)
            beta = torch.sigmoid(_linear(x, sd, P + "mem.w_beta").float() + mem_beta_bias)
            if has_initial is False:
                has_initial = torch.zeros(maps.seq_slots.numel(), dtype=torch.int32, device=x.device)
            if snapshots is None:
                r = packed_gated_delta_prefill(q, k, v, g, beta, maps.cu_seqlens, mem_state_table, maps.seq_slots, has_initial)
            else:
                snaps, layer, seqlens = snapshots
                r, mem_snaps, _ = packed_gated_delta_prefill(q, k, v, g, beta, maps.cu_seqlens, mem_state_table, maps.seq_slots,
                                                             has_initial, snapshot_every=snaps.page, seqlens=seqlens)
                snaps.mem[layer] = mem_snaps
            mem_out = _linear(rms_sigmoid_gate(r, _linear(x, sd, P + "mem.gate")), sd, P + "mem.proj")

    pp = dict(v_null=sd[P + "v_null"], null_base=sd[P + "null_base"], null_slope_raw=sd[P + "null_slope_raw"],
              len_gain_raw=sd[P + "len_gain_raw"], mag_beta_raw=sd[P + "mag_beta_raw"])
    if q.dtype in (torch.bfloat16, torch.float16):
        c, mag = polar_attention_packed_fwd(q, k, v, maps.tile_seq_starts, maps.tile_q_starts, maps.tile_seq_lens,
                                            window=window, **pp)
    else:                                   # fp32: sequence by sequence, as the reference's own fallback route does
        c = torch.empty_like(q)
        mag = torch.empty((total, H), device=q.device, dtype=q.dtype)
        cu = maps.cu_seqlens.tolist()
        for a, b in zip(cu[:-1], cu[1:]):
            if b > a:
                n = torch.arange(1, b - a + 1, device=q.device, dtype=torch.float32)
                ci, mi = polar_attention_fwd(q[a:b].transpose(0, 1)[None], k[a:b].transpose(0, 1)[None],
                                             v[a:b].transpose(0, 1)[None], n, window=window, **pp)
                c[a:b], mag[a:b] = ci[0].transpose(0, 1), mi[0].transpose(0, 1)
    gated = sigmoid_gate_mul(c, q_gate[..., dk:]).view(total, H * dk)       # the gate half is read in place
    out = _linear(gated, sd, P + "proj") + _linear(mag, sd, P + "mu_proj")
    if has_mem:
        if side is not cur:
            cur.wait_stream(side)
            mem_out.record_stream(cur)
        out = out + mem_out
    return out
