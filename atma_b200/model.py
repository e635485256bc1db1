"""The whole ATMA model on this package's kernels: packed prefill and paged decode.

Host-side mirror of the reference's inference model (inference/models/atma.py:716-754 ``Atma``,
:631-673 ``AtmaLFM2Conv``, :377-618 ``AtmaAttention``, :87-97 ``InferenceMLP``) and of what its
model runner prepares per step (inference/engine/model_runner.py:328-513): 16 blocks, every
fourth one (i % 4 == 2) a global Polar + gated-delta layer, the others LFM2 gated short convs,
each followed by the squared-ReLU gated MLP; final RMSNorm, LM head, logit soft-cap.  It takes
the reference's ``state_dict`` as is (inference/utils/loader.py:5-39).

Projections are cuBLAS (``F.linear``); everything between them is this library:

    prefill (packed fresh prompts)          decode (one token per sequence, CUDA-graph safe)
    add_rms_norm                            add_rms_norm
    lfm2_conv_packed                        lfm2_conv_decode_step
    qkv_prep_prefill                        qkv_prep_decode
    polar_attention_packed_fwd              polar_attention_decode (c * sigmoid(gate) written by the merge)
    packed_gated_delta_prefill              gated_delta_decode_step_fused (gates from logits, RMSNorm * sigmoid(gate))
    sigmoid_gate_mul, rms_sigmoid_gate
    squared_relu_gate, softcap_logits       squared_relu_gate, softcap_logits

In decode a global layer is six launches: one GEMM for all of its input projections (q|gate, k,
v, the two memory gates' logits, the memory's output gate - their weights concatenated once at
load time), the q/k/v glue kernel, the two Polar decode kernels, the memory step, and one GEMM for
W_o, W_mu and mem.proj together (their inputs lie side by side in one activation buffer, so the
sum of the three projections is one product).
"""

from dataclasses import dataclass, field

import torch
import torch.nn.functional as F

import hashlib

from .gated_delta import gated_delta_decode_step, gated_delta_decode_step_fused, packed_gated_delta_prefill
from .inference_ops import qkv_prep_prefill, sigmoid_gate_mul
from .polar import polar_attention_fwd
from .inference_ops import (add_rms_norm, decode_linear, decode_linear_supported, lfm2_conv_decode_step, lfm2_conv_packed,
                            qkv_prep_decode, rms_sigmoid_gate, softcap_logits, squared_relu_gate)
from .layer import PackedMaps, global_attention_prefill_packed
from .polar import DECODE_BESIDE_MAX_ROWS, polar_attention_decode

POLAR_NAMES = ("v_null", "null_base", "null_slope_raw", "len_gain_raw", "mag_beta_raw")


@dataclass
class ModelState:
    """Everything a sequence leaves on the device between steps, slot-indexed like the reference's
    tables (inference/engine/model_runner.py:200-252): per global layer a paged K/V cache, three
    Canon conv-state tables and the fp32 memory state; per local layer the gated conv's state."""
    k_cache: dict = field(default_factory=dict)      # layer -> (num_blocks, block_size, Hkv, dk)
    v_cache: dict = field(default_factory=dict)
    conv: dict = field(default_factory=dict)         # "conv_{i}" -> (rows, D, K-1); "attn_{i}_{q,k,v}" -> (rows, C, K-1)
    mem: dict = field(default_factory=dict)          # layer -> (rows, H, dk, dk) fp32


class AtmaModel:
    def __init__(self, state_dict, *, layers, hidden, head_dim, num_kv_heads, window=None, gamma_bias=3.9, beta_bias=0.0,
                 eps=1e-6, dtype=torch.bfloat16, device="cuda"):
        self.L, self.D, self.dk, self.Hkv = layers, hidden, head_dim, num_kv_heads
        self.H = hidden // head_dim
        self.window, self.gamma_bias, self.beta_bias, self.eps = window, gamma_bias, beta_bias, eps
        self.dtype, self.device = dtype, torch.device(device)
        sd = {}
        for name, t in state_dict.items():
            keep32 = name.split(".")[-1] in POLAR_NAMES
            sd[name] = t.detach().to(self.device, torch.float32 if keep32 else dtype).contiguous()
        self.sd = sd
        self.vocab = sd["proj.weight"].shape[0]
        self.global_layers = [i for i in range(layers) if i % 4 == 2]
        self.conv_k = sd["blocks.0.attn.conv.weight"].shape[-1] if "blocks.0.attn.conv.weight" in sd else 3
        self.attn_k = sd[f"blocks.{self.global_layers[0]}.attn.canon_q.weight"].shape[-1] if self.global_layers else 4
        self.small_batch_linear = True          # decode batches <= 16: weight-streaming kernel instead of cuBLAS
        self._pack_decode_weights()

    # ---- weights packed for the decode step -------------------------------------------------------
    def _pack_decode_weights(self):
        H, dk, Hkv = self.H, self.dk, self.Hkv
        self.packed = {}
        for i in self.global_layers:
            P = f"blocks.{i}.attn."
            sd = self.sd
            names_in = ["q", "k", "v", "mem.w_gamma", "mem.w_beta", "mem.gate"]
            w_in = torch.cat([sd[P + n + ".weight"] for n in names_in]).contiguous()
            b_in = torch.cat([sd[P + n + ".bias"] for n in names_in]).contiguous()
            w_out = torch.cat([sd[P + "proj.weight"], sd[P + "mu_proj.weight"], sd[P + "mem.proj.weight"]], dim=1).contiguous()
            b_out = (sd[P + "proj.bias"].float() + sd[P + "mu_proj.bias"].float() + sd[P + "mem.proj.bias"].float()).to(self.dtype)
            o_k = 2 * H * dk
            o_v = o_k + Hkv * dk
            o_g = o_v + Hkv * dk
            self.packed[i] = dict(w_in=w_in, b_in=b_in, w_out=w_out, b_out=b_out, o_k=o_k, o_v=o_v, o_g=o_g, o_b=o_g + H,
                                  o_mg=o_g + 2 * H,
                                  canon=[sd[P + f"canon_{n}.weight"].squeeze(1).contiguous() for n in ("q", "k", "v")],
                                  polar={n: sd[P + n] for n in POLAR_NAMES})

    # ---- per-sequence device state ---------------------------------------------------------------------
    def new_state(self, max_seqs, num_blocks, block_size=256):
        st = ModelState()
        dev, dt = self.device, self.dtype
        for i in range(self.L):
            if i in self.global_layers:
                st.k_cache[i] = torch.zeros(num_blocks, block_size, self.Hkv, self.dk, device=dev, dtype=dt)
                st.v_cache[i] = torch.zeros_like(st.k_cache[i])
                for n, C in (("q", self.H * self.dk), ("k", self.Hkv * self.dk), ("v", self.Hkv * self.dk)):
                    st.conv[f"attn_{i}_{n}"] = torch.zeros(max_seqs, C, self.attn_k - 1, device=dev, dtype=dt)
                st.mem[i] = torch.zeros(max_seqs, self.H, self.dk, self.dk, device=dev, dtype=torch.float32)
            else:
                st.conv[f"conv_{i}"] = torch.zeros(max_seqs, self.D, self.conv_k - 1, device=dev, dtype=dt)
        return st

    def _lin(self, x, name):
        return self._linear(x, self.sd[name + ".weight"], self.sd.get(name + ".bias"))

    def _linear(self, x, w, b):
        """Decode batches of up to 16 rows stream the weights through this library's kernel; larger ones are cuBLAS."""
        if self.small_batch_linear and decode_linear_supported(x, w):
            return decode_linear(x, w, b)
        return F.linear(x, w, b)

    def _mlp(self, h, i):
        w, b = self.sd[f"blocks.{i}.mlp.fc.weight"], self.sd.get(f"blocks.{i}.mlp.fc.bias")
        if self.small_batch_linear and decode_linear_supported(h, w, gated=True):
            act = decode_linear(h, w, b, gated=True)            # fc GEMM and the squared-ReLU gate in one launch
        else:
            fc = F.linear(h, w, b)
            half = fc.shape[-1] // 2
            act = squared_relu_gate(fc[:, :half], fc[:, half:])
        return self._lin(act, f"blocks.{i}.mlp.proj")

    def logits(self, hidden):
        """LM head + soft-cap on already-normalised hidden rows (inference/models/atma.py:750-754)."""
        return softcap_logits(self._lin(hidden, "proj"))

    # ---- packed prefill of fresh prompts ----------------------------------------------------------------------
    @torch.no_grad()
    def prefill(self, ids, seqlens, slots, state, slot_mapping, maps=None, snapshot_every=None):
        """ids (tokens,) packed prompts; seqlens / slots per sequence (host lists); slot_mapping (tokens,) cache rows.
        Conv states, memory states and K/V pages of ``state`` are written at the sequences' slots.  ``maps``: the
        batch's ``PackedMaps`` if the caller has built them already.
        Returns the final-norm hidden states of all tokens (tokens, D).

        ``snapshot_every`` (tokens; the K/V page size, a multiple of 64): also returns a ``PrefixSnapshots`` with the
        recurrent state of every layer after each full page of each sequence - the fp32 memory state and the last
        K-1 conv inputs - so that a later request whose prompt shares those pages can continue from them
        (``prefill_from_prefix``) instead of inheriting K/V without state, which the reference documents as a
        source of drift (docs/inference.md:72-75; inference/models/atma.py:477-479)."""
        sd = self.sd
        if maps is None:
            maps = PackedMaps(seqlens, slots, self.device)
        sm = slot_mapping.to(self.device, torch.int64)
        snaps = None
        if snapshot_every is not None:
            if snapshot_every % 64 != 0:
                raise ValueError("snapshot_every must be a multiple of 64 tokens")
            snaps = PrefixSnapshots(seqlens, snapshot_every, maps.cu_seqlens.tolist(), self.device)
        x = sd["embed.weight"][ids.to(self.device)]
        x, h = add_rms_norm(x, None, sd["blocks.0.norm1.weight"], self.eps)
        for i in range(self.L):
            P = f"blocks.{i}."
            if i in self.global_layers:
                mix = global_attention_prefill_packed(
                    h, sd, maps, num_heads=self.H, num_kv_heads=self.Hkv, head_dim=self.dk,
                    conv_states=[state.conv[f"attn_{i}_{n}"] for n in ("q", "k", "v")], mem_state_table=state.mem[i],
                    k_cache=state.k_cache[i].view(-1, self.Hkv, self.dk), v_cache=state.v_cache[i].view(-1, self.Hkv, self.dk),
                    slot_mapping=sm, window=self.window, mem_gamma_bias=self.gamma_bias, mem_beta_bias=self.beta_bias,
                    prefix=P + "attn.", has_initial=False, snapshots=None if snaps is None else (snaps, i, seqlens))
            else:
                proj = self._lin(h, P + "attn.in_proj")
                y = lfm2_conv_packed(proj, sd[P + "attn.conv.weight"].squeeze(1), state.conv[f"conv_{i}"],
                                     maps.token_seq_starts, maps.token_seq_ends, maps.token_seq_slots)
                if snaps is not None:                   # the conv's inputs B * x' at the rows before each page boundary
                    rows = snaps.rows(self.conv_k - 1)
                    gated = proj[rows, :self.D] * proj[rows, 2 * self.D:]
                    snaps.conv[f"conv_{i}"] = gated.view(-1, self.conv_k - 1, self.D).transpose(1, 2).contiguous()
                mix = self._lin(y, P + "attn.out_proj")
            x, h = add_rms_norm(x, mix, sd[P + "norm2.weight"], self.eps)
            nxt = sd[f"blocks.{i + 1}.norm1.weight"] if i + 1 < self.L else sd["norm.weight"]
            x, h = add_rms_norm(x, self._mlp(h, i), nxt, self.eps)
        return h if snaps is None else (h, snaps)

    # ---- one long prompt over several GPUs ----------------------------------------------------------------------
    @torch.no_grad()
    def prefill_context_parallel(self, ids_parts, positions, state, slot, slot_mappings, *, group=None, polar_mode=None):
        """The whole model over a context-parallel group: ONE prompt of T tokens, cut into 2N zig-zag segments, rank r
        holding segments r and 2N-1-r (``context_parallel.zigzag_segments``).  Token-local work (embedding, norms,
        projections, MLP, epilogues) runs on the rank's own 2L tokens as a packed batch of two pieces; what crosses
        segment borders is handed over between ranks:
          * the K-1 conv inputs before each segment (the gated LFM2 input; the normalised q, k and raw v of the three
            Canon convs, one message per layer) - ``cp_conv_halos``;
          * the Polar pass over the gathered (or ring-passed) K/V and the memory scan with its state prefix of affine
            maps - ``cp_global_layer_prefill``.
        ids_parts [lo, hi] (L,) token ids; ``positions`` [(a0, a1), (b0, b1)]; ``slot_mappings`` [lo, hi] (L,) rows of
        THIS rank's K/V pages (every rank caches its own tokens: the layout ``cp_polar_decode`` reads).  At the end the
        recurrent state of the whole prompt - final conv rows (held by the rank that owns the last segment) and memory
        states - is made the same on every rank at row ``slot`` of ``state``, so that decode can go on replicated.
        Returns [h_lo, h_hi] (L, D): the final-norm hidden states of this rank's tokens."""
        import torch.distributed as dist
        from . import context_parallel as cp
        sd, dev, D, H, Hkv, dk = self.sd, self.device, self.D, self.H, self.Hkv, self.dk
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        L = ids_parts[0].numel()
        if ids_parts[1].numel() != L or L % 64 != 0:
            raise ValueError("both segments must have the same length, a multiple of 64 tokens")
        maps = PackedMaps([L, L], [0, 1], dev)                       # the two segments as two packed pieces, rows 0 and 1
        sm = torch.cat([m.to(dev, torch.int64) for m in slot_mappings])
        last_owner = cp.segment_owner(2 * world - 1, world)          # its hi piece ends the prompt
        finals = {}

        def tail_rows(K):
            return torch.cat([torch.arange(L - (K - 1), L, device=dev), torch.arange(2 * L - (K - 1), 2 * L, device=dev)])

        x = sd["embed.weight"][torch.cat([i.to(dev) for i in ids_parts])]
        x, h = add_rms_norm(x, None, sd["blocks.0.norm1.weight"], self.eps)
        for i in range(self.L):
            P = f"blocks.{i}."
            if i in self.global_layers:
                A = P + "attn."
                q_gate = self._lin(h, A + "q").view(2 * L, H, 2 * dk)
                k = self._lin(h, A + "k").view(2 * L, Hkv, dk)
                v = self._lin(h, A + "v").view(2 * L, Hkv, dk)
                w = [sd[A + f"canon_{n}.weight"].squeeze(1) for n in ("q", "k", "v")]
                Kc = w[0].shape[1]
                # conv inputs at the piece ends: normalised q and k, raw v, side by side so that one message carries all
                eps32 = torch.finfo(torch.float32).eps
                idx = tail_rows(Kc)
                tail = torch.cat([F.rms_norm(q_gate[idx, :, :dk], (dk,), eps=eps32).reshape(idx.numel(), H * dk),
                                  F.rms_norm(k[idx], (dk,), eps=eps32).reshape(idx.numel(), Hkv * dk),
                                  v[idx].reshape(idx.numel(), Hkv * dk)], dim=1)
                halo = torch.stack(cp.cp_conv_halos([tail[:Kc - 1], tail[Kc - 1:]], Kc, group=group))   # (2, Cq+2Ckv, K-1)
                Cq, Ck = H * dk, Hkv * dk
                init = [halo[:, :Cq].contiguous(), halo[:, Cq:Cq + Ck].contiguous(), halo[:, Cq + Ck:].contiguous()]
                scratch = [torch.zeros_like(t) for t in init]
                q, k, v = qkv_prep_prefill(q_gate, k, v, *w, *scratch, maps.token_seq_starts, maps.token_seq_ends,
                                           maps.token_seq_slots, state.k_cache[i].view(-1, Hkv, dk),
                                           state.v_cache[i].view(-1, Hkv, dk), sm, initial_states=init)
                for n, t in zip(("q", "k", "v"), scratch):
                    finals[f"attn_{i}_{n}"] = t[1]
                g = F.logsigmoid(self._lin(h, A + "mem.w_gamma").float() + self.gamma_bias)
                beta = torch.sigmoid(self._lin(h, A + "mem.w_beta").float() + self.beta_bias)
                cut = lambda t: [t[:L][None], t[L:][None]]
                shard = cp.GlobalLayerShard(q=cut(q), k=cut(k), v=cut(v), g=cut(g), beta=cut(beta), positions=list(positions))
                pp = {n: sd[A + n] for n in POLAR_NAMES}
                polar, o, S = cp.cp_global_layer_prefill(shard, pp, group=group, polar_mode=polar_mode, window=self.window)
                c = torch.cat([pc[0][0].transpose(0, 1) for pc in polar]).contiguous()          # (2L, H, dk)
                mag = torch.cat([pc[1][0].transpose(0, 1) for pc in polar]).contiguous()        # (2L, H)
                r = torch.cat([oo[0] for oo in o]).contiguous()                                 # (2L, H, dk)
                state.mem[i][slot] = S
                gated = sigmoid_gate_mul(c, q_gate[..., dk:]).view(2 * L, H * dk)
                mix = self._lin(gated, A + "proj") + self._lin(mag.to(self.dtype), A + "mu_proj")
                mix = mix + self._lin(rms_sigmoid_gate(r, self._lin(h, A + "mem.gate")), A + "mem.proj")
            else:
                proj = self._lin(h, P + "attn.in_proj")
                Kc = self.conv_k
                idx = tail_rows(Kc)
                tail = proj[idx, :D] * proj[idx, 2 * D:]             # the conv's inputs B * x' at the piece ends
                init = torch.stack(cp.cp_conv_halos([tail[:Kc - 1], tail[Kc - 1:]], Kc, group=group))   # (2, D, K-1)
                scratch = torch.zeros_like(init)
                y = lfm2_conv_packed(proj, sd[P + "attn.conv.weight"].squeeze(1), scratch, maps.token_seq_starts,
                                     maps.token_seq_ends, maps.token_seq_slots, initial_state=init)
                finals[f"conv_{i}"] = scratch[1]
                mix = self._lin(y, P + "attn.out_proj")
            x, h = add_rms_norm(x, mix, sd[P + "norm2.weight"], self.eps)
            nxt = sd[f"blocks.{i + 1}.norm1.weight"] if i + 1 < self.L else sd["norm.weight"]
            x, h = add_rms_norm(x, self._mlp(h, i), nxt, self.eps)
        # the final conv rows of the prompt live on the owner of the last segment: one broadcast for all layers
        names = sorted(finals)
        flat = torch.cat([finals[n].reshape(-1) for n in names])
        if world > 1:
            src = dist.get_global_rank(group, last_owner) if group is not None else last_owner
            dist.broadcast(flat, src=src, group=group)
        off = 0
        for n in names:
            t = finals[n]
            state.conv[n][slot] = flat[off:off + t.numel()].view_as(t)
            off += t.numel()
        return [h[:L], h[L:]]

    @torch.no_grad()
    def prefill_from_prefix(self, ids_tail, prefix_len, slot, state, slot_mapping_tail, block_table_row, snapshots, index):
        """The rest of ONE prompt whose first ``prefix_len`` tokens (whole pages) are already in the K/V pages that
        ``block_table_row`` points to - cached by an earlier request - with the recurrent state of that prefix taken
        from ``snapshots[index]`` (``PrefixSnapshots``; ``index`` = the page-boundary row, e.g. from
        ``PrefixStateCache.lookup``).  The sequence's rows in the state tables are set from the snapshot, the tail's
        K/V rows go to ``slot_mapping_tail``, attention sees prefix + tail keys (what the reference's chunked-prefill
        continuation does, inference/models/atma.py:509-538).  Returns the tail's final-norm hidden states (T, D)."""
        sd, H, Hkv, dk = self.sd, self.H, self.Hkv, self.dk
        dev = self.device
        T = ids_tail.shape[0]
        maps = PackedMaps([T], [slot], dev)
        sm = slot_mapping_tail.to(dev, torch.int64)
        bs = next(iter(state.k_cache.values())).shape[1]
        if prefix_len % bs != 0:
            raise ValueError("a reused prefix must end at a page boundary")
        pages = block_table_row[:prefix_len // bs].to(dev, torch.long)
        n_keys = torch.arange(prefix_len + 1, prefix_len + T + 1, device=dev, dtype=torch.float32)
        one = torch.ones(1, dtype=torch.int32, device=dev)
        x = sd["embed.weight"][ids_tail.to(dev)]
        x, h = add_rms_norm(x, None, sd["blocks.0.norm1.weight"], self.eps)
        for i in range(self.L):
            P = f"blocks.{i}."
            if i in self.global_layers:
                A = P + "attn."
                tabs = [state.conv[f"attn_{i}_{n}"] for n in ("q", "k", "v")]
                inits = []
                for n, tab in zip(("q", "k", "v"), tabs):                # the prefix's conv state: left context of the tail
                    init = torch.zeros_like(tab)
                    init[slot] = snapshots.conv[f"attn_{i}_{n}"][index]
                    inits.append(init)
                state.mem[i][slot] = snapshots.mem[i][index]
                q_gate = self._lin(h, A + "q").view(T, H, 2 * dk)
                k = self._lin(h, A + "k").view(T, Hkv, dk)
                v = self._lin(h, A + "v").view(T, Hkv, dk)
                q, k, v = qkv_prep_prefill(q_gate, k, v, *(sd[A + f"canon_{n}.weight"].squeeze(1) for n in ("q", "k", "v")), *tabs,
                                           maps.token_seq_starts, maps.token_seq_ends, maps.token_seq_slots,
                                           state.k_cache[i].view(-1, Hkv, dk), state.v_cache[i].view(-1, Hkv, dk), sm,
                                           initial_states=inits)
                k_all = torch.cat([state.k_cache[i][pages].reshape(-1, Hkv, dk), k])     # cached prefix rows + the tail's
                v_all = torch.cat([state.v_cache[i][pages].reshape(-1, Hkv, dk), v])
                c, mag = polar_attention_fwd(q.transpose(0, 1)[None], k_all.transpose(0, 1)[None], v_all.transpose(0, 1)[None],
                                             n_keys, is_causal=False, window=self.window,
                                             **{n: sd[A + n] for n in POLAR_NAMES})
                gated = sigmoid_gate_mul(c[0].transpose(0, 1), q_gate[..., dk:]).view(T, H * dk)
                mix = self._lin(gated, A + "proj") + self._lin(mag[0].transpose(0, 1), A + "mu_proj")
                g = F.logsigmoid(self._lin(h, A + "mem.w_gamma").float() + self.gamma_bias)
                beta = torch.sigmoid(self._lin(h, A + "mem.w_beta").float() + self.beta_bias)
                r = packed_gated_delta_prefill(q, k, v, g, beta, maps.cu_seqlens, state.mem[i], maps.seq_slots, one)
                mix = mix + self._lin(rms_sigmoid_gate(r, self._lin(h, A + "mem.gate")), A + "mem.proj")
            else:
                tab = state.conv[f"conv_{i}"]
                init = torch.zeros_like(tab)
                init[slot] = snapshots.conv[f"conv_{i}"][index]
                proj = self._lin(h, P + "attn.in_proj")
                y = lfm2_conv_packed(proj, sd[P + "attn.conv.weight"].squeeze(1), tab, maps.token_seq_starts,
                                     maps.token_seq_ends, maps.token_seq_slots, initial_state=init)
                mix = self._lin(y, P + "attn.out_proj")
            x, h = add_rms_norm(x, mix, sd[P + "norm2.weight"], self.eps)
            nxt = sd[f"blocks.{i + 1}.norm1.weight"] if i + 1 < self.L else sd["norm.weight"]
            x, h = add_rms_norm(x, self._mlp(h, i), nxt, self.eps)
        return h

    # ---- one decode step ---------------------------------------------------------------------------------
    @torch.no_grad()
    def decode(self, ids, state, seq_slots, slot_mapping, block_tables, context_lens, *, local_lens=None, group=None):
        """One token per sequence: ids (B,), seq_slots (B,) int64 state rows, slot_mapping (B,) int32 cache rows
        of the new token, block_tables (B, max_blocks) int32, context_lens (B,) int32 INCLUDING the new token.
        All arguments are device tensors with fixed shapes, nothing synchronises: the call can be captured in
        a CUDA graph (inference/engine/model_runner.py:254-310).  Returns soft-capped logits (B, vocab).

        ``local_lens`` (B,) int32: the step runs over a cache that a context-parallel prefill left spread over the
        ranks of ``group``.  Every rank makes the same call with the same ids and state (the step is replicated);
        ``block_tables`` and ``local_lens`` then describe THIS rank's pages and key count (the new token included on
        the one rank whose ``slot_mapping`` entry is not -1, which stores its K/V row), ``context_lens`` stays the
        whole context.  The attention of each global layer becomes ``cp_polar_decode``: local partial statistics,
        one small all-gather, the single-GPU merge; full-context attention only."""
        sd, H, Hkv, dk, D = self.sd, self.H, self.Hkv, self.dk, self.D
        B = ids.shape[0]
        x = sd["embed.weight"][ids]
        x, h = add_rms_norm(x, None, sd["blocks.0.norm1.weight"], self.eps)
        for i in range(self.L):
            P = f"blocks.{i}."
            if i in self.global_layers:
                pk = self.packed[i]
                z = self._linear(h, pk["w_in"], pk["b_in"])                              # every input projection at once
                q_gate = z[:, :pk["o_k"]].view(B, H, 2 * dk)
                k = z[:, pk["o_k"]:pk["o_v"]].view(B, Hkv, dk)
                v = z[:, pk["o_v"]:pk["o_g"]].view(B, Hkv, dk)
                q, k, v = qkv_prep_decode(q_gate, k, v, *pk["canon"],
                                          *(state.conv[f"attn_{i}_{n}"] for n in ("q", "k", "v")), seq_slots,
                                          state.k_cache[i], state.v_cache[i], slot_mapping)
                act = torch.empty((B, 2 * H * dk + H), device=x.device, dtype=x.dtype)   # [c * sig(gate) | mag | norm(r) * sig(gate)]
                r_out = act[:, H * dk + H:]
                mem_gate = z[:, pk["o_mg"]:]
                # The memory branch shares nothing it writes with the attention branch (its slice of ``act``, its own
                # state table), so it runs beside the paged attention on a second stream: fork here, join before W_out.
                # Small batches hand it to the decode call instead, which runs it beside the merge launch: the key-range
                # launch then has the machine to itself (polar.DECODE_BESIDE_MAX_ROWS).
                cur = torch.cuda.current_stream(x.device)

                def memory_step():
                    return gated_delta_decode_step_fused(q, k, v, state.mem[i], seq_slots,
                                                         gate_logits=(z[:, pk["o_g"]:pk["o_b"]], z[:, pk["o_b"]:pk["o_mg"]]),
                                                         gamma_bias=self.gamma_bias, beta_bias=self.beta_bias, gate=mem_gate,
                                                         out=r_out)
                beside = dk == 128 and local_lens is None and B <= DECODE_BESIDE_MAX_ROWS
                forked = dk == 128 and not beside
                if forked:
                    side = self._decode_side_stream()
                    side.wait_stream(cur)
                    with torch.cuda.stream(side):
                        memory_step()
                elif beside:
                    pass                                                         # launched by the decode call below
                else:                                                            # other head sizes: the separate kernels
                    G = H // Hkv
                    gamma = torch.sigmoid(z[:, pk["o_g"]:pk["o_b"]].float() + self.gamma_bias)
                    beta = torch.sigmoid(z[:, pk["o_b"]:pk["o_mg"]].float() + self.beta_bias)
                    r = gated_delta_decode_step(q, k.repeat_interleave(G, 1), v.repeat_interleave(G, 1), gamma, beta,
                                                state.mem[i], seq_slots)
                    r_out.copy_(rms_sigmoid_gate(r.to(x.dtype), mem_gate))
                if local_lens is None:
                    polar_attention_decode(q, state.k_cache[i], state.v_cache[i], block_tables, context_lens, window=self.window,
                                           gate=q_gate[..., dk:], out=(act[:, :H * dk].view(B, H, dk), act[:, H * dk:H * dk + H]),
                                           beside=memory_step if beside else None, **pk["polar"])
                else:
                    from .context_parallel import cp_polar_decode
                    if self.window is not None:
                        raise ValueError("decode over a context-parallel cache is full-context attention only")
                    c, mag = cp_polar_decode(q, state.k_cache[i], state.v_cache[i], block_tables, local_lens, context_lens,
                                             pk["polar"], group=group)
                    act[:, :H * dk] = sigmoid_gate_mul(c, q_gate[..., dk:]).view(B, H * dk)
                    act[:, H * dk:H * dk + H] = mag
                if forked:
                    cur.wait_stream(side)                                        # join the memory branch
                mix = self._linear(act, pk["w_out"], pk["b_out"])                          # W_o, W_mu and mem.proj in one product
            else:
                proj = self._lin(h, P + "attn.in_proj")
                y = lfm2_conv_decode_step(proj, sd[P + "attn.conv.weight"].squeeze(1), seq_slots, state.conv[f"conv_{i}"])
                mix = self._lin(y, P + "attn.out_proj")
            x, h = add_rms_norm(x, mix, sd[P + "norm2.weight"], self.eps)
            nxt = sd[f"blocks.{i + 1}.norm1.weight"] if i + 1 < self.L else sd["norm.weight"]
            x, h = add_rms_norm(x, self._mlp(h, i), nxt, self.eps)
        return self.logits(h)

    def _decode_side_stream(self):
        if getattr(self, "_side", None) is None:
            self._side = torch.cuda.Stream(device=self.device)
        return self._side

    def decode_bytes(self, batch, context):
        """Algorithmic HBM bytes of one decode step: every weight once, the K/V rows of the context, the memory
        and conv states read and written, the activations (scripts/roofline_inference.py:66-77 in the reference)."""
        n_w = sum(t.numel() * t.element_size() for n, t in self.sd.items() if n != "embed.weight")
        kv = len(self.global_layers) * 2 * context * self.Hkv * self.dk * 2
        mem = len(self.global_layers) * 2 * self.H * self.dk * self.dk * 4
        conv = 2 * 2 * (len(self.global_layers) * (self.H + 2 * self.Hkv) * self.dk * (self.attn_k - 1) +
                        (self.L - len(self.global_layers)) * self.D * (self.conv_k - 1))
        act = 2 * self.D * 2
        return n_w + batch * (kv + mem + conv + act)


class PrefixSnapshots:
    """Recurrent state of every layer at the page boundaries of a packed prefill.  Row r of every tensor belongs
    to one (sequence, page boundary): sequence i's j-th full page is row ``offsets[i] + j`` (j = 0 is the state
    after the first ``page`` tokens).  ``mem[layer]`` (rows, H, dk, dk) fp32; ``conv[name]`` (rows, C, K-1) in the
    conv-state tables' layout (oldest input first)."""

    def __init__(self, seqlens, page, cu_seqlens, device):
        self.page = page
        counts = [int(n) // page for n in seqlens]
        self.offsets = [0]
        for c in counts:
            self.offsets.append(self.offsets[-1] + c)
        self.n_rows = self.offsets.pop()
        self.ends = [cu_seqlens[i] + (j + 1) * page for i, c in enumerate(counts) for j in range(c)]   # packed token index after each page
        self.device = device
        self.mem, self.conv = {}, {}

    def rows(self, k_minus_1):
        """Packed token indices of the last K-1 inputs before every page boundary, oldest first (rows * (K-1),)."""
        ends = torch.tensor(self.ends, dtype=torch.long, device=self.device)
        return (ends[:, None] + torch.arange(-k_minus_1, 0, device=self.device)[None, :]).reshape(-1)


class PrefixStateCache:
    """Which snapshot goes with which cached page: the bookkeeping an engine keeps beside its block manager's
    hash table.  A page is named by the chained hash of the token ids up to and including it (the scheme of the
    reference's block manager, inference/engine/block_manager.py:42-57); ``register`` files the snapshot rows of a
    finished prefill under those names, ``lookup`` returns the longest run of leading pages of a new prompt that
    has both K/V pages and state on record."""

    def __init__(self, page):
        self.page = page
        self.table = {}                       # chained page hash -> (snapshots, row, physical page id)

    @staticmethod
    def _chain(prev, token_ids):
        h = hashlib.blake2b(digest_size=8)
        h.update(prev.to_bytes(8, "little"))
        h.update(torch.as_tensor(token_ids, dtype=torch.int64).numpy().tobytes())
        return int.from_bytes(h.digest(), "little")

    def page_hashes(self, token_ids):
        out, prev = [], 0
        for j in range(len(token_ids) // self.page):
            prev = self._chain(prev, token_ids[j * self.page:(j + 1) * self.page])
            out.append(prev)
        return out

    def register(self, token_ids, snapshots, seq_index, block_table_row):
        for j, hsh in enumerate(self.page_hashes(token_ids)):
            self.table.setdefault(hsh, (snapshots, snapshots.offsets[seq_index] + j, int(block_table_row[j])))

    def lookup(self, token_ids):
        """(n_pages, physical page ids, snapshots, row of the last shared page) or (0, [], None, None).  At least one
        token of the prompt is left for the tail."""
        hit = []
        for hsh in self.page_hashes(token_ids[:max(len(token_ids) - 1, 0)]):
            if hsh not in self.table:
                break
            hit.append(self.table[hsh])
        if not hit:
            return 0, [], None, None
        return len(hit), [p for _, _, p in hit], hit[-1][0], hit[-1][1]


def random_state_dict(*, layers, hidden, head_dim, num_kv_heads, vocab, seed, device, dtype=torch.bfloat16, kernel_attn=4,
                      kernel_conv=3):
    """Random weights in the reference's key layout (model/reference.py:236-262), drawn on the device: the default
    initialisation's distributions (uniform +-1/sqrt(fan_in) for linears and convs, ones for norms, the Polar
    constants of model/reference.py:17-20), except that ``mem.proj`` is random instead of zero so that the memory
    branch contributes.  For benchmarks - checkpoints load through ``AtmaModel(state_dict, ...)`` directly."""
    g = torch.Generator(device=device).manual_seed(seed)
    H, dk, Hkv, D = hidden // head_dim, head_dim, num_kv_heads, hidden
    sd = {}

    def uni(shape, fan):
        return ((torch.rand(*shape, device=device, generator=g) * 2 - 1) * fan ** -0.5).to(dtype)

    def lin(name, out_f, in_f):
        sd[name + ".weight"], sd[name + ".bias"] = uni((out_f, in_f), in_f), uni((out_f,), in_f)

    sd["embed.weight"] = torch.randn(vocab, D, device=device, generator=g).to(dtype)
    for i in range(layers):
        P = f"blocks.{i}."
        if i % 4 == 2:
            lin(P + "attn.q", 2 * H * dk, D); lin(P + "attn.k", Hkv * dk, D); lin(P + "attn.v", Hkv * dk, D)
            for n, C in (("q", H * dk), ("k", Hkv * dk), ("v", Hkv * dk)):
                sd[P + f"attn.canon_{n}.weight"] = uni((C, 1, kernel_attn), kernel_attn)
            lin(P + "attn.proj", D, H * dk); lin(P + "attn.mu_proj", D, H)
            sd[P + "attn.v_null"] = torch.zeros(H, dk, device=device)
            for n, val in (("null_base", 2.0), ("null_slope_raw", 0.5), ("len_gain_raw", -1.0), ("mag_beta_raw", -1.5)):
                sd[P + "attn." + n] = torch.full((H,), val, device=device)
            lin(P + "attn.mem.w_gamma", H, D); lin(P + "attn.mem.w_beta", H, D); lin(P + "attn.mem.gate", H * dk, D)
            lin(P + "attn.mem.proj", D, H * dk)
        else:
            lin(P + "attn.in_proj", 3 * D, D)
            sd[P + "attn.conv.weight"] = uni((D, 1, kernel_conv), kernel_conv)
            lin(P + "attn.out_proj", D, D)
        lin(P + "mlp.fc", 8 * D, D); lin(P + "mlp.proj", D, 4 * D)
        sd[P + "norm1.weight"] = torch.ones(D, device=device, dtype=dtype)
        sd[P + "norm2.weight"] = torch.ones(D, device=device, dtype=dtype)
    lin("proj", vocab, D)
    sd["norm.weight"] = torch.ones(D, device=device, dtype=dtype)
    return sd


class CapturedDecode:
    """The decode step of one batch size, captured once and replayed (what the reference's model runner does per
    batch bucket, inference/engine/model_runner.py:254-310,500-512): fill the static inputs, call ``replay``."""

    def __init__(self, model, state, batch, max_blocks, warmup=2):
        dev = model.device
        self.model, self.state = model, state
        self.ids = torch.zeros(batch, dtype=torch.long, device=dev)
        self.seq_slots = torch.arange(batch, dtype=torch.int64, device=dev)
        self.slot_mapping = torch.full((batch,), -1, dtype=torch.int32, device=dev)
        self.block_tables = torch.zeros(batch, max_blocks, dtype=torch.int32, device=dev)
        self.context_lens = torch.zeros(batch, dtype=torch.int32, device=dev)
        self.graph = None
        self.warmup = warmup
        self.logits = None

    def capture(self):
        """Call after the static inputs hold a valid step (warm-up runs execute it for real)."""
        dev = self.model.device
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(self.warmup):
                self._run()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.logits = self._run()
        return self

    def _run(self):
        return self.model.decode(self.ids, self.state, self.seq_slots, self.slot_mapping, self.block_tables, self.context_lens)

    def replay(self):
        self.graph.replay()
        return self.logits
