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

from .gated_delta import gated_delta_decode_step, gated_delta_decode_step_fused
from .inference_ops import (add_rms_norm, lfm2_conv_decode_step, lfm2_conv_packed, qkv_prep_decode, rms_sigmoid_gate,
                            softcap_logits, squared_relu_gate)
from .layer import PackedMaps, global_attention_prefill_packed
from .polar import polar_attention_decode

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
        return F.linear(x, self.sd[name + ".weight"], self.sd.get(name + ".bias"))

    def _mlp(self, h, i):
        fc = self._lin(h, f"blocks.{i}.mlp.fc")
        half = fc.shape[-1] // 2
        return self._lin(squared_relu_gate(fc[:, :half], fc[:, half:]), f"blocks.{i}.mlp.proj")

    def logits(self, hidden):
        """LM head + soft-cap on already-normalised hidden rows (inference/models/atma.py:750-754)."""
        return softcap_logits(self._lin(hidden, "proj"))

    # ---- packed prefill of fresh prompts ----------------------------------------------------------------------
    @torch.no_grad()
    def prefill(self, ids, seqlens, slots, state, slot_mapping):
        """ids (tokens,) packed prompts; seqlens / slots per sequence (host lists); slot_mapping (tokens,) cache rows.
        Conv states, memory states and K/V pages of ``state`` are written at the sequences' slots.
        Returns the final-norm hidden states of all tokens (tokens, D)."""
        sd = self.sd
        maps = PackedMaps(seqlens, slots, self.device)
        sm = slot_mapping.to(self.device, torch.int64)
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
                    prefix=P + "attn.", has_initial=False)
            else:
                proj = self._lin(h, P + "attn.in_proj")
                y = lfm2_conv_packed(proj, sd[P + "attn.conv.weight"].squeeze(1), state.conv[f"conv_{i}"],
                                     maps.token_seq_starts, maps.token_seq_ends, maps.token_seq_slots)
                mix = self._lin(y, P + "attn.out_proj")
            x, h = add_rms_norm(x, mix, sd[P + "norm2.weight"], self.eps)
            nxt = sd[f"blocks.{i + 1}.norm1.weight"] if i + 1 < self.L else sd["norm.weight"]
            x, h = add_rms_norm(x, self._mlp(h, i), nxt, self.eps)
        return h

    # ---- one decode step ---------------------------------------------------------------------------------
    @torch.no_grad()
    def decode(self, ids, state, seq_slots, slot_mapping, block_tables, context_lens):
        """One token per sequence: ids (B,), seq_slots (B,) int64 state rows, slot_mapping (B,) int32 cache rows
        of the new token, block_tables (B, max_blocks) int32, context_lens (B,) int32 INCLUDING the new token.
        All arguments are device tensors with fixed shapes, nothing synchronises: the call can be captured in
        a CUDA graph (inference/engine/model_runner.py:254-310).  Returns soft-capped logits (B, vocab)."""
        sd, H, Hkv, dk, D = self.sd, self.H, self.Hkv, self.dk, self.D
        B = ids.shape[0]
        x = sd["embed.weight"][ids]
        x, h = add_rms_norm(x, None, sd["blocks.0.norm1.weight"], self.eps)
        for i in range(self.L):
            P = f"blocks.{i}."
            if i in self.global_layers:
                pk = self.packed[i]
                z = F.linear(h, pk["w_in"], pk["b_in"])                              # every input projection at once
                q_gate = z[:, :pk["o_k"]].view(B, H, 2 * dk)
                k = z[:, pk["o_k"]:pk["o_v"]].view(B, Hkv, dk)
                v = z[:, pk["o_v"]:pk["o_g"]].view(B, Hkv, dk)
                q, k, v = qkv_prep_decode(q_gate, k, v, *pk["canon"],
                                          *(state.conv[f"attn_{i}_{n}"] for n in ("q", "k", "v")), seq_slots,
                                          state.k_cache[i], state.v_cache[i], slot_mapping)
                act = torch.empty((B, 2 * H * dk + H), device=x.device, dtype=x.dtype)   # [c * sig(gate) | mag | norm(r) * sig(gate)]
                polar_attention_decode(q, state.k_cache[i], state.v_cache[i], block_tables, context_lens, window=self.window,
                                       gate=q_gate[..., dk:], out=(act[:, :H * dk].view(B, H, dk), act[:, H * dk:H * dk + H]),
                                       **pk["polar"])
                r_out = act[:, H * dk + H:]
                mem_gate = z[:, pk["o_mg"]:]
                if dk == 128:
                    gated_delta_decode_step_fused(q, k, v, state.mem[i], seq_slots,
                                                  gate_logits=(z[:, pk["o_g"]:pk["o_b"]], z[:, pk["o_b"]:pk["o_mg"]]),
                                                  gamma_bias=self.gamma_bias, beta_bias=self.beta_bias, gate=mem_gate, out=r_out)
                else:                                                            # other head sizes: the separate kernels
                    G = H // Hkv
                    gamma = torch.sigmoid(z[:, pk["o_g"]:pk["o_b"]].float() + self.gamma_bias)
                    beta = torch.sigmoid(z[:, pk["o_b"]:pk["o_mg"]].float() + self.beta_bias)
                    r = gated_delta_decode_step(q, k.repeat_interleave(G, 1), v.repeat_interleave(G, 1), gamma, beta,
                                                state.mem[i], seq_slots)
                    r_out.copy_(rms_sigmoid_gate(r.to(x.dtype), mem_gate))
                mix = F.linear(act, pk["w_out"], pk["b_out"])                          # W_o, W_mu and mem.proj in one product
            else:
                proj = self._lin(h, P + "attn.in_proj")
                y = lfm2_conv_decode_step(proj, sd[P + "attn.conv.weight"].squeeze(1), seq_slots, state.conv[f"conv_{i}"])
                mix = self._lin(y, P + "attn.out_proj")
            x, h = add_rms_norm(x, mix, sd[P + "norm2.weight"], self.eps)
            nxt = sd[f"blocks.{i + 1}.norm1.weight"] if i + 1 < self.L else sd["norm.weight"]
            x, h = add_rms_norm(x, self._mlp(h, i), nxt, self.eps)
        return self.logits(h)

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
