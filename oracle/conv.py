"""Depthwise causal convolution and KV-cache scatter on the CPU - checkers.

TEST INFRASTRUCTURE: see the package docstring.

y_t[c] = sum_{j=0}^{K-1} w[c, j] * x_{t-(K-1)+j}[c], zero (or carried-state) left
context, no bias (model/reference.py:43-47; model/blocks.py:501,526-528).  The
recurrent state is the last K-1 inputs, oldest first
(inference/models/atma.py:137,186; kernel/causal_conv1d_triton.py:36-41).
"""

import torch


def causal_conv1d_prefill(x, weight, state_in=None):
    """x (T, C); weight (C, K); state_in (C, K-1) or None (fresh prompt).
    Returns out (T, C) fp32 and the final state (C, K-1) in x.dtype
    (inference/models/atma.py:128-137)."""
    T, C = x.shape
    K = weight.shape[1]
    left = x.new_zeros(K - 1, C) if state_in is None else state_in.to(x.dtype).transpose(0, 1)
    padded = torch.cat([left, x], dim=0)                                        # (T+K-1, C)
    out = torch.zeros(T, C, dtype=torch.float32)
    wf = weight.float()
    for j in range(K):
        out += padded[j:j + T].float() * wf[:, j][None, :]
    return out, padded[-(K - 1):].transpose(0, 1).contiguous()


def causal_conv1d_step(x, weight, slots, state_table):
    """One decode step, in place on state_table[slots]
    (kernel/causal_conv1d_triton.py:17-42; inference/models/atma.py:181-187).
    x (B, C); weight (C, K); state_table (max_seqs, C, K-1) - MUTATED.  Returns fp32."""
    K = weight.shape[1]
    st = state_table[slots.long()]                                              # (B, C, K-1)
    out = (st.float() * weight.float()[None, :, :K - 1]).sum(-1) + x.float() * weight.float()[None, :, K - 1]
    state_table[slots.long()] = torch.cat([st[:, :, 1:], x.to(st.dtype)[:, :, None]], dim=2)
    return out


def packed_causal_conv1d_oracle(x, weight, state_table, token_seq_starts, token_seq_ends,
                                token_seq_slots):
    """Fresh-prompt conv over packed ragged sequences plus the final-state write
    (kernel/inference_ops_triton.py:17-63).  x (tokens, C); the three maps are
    per-token int32.  state_table (max_seqs, C, K-1) - MUTATED.  Returns fp32."""
    total = x.shape[0]
    out = torch.zeros(total, x.shape[1], dtype=torch.float32)
    seen = set()
    for t in range(total):
        s, e, slot = int(token_seq_starts[t]), int(token_seq_ends[t]), int(token_seq_slots[t])
        if (s, e) in seen:
            continue
        seen.add((s, e))
        o, st = causal_conv1d_prefill(x[s:e], weight, None)
        out[s:e] = o
        state_table[slot] = st.to(state_table.dtype)
    return out


def store_kvcache_oracle(key, value, k_cache, v_cache, slot_mapping):
    """Scatter rows into flat cache slots, skipping slot -1
    (inference/layers/attention.py:39-47).  Caches are MUTATED."""
    N, h, d = key.shape
    kf, vf = k_cache.view(-1, h, d), v_cache.view(-1, h, d)
    for i in range(N):
        s = int(slot_mapping[i])
        if s >= 0:
            kf[s] = key[i]
            vf[s] = value[i]


def qkv_prep_prefill_oracle(q_gate, k, v, w_q, w_k, w_v, state_q, state_k, state_v, token_seq_starts, token_seq_ends,
                            token_seq_slots, k_cache, v_cache, slot_mapping, initial_states=None, eps=None):
    """The q/k/v preparation of a global layer's packed prefill, op by op as the reference runs it
    (inference/models/atma.py:391-399 rms_norm of q and k per head; :431-441 x + packed conv for
    q, k, v; :468-471 store_kvcache).  q_gate (tokens, H, 2*dk); k, v (tokens, Hkv, dk); conv
    weights (C, K); state tables (rows, C, K-1) MUTATED; caches MUTATED.  ``initial_states`` =
    (iq, ik, iv) tables read as left context of every sequence (a continued prefix), None = fresh
    prompts as in the reference's packed path.  Every op rounds to the input dtype as eager does.
    Returns q (tokens, H, dk), k, v (tokens, Hkv, dk) in the input dtype."""
    import torch.nn.functional as F
    total, H, two_dk = q_gate.shape
    dk = two_dk // 2
    dt = q_gate.dtype
    qn = F.rms_norm(q_gate[..., :dk], (dk,), eps=eps).reshape(total, -1)
    kn = F.rms_norm(k, (dk,), eps=eps).reshape(total, -1)
    vn = v.reshape(total, -1)
    outs = []
    for x, w, st, idx in ((qn, w_q, state_q, 0), (kn, w_k, state_k, 1), (vn, w_v, state_v, 2)):
        conv = torch.zeros(total, x.shape[1], dtype=torch.float32)
        done = set()
        for t in range(total):
            s, e, slot = int(token_seq_starts[t]), int(token_seq_ends[t]), int(token_seq_slots[t])
            if (s, e) in done:
                continue
            done.add((s, e))
            init = None
            if initial_states is not None and slot >= 0:
                init = initial_states[idx][slot]
            o, fin = causal_conv1d_prefill(x[s:e], w, init)
            conv[s:e] = o
            if slot >= 0:
                st[slot] = fin.to(st.dtype)
        outs.append((x.float() + conv.to(dt).float()).to(dt))
    q_out = outs[0].view(total, H, dk)
    k_out = outs[1].view(total, -1, dk)
    v_out = outs[2].view(total, -1, dk)
    if k_cache is not None:
        store_kvcache_oracle(k_out, v_out, k_cache, v_cache, slot_mapping)
    return q_out, k_out, v_out


def lfm2_conv_step_oracle(projected, weight, slots, state_table):
    """Decode step of the local layers' gated conv, op by op (inference/models/atma.py:633-636,668-673):
    chunk, B*x', conv step on the slot-indexed table (MUTATED), C*conv.  Returns (B, D) in the input dtype."""
    Bv, Cv, xp = projected.chunk(3, dim=-1)
    x_gated = Bv * xp
    conv = causal_conv1d_step(x_gated, weight, slots, state_table).to(projected.dtype)
    return Cv * conv


def lfm2_conv_packed_oracle(projected, weight, state_table, token_seq_starts, token_seq_ends, token_seq_slots,
                            initial_state=None):
    """Packed prefill of the same block (inference/models/atma.py:648-653), sequence by sequence."""
    Bv, Cv, xp = projected.chunk(3, dim=-1)
    x_gated = Bv * xp
    total = projected.shape[0]
    conv = torch.zeros(total, weight.shape[0], dtype=torch.float32)
    done = set()
    for t in range(total):
        s, e, slot = int(token_seq_starts[t]), int(token_seq_ends[t]), int(token_seq_slots[t])
        if (s, e) in done:
            continue
        done.add((s, e))
        init = initial_state[slot] if (initial_state is not None and slot >= 0) else None
        o, fin = causal_conv1d_prefill(x_gated[s:e], weight, init)
        conv[s:e] = o
        if slot >= 0:
            state_table[slot] = fin.to(state_table.dtype)
    return Cv * conv.to(projected.dtype)
