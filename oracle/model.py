"""Block- and model-level forward on the CPU - checker for the composed layers and the model harness.

TEST INFRASTRUCTURE: see the package docstring.

Restates the reference's pure-PyTorch model (model/reference.py) from the per-op checkers of
this package, taking the reference's ``state_dict`` key layout:

    local block   x + out_proj(C * conv(B * x'))  with [B, C, x'] = in_proj(norm1 x)     model/reference.py:31-49
    global block  x + Polar(q, k, v) channels + memory channel                          model/reference.py:127-195
    both          x + proj(gate * relu(fc x)^2) after norm2                             model/layers.py:19-31, reference.py:230-233
    model         embed, blocks (i % 4 == 2 global), final norm, LM head, 15 x / sqrt(x^2 + 225)   reference.py:236-269
"""

import torch
import torch.nn.functional as F

from .conv import causal_conv1d_prefill
from .gated_delta import gated_delta_chunked
from .polar import polar_materialized


def _lin(x, sd, name):
    return F.linear(x, sd[name + ".weight"].to(x.dtype), sd[name + ".bias"].to(x.dtype) if name + ".bias" in sd else None)


def _conv_btc(x, weight, state_in=None):
    """Depthwise causal conv of a (B, T, C) tensor with an nn.Conv1d weight (C, 1, K); fp32."""
    return torch.stack([causal_conv1d_prefill(x[b], weight.squeeze(1), None if state_in is None else state_in[b])[0]
                        for b in range(x.shape[0])]).to(x.dtype)


def mlp_oracle(h, sd, prefix):
    fc = _lin(h, sd, prefix + "mlp.fc")
    a, gate = fc.chunk(2, dim=-1)
    return _lin(gate * a.relu().square(), sd, prefix + "mlp.proj")


def lfm2_mix_oracle(h, sd, prefix):
    """LFM2Conv.forward (model/reference.py:37-49)."""
    Bg, Cg, xp = _lin(h, sd, prefix + "in_proj").chunk(3, dim=-1)
    return _lin(Cg * _conv_btc(Bg * xp, sd[prefix + "conv.weight"]), sd, prefix + "out_proj")


def memory_readout_oracle(x, q_t, k_t, v_t, sd, prefix, gamma_bias=3.9, beta_bias=0.0, chunk=64, S0=None):
    """TitansMemory.forward, torch backend (model/blocks.py:463-490).  q_t, k_t, v_t (B, H, T, dk) with
    the KV heads expanded.  Returns (out (B, T, D), final state (B, H, dv, dk))."""
    B, H, T, dk = q_t.shape
    gamma = torch.sigmoid(_lin(x, sd, prefix + "w_gamma").float() + gamma_bias).transpose(1, 2)
    beta = torch.sigmoid(_lin(x, sd, prefix + "w_beta").float() + beta_bias).transpose(1, 2)
    r, S = gated_delta_chunked(F.normalize(q_t.float(), dim=-1), F.normalize(k_t.float(), dim=-1), v_t.float(),
                               gamma, beta, chunk=chunk, S0=S0)
    r = F.rms_norm(r.transpose(1, 2), (dk,)).reshape(B, T, H * dk).to(x.dtype)
    return _lin(r * torch.sigmoid(_lin(x, sd, prefix + "gate")), sd, prefix + "proj"), S


def polar_mix_oracle(h, sd, prefix, head_dim, num_kv_heads, window=None, return_parts=False):
    """PolarAttention.forward (model/reference.py:127-195)."""
    B, T, D = h.shape
    dk, Hkv = head_dim, num_kv_heads
    H = sd[prefix + "null_base"].shape[0]
    q_gate = _lin(h, sd, prefix + "q").view(B, T, H, 2 * dk)
    q, gate = q_gate.chunk(2, dim=-1)
    k = _lin(h, sd, prefix + "k").view(B, T, Hkv, dk)
    v = _lin(h, sd, prefix + "v").view(B, T, Hkv, dk)
    q, k = F.rms_norm(q, (dk,)), F.rms_norm(k, (dk,))
    q = (q.reshape(B, T, -1) + _conv_btc(q.reshape(B, T, -1), sd[prefix + "canon_q.weight"])).view(B, T, H, dk)
    k = (k.reshape(B, T, -1) + _conv_btc(k.reshape(B, T, -1), sd[prefix + "canon_k.weight"])).view(B, T, Hkv, dk)
    v = (v.reshape(B, T, -1) + _conv_btc(v.reshape(B, T, -1), sd[prefix + "canon_v.weight"])).view(B, T, Hkv, dk)
    q_t, k_t, v_t = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    n_keys = torch.arange(1, T + 1, dtype=torch.float32)
    params = {n: sd[prefix + n] for n in ("v_null", "null_base", "null_slope_raw", "len_gain_raw", "mag_beta_raw")}
    c, mag = polar_materialized(q_t, k_t, v_t, n_keys, window=window, **params)
    out = _lin(c.transpose(1, 2).reshape(B, T, H * dk) * torch.sigmoid(gate.reshape(B, T, -1)), sd, prefix + "proj")
    out = out + _lin(mag.transpose(1, 2), sd, prefix + "mu_proj")
    S = None
    if prefix + "mem.proj.weight" in sd:
        G = H // Hkv
        mem, S = memory_readout_oracle(h, q_t, k_t.repeat_interleave(G, 1), v_t.repeat_interleave(G, 1), sd, prefix + "mem.")
        out = out + mem
    if return_parts:
        return out, dict(q=q, k=k, v=v, S=S)
    return out


def block_oracle(x, sd, prefix, *, attention, head_dim, num_kv_heads, window=None, eps=1e-6):
    """Block.forward (model/reference.py:230-233)."""
    D = x.shape[-1]
    h = F.rms_norm(x, (D,), weight=sd[prefix + "norm1.weight"], eps=eps)
    mix = (polar_mix_oracle(h, sd, prefix + "attn.", head_dim, num_kv_heads, window) if attention
           else lfm2_mix_oracle(h, sd, prefix + "attn."))
    x = x + mix
    h2 = F.rms_norm(x, (D,), weight=sd[prefix + "norm2.weight"], eps=eps)
    return x + mlp_oracle(h2, sd, prefix)


def model_oracle(ids, sd, *, layers, head_dim, num_kv_heads, window=None, eps=1e-6):
    """ReferenceModel.forward (model/reference.py:262-269): logits (B, T, vocab) fp32 for every position."""
    x = sd["embed.weight"][ids]
    for i in range(layers):
        x = block_oracle(x, sd, f"blocks.{i}.", attention=(i % 4 == 2), head_dim=head_dim, num_kv_heads=num_kv_heads,
                         window=window, eps=eps)
    logits = _lin(F.rms_norm(x, (x.shape[-1],), weight=sd["norm.weight"], eps=eps), sd, "proj").float()
    return 15.0 * logits * (logits.square() + 225.0).rsqrt()
