"""One ATMA global block forward on the GPU, composed from this package's kernels.

Host-side mirror of the reference's ``Block.forward`` with a Polar attention core and the
gated-delta memory branch (model/reference.py:127-195,230-233; model/blocks.py:463-490;
model/layers.py:19-31): pre-norm RMSNorm, q/k/v projections, per-head RMSNorm of q and k,
the three Canon depthwise convs (residual form), Polar attention, the additive memory channel,
then the squared-ReLU gated MLP.  Projections and norms are library calls (cuBLAS through
``F.linear``, ``F.rms_norm``); every mixing step goes through the C ABI:

    Canon convs        -> causal_conv1d_fn (packed prefill conv kernel)
    Polar core         -> polar_attention_fwd (un-expanded KV heads, (B,T,H,dk) storage viewed as (B,H,T,dk))
    memory scan        -> chunk_gated_delta_rule (in-kernel L2 norm, [K,V] fp32 state)
    MLP gate           -> squared_relu_gate

It takes the reference block's ``state_dict`` as is, so a parity test can load the oracle's
weights and compare outputs.
"""

import torch
import torch.nn.functional as F

from .causal_conv1d import causal_conv1d_fn
from .gated_delta import chunk_gated_delta_rule
from .inference_ops import squared_relu_gate
from .polar import polar_attention_fwd


def _linear(x, sd, name):
    w = sd[name + ".weight"].to(x.dtype)
    b = sd.get(name + ".bias")
    return F.linear(x, w, None if b is None else b.to(x.dtype))


def _canon(x_btc, weight):
    """x + depthwise causal conv(x); x (B, T, C), weight (C, 1, K) as nn.Conv1d stores it."""
    out = causal_conv1d_fn(x_btc.transpose(1, 2), weight.squeeze(1).to(x_btc.dtype))
    return x_btc + out.transpose(1, 2)


@torch.no_grad()
def global_block_forward(x, sd, *, head_dim, num_kv_heads, window=None, mem_chunk=64, mem_gamma_bias=3.9,
                         mem_beta_bias=0.0, eps=1e-6, initial_state=None, return_state=False):
    """x (B, T, D) on the GPU; ``sd`` the reference block's state_dict (tensors on the same
    device).  Returns the block output (B, T, D) (and the memory's final [K,V] state)."""
    if mem_chunk != 64:
        raise ValueError("the scan kernels use 64-token chunks (the result does not depend on the chunk size)")
    B, T, D = x.shape
    dk = head_dim
    H = sd["attn.null_base"].shape[0]
    Hkv = num_kv_heads
    h = F.rms_norm(x, (D,), weight=sd["norm1.weight"].to(x.dtype), eps=eps)

    q_gate = _linear(h, sd, "attn.q").view(B, T, H, 2 * dk)
    q, gate = q_gate[..., :dk], q_gate[..., dk:]
    k = _linear(h, sd, "attn.k").view(B, T, Hkv, dk)
    v = _linear(h, sd, "attn.v").view(B, T, Hkv, dk)
    q = F.rms_norm(q, (dk,))
    k = F.rms_norm(k, (dk,))
    q = _canon(q.reshape(B, T, H * dk), sd["attn.canon_q.weight"]).view(B, T, H, dk)
    k = _canon(k.reshape(B, T, Hkv * dk), sd["attn.canon_k.weight"]).view(B, T, Hkv, dk)
    v = _canon(v.reshape(B, T, Hkv * dk), sd["attn.canon_v.weight"]).view(B, T, Hkv, dk)

    n_keys = torch.arange(1, T + 1, device=x.device, dtype=torch.float32)
    c, mag = polar_attention_fwd(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), n_keys,
                                 v_null=sd["attn.v_null"], null_base=sd["attn.null_base"],
                                 null_slope_raw=sd["attn.null_slope_raw"], len_gain_raw=sd["attn.len_gain_raw"],
                                 mag_beta_raw=sd["attn.mag_beta_raw"], window=window)
    c_flat = c.transpose(1, 2).reshape(B, T, H * dk)
    out = _linear(c_flat * torch.sigmoid(gate.reshape(B, T, H * dk)), sd, "attn.proj")
    out = out + _linear(mag.transpose(1, 2), sd, "attn.mu_proj")

    S = None
    if "attn.mem.proj.weight" in sd:
        g_logit = _linear(h, sd, "attn.mem.w_gamma").float() + mem_gamma_bias
        b_logit = _linear(h, sd, "attn.mem.w_beta").float() + mem_beta_bias
        r, S = chunk_gated_delta_rule(q=q.contiguous(), k=k.contiguous(), v=v.contiguous(), g=F.logsigmoid(g_logit),
                                      beta=torch.sigmoid(b_logit), scale=1.0, initial_state=initial_state,
                                      output_final_state=True, use_qk_l2norm_in_kernel=True)
        r = F.rms_norm(r.float(), (dk,)).reshape(B, T, H * dk).to(x.dtype)
        out = out + _linear(r * torch.sigmoid(_linear(h, sd, "attn.mem.gate")), sd, "attn.mem.proj")
    x = x + out

    h2 = F.rms_norm(x, (D,), weight=sd["norm2.weight"].to(x.dtype), eps=eps)
    fc = _linear(h2, sd, "mlp.fc")
    half = fc.shape[-1] // 2
    act = squared_relu_gate(fc[..., :half].reshape(B * T, half), fc[..., half:].reshape(B * T, half)).view(B, T, half)
    x = x + _linear(act, sd, "mlp.proj")
    return (x, S) if return_state else x
