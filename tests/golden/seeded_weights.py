"""Seeded weights with the reference's ``state_dict`` key layout.

The large parity cases (one global block at hidden 1024; a whole small model) cannot ship
their weights as fixtures, so both sides regenerate them from a seed with this file:
``make_golden.py`` loads them into the unmodified reference modules (``load_state_dict`` with
``strict=True``, which pins names and shapes) and stores only the outputs; the tests rebuild
the same tensors (CPU generator, deterministic) and feed them to this package.

Distributions follow the reference's default initialisation (model/reference.py:17-20,117;
``nn.Linear`` / ``nn.Conv1d`` uniform +-1/sqrt(fan_in)), except where that default would hide a
branch: ``mem.proj`` (zero-initialised, model/blocks.py:458-461) and ``v_null`` (zeros) are
random, as the reference's own tests make them (tests/verify.py:363), and the five Polar
scalars are jittered per head.
"""

import torch


def _uniform(gen, shape, bound):
    return (torch.rand(*shape, generator=gen) * 2.0 - 1.0) * bound


def _linear(sd, name, gen, out_f, in_f, bias=True):
    sd[name + ".weight"] = _uniform(gen, (out_f, in_f), in_f ** -0.5)
    if bias:
        sd[name + ".bias"] = _uniform(gen, (out_f,), in_f ** -0.5)


def attention_state(gen, dim, head_dim, num_kv_heads, kernel_size=4, mem=True, prefix="attn."):
    """Tensors of ``PolarAttention`` / ``AtmaAttention`` (model/reference.py:101-125, model/blocks.py:505-532)."""
    H, dk, Hkv = dim // head_dim, head_dim, num_kv_heads
    sd = {}
    _linear(sd, prefix + "q", gen, 2 * H * dk, dim)
    _linear(sd, prefix + "k", gen, Hkv * dk, dim)
    _linear(sd, prefix + "v", gen, Hkv * dk, dim)
    for n, c in (("q", H * dk), ("k", Hkv * dk), ("v", Hkv * dk)):
        sd[prefix + f"canon_{n}.weight"] = _uniform(gen, (c, 1, kernel_size), kernel_size ** -0.5)
    _linear(sd, prefix + "proj", gen, dim, H * dk)
    _linear(sd, prefix + "mu_proj", gen, dim, H)
    sd[prefix + "v_null"] = torch.randn(H, dk, generator=gen) * 0.2
    sd[prefix + "null_base"] = 2.0 + 0.3 * torch.randn(H, generator=gen)
    sd[prefix + "null_slope_raw"] = 0.5 + 0.3 * torch.randn(H, generator=gen)
    sd[prefix + "len_gain_raw"] = -1.0 + 0.3 * torch.randn(H, generator=gen)
    sd[prefix + "mag_beta_raw"] = -1.5 + 0.3 * torch.randn(H, generator=gen)
    if mem:
        _linear(sd, prefix + "mem.w_gamma", gen, H, dim)
        _linear(sd, prefix + "mem.w_beta", gen, H, dim)
        _linear(sd, prefix + "mem.gate", gen, H * dk, dim)
        sd[prefix + "mem.proj.weight"] = torch.randn(dim, H * dk, generator=gen) * 0.05
        sd[prefix + "mem.proj.bias"] = torch.randn(dim, generator=gen) * 0.01
    return sd


def lfm2_state(gen, dim, kernel_size=3, prefix="attn."):
    """Tensors of ``LFM2Conv`` (model/blocks.py:493-503)."""
    sd = {}
    _linear(sd, prefix + "in_proj", gen, 3 * dim, dim)
    sd[prefix + "conv.weight"] = _uniform(gen, (dim, 1, kernel_size), kernel_size ** -0.5)
    _linear(sd, prefix + "out_proj", gen, dim, dim)
    return sd


def block_state(seed, dim, head_dim, num_kv_heads, attention=True, mem=True, gen=None, prefix=""):
    """Tensors of ``Block`` (model/reference.py:198-233): mixing module, MLP, two RMSNorms."""
    gen = gen or torch.Generator().manual_seed(seed)
    sd = (attention_state(gen, dim, head_dim, num_kv_heads, mem=mem, prefix=prefix + "attn.") if attention
          else lfm2_state(gen, dim, prefix=prefix + "attn."))
    _linear(sd, prefix + "mlp.fc", gen, 8 * dim, dim)
    _linear(sd, prefix + "mlp.proj", gen, dim, 4 * dim)
    sd[prefix + "norm1.weight"] = 1.0 + 0.1 * torch.randn(dim, generator=gen)
    sd[prefix + "norm2.weight"] = 1.0 + 0.1 * torch.randn(dim, generator=gen)
    return sd


def model_state(seed, vocab, layers, dim, head_dim, num_kv_heads):
    """Tensors of ``ReferenceModel`` / the inference ``Atma`` (model/reference.py:236-262): embedding,
    ``layers`` blocks (every fourth one, i % 4 == 2, global), final norm, LM head."""
    gen = torch.Generator().manual_seed(seed)
    sd = {"embed.weight": torch.randn(vocab, dim, generator=gen)}
    for i in range(layers):
        sd.update(block_state(0, dim, head_dim, num_kv_heads, attention=(i % 4 == 2), gen=gen, prefix=f"blocks.{i}."))
    _linear(sd, "proj", gen, vocab, dim)
    sd["norm.weight"] = 1.0 + 0.1 * torch.randn(dim, generator=gen)
    return sd
