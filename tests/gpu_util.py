"""Helpers shared by the GPU parity tests."""

import torch


def polar_params(H, dk, seed=0, device="cuda", random=True):
    g = torch.Generator().manual_seed(1000 + seed)
    if random:
        p = dict(v_null=torch.randn(H, dk, generator=g) * 0.3,
                 null_base=2.0 + 0.5 * torch.randn(H, generator=g),
                 null_slope_raw=0.5 + 0.5 * torch.randn(H, generator=g),
                 len_gain_raw=-1.0 + 0.5 * torch.randn(H, generator=g),
                 mag_beta_raw=-1.5 + 0.5 * torch.randn(H, generator=g))
    else:   # the reference's default init (model/reference.py:17-20,117)
        p = dict(v_null=torch.zeros(H, dk), null_base=torch.full((H,), 2.0),
                 null_slope_raw=torch.full((H,), 0.5), len_gain_raw=torch.full((H,), -1.0),
                 mag_beta_raw=torch.full((H,), -1.5))
    return p, {k: v.to(device) for k, v in p.items()}


def rand(shape, seed, dtype=torch.float32, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)
