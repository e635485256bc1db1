"""Polar Attention on the CPU - checker for the CUDA prefill / decode kernels.

TEST INFRASTRUCTURE: see the package docstring.  Two restatements are kept:

* ``polar_materialized`` follows the reference's validated materialised oracle
  ``polar_reduce`` (model/blocks.py:120-164) with the per-query temperature and
  null floor of ``polar_temp_null`` (model/blocks.py:104-117), the causal /
  sliding-window masks built the way the reference callers build them
  (model/reference.py:163-172, inference/models/atma.py:235-244).
* ``polar_streaming`` follows the tile-streaming form the reference's device
  kernels implement (kernel/polar_triton.py:85-178): running (m, L, Q2, S) over
  key tiles, Q2 rescaled by alpha squared, null sink folded once at the end, a
  1e-30 floor on Q2.  It differs from the materialised form only when the real
  keys hold less than ~1e-6 of the softmax mass (mag ~ 0 either way).

Inputs use the kernel-API layout: q (B, H, Tq, dk); k, v (B, Hkv, Tk, dk) with
Hkv dividing H (the reference expands K/V heads before its kernels; expansion
is a pure index map, so it is done here by indexing).
"""

import math

import torch
import torch.nn.functional as F


def polar_params_host(len_gain_raw, null_slope_raw, mag_beta_raw):
    """softplus of the three raw per-head parameters, done on the host before the
    launch exactly as kernel/polar_triton.py:540-542 does."""
    return (F.softplus(len_gain_raw.float()), F.softplus(null_slope_raw.float()),
            F.softplus(mag_beta_raw.float()))


def _temp_null(n_keys, window, spg, null_base, sps, cd):
    """Per (head, query) temperature and null logit (model/blocks.py:104-117;
    windowed count as kernel/polar_triton.py:93-96)."""
    n = n_keys.to(cd)
    if window is not None:
        n = torch.minimum(n, torch.tensor(float(window), dtype=cd))
    n = n.clamp(min=1.0)
    temp = 1.0 + spg.to(cd)[:, None] * torch.log(n)[None, :]                     # (H, Tq)
    null = null_base.to(cd)[:, None] + sps.to(cd)[:, None] * torch.sqrt(torch.log(n + 1.0))[None, :]
    return temp, null


def _valid_mask(n_keys, Tk, window):
    """valid[i, j] = key j visible to query i: j < n_i and (window) j >= n_i - W
    (kernel/polar_triton.py:136-138)."""
    j = torch.arange(Tk, dtype=torch.float64)[None, :]
    n = n_keys.to(torch.float64)[:, None]
    valid = j < n
    if window is not None:
        valid = valid & (j >= n - float(window))
    return valid


def polar_materialized(q, k, v, n_keys, *, v_null, null_base, null_slope_raw,
                       len_gain_raw, mag_beta_raw, eps=1e-6, window=None,
                       compute_dtype=torch.float32, row_block=512):
    """Materialised softmax over [temp*sigma, temp*null] (model/blocks.py:141-161),
    evaluated in query-row blocks (the function is row-independent, so blocking is
    exact).  Returns c (B, H, Tq, dk) and mag (B, H, Tq) in ``compute_dtype``."""
    cd = compute_dtype
    B, H, Tq, dk = q.shape
    Hkv, Tk = k.shape[1], k.shape[2]
    G = H // Hkv
    head_map = torch.arange(H) // G
    spg = F.softplus(len_gain_raw.to(cd))
    sps = F.softplus(null_slope_raw.to(cd))
    beta = F.softplus(mag_beta_raw.to(cd))
    temp, null = _temp_null(n_keys, window, spg, null_base, sps, cd)
    valid = _valid_mask(n_keys, Tk, window)
    qf, kf, vf = q.to(cd), k.to(cd)[:, head_map], v.to(cd)[:, head_map]
    vn = v_null.to(cd).view(1, H, 1, dk)
    c = torch.empty(B, H, Tq, dk, dtype=cd)
    mag = torch.empty(B, H, Tq, dtype=cd)
    scale = 1.0 / math.sqrt(dk)
    for r0 in range(0, Tq, row_block):
        r1 = min(r0 + row_block, Tq)
        sig = torch.matmul(qf[:, :, r0:r1], kf.transpose(-1, -2)) * scale          # (B,H,R,Tk)
        t = temp[None, :, r0:r1, None]
        real = (sig * t).masked_fill(~valid[None, None, r0:r1], float("-inf"))
        logits = torch.cat([real, (null[None, :, r0:r1, None] * t).expand(B, H, r1 - r0, 1)], dim=-1)
        w = torch.softmax(logits, dim=-1)
        w_null, w_r = w[..., -1:], w[..., :-1]
        s = torch.matmul(w_r, vf) + w_null * vn
        c[:, :, r0:r1] = s / s.norm(dim=-1, keepdim=True).clamp_min(eps)
        denom = w_r.sum(-1, keepdim=True).clamp_min(eps)
        n_eff = 1.0 / (w_r / denom).square().sum(-1).clamp_min(eps)
        m_eff = n_eff * (1.0 - w_null.squeeze(-1))
        mag[:, :, r0:r1] = torch.tanh(beta.view(1, H, 1) * torch.log1p(m_eff))
    return c, mag


def polar_streaming_stats(q, k, v, n_keys, *, len_gain_raw, window=None,
                          compute_dtype=torch.float32, tile=64, key_offset=0, carry=None):
    """The running statistics (m, L, Q2, S) after streaming the given keys in tiles
    (kernel/polar_triton.py:105-149), BEFORE the null sink is folded.  ``key_offset``
    is the absolute position of k[:, :, 0]; ``carry`` continues from an earlier key
    block, which is how a ring pass over remote K/V blocks accumulates."""
    cd = compute_dtype
    B, H, Tq, dk = q.shape
    Hkv, Tk = k.shape[1], k.shape[2]
    head_map = torch.arange(H) // (H // Hkv)
    spg = F.softplus(len_gain_raw.to(cd))
    n = n_keys.to(cd)
    nc = n if window is None else torch.minimum(n, torch.tensor(float(window), dtype=cd))
    temp = 1.0 + spg[:, None] * torch.log(nc.clamp(min=1.0))[None, :]           # (H,Tq)
    qf, kf, vf = q.to(cd), k.to(cd)[:, head_map], v.to(cd)[:, head_map]
    if carry is None:
        m = torch.full((B, H, Tq), -1e38, dtype=cd)
        L = torch.zeros(B, H, Tq, dtype=cd)
        Q2 = torch.zeros(B, H, Tq, dtype=cd)
        S = torch.zeros(B, H, Tq, dk, dtype=cd)
    else:
        m, L, Q2, S = (x.clone().to(cd) for x in carry)
    scale = 1.0 / math.sqrt(dk)
    nn_ = n_keys.to(torch.float64)[:, None]
    for j0 in range(0, Tk, tile):
        j1 = min(j0 + tile, Tk)
        pos = (torch.arange(j0, j1, dtype=torch.float64) + key_offset)[None, :]
        valid = pos < nn_
        if window is not None:
            valid = valid & (pos >= nn_ - float(window))
        a = torch.matmul(qf, kf[:, :, j0:j1].transpose(-1, -2)) * scale * temp[None, :, :, None]
        a = torch.where(valid[None, None], a, torch.tensor(-1e38, dtype=cd))
        m_new = torch.maximum(m, a.amax(-1))
        alpha = torch.exp(m - m_new)
        p = torch.where(valid[None, None], torch.exp(a - m_new[..., None]), torch.zeros((), dtype=cd))
        L = L * alpha + p.sum(-1)
        Q2 = Q2 * alpha * alpha + p.square().sum(-1)
        S = S * alpha[..., None] + torch.matmul(p, vf[:, :, j0:j1])
        m = m_new
    return m, L, Q2, S


def polar_finalize(stats, n_keys, *, v_null, null_base, null_slope_raw, len_gain_raw,
                   mag_beta_raw, eps=1e-6, window=None, compute_dtype=torch.float32):
    """Fold the null sink into streamed statistics and emit (c, mag)
    (kernel/polar_triton.py:151-178)."""
    cd = compute_dtype
    m, L, Q2, S = (x.to(cd) for x in stats)
    H = S.shape[1]
    spg = F.softplus(len_gain_raw.to(cd))
    sps = F.softplus(null_slope_raw.to(cd))
    beta = F.softplus(mag_beta_raw.to(cd))
    temp, null = _temp_null(n_keys, window, spg, null_base, sps, cd)
    a_n = (temp * null)[None]                                                   # (1,H,Tq)
    m_new = torch.maximum(m, a_n)
    alpha = torch.exp(m - m_new)
    L, Q2, S = L * alpha, Q2 * alpha * alpha, S * alpha[..., None]
    p_n = torch.exp(a_n - m_new)
    Z = L + p_n
    s = S + p_n[..., None] * v_null.to(cd).view(1, H, 1, -1)
    c = s / s.norm(dim=-1, keepdim=True).clamp_min(eps)
    n_eff = L * L / Q2.clamp_min(1e-30)
    m_eff = n_eff * (L / Z.clamp_min(eps))
    mag = torch.tanh(beta.view(1, H, 1) * torch.log1p(m_eff))
    return c, mag


def polar_streaming(q, k, v, n_keys, *, v_null, null_base, null_slope_raw, len_gain_raw,
                    mag_beta_raw, eps=1e-6, window=None, compute_dtype=torch.float32, tile=64):
    """Tile-streaming Polar attention: the exact target of the device kernels."""
    stats = polar_streaming_stats(q, k, v, n_keys, len_gain_raw=len_gain_raw, window=window,
                                  compute_dtype=compute_dtype, tile=tile)
    return polar_finalize(stats, n_keys, v_null=v_null, null_base=null_base,
                          null_slope_raw=null_slope_raw, len_gain_raw=len_gain_raw,
                          mag_beta_raw=mag_beta_raw, eps=eps, window=window,
                          compute_dtype=compute_dtype)


def polar_prefill_oracle(q, k, v, n_keys, params, *, eps=1e-6, window=None,
                         compute_dtype=torch.float32):
    """Checker for polar_attention_fwd: materialised form, kernel-API layout."""
    return polar_materialized(q, k, v, n_keys, eps=eps, window=window,
                              compute_dtype=compute_dtype, **params)


def polar_decode_oracle(q, k_cache, v_cache, block_tables, context_lens, params, *,
                        eps=1e-6, window=None, compute_dtype=torch.float32):
    """Checker for polar_attention_decode (kernel/polar_triton.py:681-858): for each
    sequence gather its keys through the page table, then run the materialised form
    with Tq = 1 and n = context_len.  q (B, H, dk); caches (num_blocks, block_size,
    Hkv, dk); block_tables (B, max_blocks) int32; context_lens (B,) int32."""
    B, H, dk = q.shape
    bs = k_cache.shape[1]
    c = torch.empty(B, H, dk, dtype=compute_dtype)
    mag = torch.empty(B, H, dtype=compute_dtype)
    for b in range(B):
        n = int(context_lens[b])
        nblk = (n + bs - 1) // bs
        if nblk == 0:
            kk = k_cache.new_zeros(1, k_cache.shape[2], 1, dk)
            vv = kk.clone()
        else:
            phys = block_tables[b, :nblk].long()
            kk = k_cache[phys].reshape(nblk * bs, -1, dk)[:n].permute(1, 0, 2)[None]   # (1,Hkv,n,dk)
            vv = v_cache[phys].reshape(nblk * bs, -1, dk)[:n].permute(1, 0, 2)[None]
        cb, mb = polar_materialized(q[b][None, :, None, :], kk, vv,
                                    torch.tensor([float(n)]), eps=eps, window=window,
                                    compute_dtype=compute_dtype, **params)
        c[b], mag[b] = cb[0, :, 0], mb[0, :, 0]
    return c, mag
