"""Gated-delta ("Titans MAG") memory on the CPU - checker for the CUDA scan and step.

TEST INFRASTRUCTURE: see the package docstring.

Recurrence per head, state M (dv x dk), unit-norm k_t and q_t
(scripts/titans_proto.py:53-74):

    M <- gamma_t M;  pred = M k_t;  M <- M + beta_t (v_t - pred) k_t^T;  r_t = M q_t

``gated_delta_sequential`` is that definition.  ``gated_delta_chunked`` is the
chunk-parallel form of model/blocks.py:375-423, restated with an explicit forward
substitution in place of the library triangular solve.  The device API uses the
flash-linear-attention convention (inference/models/atma.py:285-287): tensors are
(B, T, H, d), the decay arrives as a log (g = log gamma), the state table is
[K, V] = M transposed, and q, k are L2-normalised inside the kernel.
"""

import torch
import torch.nn.functional as F


def gated_delta_sequential(q, k, v, gamma, beta, S0=None):
    """Token-by-token definition.  q, k (B,H,N,dk) unit norm; v (B,H,N,dv);
    gamma, beta (B,H,N).  Returns R (B,H,N,dv), M_final (B,H,dv,dk)."""
    B, H, N, dk = q.shape
    dv = v.shape[-1]
    M = torch.zeros(B, H, dv, dk, dtype=q.dtype) if S0 is None else S0.clone()
    R = torch.empty(B, H, N, dv, dtype=q.dtype)
    for t in range(N):
        M = M * gamma[:, :, t, None, None]
        pred = torch.einsum("bhvk,bhk->bhv", M, k[:, :, t])
        u = beta[:, :, t, None] * (v[:, :, t] - pred)
        M = M + u[..., :, None] * k[:, :, t, None, :]
        R[:, :, t] = torch.einsum("bhvk,bhk->bhv", M, q[:, :, t])
    return R, M


def gated_delta_chunked(q, k, v, gamma, beta, chunk=64, S0=None, substitution=False):
    """Chunk-parallel form (model/blocks.py:393-423).  Inside a chunk with inclusive
    cumulative decay g_p: A[p,s] = beta_p (g_p/g_s)(k_s.k_p) for s<p; solve
    (I + A) U = diag(beta)(V - g (.) (M0 K^T)^T); R = g (.) (M0 Q^T)^T + Rq U with
    Rq[p,s] = (g_p/g_s)(k_s.q_p) for s<=p; M_C = g_C M0 + sum_s (g_C/g_s) u_s k_s^T.
    ``substitution=True`` solves the unit-lower-triangular system row by row instead
    of calling the library triangular solve (the two are cross-checked in the tests)."""
    B, H, N, dk = q.shape
    dv = v.shape[-1]
    M = torch.zeros(B, H, dv, dk, dtype=q.dtype) if S0 is None else S0.clone()
    R = torch.empty(B, H, N, dv, dtype=q.dtype)
    for c0 in range(0, N, chunk):
        c1 = min(c0 + chunk, N)
        C = c1 - c0
        qc, kc, vc = q[:, :, c0:c1], k[:, :, c0:c1], v[:, :, c0:c1]
        lg = torch.cumsum(torch.log(gamma[:, :, c0:c1]), dim=-1)               # log g_p
        ratio = torch.exp(lg[..., :, None] - lg[..., None, :])                 # g_p / g_s
        idx = torch.arange(C)
        strict = (idx[:, None] > idx[None, :])
        incl = (idx[:, None] >= idx[None, :])
        kk = torch.matmul(kc, kc.transpose(-1, -2))
        qk = torch.matmul(qc, kc.transpose(-1, -2))
        A = torch.where(strict, ratio * kk, torch.zeros((), dtype=q.dtype)) * beta[:, :, c0:c1, None]
        Rq = torch.where(incl, ratio * qk, torch.zeros((), dtype=q.dtype))
        g = torch.exp(lg)
        rhs = beta[:, :, c0:c1, None] * (vc - g[..., None] * torch.matmul(kc, M.transpose(-1, -2)))
        if substitution:                                                       # explicit forward substitution
            U = torch.empty_like(rhs)
            for p in range(C):
                U[:, :, p] = rhs[:, :, p] - torch.einsum("bhs,bhsv->bhv", A[:, :, p, :p], U[:, :, :p])
        else:                                                                  # same system, LAPACK trsm
            U = torch.linalg.solve_triangular(A, rhs, upper=False, unitriangular=True)
        R[:, :, c0:c1] = g[..., None] * torch.matmul(qc, M.transpose(-1, -2)) + torch.matmul(Rq, U)
        tail = torch.exp(lg[..., -1:] - lg)                                    # g_C / g_s
        M = g[..., -1, None, None] * M + torch.matmul((tail[..., None] * U).transpose(-1, -2), kc)
    return R, M


def gated_delta_step(q, k, v, gamma, beta, state_table, slots, eps=1e-12):
    """One in-place decode step on a slot-indexed [K, V] state table
    (kernel/gated_delta_triton.py:56-75; torch fallback inference/models/atma.py:362-371).
    q, k, v (B,H,d); gamma, beta (B,H); state_table (max_seqs,H,dk,dv) fp32 - MUTATED.
    Returns r (B,H,dv) fp32."""
    qn = q.float() / q.float().norm(dim=-1, keepdim=True).clamp_min(eps)
    kn = k.float() / k.float().norm(dim=-1, keepdim=True).clamp_min(eps)
    S = state_table[slots.long()].float()                                      # (B,H,dk,dv)
    Sd = gamma.float()[..., None, None] * S
    pred = torch.einsum("bhk,bhkv->bhv", kn, Sd)
    u = beta.float()[..., None] * (v.float() - pred)
    S_new = Sd + kn[..., :, None] * u[..., None, :]
    state_table[slots.long()] = S_new.to(state_table.dtype)
    return torch.einsum("bhk,bhkv->bhv", qn, S_new)


def chunk_gated_delta_rule_oracle(q, k, v, g, beta, initial_state=None, chunk=64,
                                  compute_dtype=torch.float32, sequential=False):
    """Checker for the device scan in its production calling convention
    (inference/models/atma.py:280-288): q, k, v (B,T,H,d); g (B,T,H) log-decay;
    beta (B,T,H); initial_state (B,H,dk,dv) [K,V].  q, k are L2-normalised here
    (F.normalize, eps 1e-12) as the in-kernel normalisation does.  Returns
    o (B,T,H,dv) and the final state (B,H,dk,dv), both in ``compute_dtype``."""
    cd = compute_dtype
    if k.shape[2] != q.shape[2]:                     # un-expanded KV heads: head h reads KV head h // G
        G = q.shape[2] // k.shape[2]
        k, v = k.repeat_interleave(G, dim=2), v.repeat_interleave(G, dim=2)
    qn = F.normalize(q.to(cd), dim=-1).transpose(1, 2)
    kn = F.normalize(k.to(cd), dim=-1).transpose(1, 2)
    vt = v.to(cd).transpose(1, 2)
    gamma = torch.exp(g.to(cd)).transpose(1, 2)
    bt = beta.to(cd).transpose(1, 2)
    S0 = None if initial_state is None else initial_state.to(cd).transpose(-1, -2).contiguous()
    if sequential:
        R, M = gated_delta_sequential(qn, kn, vt, gamma, bt, S0)
    else:
        R, M = gated_delta_chunked(qn, kn, vt, gamma, bt, chunk=chunk, S0=S0)
    return R.transpose(1, 2).contiguous(), M.transpose(-1, -2).contiguous()
