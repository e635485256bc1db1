"""CPU (gloo, world_size 2 and 3): the context-parallel routing - zig-zag segments, ring plan,
statistics carry, affine state prefix, conv halos - reproduces the single-process result.
The compute backend here is the CPU oracle; the GPU path swaps in the CUDA kernels only."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from oracle.polar import polar_streaming_stats, polar_finalize
from atma_b200 import context_parallel as cp


class OracleBackend:
    def prepare_params(self, params, device):
        return params

    def polar_block(self, q, k, v, n_keys, params, key_offset, stats_in, finalize, eps, window):
        stats = polar_streaming_stats(q, k, v, n_keys, len_gain_raw=params["len_gain_raw"], window=window,
                                      key_offset=key_offset, carry=stats_in, tile=8)
        if not finalize:
            return stats
        return polar_finalize(stats, n_keys, eps=eps, window=window, **params)

    def decode_partials(self, q, k_cache, v_cache, block_tables, local_lens, total_lens, params, eps):
        B, H, dk = q.shape
        bs = k_cache.shape[1]
        stats, sums = torch.zeros(B, H, 1, 4), torch.zeros(B, H, 1, dk)
        for b in range(B):
            n = int(local_lens[b])
            pages = block_tables[b, :(n + bs - 1) // bs].long()
            kk = k_cache[pages].reshape(-1, k_cache.shape[2], dk)[:n].permute(1, 0, 2)[None]
            vv = v_cache[pages].reshape(-1, k_cache.shape[2], dk)[:n].permute(1, 0, 2)[None]
            m, L, Q2, S = polar_streaming_stats(q[b][None, :, None, :], kk, vv, torch.tensor([float(total_lens[b])]),
                                                len_gain_raw=params["len_gain_raw"], tile=8)
            stats[b, :, 0, 0], stats[b, :, 0, 1], stats[b, :, 0, 2] = m[0, :, 0], L[0, :, 0], Q2[0, :, 0]
            sums[b, :, 0] = S[0, :, 0]
        return stats, sums

    def decode_merge(self, stats, sums, total_lens, params, dtype, eps):
        m = stats[..., 0].amax(-1)                                          # the merge rule of the device kernel
        w = torch.exp(stats[..., 0] - m[..., None])
        L = (stats[..., 1] * w).sum(-1)
        Q2 = (stats[..., 2] * w * w).sum(-1)
        S = (sums * w[..., None]).sum(-2)
        cs, ms = [], []
        for b in range(m.shape[0]):                                         # the null sink depends on each sequence's length
            c, mag = polar_finalize((m[b:b + 1, :, None], L[b:b + 1, :, None], Q2[b:b + 1, :, None], S[b:b + 1, :, None]),
                                    total_lens[b:b + 1].float(), eps=eps, **params)
            cs.append(c[:, :, 0])
            ms.append(mag[:, :, 0])
        return torch.cat(cs).to(dtype), torch.cat(ms).to(dtype)

    def scan_factors(self, q, k, v, g, beta):
        return (q, k, v, g, beta)

    def scan_recur(self, factors, rec_of, initial_state, zero_value, want_output):
        q, k, v, g, beta = factors
        idx = torch.tensor(rec_of)
        vv = v[idx].clone()
        for i, z in enumerate(zero_value or []):
            if z:
                vv[i] = 0
        o, S = oracle.chunk_gated_delta_rule_oracle(q[idx], k[idx], vv, g[idx], beta[idx], initial_state=initial_state, chunk=8)
        return (o if want_output else None), S


def _inputs(T, H, Hkv, dk):
    g = torch.Generator().manual_seed(0)
    t = dict(q=torch.randn(1, T, H, dk, generator=g), k=torch.randn(1, T, Hkv, dk, generator=g),
             v=torch.randn(1, T, Hkv, dk, generator=g),
             g=-torch.nn.functional.softplus(torch.randn(1, T, H, generator=g)),
             beta=torch.sigmoid(torch.randn(1, T, H, generator=g)))
    params = dict(v_null=torch.randn(H, dk, generator=g) * 0.3, null_base=torch.full((H,), 2.0),
                  null_slope_raw=torch.full((H,), 0.5), len_gain_raw=torch.full((H,), -1.0),
                  mag_beta_raw=torch.full((H,), -1.5))
    x = torch.randn(T, 6, generator=g)
    return t, params, x


def _worker(rank, world, port, T, mode, window, ret):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        H, Hkv, dk = 4, 2, 16
        t, params, x = _inputs(T, H, Hkv, dk)
        shard = cp.shard_sequence(t, rank, world)
        polar, o, S = cp.cp_global_layer_prefill(shard, params, backend=OracleBackend(), polar_mode=mode, window=window)
        halos = cp.cp_conv_halos([x[a:b] for a, b in shard.positions], 4)
        ret[rank] = dict(pos=shard.positions, c=[p[0] for p in polar], mag=[p[1] for p in polar], o=o, S=S, halos=halos)
    finally:
        dist.destroy_process_group()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


@pytest.mark.parametrize("world,T,mode,window", [(2, 64, "ring", None), (3, 96, "ring", None), (2, 64, "gather", None),
                                                 (3, 96, "gather", None), (2, 64, "ring", 20), (2, 64, "gather", 20)])
def test_context_parallel_matches_single_process(world, T, mode, window):
    H, Hkv, dk = 4, 2, 16
    t, params, x = _inputs(T, H, Hkv, dk)
    n = torch.arange(1, T + 1, dtype=torch.float32)
    c_ref, m_ref = oracle.polar_prefill_oracle(t["q"].transpose(1, 2), t["k"].transpose(1, 2), t["v"].transpose(1, 2), n, params, window=window)
    ke, ve = t["k"].repeat_interleave(H // Hkv, 2), t["v"].repeat_interleave(H // Hkv, 2)
    o_ref, S_ref = oracle.chunk_gated_delta_rule_oracle(t["q"], ke, ve, t["g"], t["beta"], chunk=8)
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), T, mode, window, ret), nprocs=world, join=True)
    assert len(ret) == world
    for rank in range(world):
        r = ret[rank]
        for part, (a, b) in enumerate(r["pos"]):
            assert (r["c"][part] - c_ref[:, :, a:b]).abs().max() < 1e-5
            assert (r["mag"][part] - m_ref[:, :, a:b]).abs().max() < 1e-5
            assert (r["o"][part] - o_ref[:, a:b]).abs().max() < 1e-4
            expect = torch.zeros(3, 6) if a == 0 else x[a - 3:a]
            assert torch.equal(r["halos"][part], expect.t())
        assert (r["S"] - S_ref[0]).abs().max() < 1e-4


def test_zigzag_and_plan_cover_the_causal_triangle():
    for world in (1, 2, 4, 8):
        segs = cp.zigzag_segments(16 * world, world)
        flat = sorted(s for pair in segs for s in pair)
        assert flat == [(i * 8, (i + 1) * 8) for i in range(2 * world)]
        seen = set()
        for rank in range(world):
            plan = cp.ring_plan(rank, world)
            assert [a for a, _ in plan] == [(rank - s) % world for s in range(world)]
            loads = [len(p) for _, p in plan]
            assert loads[0] == (3 if True else 2) and all(x == 2 for x in loads[1:])      # balanced steps
            for a, prods in plan:
                for qp, kp, diag in prods:
                    qs = rank if qp == 0 else 2 * world - 1 - rank
                    ks = a if kp == 0 else 2 * world - 1 - a
                    assert ks <= qs and diag == (ks == qs)
                    seen.add((qs, ks))
        assert seen == {(i, j) for i in range(2 * world) for j in range(i + 1)}
    with pytest.raises(ValueError):
        cp.zigzag_segments(100, 8)


def test_state_prefix_composition():
    g = torch.Generator().manual_seed(1)
    P = torch.randn(5, 2, 4, 4, generator=g) * 0.5
    Q = torch.randn(5, 2, 4, 3, generator=g)
    S0 = torch.randn(2, 4, 3, generator=g)
    states, final = cp.compose_state_prefix(P, Q, S0)
    S = S0
    for i in range(5):
        assert torch.allclose(states[i], S)
        S = P[i] @ S + Q[i]
    assert torch.allclose(final, S)


def _decode_worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        B, H, Hkv, dk, bs, T = 3, 4, 2, 16, 8, 48
        g = torch.Generator().manual_seed(5)
        k = torch.randn(B, T, Hkv, dk, generator=g)
        v = torch.randn(B, T, Hkv, dk, generator=g)
        q = torch.randn(B, H, dk, generator=g)
        lens = torch.tensor([48, 31, 17])
        params = dict(v_null=torch.randn(H, dk, generator=g) * 0.3, null_base=torch.full((H,), 2.0),
                      null_slope_raw=torch.full((H,), 0.5), len_gain_raw=torch.full((H,), -1.0),
                      mag_beta_raw=torch.full((H,), -1.5))
        # this rank's share of every sequence: the zig-zag segments it owns, packed into its own pages
        segs = cp.zigzag_segments(T, world)[rank]
        pages_per = T // bs
        kc, vc = torch.zeros(B * pages_per, bs, Hkv, dk), torch.zeros(B * pages_per, bs, Hkv, dk)
        bt = torch.arange(B * pages_per).view(B, pages_per).int()
        local = torch.zeros(B, dtype=torch.int32)
        for b in range(B):
            idx = torch.cat([torch.arange(a, min(e, int(lens[b]))) for a, e in segs if a < int(lens[b])] or [torch.zeros(0, dtype=torch.long)])
            local[b] = idx.numel()
            flat_k, flat_v = kc.view(-1, Hkv, dk), vc.view(-1, Hkv, dk)
            base = int(bt[b, 0]) * bs
            flat_k[base:base + idx.numel()] = k[b, idx]
            flat_v[base:base + idx.numel()] = v[b, idx]
        c, mag = cp.cp_polar_decode(q, kc, vc, bt, local, lens.int(), params, backend=OracleBackend())
        ret[rank] = (c, mag)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_decode_over_a_context_parallel_cache_matches_single_process(world):
    """Every rank holds the K/V of its own segments; partial statistics are all-gathered and merged: the result is
    the decode over the whole cache, on every rank (ragged lengths, one sequence shorter than a segment)."""
    B, H, Hkv, dk, bs, T = 3, 4, 2, 16, 8, 48
    g = torch.Generator().manual_seed(5)
    k = torch.randn(B, T, Hkv, dk, generator=g)
    v = torch.randn(B, T, Hkv, dk, generator=g)
    q = torch.randn(B, H, dk, generator=g)
    lens = torch.tensor([48, 31, 17], dtype=torch.int32)
    params = dict(v_null=torch.randn(H, dk, generator=g) * 0.3, null_base=torch.full((H,), 2.0),
                  null_slope_raw=torch.full((H,), 0.5), len_gain_raw=torch.full((H,), -1.0),
                  mag_beta_raw=torch.full((H,), -1.5))
    kc, vc = k.reshape(B * T // bs, bs, Hkv, dk), v.reshape(B * T // bs, bs, Hkv, dk)
    bt = torch.arange(B * T // bs).view(B, T // bs).int()
    c_ref, m_ref = oracle.polar_decode_oracle(q, kc, vc, bt, lens, params)
    ret = mp.Manager().dict()
    mp.spawn(_decode_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    for rank in range(world):
        c, mag = ret[rank]
        assert (c - c_ref).abs().max() < 1e-5 and (mag - m_ref).abs().max() < 1e-5
