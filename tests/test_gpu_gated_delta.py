"""GPU parity: gated-delta decode step and chunked scan (through the C ABI) against the CPU
oracle and the golden vectors."""

import pytest
import torch
import torch.nn.functional as F

import atma_b200
import oracle
from conftest import max_abs, max_rel
from gpu_util import rand

pytestmark = pytest.mark.gpu


def test_step_golden(golden):
    g = golden["delta_step"]
    table = g["table"].cuda()
    r = atma_b200.gated_delta_decode_step(g["q"].cuda(), g["k"].cuda(), g["v"].cuda(), g["gamma"].cuda(),
                                          g["beta"].cuda(), table, g["slots"].cuda())
    assert max_abs(r, g["r"]) < 2e-5 and max_abs(table, g["table_out"]) < 2e-6


# tests/test_decode_kernels.py:27-53 of the reference (bf16 inputs, dim 64), plus the model's shape
@pytest.mark.parametrize("batch,heads,dim,dtype", [(2, 2, 64, torch.bfloat16), (5, 8, 128, torch.bfloat16),
                                                   (3, 4, 128, torch.float32), (2, 2, 32, torch.float16)])
def test_step_matches_oracle(batch, heads, dim, dtype):
    q, k, v = rand((batch, heads, dim), 4, dtype), rand((batch, heads, dim), 5, dtype), rand((batch, heads, dim), 6, dtype)
    g = torch.Generator().manual_seed(7)
    gamma, beta = torch.rand(batch, heads, generator=g), torch.rand(batch, heads, generator=g)
    slots = torch.randperm(batch + 3, generator=g)[:batch]
    table = torch.randn(batch + 3, heads, dim, dim, generator=g)
    expect_table = table.clone()
    r_ref = oracle.gated_delta_step(q, k, v, gamma, beta, expect_table, slots)
    tg = table.cuda()
    r = atma_b200.gated_delta_decode_step(q.cuda(), k.cuda(), v.cuda(), gamma.cuda(), beta.cuda(), tg, slots.cuda())
    torch.testing.assert_close(r.cpu(), r_ref, atol=2e-4, rtol=2e-4)
    torch.testing.assert_close(tg.cpu(), expect_table, atol=2e-5, rtol=2e-5)
    untouched = [i for i in range(batch + 3) if i not in slots.tolist()]
    assert torch.equal(tg.cpu()[untouched], table[untouched])


def test_step_strided_inputs_and_padded_slot():
    B, H, d = 3, 4, 64
    big = rand((B, 3, H, d), 8, torch.bfloat16).cuda()       # q, k, v interleaved: strided views
    q, k, v = big[:, 0], big[:, 1], big[:, 2]
    gamma, beta = torch.rand(B, H, device="cuda"), torch.rand(B, H, device="cuda")
    table = torch.randn(4, H, d, d, device="cuda")
    keep = table.clone()
    slots = torch.tensor([2, -1, 0], device="cuda")
    r = atma_b200.gated_delta_decode_step(q, k, v, gamma, beta, table, slots)
    ref_table = keep.cpu().clone()
    r_ref = oracle.gated_delta_step(q.cpu()[[0, 2]], k.cpu()[[0, 2]], v.cpu()[[0, 2]], gamma.cpu()[[0, 2]],
                                    beta.cpu()[[0, 2]], ref_table, torch.tensor([2, 0]))
    assert max_abs(r[[0, 2]], r_ref) < 2e-4 and float(r[1].abs().max()) == 0.0
    assert max_abs(table, ref_table) < 2e-5


def _scan_inputs(B, T, H, dk, dv, dtype, seed, gamma_bias):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, T, H, dk, generator=g).to(dtype)
    k = torch.randn(B, T, H, dk, generator=g).to(dtype)
    v = torch.randn(B, T, H, dv, generator=g).to(dtype)
    glog = F.logsigmoid(torch.randn(B, T, H, generator=g) + gamma_bias)
    beta = torch.sigmoid(torch.randn(B, T, H, generator=g))
    S0 = torch.randn(B, H, dk, dv, generator=g) * 0.3
    return q, k, v, glog, beta, S0


def _scan(q, k, v, glog, beta, S0):
    return atma_b200.chunk_gated_delta_rule(q=q.cuda(), k=k.cuda(), v=v.cuda(), g=glog.cuda(), beta=beta.cuda(),
                                            scale=1.0, initial_state=None if S0 is None else S0.cuda(),
                                            output_final_state=True, use_qk_l2norm_in_kernel=True)


@pytest.mark.parametrize("name", ["delta_small", "delta_carry", "delta_d128"])
def test_scan_golden(golden, name):
    """The golden inputs are already unit-norm (B,H,N,d); re-normalising in-kernel is a no-op."""
    g = golden[name]
    S0 = g["S0"].transpose(-1, -2).contiguous() if g["S0"].numel() else None
    o, S = _scan(g["q"].transpose(1, 2), g["k"].transpose(1, 2), g["v"].transpose(1, 2),
                 torch.log(g["gamma"]).transpose(1, 2), g["beta"].transpose(1, 2), S0)
    assert max_abs(o, g["R"].transpose(1, 2)) < 1e-4
    assert max_abs(S, g["S"].transpose(-1, -2)) < 1e-4


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("B,T,H,dk,dv,bias", [(2, 256, 4, 128, 128, 3.9), (1, 1000, 2, 128, 128, 0.0),
                                              (2, 130, 3, 64, 64, 3.9), (1, 63, 2, 128, 128, 3.9), (1, 1, 1, 128, 128, 0.0)])
def test_scan_matches_oracle(dtype, tol, B, T, H, dk, dv, bias):
    q, k, v, glog, beta, S0 = _scan_inputs(B, T, H, dk, dv, dtype, seed=T + H, gamma_bias=bias)
    o_ref, S_ref = oracle.chunk_gated_delta_rule_oracle(q, k, v, glog, beta, initial_state=S0)
    o, S = _scan(q, k, v, glog, beta, S0)
    assert o.dtype == dtype and S.dtype == torch.float32
    if dtype == torch.float32:
        assert max_abs(o, o_ref) < tol and max_abs(S, S_ref) < tol
    else:
        assert max_rel(o, o_ref) < tol and max_rel(S, S_ref) < tol


def test_scan_state_carry_layout_and_decode_continuity():
    """The checks of the reference's tests/verify_fla.py:29-121: (1) splitting the prompt at a
    non-multiple of the chunk and carrying the state == one pass; (2) the final state is [K,V]
    (the transpose of the oracle's [V,K]); (3) single-token steps from the scan's final state
    continue the scan."""
    B, H, T, dk, Tdec = 2, 8, 256, 128, 8
    q, k, v, glog, beta, _ = _scan_inputs(B, T + Tdec, H, dk, dk, torch.bfloat16, seed=1, gamma_bias=3.9)
    o_full, S_full = _scan(q, k, v, glog, beta, None)
    T1 = 100
    _, S_a = _scan(q[:, :T1], k[:, :T1], v[:, :T1], glog[:, :T1], beta[:, :T1], None)
    o_b, _ = _scan(q[:, T1:T], k[:, T1:T], v[:, T1:T], glog[:, T1:T], beta[:, T1:T], S_a.cpu())
    assert max_rel(o_b, o_full[:, T1:T]) < 2e-2
    o_pre, S_pre = _scan(q[:, :T], k[:, :T], v[:, :T], glog[:, :T], beta[:, :T], None)
    qn = F.normalize(q[:, :T].float().transpose(1, 2), dim=-1)
    kn = F.normalize(k[:, :T].float().transpose(1, 2), dim=-1)
    r_t, S_t = oracle.gated_delta_chunked(qn, kn, v[:, :T].float().transpose(1, 2),
                                          torch.exp(glog[:, :T]).transpose(1, 2), beta[:, :T].transpose(1, 2), chunk=64)
    assert max_rel(o_pre, r_t.transpose(1, 2)) < 2e-2
    assert max_rel(S_pre, S_t.transpose(-1, -2)) < 2e-2
    assert max_rel(S_pre, S_t) > 0.2                      # the un-transposed compare must be far off
    table = torch.zeros(4, H, dk, dk, device="cuda")
    slots = torch.tensor([2, 0], device="cuda")
    table[slots] = S_pre
    outs = []
    for t in range(T, T + Tdec):
        outs.append(atma_b200.gated_delta_decode_step(q[:, t].cuda(), k[:, t].cuda(), v[:, t].cuda(),
                                                      torch.exp(glog[:, t]).cuda(), beta[:, t].cuda(), table, slots))
    assert max_rel(torch.stack(outs, 1), o_full[:, T:].float()) < 2e-2
    assert max_rel(table[slots], S_full) < 2e-2


# ---- packed ("varlen") scan: several sequences on one token axis, one call ------------------------------
def _packed_inputs(lens, H, Hkv, d, dtype, seed):
    total = sum(lens)
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(total, H, d, generator=g).to(dtype)
    k = torch.randn(total, Hkv, d, generator=g).to(dtype)
    v = torch.randn(total, Hkv, d, generator=g).to(dtype)
    glog = F.logsigmoid(torch.randn(total, H, generator=g) + 3.0)
    beta = torch.sigmoid(torch.randn(total, H, generator=g))
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    return q, k, v, glog, beta, cu


@pytest.mark.parametrize("dtype,d,tol", [(torch.bfloat16, 128, 2e-2), (torch.float16, 128, 2e-2), (torch.float32, 64, 1e-4)])
def test_packed_scan_matches_oracle_per_sequence(dtype, d, tol):
    """Ragged lengths (below one chunk, exact chunk multiples, odd tails, an empty sequence) in one
    call == the oracle run sequence by sequence, outputs and final states, with initial states."""
    lens, H, Hkv = [130, 64, 7, 0, 300, 1], 4, 2
    q, k, v, glog, beta, cu = _packed_inputs(lens, H, Hkv, d, dtype, seed=21)
    S0 = torch.randn(len(lens), H, d, d, generator=torch.Generator().manual_seed(3)) * 0.3
    o, S = atma_b200.chunk_gated_delta_rule(q=q.cuda()[None], k=k.cuda()[None], v=v.cuda()[None], g=glog.cuda()[None],
                                            beta=beta.cuda()[None], scale=1.0, initial_state=S0.cuda(),
                                            output_final_state=True, use_qk_l2norm_in_kernel=True, cu_seqlens=cu.cuda())
    assert o.shape == (1, sum(lens), H, d) and S.shape == (len(lens), H, d, d)
    err = max_rel if dtype != torch.float32 else max_abs
    for i, n in enumerate(lens):
        a, b = int(cu[i]), int(cu[i + 1])
        if n == 0:
            assert torch.equal(S[i].cpu(), S0[i])                  # an empty sequence passes its state through
            continue
        o_ref, S_ref = oracle.chunk_gated_delta_rule_oracle(q[None, a:b], k[None, a:b], v[None, a:b], glog[None, a:b],
                                                            beta[None, a:b], initial_state=S0[i:i + 1])
        assert err(o[0, a:b], o_ref[0]) < tol, (i, n)
        assert err(S[i], S_ref[0]) < tol, (i, n)


def test_packed_prefill_updates_the_slot_table_in_place():
    """packed_gated_delta_prefill == the reference's per-sequence loop (scan from the slot's row when the
    sequence continues a cached prefix, else from zero; copy the final state back): bit-identical to
    the dense kernel called sequence by sequence, rows of other slots untouched."""
    lens, H, Hkv, d = [200, 65, 511, 33], 8, 2, 128
    q, k, v, glog, beta, cu = _packed_inputs(lens, H, Hkv, d, torch.bfloat16, seed=5)
    gen = torch.Generator().manual_seed(9)
    table = (torch.randn(7, H, d, d, generator=gen) * 0.2).cuda()
    slots = torch.tensor([5, 0, 3, 6])
    has_initial = torch.tensor([1, 0, 1, 0])
    expect = table.clone()
    qc, kc, vc, gc, bc = q.cuda(), k.cuda(), v.cuda(), glog.cuda(), beta.cuda()
    o_expect = torch.empty(sum(lens), H, d, dtype=torch.bfloat16, device="cuda")
    for i in range(len(lens)):
        a, b = int(cu[i]), int(cu[i + 1])
        s0 = expect[slots[i]][None].clone() if has_initial[i] else None
        oi, Si = atma_b200.chunk_gated_delta_rule(q=qc[None, a:b], k=kc[None, a:b], v=vc[None, a:b], g=gc[None, a:b],
                                                  beta=bc[None, a:b], scale=1.0, initial_state=s0,
                                                  output_final_state=True, use_qk_l2norm_in_kernel=True)
        o_expect[a:b] = oi[0]
        expect[slots[i]] = Si[0]
    o = atma_b200.packed_gated_delta_prefill(qc, kc, vc, gc, bc, cu, table, slots, has_initial)
    assert torch.equal(o, o_expect)
    assert torch.equal(table, expect)
    # every sequence continuing from its row (has_initial=None), device-resident cu_seqlens
    table2 = expect.clone()
    o2 = atma_b200.packed_gated_delta_prefill(qc, kc, vc, gc, bc, cu.cuda(), table2, slots.cuda())
    a, b = int(cu[1]), int(cu[2])
    o_ref, S_ref = atma_b200.chunk_gated_delta_rule(q=qc[None, a:b], k=kc[None, a:b], v=vc[None, a:b], g=gc[None, a:b],
                                                    beta=bc[None, a:b], scale=1.0, initial_state=expect[0][None],
                                                    output_final_state=True, use_qk_l2norm_in_kernel=True)
    assert torch.equal(o2[a:b], o_ref[0]) and torch.equal(table2[0], S_ref[0])


def test_packed_prefill_state_snapshots_give_exact_prefix_reuse():
    """Snapshots at every 256-token page boundary == the final state of a scan over exactly that prefix
    (bit-identical: same kernels, same chunks), and a second request that shares the first two pages
    and starts from the page-2 snapshot reproduces the outputs of the full-length scan."""
    lens, H, Hkv, d, page = [700, 256, 90, 513], 8, 2, 128, 256
    q, k, v, glog, beta, cu = _packed_inputs(lens, H, Hkv, d, torch.bfloat16, seed=31)
    qc, kc, vc, gc, bc = q.cuda(), k.cuda(), v.cuda(), glog.cuda(), beta.cuda()
    table = torch.zeros(5, H, d, d, device="cuda")
    slots = torch.tensor([3, 1, 0, 4])
    o, snaps, offs = atma_b200.packed_gated_delta_prefill(qc, kc, vc, gc, bc, cu, table, slots, snapshot_every=page,
                                                         seqlens=lens)
    assert offs == [0, 2, 3, 3] and snaps.shape == (5, H, d, d)
    plain_table = torch.zeros_like(table)
    o_plain = atma_b200.packed_gated_delta_prefill(qc, kc, vc, gc, bc, cu, plain_table, slots)
    assert torch.equal(o, o_plain) and torch.equal(table, plain_table)       # snapshots do not disturb the scan
    for i, n in enumerate(lens):
        a = int(cu[i])
        for j in range(n // page):
            _, S_ref = atma_b200.chunk_gated_delta_rule(q=qc[None, a:a + (j + 1) * page], k=kc[None, a:a + (j + 1) * page],
                                                        v=vc[None, a:a + (j + 1) * page], g=gc[None, a:a + (j + 1) * page],
                                                        beta=bc[None, a:a + (j + 1) * page], scale=1.0,
                                                        output_final_state=True, use_qk_l2norm_in_kernel=True)
            assert torch.equal(snaps[offs[i] + j], S_ref[0]), (i, j)
    # prefix reuse: sequence 0's tokens 512..699 scanned from the page-2 snapshot
    a = int(cu[0])
    table2 = torch.zeros_like(table)
    table2[2] = snaps[offs[0] + 1]
    tail = slice(a + 2 * page, a + lens[0])
    o_tail = atma_b200.packed_gated_delta_prefill(qc[tail], kc[tail], vc[tail], gc[tail], bc[tail],
                                                  torch.tensor([0, lens[0] - 2 * page], dtype=torch.int32), table2,
                                                  torch.tensor([2]))
    assert torch.equal(o_tail, o[tail]) and torch.equal(table2[2], table[3])


@pytest.mark.parametrize("B,T,segments", [(1, 8192, 4), (1, 4500, 0), (2, 4096 + 37, 3), (1, 16384, 8)])
def test_scan_cut_into_segments_equals_the_single_pass(B, T, segments):
    """A long sequence of a small batch is walked as several segments side by side (transfer maps,
    chained states, second pass): outputs and final state agree with the single pass and with the
    oracle; `segments=0` lets the library choose, 1 forces the single pass."""
    H, Hkv, d = 8, 2, 128
    g = torch.Generator().manual_seed(T)
    q = torch.randn(B, T, H, d, generator=g).bfloat16()
    k = torch.randn(B, T, Hkv, d, generator=g).bfloat16()
    v = torch.randn(B, T, Hkv, d, generator=g).bfloat16()
    glog = F.logsigmoid(torch.randn(B, T, H, generator=g) + 3.9)
    beta = torch.sigmoid(torch.randn(B, T, H, generator=g))
    S0 = torch.randn(B, H, d, d, generator=g) * 0.3
    kw = dict(q=q.cuda(), k=k.cuda(), v=v.cuda(), g=glog.cuda(), beta=beta.cuda(), scale=1.0, initial_state=S0.cuda(),
              output_final_state=True, use_qk_l2norm_in_kernel=True)
    o1, S1 = atma_b200.chunk_gated_delta_rule(segments=1, **kw)
    o2, S2 = atma_b200.chunk_gated_delta_rule(segments=segments, **kw)
    assert max_rel(o2, o1) < 1e-2 and max_rel(S2, S1) < 1e-2
    o_ref, S_ref = oracle.chunk_gated_delta_rule_oracle(q, k, v, glog, beta, initial_state=S0)
    assert max_rel(o2, o_ref) < 2e-2 and max_rel(S2, S_ref) < 2e-2
    assert atma_b200.device_status() == 0            # no bounded wait of the tcgen05 scan kernels ran out
