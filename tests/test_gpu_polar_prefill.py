"""GPU parity: Polar prefill (through the C ABI) against the CPU oracle and the golden vectors.

Tolerances: fp32 path atol 1e-4 (tests/verify.py:57 of the reference); 16-bit path max error
relative to the tensor's largest magnitude <= 2e-2 with fp32 accumulation."""

import pytest
import torch

import atma_b200
import oracle
from oracle.polar import polar_streaming_stats
from conftest import max_abs, max_rel
from gpu_util import polar_params, rand

pytestmark = pytest.mark.gpu
PKEYS = ("v_null", "null_base", "null_slope_raw", "len_gain_raw", "mag_beta_raw")
FP32_ATOL = 1e-4
BF16_REL = 2e-2


def run_case(B, H, Hkv, Tq, Tk, dk, dtype, seed, window=None, n_keys=None, transposed=False):
    q = rand((B, H, Tq, dk), seed, dtype)
    k = rand((B, Hkv, Tk, dk), seed + 1, dtype)
    v = rand((B, Hkv, Tk, dk), seed + 2, dtype)
    if n_keys is None:
        n_keys = torch.arange(1, Tq + 1, dtype=torch.float32) + (Tk - Tq)
    pc, pg = polar_params(H, dk, seed)
    c_ref, m_ref = oracle.polar_prefill_oracle(q, k, v, n_keys, pc, window=window)
    if transposed:   # (B,T,H,dk) storage viewed as (B,H,T,dk): the real call site's layout
        qg = q.transpose(1, 2).contiguous().cuda().transpose(1, 2)
        kg = k.transpose(1, 2).contiguous().cuda().transpose(1, 2)
        vg = v.transpose(1, 2).contiguous().cuda().transpose(1, 2)
    else:
        qg, kg, vg = q.cuda(), k.cuda(), v.cuda()
    c, m = atma_b200.polar_attention_fwd(qg, kg, vg, n_keys.cuda(), is_causal=(Tq == Tk), window=window, **pg)
    assert c.dtype == dtype and m.dtype == dtype and c.shape == (B, H, Tq, dk) and m.shape == (B, H, Tq)
    if dtype == torch.float32:
        assert max_abs(c, c_ref) < FP32_ATOL and max_abs(m, m_ref) < FP32_ATOL
    else:
        assert max_rel(c, c_ref) < BF16_REL and max_abs(m, m_ref) < BF16_REL
    cf = c.float()
    assert cf.norm(dim=-1).max() <= 1.0 + (1e-4 if dtype == torch.float32 else 1e-2)
    assert m.float().min() >= 0 and m.float().max() <= 1.0
    return c, m


@pytest.mark.parametrize("name", ["polar_causal_small", "polar_causal_dk128", "polar_window",
                                  "polar_offset_prefill", "polar_padding_queries", "polar_causal_bf16"])
def test_golden(golden, name):
    g = golden[name]
    window = None if int(g["window"]) < 0 else int(g["window"])
    params = {k: g[k].cuda() for k in PKEYS}
    Tq, Tk = g["q"].shape[2], g["k"].shape[2]
    c, m = atma_b200.polar_attention_fwd(g["q"].cuda(), g["k"].cuda(), g["v"].cuda(), g["n_keys"].cuda(),
                                         is_causal=(Tq == Tk), window=window, **params)
    if g["q"].dtype == torch.float32:
        assert max_abs(c, g["c"]) < FP32_ATOL and max_abs(m, g["mag"]) < FP32_ATOL
    else:
        assert max_rel(c, g["c"]) < BF16_REL and max_abs(m, g["mag"]) < BF16_REL


# shapes of the reference's own forward parity loop (kernel/test_polar_kernel.py:51-73)
@pytest.mark.parametrize("B,H,T,dk", [(1, 1, 16, 64), (2, 4, 128, 64), (2, 8, 200, 128),
                                      (1, 2, 512, 128), (3, 4, 65, 128), (2, 3, 1000, 128)])
def test_fp32_reference_shapes(B, H, T, dk):
    run_case(B, H, H, T, T, dk, torch.float32, seed=B * 100 + T)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,H,Hkv,T,dk", [(1, 8, 2, 384, 128), (2, 4, 1, 200, 128), (1, 4, 4, 129, 128),
                                          (2, 2, 2, 96, 64)])
def test_16bit_shapes(dtype, B, H, Hkv, T, dk):
    run_case(B, H, Hkv, T, T, dk, dtype, seed=T)


# edge shapes: T=1, T smaller than a tile, odd T (kernel/test_polar_kernel.py:120-123)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,H,T,dk", [(1, 4, 8, 128), (2, 2, 1, 128), (1, 4, 17, 64), (3, 2, 33, 128), (1, 8, 127, 128),
                                      (1, 8, 257, 128)])
def test_edge_shapes(dtype, B, H, T, dk):
    run_case(B, H, max(1, H // 2), T, T, dk, dtype, seed=7 * T)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [4, 64, 300])
def test_window(dtype, window):
    run_case(1, 4, 2, 333, 333, 128, dtype, seed=window, window=window)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_offset_prefill_and_padding_queries(dtype):
    # continuation chunk: 70 new queries over 70 + 186 cached keys (inference/models/atma.py:514-538)
    run_case(1, 8, 2, 70, 256, 128, dtype, seed=3)
    # n_keys = 0 rows drain to the null sink (kernel/test_polar_kernel.py:144-158)
    run_case(2, 3, 3, 4, 16, 128, dtype, seed=4, n_keys=torch.tensor([5., 0., 12., 0.]))
    # arbitrary, non-monotone counts
    run_case(1, 4, 2, 150, 200, 128, dtype, seed=5,
             n_keys=torch.randint(0, 201, (150,), generator=torch.Generator().manual_seed(9)).float())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_transposed_views_and_gqa_equivalence(dtype):
    c1, m1 = run_case(2, 8, 2, 160, 160, 128, dtype, seed=11, transposed=True)
    # expanded K/V (what the reference's caller passes) gives the same result as un-expanded
    q = rand((2, 8, 160, 128), 11, dtype).cuda()
    k = rand((2, 2, 160, 128), 12, dtype).cuda().repeat_interleave(4, dim=1)
    v = rand((2, 2, 160, 128), 13, dtype).cuda().repeat_interleave(4, dim=1)
    _, pg = polar_params(8, 128, 11)
    n = torch.arange(1, 161, dtype=torch.float32).cuda()
    c2, m2 = atma_b200.polar_attention_fwd(q, k, v, n, **pg)
    assert torch.equal(c1, c2) and torch.equal(m1, m2)


def test_default_init_params_and_is_causal_guard():
    pc, pg = polar_params(8, 128, random=False)
    q, k, v = rand((1, 8, 300, 128), 1, torch.bfloat16), rand((1, 2, 300, 128), 2, torch.bfloat16), rand((1, 2, 300, 128), 3, torch.bfloat16)
    n = torch.arange(1, 301, dtype=torch.float32)
    c_ref, m_ref = oracle.polar_prefill_oracle(q, k, v, n, pc)
    c, m = atma_b200.polar_attention_fwd(q.cuda(), k.cuda(), v.cuda(), n.cuda(), **pg)
    assert max_rel(c, c_ref) < BF16_REL and max_abs(m, m_ref) < BF16_REL
    with pytest.raises(ValueError):
        atma_b200.polar_attention_fwd(q.cuda()[:, :, :10], k.cuda(), v.cuda(), n.cuda()[:10], is_causal=True, **pg)
    with pytest.raises(ValueError):
        atma_b200.polar_attention_fwd(q.cuda()[..., :96], k.cuda()[..., :96], v.cuda()[..., :96], n.cuda(), **pg)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_statistics_carry_across_key_blocks(dtype):
    """A ring pass: keys arrive in blocks with absolute offsets, statistics carried between
    calls, null sink folded after the last block == one call over all keys."""
    B, H, Hkv, Tq, Tk, dk = 1, 8, 2, 192, 448, 128
    q, k, v = rand((B, H, Tq, dk), 21, dtype), rand((B, Hkv, Tk, dk), 22, dtype), rand((B, Hkv, Tk, dk), 23, dtype)
    n = torch.arange(1, Tq + 1, dtype=torch.float32) + (Tk - Tq)
    pc, pg = polar_params(H, dk, 21)
    from atma_b200.polar import _params
    params = _params(device="cuda", **pg)
    c_full, m_full = atma_b200.polar_prefill_raw(q.cuda(), k.cuda(), v.cuda(), n.cuda(), params)
    stats, bounds = None, [0, 128, 320, 448]
    for i in range(3):
        lo, hi = bounds[i], bounds[i + 1]
        last = i == 2
        out = atma_b200.polar_prefill_raw(q.cuda(), k[:, :, lo:hi].cuda(), v[:, :, lo:hi].cuda(), n.cuda(), params,
                                          key_offset=lo, stats_in=stats, finalize=last)
        stats = None if last else out
        if i == 0:     # carried statistics match the oracle's running statistics
            ref = polar_streaming_stats(q, k[:, :, lo:hi], v[:, :, lo:hi], n, len_gain_raw=pc["len_gain_raw"], tile=64)
            lse_ref = ref[0] + torch.log(ref[1].clamp_min(1e-30))
            lse = out[0].cpu() + torch.log(out[1].cpu().clamp_min(1e-30))
            seen = ref[1] > 0
            assert max_abs(lse[seen], lse_ref[seen]) < (1e-3 if dtype == torch.float32 else 5e-2)
    c, m = out
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert max_abs(c, c_full) < tol and max_abs(m, m_full) < tol


# tests/test_decode_kernels.py:69-111 of the reference: packed == per-sequence, lengths 33/65/129
@pytest.mark.parametrize("window", [None, 64])
@pytest.mark.parametrize("hkv", [2, 1])
def test_packed_matches_per_sequence(window, hkv):
    lengths, heads, dim = [33, 65, 129, 300], 2, 128
    total = sum(lengths)
    q = rand((total, heads, dim), 6, torch.bfloat16).cuda()
    k, v = rand((total, hkv, dim), 7, torch.bfloat16).cuda(), rand((total, hkv, dim), 8, torch.bfloat16).cuda()
    _, pg = polar_params(heads, dim, 6)
    seq_starts, query_starts, seq_lens, start = [], [], [], 0
    for length in lengths:
        for qs in range(0, length, 128):
            seq_starts.append(start); query_starts.append(qs); seq_lens.append(length)
        start += length
    tile_map = [torch.tensor(x, device="cuda", dtype=torch.int32) for x in (seq_starts, query_starts, seq_lens)]
    c, m = atma_b200.polar_attention_packed_fwd(q, k, v, *tile_map, window=window, **pg)
    start = 0
    for length in lengths:
        sl = slice(start, start + length)
        n = torch.arange(1, length + 1, device="cuda", dtype=torch.float32)
        ce, me = atma_b200.polar_attention_fwd(q[sl].transpose(0, 1)[None], k[sl].transpose(0, 1)[None],
                                               v[sl].transpose(0, 1)[None], n, window=window, **pg)
        torch.testing.assert_close(c[sl], ce[0].transpose(0, 1))
        torch.testing.assert_close(m[sl], me[0].transpose(0, 1))
        start += length
    with pytest.raises(ValueError):
        atma_b200.polar_attention_packed_fwd(q.float(), k.float(), v.float(), *tile_map, **pg)


def test_full_size_config_rows_against_oracle():
    """BASELINE config 2 (q [4,8192,8,128], k/v [4,8192,2,128], bf16, seed 1, default Polar
    parameters): the whole tensor is computed on the GPU; a sample of query rows is checked
    against the fp32 materialised oracle (rows are independent, so sampling rows is exact)."""
    torch.manual_seed(1)
    B, T, H, Hkv, dk = 4, 8192, 8, 2, 128
    q = torch.randn(B, T, H, dk).to(torch.bfloat16)
    k = torch.randn(B, T, Hkv, dk).to(torch.bfloat16)
    v = torch.randn(B, T, Hkv, dk).to(torch.bfloat16)
    pc, pg = polar_params(H, dk, random=False)
    n = torch.arange(1, T + 1, dtype=torch.float32)
    c, m = atma_b200.polar_attention_fwd(q.cuda().transpose(1, 2), k.cuda().transpose(1, 2),
                                         v.cuda().transpose(1, 2), n.cuda(), **pg)
    assert torch.isfinite(c.float()).all() and torch.isfinite(m.float()).all()
    rows = torch.cat([torch.tensor([0, 1, 127, 128, 129, 4095, 4096, T - 1]),
                      torch.randint(0, T, (40,), generator=torch.Generator().manual_seed(5))])
    for b in (0, B - 1):
        c_ref, m_ref = oracle.polar_prefill_oracle(q[b:b + 1, rows].transpose(1, 2), k[b:b + 1].transpose(1, 2),
                                                   v[b:b + 1].transpose(1, 2), n[rows], pc)
        assert max_rel(c[b:b + 1, :, rows], c_ref) < BF16_REL
        assert max_abs(m[b:b + 1, :, rows], m_ref) < BF16_REL
    # size-independent property: c is a unit vector wherever any mass exists, mag in [0, 1)
    norms = c.float().norm(dim=-1)
    assert norms.max() < 1.01 and norms.min() > 0.98


def test_tensor_core_path_is_taken_and_no_wait_ran_out():
    """16-bit dk=128 inputs must run on the tcgen05 kernel, and none of its bounded waits may
    have expired during this test session."""
    from ctypes import byref, c_int
    from atma_b200 import _lib
    lib = _lib.load()
    probe = _lib.PolarPrefillArgs()
    probe.dtype, probe.dk, probe.H, probe.Hkv, probe.finalize = 1, 128, 8, 2, 1
    assert lib.atma_polar_prefill_path(byref(probe)) == 1
    probe.dtype = 0
    assert lib.atma_polar_prefill_path(byref(probe)) == 0
    status = c_int(-1)
    _lib.check(lib.atma_device_status(byref(status)))
    assert status.value == 0
