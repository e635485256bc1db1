"""GPU parity: paged Polar decode (through the C ABI) against the CPU oracle."""

import pytest
import torch

import atma_b200
import oracle
from conftest import max_abs, max_rel
from gpu_util import polar_params, rand

pytestmark = pytest.mark.gpu


def make_paged(B, Hkv, dk, block_size, lens, dtype, seed, extra_blocks=3):
    """Random K/V per sequence laid out in a paged cache through a random page permutation."""
    max_blocks = max(1, max((n + block_size - 1) // block_size for n in lens))
    need = sum((n + block_size - 1) // block_size for n in lens)
    num_blocks = need + extra_blocks
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(num_blocks, generator=g)
    k_cache = torch.randn(num_blocks, block_size, Hkv, dk, generator=g).to(dtype)   # stale data in unused rows
    v_cache = torch.randn(num_blocks, block_size, Hkv, dk, generator=g).to(dtype)
    bt = torch.full((B, max_blocks), -1, dtype=torch.int32)
    used = 0
    for b, n in enumerate(lens):
        nb = (n + block_size - 1) // block_size
        bt[b, :nb] = perm[used:used + nb].int()
        used += nb
    return k_cache, v_cache, bt, torch.tensor(lens, dtype=torch.int32)


def run_decode(B, H, Hkv, dk, block_size, lens, dtype, seed, window=None, num_splits=None):
    k_cache, v_cache, bt, cl = make_paged(B, Hkv, dk, block_size, lens, dtype, seed)
    q = rand((B, H, dk), seed + 5, dtype)
    pc, pg = polar_params(H, dk, seed)
    c_ref, m_ref = oracle.polar_decode_oracle(q, k_cache, v_cache, bt, cl, pc, window=window)
    c, m = atma_b200.polar_attention_decode(q.cuda(), k_cache.cuda(), v_cache.cuda(), bt.cuda(), cl.cuda(),
                                            window=window, num_splits=num_splits, **pg)
    assert c.shape == (B, H, dk) and m.shape == (B, H) and c.dtype == dtype
    if dtype == torch.float32:
        assert max_abs(c, c_ref) < 1e-4 and max_abs(m, m_ref) < 1e-4
    else:
        assert max_rel(c, c_ref) < 2e-2 and max_abs(m, m_ref) < 2e-2
    return c, m


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_ragged_batch(dtype):
    run_decode(5, 8, 2, 128, 16, [1, 15, 16, 17, 200], dtype, seed=1)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dk,H,Hkv", [(64, 4, 2), (128, 8, 8), (128, 4, 1), (32, 2, 1), (128, 16, 2)])
def test_head_layouts(dtype, dk, H, Hkv):
    run_decode(3, H, Hkv, dk, 32, [40, 129, 77], dtype, seed=dk + H)


@pytest.mark.parametrize("window", [4, 64])
def test_window(window):
    run_decode(4, 8, 2, 128, 16, [3, 64, 65, 300], torch.float32, seed=2, window=window)
    run_decode(4, 8, 2, 128, 16, [3, 64, 65, 300], torch.bfloat16, seed=2, window=window)


def test_empty_and_padded_rows():
    """context_len 0 (a padded CUDA-graph row): everything drains to the null sink; the
    -1 page ids of unused table entries are never dereferenced."""
    c, m = run_decode(3, 4, 2, 128, 16, [0, 5, 0], torch.float32, seed=3)
    assert float(m[0].abs().max()) < 1e-6


@pytest.mark.parametrize("splits", [1, 2, 7, 32])
def test_split_count_does_not_change_the_result(splits):
    c1, m1 = run_decode(2, 8, 2, 128, 256, [2048, 777], torch.bfloat16, seed=4, num_splits=1)
    c2, m2 = run_decode(2, 8, 2, 128, 256, [2048, 777], torch.bfloat16, seed=4, num_splits=splits)
    assert max_abs(c1, c2) < 4e-3 and max_abs(m1, m2) < 4e-3


def test_decode_equals_last_prefill_row():
    """Engine invariant: decoding token T over a cache holding the prompt == row T-1 of prefill."""
    B, H, Hkv, T, dk, bs = 2, 8, 2, 700, 128, 256
    q = rand((B, H, T, dk), 31, torch.bfloat16).cuda()
    k = rand((B, Hkv, T, dk), 32, torch.bfloat16).cuda()
    v = rand((B, Hkv, T, dk), 33, torch.bfloat16).cuda()
    _, pg = polar_params(H, dk, 31)
    n = torch.arange(1, T + 1, dtype=torch.float32).cuda()
    c_pre, m_pre = atma_b200.polar_attention_fwd(q, k, v, n, **pg)
    nb = (T + bs - 1) // bs
    k_cache = torch.zeros(B * nb, bs, Hkv, dk, dtype=torch.bfloat16, device="cuda")
    v_cache = torch.zeros_like(k_cache)
    slots = torch.arange(B * nb * bs, device="cuda", dtype=torch.int32).view(B, nb * bs)[:, :T].reshape(-1)
    atma_b200.store_kvcache(k.transpose(1, 2).reshape(B * T, Hkv, dk), v.transpose(1, 2).reshape(B * T, Hkv, dk),
                            k_cache, v_cache, slots)
    bt = torch.arange(B * nb, device="cuda", dtype=torch.int32).view(B, nb)
    cl = torch.full((B,), T, device="cuda", dtype=torch.int32)
    c, m = atma_b200.polar_attention_decode(q[:, :, -1].contiguous(), k_cache, v_cache, bt, cl, **pg)
    assert max_rel(c, c_pre[:, :, -1]) < 2e-2 and max_abs(m, m_pre[:, :, -1]) < 2e-2


def test_cuda_graph_capture_and_replay():
    """The decode call has fixed launch shapes and reads lengths on the device, so it can be
    captured once and replayed with new lengths (inference/engine/model_runner.py:254-310)."""
    B, H, Hkv, dk, bs = 4, 8, 2, 128, 64
    lens = [100, 64, 1, 250]
    k_cache, v_cache, bt, cl = make_paged(B, Hkv, dk, bs, [256] * B, torch.bfloat16, 5)
    q = rand((B, H, dk), 6, torch.bfloat16).cuda()
    pc, pg = polar_params(H, dk, 5)
    kc, vc, btg = k_cache.cuda(), v_cache.cuda(), bt.cuda()
    clg = torch.tensor([256] * B, dtype=torch.int32, device="cuda")
    atma_b200.polar_attention_decode(q, kc, vc, btg, clg, **pg)          # warm scratch outside capture
    graph = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        with torch.cuda.graph(graph, stream=s):
            c, m = atma_b200.polar_attention_decode(q, kc, vc, btg, clg, **pg)
    clg.copy_(torch.tensor(lens, dtype=torch.int32))
    graph.replay()
    torch.cuda.synchronize()
    c_ref, m_ref = oracle.polar_decode_oracle(q.cpu(), k_cache, v_cache, bt, torch.tensor(lens, dtype=torch.int32), pc)
    assert max_rel(c, c_ref) < 2e-2 and max_abs(m, m_ref) < 2e-2


def test_decode_step_is_graph_capturable():
    """KV scatter + paged decode + memory step captured in a CUDA graph (fixed launch shapes, no host
    synchronisation, scratch at a stable address) and replayed: same results as the eager calls."""
    B, H, Hkv, dk, bs, ctx = 4, 8, 2, 128, 64, 512
    k_cache, v_cache, bt, cl = make_paged(B, Hkv, dk, bs, [ctx - 1] * B, torch.bfloat16, 7)
    kc, vc, btg, clg = k_cache.cuda(), v_cache.cuda(), bt.cuda(), (cl + 1).cuda()
    g = torch.Generator().manual_seed(2)
    q = torch.randn(B, H, dk, generator=g).bfloat16().cuda()
    kn, vn = torch.randn(B, Hkv, dk, generator=g).bfloat16().cuda(), torch.randn(B, Hkv, dk, generator=g).bfloat16().cuda()
    slot_map = torch.tensor([int(bt[b, (ctx - 1) // bs]) * bs + (ctx - 1) % bs for b in range(B)], dtype=torch.int32).cuda()
    params = dict(v_null=torch.zeros(H, dk).cuda(), null_base=torch.full((H,), -2.0).cuda(), null_slope_raw=torch.full((H,), -1.0).cuda(),
                  len_gain_raw=torch.full((H,), -2.0).cuda(), mag_beta_raw=torch.full((H,), 0.5).cuda())
    state0 = (torch.randn(B, H, dk, dk, generator=g) * 0.1).cuda()
    gamma, beta, slots = torch.rand(B, H, generator=g).cuda(), torch.rand(B, H, generator=g).cuda(), torch.arange(B).cuda()

    def step(state):
        atma_b200.store_kvcache(kn, vn, kc, vc, slot_map)
        c, mag = atma_b200.polar_attention_decode(q, kc, vc, btg, clg, **params)
        r = atma_b200.gated_delta_decode_step(q, kn.repeat_interleave(H // Hkv, 1), vn.repeat_interleave(H // Hkv, 1), gamma, beta, state, slots)
        return c, mag, r

    st_e = state0.clone()
    want = step(st_e)                                            # also warms the scratch cache up
    torch.cuda.synchronize()
    st_g = state0.clone()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        got = step(st_g)
    st_g.copy_(state0)
    graph.replay()
    torch.cuda.synchronize()
    for a, b in zip(got, want):
        assert torch.equal(a, b)
    assert torch.equal(st_g, st_e)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_partials_of_two_caches_merge_to_the_decode_of_the_whole_context(dtype):
    """A context whose keys lie in two caches (as after a context-parallel prefill): the key-range pass over each
    cache with the whole length setting the temperature, then one merge of all partials == decode over one cache
    that holds every key, and == the oracle."""
    from atma_b200.polar import _params, polar_decode_merge, polar_decode_partials
    B, H, Hkv, dk, bs = 3, 8, 2, 128, 16
    lens = [300, 17, 129]
    k_cache, v_cache, bt, cl = make_paged(B, Hkv, dk, bs, lens, dtype, seed=9)
    q = rand((B, H, dk), 3, dtype)
    pc, pg = polar_params(H, dk, 4)
    c_ref, m_ref = oracle.polar_decode_oracle(q, k_cache, v_cache, bt, cl, pc)
    # cache A holds the first `cut` keys of every sequence, cache B the rest (own pages, own tables)
    cuts = [160, 16, 1]
    parts = []
    for lo_hi in (lambda n, c: (0, min(c, n)), lambda n, c: (min(c, n), n)):
        kc, vc = torch.zeros_like(k_cache), torch.zeros_like(v_cache)
        local = []
        for b, n in enumerate(lens):
            lo, hi = lo_hi(n, cuts[b])
            pages = bt[b, :(n + bs - 1) // bs].long()
            rows_k = k_cache[pages].reshape(-1, Hkv, dk)[lo:hi]
            rows_v = v_cache[pages].reshape(-1, Hkv, dk)[lo:hi]
            dst = (pages[:, None] * bs + torch.arange(bs)[None, :]).reshape(-1)[:hi - lo]
            kc.view(-1, Hkv, dk)[dst] = rows_k
            vc.view(-1, Hkv, dk)[dst] = rows_v
            local.append(hi - lo)
        prepared = _params(device=torch.device("cuda"), **pg)
        parts.append(polar_decode_partials(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), torch.tensor(local).cuda(), cl.cuda(),
                                           prepared, num_splits=3))
    stats = torch.cat([p[0] for p in parts], dim=2)
    sums = torch.cat([p[1] for p in parts], dim=2)
    c, m = polar_decode_merge(stats, sums, cl.cuda(), prepared, dtype)
    if dtype == torch.float32:
        assert max_abs(c, c_ref) < 1e-4 and max_abs(m, m_ref) < 1e-4
    else:
        assert max_rel(c, c_ref) < 2e-2 and max_abs(m, m_ref) < 2e-2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("ctx", [[1, 70, 513, 64], [300, 2, 129, 1000]])
def test_decode_that_stores_the_new_token_itself_equals_scatter_then_decode(dtype, ctx):
    """``append=``: the decode call stores the new token's K/V rows before it reads the cache (16-bit: inside the
    key-range kernel; fp32: by the separate scatter): cache contents and outputs equal store_kvcache + decode."""
    g = torch.Generator().manual_seed(sum(ctx))
    B, H, Hkv, dk, bs = len(ctx), 8, 2, 128, 64
    per = (max(ctx) + bs - 1) // bs
    nblk = B * per + 2
    kc = torch.randn(nblk, bs, Hkv, dk, generator=g).to(dtype).cuda()
    vc = torch.randn(nblk, bs, Hkv, dk, generator=g).to(dtype).cuda()
    bt = torch.randperm(nblk, generator=g)[:B * per].view(B, per).int().cuda()
    cl = torch.tensor(ctx, dtype=torch.int32).cuda()
    q = torch.randn(B, H, dk, generator=g).to(dtype).cuda()
    kn = torch.randn(B, Hkv, dk, generator=g).to(dtype).cuda()
    vn = torch.randn(B, Hkv, dk, generator=g).to(dtype).cuda()
    last = cl.long() - 1
    sm = (bt.long()[torch.arange(B), last // bs] * bs + last % bs).int()
    _, P = polar_params(H, dk, 4)
    kc1, vc1 = kc.clone(), vc.clone()
    atma_b200.store_kvcache(kn, vn, kc1, vc1, sm)
    c1, m1 = atma_b200.polar_attention_decode(q, kc1, vc1, bt, cl, **P)
    kc2, vc2 = kc.clone(), vc.clone()
    c2, m2 = atma_b200.polar_attention_decode(q, kc2, vc2, bt, cl, append=(kn, vn, sm), **P)
    assert torch.equal(kc1, kc2) and torch.equal(vc1, vc2)
    assert torch.equal(c1, c2) and torch.equal(m1, m2)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_side_work_runs_between_the_key_range_and_merge_launches(dtype):
    """``beside=``: the callable's work goes to a side stream after the key-range kernel and is joined before the
    call returns; c, mag equal the plain call (also with ``append`` and ``gate``), the callable's result comes back,
    and what it wrote is complete once the current stream is synchronised."""
    g = torch.Generator().manual_seed(11)
    ctx = [300, 2, 129, 1000]
    B, H, Hkv, dk, bs = len(ctx), 8, 2, 128, 64
    per = (max(ctx) + bs - 1) // bs
    nblk = B * per + 2
    kc = torch.randn(nblk, bs, Hkv, dk, generator=g).to(dtype).cuda()
    vc = torch.randn(nblk, bs, Hkv, dk, generator=g).to(dtype).cuda()
    bt = torch.randperm(nblk, generator=g)[:B * per].view(B, per).int().cuda()
    cl = torch.tensor(ctx, dtype=torch.int32).cuda()
    q = torch.randn(B, H, dk, generator=g).to(dtype).cuda()
    kn = torch.randn(B, Hkv, dk, generator=g).to(dtype).cuda()
    vn = torch.randn(B, Hkv, dk, generator=g).to(dtype).cuda()
    gate = torch.randn(B, H, dk, generator=g).to(dtype).cuda()
    last = cl.long() - 1
    sm = (bt.long()[torch.arange(B), last // bs] * bs + last % bs).int()
    _, P = polar_params(H, dk, 4)
    state = (torch.randn(B, H, dk, dk, generator=g) * 0.1).cuda()
    gamma, beta = torch.rand(B, H, generator=g).cuda(), torch.rand(B, H, generator=g).cuda()
    slots = torch.arange(B).cuda()
    kc1, vc1, st1 = kc.clone(), vc.clone(), state.clone()
    c1, m1 = atma_b200.polar_attention_decode(q, kc1, vc1, bt, cl, append=(kn, vn, sm), gate=gate, **P)
    r1 = atma_b200.gated_delta_decode_step_fused(q, kn, vn, st1, slots, gamma=gamma, beta=beta)
    kc2, vc2, st2 = kc.clone(), vc.clone(), state.clone()
    c2, m2, r2 = atma_b200.polar_attention_decode(
        q, kc2, vc2, bt, cl, append=(kn, vn, sm), gate=gate,
        beside=lambda: atma_b200.gated_delta_decode_step_fused(q, kn, vn, st2, slots, gamma=gamma, beta=beta), **P)
    torch.cuda.current_stream().synchronize()
    assert torch.equal(c1, c2) and torch.equal(m1, m2) and torch.equal(kc1, kc2) and torch.equal(vc1, vc2)
    assert torch.equal(r1, r2) and torch.equal(st1, st2)
    assert atma_b200.device_status() == 0
