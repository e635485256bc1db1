"""GPU parity: depthwise causal convs, KV-cache scatter and the elementwise decode fusions."""

import pytest
import torch
import torch.nn.functional as F

import atma_b200
import oracle
from conftest import max_abs, max_rel
from gpu_util import rand

pytestmark = pytest.mark.gpu


def test_conv_golden(golden):
    g = golden["conv"]
    x, w = g["x"].cuda(), g["w"].cuda()
    fresh, st = atma_b200.causal_conv1d_fn(x[:11].t()[None], w, None, return_final_states=True)
    assert max_abs(fresh[0].t(), g["fresh"]) < 1e-5 and torch.equal(st[0].cpu(), g["st_fresh"])
    cont, st2 = atma_b200.causal_conv1d_fn(x[11:].t()[None], w, None, return_final_states=True, initial_states=st)
    assert max_abs(cont[0].t(), g["cont"]) < 1e-5 and torch.equal(st2[0].cpu(), g["st_cont"])
    table = torch.zeros(3, w.shape[0], 3, device="cuda")
    table[1] = st2[0]
    step = atma_b200.causal_conv1d_decode_step(g["xs"].cuda(), w, g["slots"].cuda(), table)
    assert max_abs(step, g["step"]) < 1e-5 and torch.equal(table.cpu(), g["table_after_step"])
    g3 = golden["conv_k3_T1"]
    o, s3 = atma_b200.causal_conv1d_fn(g3["x"].cuda().t()[None], g3["w"].cuda(), None, return_final_states=True)
    assert max_abs(o[0].t(), g3["out"]) < 1e-6 and torch.equal(s3[0].cpu(), g3["st"])


# tests/test_decode_kernels.py:8-24 of the reference
@pytest.mark.parametrize("kernel", [3, 4])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_conv_decode_step(kernel, dtype):
    batch, channels = 7, 256
    g = torch.Generator().manual_seed(3)
    slots = torch.randperm(batch + 3, generator=g)[:batch]
    x, weight = rand((batch, channels), 1, dtype), rand((channels, kernel), 2, dtype)
    state = rand((batch + 3, channels, kernel - 1), 3, dtype)
    expect_state = state.clone()
    expected = oracle.causal_conv1d_step(x, weight, slots, expect_state)
    sg = state.cuda()
    actual = atma_b200.causal_conv1d_decode_step(x.cuda(), weight.cuda(), slots.cuda(), sg)
    torch.testing.assert_close(actual.float().cpu(), expected, atol=0.04 if dtype == torch.bfloat16 else 1e-5, rtol=0.02)
    assert torch.equal(sg.cpu(), expect_state)


# tests/test_decode_kernels.py:135-165 of the reference: lengths 1/3/7/17, 257 channels
@pytest.mark.parametrize("kernel", [3, 4])
@pytest.mark.parametrize("channels", [257, 256])          # the scalar kernel; the 16-byte vector kernel
def test_packed_conv_boundaries_and_states(kernel, channels):
    lengths = [1, 3, 7, 17, 40]
    total = sum(lengths)
    x, weight = rand((total, channels), 8, torch.bfloat16), rand((channels, kernel), 9, torch.bfloat16)
    starts, ends, slots, p = [], [], [], 0
    for slot, length in enumerate(lengths):
        starts += [p] * length; ends += [p + length] * length; slots += [slot] * length; p += length
    exp_state = torch.zeros(len(lengths), channels, kernel - 1, dtype=torch.bfloat16)
    expected = oracle.packed_causal_conv1d_oracle(x, weight, exp_state, starts, ends, slots)
    maps = [torch.tensor(t, device="cuda", dtype=torch.int32) for t in (starts, ends, slots)]
    state = torch.zeros(len(lengths), channels, kernel - 1, device="cuda", dtype=torch.bfloat16)
    actual = atma_b200.packed_causal_conv1d(x.cuda(), weight.cuda(), state, *maps)
    torch.testing.assert_close(actual.float().cpu(), expected, atol=0.04, rtol=0.02)
    assert torch.equal(state.cpu(), exp_state)
    with pytest.raises(ValueError):
        atma_b200.packed_causal_conv1d(x.cuda(), rand((channels, 5), 1, torch.bfloat16).cuda(), state, *maps)


def test_prefill_then_decode_conv_is_one_stream():
    """Prefill of T tokens then one decode step == prefill of T+1 tokens (last row)."""
    C, K, T = 96, 4, 21
    x, w = rand((T + 1, C), 1).cuda(), rand((C, K), 2).cuda()
    full, _ = atma_b200.causal_conv1d_fn(x.t()[None], w, None, return_final_states=True)
    _, st = atma_b200.causal_conv1d_fn(x[:T].t()[None], w, None, return_final_states=True)
    step = atma_b200.causal_conv1d_decode_step(x[T:], w, torch.zeros(1, dtype=torch.long, device="cuda"), st.contiguous())
    assert max_abs(step[0], full[0, :, -1]) < 1e-5


def test_store_kvcache():
    N, Hkv, dk, slots_total = 9, 2, 128, 64
    key, value = rand((N, Hkv, dk), 1, torch.bfloat16), rand((N, Hkv, dk), 2, torch.bfloat16)
    mapping = torch.tensor([5, -1, 0, 63, 17, -1, 2, 3, 40], dtype=torch.int32)
    kc, vc = torch.zeros(4, 16, Hkv, dk, dtype=torch.bfloat16), torch.zeros(4, 16, Hkv, dk, dtype=torch.bfloat16)
    ek, ev = kc.clone(), vc.clone()
    oracle.store_kvcache_oracle(key, value, ek, ev, mapping)
    kg, vg = kc.cuda(), vc.cuda()
    # strided source rows (a slice of a wider projection output), as at the call site
    wide = torch.zeros(N, 3, Hkv, dk, dtype=torch.bfloat16, device="cuda")
    wide[:, 0], wide[:, 1] = key.cuda(), value.cuda()
    atma_b200.store_kvcache(wide[:, 0], wide[:, 1], kg, vg, mapping.cuda())
    assert torch.equal(kg.cpu(), ek) and torch.equal(vg.cpu(), ev)


# tests/test_decode_kernels.py:56-66 of the reference: exact against eager bf16 on the device
def test_elementwise_fusions_are_exact(golden):
    packed = rand((32, 1024), 5, torch.bfloat16).cuda()
    x, gate = packed.chunk(2, dim=-1)
    torch.testing.assert_close(atma_b200.squared_relu_gate(x, gate), gate * x.relu().square(), atol=0, rtol=0)
    logits = rand((32, 50304), 6, torch.bfloat16).cuda()
    expected = 15.0 * logits * (logits.square() + 225.0).rsqrt()
    got = atma_b200.softcap_logits(logits)
    torch.testing.assert_close(got, expected)
    assert (got != expected).float().mean() < 1e-3            # rsqrt may differ by an ulp on rare inputs
    g = golden["elementwise"]
    xx, gg = g["packed"].cuda().chunk(2, dim=-1)
    assert torch.equal(atma_b200.squared_relu_gate(xx, gg).cpu(), g["sq"])
    assert torch.equal(atma_b200.softcap_logits(g["logits"].cuda()).cpu(), oracle.softcap_logits_oracle(g["logits"]))
    assert max_abs(atma_b200.softcap_logits(g["logits32"].cuda()), g["capped32"]) < 2e-6
    x32 = rand((7, 100), 7).cuda()                           # fp32, odd width: scalar path
    torch.testing.assert_close(atma_b200.squared_relu_gate(x32, -x32), -x32 * x32.relu().square())


# tests/test_decode_kernels.py:114-132 of the reference
@pytest.mark.parametrize("gated,heads", [(False, 2), (True, 8)])
def test_linear_head_rms(gated, heads):
    rows, hidden, head_dim = 33, 1024, 128
    width = head_dim * (2 if gated else 1)
    x = rand((rows, hidden), 1, torch.bfloat16)
    weight = rand((heads * width, hidden), 2, torch.bfloat16)
    bias = rand((heads * width,), 3, torch.bfloat16)
    expected = oracle.linear_head_rms_oracle(x, weight, bias, num_heads=heads, head_dim=head_dim, gated=gated)
    actual = atma_b200.linear_head_rms(x.cuda(), weight.cuda(), bias.cuda(), num_heads=heads, head_dim=head_dim, gated=gated)
    torch.testing.assert_close(actual.float().cpu(), expected, atol=0.02, rtol=0.02)


# ---- fused q/k/v preparation of the packed prefill (RMSNorm + 3 residual convs + state rows + cache scatter) ----
def _prep_case(dtype, lens, H=4, Hkv=2, dk=128, K=4, seed=0, rows=6):
    g = torch.Generator().manual_seed(seed)
    total = sum(lens)
    q_gate = torch.randn(total, H, 2 * dk, generator=g).to(dtype)
    k = torch.randn(total, Hkv, dk, generator=g).to(dtype)
    v = torch.randn(total, Hkv, dk, generator=g).to(dtype)
    w = [(torch.randn(C, K, generator=g) * 0.3).to(dtype) for C in (H * dk, Hkv * dk, Hkv * dk)]
    states = [torch.randn(rows, C, K - 1, generator=g).to(dtype) for C in (H * dk, Hkv * dk, Hkv * dk)]
    slots = torch.randperm(rows, generator=g)[:len(lens)].tolist()
    slots[-1] = -1                                            # a sequence whose state is not kept
    starts, ends, sl = [], [], []
    pos = 0
    for n, s in zip(lens, slots):
        starts += [pos] * n; ends += [pos + n] * n; sl += [s] * n
        pos += n
    i32 = lambda x: torch.tensor(x, dtype=torch.int32)
    n_cache = total + 5
    k_cache = torch.randn(n_cache, Hkv, dk, generator=g).to(dtype)
    v_cache = torch.randn(n_cache, Hkv, dk, generator=g).to(dtype)
    slot_mapping = torch.randperm(n_cache, generator=g)[:total].to(torch.int64)
    slot_mapping[3] = -1
    return q_gate, k, v, w, states, i32(starts), i32(ends), i32(sl), k_cache, v_cache, slot_mapping


@pytest.mark.parametrize("dtype,tol,dk,lens", [(torch.bfloat16, 2e-2, 128, [2, 37, 1, 64, 29]),      # direct form, border runs
                                                (torch.bfloat16, 2e-2, 128, [300, 5, 1, 260, 70]),    # direct form, long runs
                                                (torch.float16, 4e-3, 128, [2, 37, 1, 64, 29]),
                                                (torch.bfloat16, 2e-2, 64, [2, 37, 1, 64, 29]),       # shared-memory tile form
                                                (torch.float32, 1e-4, 128, [2, 37, 1, 64, 29])])
@pytest.mark.parametrize("continued", [False, True])
def test_qkv_prep_prefill_matches_the_op_by_op_oracle(dtype, tol, dk, lens, continued):
    _check_prep_against_oracle(dtype, tol, dk, lens, continued)


@pytest.mark.parametrize("H,Hkv", [(3, 1), (5, 2), (1, 1)])
def test_qkv_prep_prefill_with_an_odd_number_of_head_rows(H, Hkv):
    """The direct form pairs head rows two to a warp; with H + 2 Hkv odd the last pair is half empty and
    with H odd a q head shares its warp with a k head.  Same check as above on those shapes."""
    _check_prep_against_oracle(torch.bfloat16, 2e-2, 128, [300, 5, 1, 260, 70], True, H=H, Hkv=Hkv)


def _check_prep_against_oracle(dtype, tol, dk, lens, continued, H=4, Hkv=2):
    """Ragged packed sequences (shorter than the kernel, crossing the 32-token tile, one without a
    state slot): the fused launch == rms_norm + x + conv(x) + state write + store_kvcache run op by
    op on the CPU; state rows and cache rows that nothing addresses stay as they were."""
    q_gate, k, v, w, states, s0, e0, sl, k_cache, v_cache, sm = _prep_case(dtype, lens, H=H, Hkv=Hkv, dk=dk, seed=3)
    init = [s.clone() for s in states] if continued else None
    ref_states = [s.clone() for s in states]
    ref_kc, ref_vc = k_cache.clone(), v_cache.clone()
    q_ref, k_ref, v_ref = oracle.qkv_prep_prefill_oracle(q_gate, k, v, *w, *ref_states, s0, e0, sl, ref_kc, ref_vc, sm,
                                                         initial_states=init)
    dev_states = [s.cuda() for s in states]
    kc, vc = k_cache.cuda(), v_cache.cuda()
    q_o, k_o, v_o = atma_b200.qkv_prep_prefill(q_gate.cuda(), k.cuda(), v.cuda(), *(x.cuda() for x in w), *dev_states,
                                               s0.cuda(), e0.cuda(), sl.cuda(), kc, vc, sm.cuda(),
                                               initial_states=None if init is None else [x.cuda() for x in init])
    err = max_rel if dtype != torch.float32 else max_abs
    for got, want in ((q_o, q_ref), (k_o, k_ref), (v_o, v_ref)):
        assert got.dtype == dtype and err(got, want) < tol
    for got, want, before in zip(dev_states, ref_states, states):
        assert err(got, want) < tol
        untouched = [r for r in range(before.shape[0]) if r not in sl.tolist()]
        assert torch.equal(got.cpu()[untouched], before[untouched])
    assert err(kc, ref_kc) < tol and err(vc, ref_vc) < tol
    unused = [r for r in range(k_cache.shape[0]) if r not in sm.tolist()]
    assert torch.equal(kc.cpu()[unused], k_cache[unused]) and torch.equal(vc.cpu()[unused], v_cache[unused])
    assert torch.equal(kc[sm[5]], k_o[5]) and torch.equal(vc[sm[5]], v_o[5])      # the cache holds the post-conv rows


def test_qkv_prep_prefill_equals_the_separate_kernels():
    """Against this library's own unfused calls (F.rms_norm, packed_causal_conv1d, store_kvcache) in bf16:
    same rounding points, so q, k, v and the cache rows agree to the last bit or one bf16 ulp."""
    import torch.nn.functional as F
    lens = [100, 31, 70]
    q_gate, k, v, w, states, s0, e0, sl, k_cache, v_cache, sm = _prep_case(torch.bfloat16, lens, seed=11)
    sl = torch.where(sl < 0, torch.zeros_like(sl) + 5, sl)
    dk = k.shape[-1]
    qg, kg, vg = q_gate.cuda(), k.cuda(), v.cuda()
    wg = [x.cuda() for x in w]
    st_f = [s.cuda() for s in states]
    kc, vc = k_cache.cuda(), v_cache.cuda()
    q_o, k_o, v_o = atma_b200.qkv_prep_prefill(qg, kg, vg, *wg, *st_f, s0.cuda(), e0.cuda(), sl.cuda(), kc, vc, sm.cuda())
    st_u = [s.cuda() for s in states]
    xs = [F.rms_norm(qg[..., :dk], (dk,)).reshape(len(qg), -1), F.rms_norm(kg, (dk,)).reshape(len(kg), -1),
          vg.reshape(len(vg), -1)]
    outs = [x + atma_b200.packed_causal_conv1d(x, wi, si, s0.cuda(), e0.cuda(), sl.cuda()) for x, wi, si in zip(xs, wg, st_u)]
    for got, want in zip((q_o, k_o, v_o), outs):
        assert max_rel(got.reshape(want.shape), want) < 8e-3
        assert (got.reshape(want.shape) != want).float().mean() < 0.02
    for a, b in zip(st_f, st_u):
        assert max_rel(a, b) < 8e-3


# ---- gate epilogues ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_sigmoid_gate_mul_reads_the_gate_half_in_place(dtype):
    """c * sigmoid(gate) with gate = the second half of the q|gate projection (a strided view) and c in
    the (H, tokens, dk) layout viewed as (tokens, H, dk): equals the eager expression on the CPU."""
    g = torch.Generator().manual_seed(8)
    tokens, H, dk = 77, 8, 128
    q_gate = torch.randn(tokens, H, 2 * dk, generator=g).to(dtype)
    c_ht = torch.randn(H, tokens, dk, generator=g).to(dtype)
    want = oracle.sigmoid_gate_mul_oracle(c_ht.transpose(0, 1), q_gate[..., dk:])
    got = atma_b200.sigmoid_gate_mul(c_ht.cuda().transpose(0, 1), q_gate.cuda()[..., dk:])
    assert got.shape == (tokens, H, dk) and got.is_contiguous()
    if dtype == torch.float32:
        assert max_abs(got, want) < 1e-5
    else:
        assert max_rel(got, want) < 8e-3 and (got.cpu() != want).float().mean() < 0.02


@pytest.mark.parametrize("dtype,dk", [(torch.bfloat16, 128), (torch.float16, 64), (torch.float32, 128), (torch.bfloat16, 32)])
def test_rms_sigmoid_gate_matches_eager(dtype, dk):
    g = torch.Generator().manual_seed(9)
    tokens, H = 203, 4
    r = (torch.randn(tokens, H, dk, generator=g) * 3).to(dtype)
    gate_wide = torch.randn(tokens, H * dk + 16, generator=g).to(dtype)
    gate = gate_wide[:, :H * dk]                                  # a row stride larger than the width
    want = oracle.rms_sigmoid_gate_oracle(r, gate)
    got = atma_b200.rms_sigmoid_gate(r.cuda(), gate_wide.cuda()[:, :H * dk])
    assert got.shape == (tokens, H * dk)
    if dtype == torch.float32:
        assert max_abs(got, want) < 1e-5
    else:
        assert max_rel(got, want) < 8e-3 and (got.cpu() != want).float().mean() < 0.03


# ---- gated short conv of the local layers (chunk, B*x', conv, C*conv in one pass) ------------------------------
@pytest.mark.parametrize("dtype,K", [(torch.bfloat16, 3), (torch.float16, 4), (torch.float32, 3), (torch.bfloat16, 2)])
def test_lfm2_conv_decode_step_matches_the_op_by_op_oracle(dtype, K):
    g = torch.Generator().manual_seed(K)
    B, D, rows = 5, 384, 9
    proj = torch.randn(B, 3 * D, generator=g).to(dtype)
    w = (torch.randn(D, K, generator=g) * 0.5).to(dtype)
    table = torch.randn(rows, D, K - 1, generator=g).to(dtype)
    slots = torch.tensor([4, 0, 7, 2, 8])
    ref_table = table.clone()
    want = oracle.lfm2_conv_step_oracle(proj, w, slots, ref_table)
    tg = table.cuda()
    got = atma_b200.lfm2_conv_decode_step(proj.cuda(), w.cuda(), slots.cuda(), tg)
    if dtype == torch.float32:
        assert max_abs(got, want) < 1e-5 and max_abs(tg, ref_table) < 1e-6
    else:
        assert max_rel(got, want) < 8e-3 and (got.cpu() != want).float().mean() < 0.03
        assert torch.equal(tg.cpu(), ref_table)                    # the state holds the rounded B*x' exactly
    untouched = [r for r in range(rows) if r not in slots.tolist()]
    assert torch.equal(tg.cpu()[untouched], table[untouched])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("continued", [False, True])
@pytest.mark.parametrize("D,K", [(256, 3), (100, 3), (256, 4)])   # 100 channels of bf16: the scalar kernel
def test_lfm2_conv_packed_matches_the_op_by_op_oracle(dtype, continued, D, K):
    g = torch.Generator().manual_seed(12)
    lens, slots, rows = [1, 40, 17, 2, 33], [3, 0, -1, 5, 1], 6
    total = sum(lens)
    proj = torch.randn(total, 3 * D, generator=g).to(dtype)
    w = (torch.randn(D, K, generator=g) * 0.5).to(dtype)
    table = torch.randn(rows, D, K - 1, generator=g).to(dtype)
    s0, e0, sl, pos = [], [], [], 0
    for n, s in zip(lens, slots):
        s0 += [pos] * n; e0 += [pos + n] * n; sl += [s] * n
        pos += n
    s0, e0, sl = (torch.tensor(x, dtype=torch.int32) for x in (s0, e0, sl))
    init = table.clone() if continued else None
    ref_table = table.clone()
    want = oracle.lfm2_conv_packed_oracle(proj, w, ref_table, s0, e0, sl, initial_state=init)
    tg = table.cuda()
    got = atma_b200.lfm2_conv_packed(proj.cuda(), w.cuda(), tg, s0.cuda(), e0.cuda(), sl.cuda(),
                                     initial_state=None if init is None else init.cuda())
    if dtype == torch.float32:
        assert max_abs(got, want) < 1e-5 and max_abs(tg, ref_table) < 1e-6
    else:
        assert max_rel(got, want) < 8e-3 and (got.cpu() != want).float().mean() < 0.03
        assert torch.equal(tg.cpu(), ref_table)
    assert torch.equal(tg.cpu()[[2, 4]], table[[2, 4]])             # rows no sequence owns


def test_empty_inputs_are_accepted_by_the_fused_entries():
    """Zero tokens / zero rows: every fused entry returns an empty result and touches nothing."""
    dev = "cuda"
    bf = torch.bfloat16
    z = lambda *s: torch.zeros(*s, dtype=bf, device=dev)
    i32 = torch.zeros(0, dtype=torch.int32, device=dev)
    st = [z(2, 512, 3), z(2, 256, 3), z(2, 256, 3)]
    q, k, v = atma_b200.qkv_prep_prefill(z(0, 4, 256), z(0, 2, 128), z(0, 2, 128), z(512, 4), z(256, 4), z(256, 4), *st, i32, i32, i32)
    assert q.shape == (0, 4, 128) and k.shape == (0, 2, 128) and v.shape == (0, 2, 128)
    assert atma_b200.sigmoid_gate_mul(z(0, 4, 128), z(0, 4, 128)).shape == (0, 4, 128)
    assert atma_b200.rms_sigmoid_gate(z(0, 4, 128), z(0, 512)).shape == (0, 512)
    assert atma_b200.lfm2_conv_decode_step(z(0, 768), z(256, 3), torch.zeros(0, dtype=torch.long, device=dev), z(2, 256, 2)).shape == (0, 256)
    assert atma_b200.lfm2_conv_packed(z(0, 768), z(256, 3), z(2, 256, 2), i32, i32, i32).shape == (0, 256)
    table = torch.ones(2, 4, 128, 128, device=dev)
    o = atma_b200.packed_gated_delta_prefill(z(0, 4, 128), z(0, 2, 128), z(0, 2, 128), torch.zeros(0, 4, device=dev),
                                             torch.zeros(0, 4, device=dev), torch.zeros(1, dtype=torch.int32), table,
                                             torch.zeros(0, dtype=torch.long))
    assert o.shape == (0, 4, 128) and bool((table == 1).all())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,N,K,gated,bias", [(1, 8192, 1024, True, True), (8, 8192, 1024, True, False), (16, 1024, 4096, False, True),
                                               (13, 3072, 1024, False, False), (5, 50304, 1024, False, False),
                                               (3, 48, 64, False, True), (9, 64, 96, True, True)])
def test_decode_linear_matches_the_separate_ops(dtype, B, N, K, gated, bias):
    """The weight-streaming linear for decode batches against F.linear (+ squared_relu_gate): same fp32 accumulation and
    rounding points, so nearly every element is identical and none is off by more than an ulp or two of the 16-bit type."""
    g = torch.Generator().manual_seed(N + K + B)
    x = torch.randn(B, K, generator=g).to(dtype).cuda()
    w = (torch.randn(N, K, generator=g) / K ** 0.5).to(dtype).cuda()
    b = (torch.randn(N, generator=g) * 0.1).to(dtype).cuda() if bias else None
    got = atma_b200.decode_linear(x, w, b, gated=gated)
    y32 = F.linear(x.float(), w.float(), None if b is None else b.float())
    want = F.linear(x, w, b)
    if gated:
        h = N // 2
        want = atma_b200.squared_relu_gate(want[:, :h], want[:, h:])
        y16 = y32.to(dtype).float()
        sq = torch.relu(y16[:, :h]) ** 2
        ref32 = y16[:, h:] * (sq.to(dtype).float() if dtype == torch.bfloat16 else sq)
    else:
        ref32 = y32
    assert got.shape == want.shape
    scale = float(ref32.abs().max())
    assert float((got.float() - ref32).abs().max()) < 2e-2 * scale
    assert float((got.float() - want.float()).abs().max()) < 2e-2 * scale
    assert float((got != want).float().mean()) < 0.05


def test_decode_linear_rejects_what_it_does_not_serve():
    x = torch.zeros(17, 64, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(32, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        atma_b200.decode_linear(x, w)                                     # more than 16 rows
    with pytest.raises(ValueError):
        atma_b200.decode_linear(x[:4, :48].contiguous(), w[:, :48].contiguous())   # K not a multiple of 32
    assert atma_b200.decode_linear(x[:0], w).shape == (0, 32)
    assert atma_b200.device_status() == 0
