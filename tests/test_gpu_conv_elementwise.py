"""GPU parity: depthwise causal convs, KV-cache scatter and the elementwise decode fusions."""

import pytest
import torch

import atma_b200
import oracle
from conftest import max_abs
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
def test_packed_conv_boundaries_and_states(kernel):
    lengths, channels = [1, 3, 7, 17, 40], 257
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
