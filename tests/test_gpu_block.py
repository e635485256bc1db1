"""GPU parity: one global block (BASELINE config 1's block at a small shape) composed from the
kernels reproduces the reference block's output on the reference's own weights (golden)."""

import pytest
import torch

from atma_b200.block import global_block_forward
from conftest import max_abs

pytestmark = pytest.mark.gpu


def test_global_block_matches_reference_fp32(golden):
    g = golden["block"]
    sd = {k: v.cuda() for k, v in g["state"].items()}
    assert sd["attn.mem.proj.weight"].abs().max() > 0 and sd["attn.v_null"].abs().max() > 0   # both branches visible
    y = global_block_forward(g["x"].cuda(), sd, head_dim=32, num_kv_heads=2)
    assert max_abs(y, g["y"]) < 1e-4


@pytest.mark.gpu
def test_host_fed_pipeline_matches_direct_calls():
    """Three steps through the three-stream pipeline (distinct inputs per step, result slots reused)
    give bit-identical results to the direct call on device-resident inputs."""
    from atma_b200.mixing import HostFedMixing, global_layer_mixing
    dev = torch.device("cuda", 0)
    B, T, H, Hkv, dk = 1, 1024, 8, 2, 128
    params = dict(v_null=torch.zeros(H, dk, device=dev), null_base=torch.full((H,), -2.0, device=dev),
                  null_slope_raw=torch.full((H,), -1.0, device=dev), len_gain_raw=torch.full((H,), -2.0, device=dev),
                  mag_beta_raw=torch.full((H,), 0.5, device=dev))
    n_keys = torch.arange(1, T + 1, dtype=torch.float32, device=dev)
    gen = torch.Generator().manual_seed(11)

    def inputs():
        t = {"q": torch.randn(B, T, H, dk, generator=gen).bfloat16(), "k": torch.randn(B, T, Hkv, dk, generator=gen).bfloat16(),
             "v": torch.randn(B, T, Hkv, dk, generator=gen).bfloat16(),
             "g": torch.nn.functional.logsigmoid(torch.randn(B, T, H, generator=gen) + 3.9),
             "beta": torch.sigmoid(torch.randn(B, T, H, generator=gen))}
        return {n: x.pin_memory() for n, x in t.items()}

    steps = [inputs() for _ in range(3)]
    pipe = HostFedMixing(dev)
    tickets, got = [], []
    for i, h in enumerate(steps):
        tickets.append(pipe.submit(h, n_keys, params))
        if i >= 1:                                   # read step i-1 while step i is in flight
            got.append([x.clone() for x in pipe.results(tickets[i - 1])])
    got.append([x.clone() for x in pipe.results(tickets[-1])])
    with pytest.raises(ValueError):
        pipe.results(tickets[0])                     # its slot has been reused by the third submit
    for h, g in zip(steps, got):
        d = {n: x.to(dev) for n, x in h.items()}
        want = global_layer_mixing(d["q"], d["k"], d["v"], d["g"], d["beta"], n_keys, params)
        for a, b in zip(g, want):
            assert torch.equal(a, b.cpu())


@pytest.mark.gpu
def test_packed_global_attention_prefill_matches_oracle_per_sequence():
    """The packed prefill of one global attention layer (fused q/k/v preparation, one packed Polar
    launch, one packed memory call, side stream) against the oracle run sequence by sequence in
    fp32: layer output, conv-state rows, memory-state rows and K/V cache rows."""
    import oracle
    import torch.nn.functional as F
    from atma_b200.layer import PackedMaps, global_attention_prefill_packed
    from conftest import max_rel
    D, H, Hkv, dk, K = 128, 4, 2, 128, 4
    lens, slots = [70, 200, 5], [2, 0, 3]
    total = sum(lens)
    g = torch.Generator().manual_seed(17)
    rn = lambda *s, std=1.0: torch.randn(*s, generator=g) * std
    sd = {"attn.q.weight": rn(H * 2 * dk, D, std=D ** -0.5), "attn.k.weight": rn(Hkv * dk, D, std=D ** -0.5),
          "attn.v.weight": rn(Hkv * dk, D, std=D ** -0.5), "attn.proj.weight": rn(D, H * dk, std=(H * dk) ** -0.5),
          "attn.mu_proj.weight": rn(D, H, std=0.5), "attn.canon_q.weight": rn(H * dk, 1, K, std=0.3),
          "attn.canon_k.weight": rn(Hkv * dk, 1, K, std=0.3), "attn.canon_v.weight": rn(Hkv * dk, 1, K, std=0.3),
          "attn.v_null": rn(H, dk, std=0.3), "attn.null_base": torch.full((H,), 1.0),
          "attn.null_slope_raw": torch.full((H,), 0.3), "attn.len_gain_raw": torch.full((H,), -1.0),
          "attn.mag_beta_raw": torch.full((H,), -0.5), "attn.mem.w_gamma.weight": rn(H, D, std=D ** -0.5),
          "attn.mem.w_beta.weight": rn(H, D, std=D ** -0.5), "attn.mem.gate.weight": rn(H * dk, D, std=D ** -0.5),
          "attn.mem.proj.weight": rn(D, H * dk, std=(H * dk) ** -0.5)}
    sd = {n: t.bfloat16().float() if t.ndim > 1 else t for n, t in sd.items()}        # weights exactly representable
    x = rn(total, D).bfloat16()
    rows = 4
    conv0 = [torch.zeros(rows, C, K - 1) for C in (H * dk, Hkv * dk, Hkv * dk)]
    mem0 = rn(rows, H, dk, dk, std=0.1)
    n_cache = total + 3
    sm = torch.randperm(n_cache, generator=g)[:total]

    # ---- oracle, fp32 ----
    xf = x.float()
    lin = lambda t, n: t @ sd[n + ".weight"].t()
    q_gate = lin(xf, "attn.q").view(total, H, 2 * dk)
    maps_cpu = PackedMaps(lens, slots, "cpu")
    conv_ref = [c.clone() for c in conv0]
    kc_ref, vc_ref = torch.zeros(n_cache, Hkv, dk), torch.zeros(n_cache, Hkv, dk)
    q_r, k_r, v_r = oracle.qkv_prep_prefill_oracle(q_gate, lin(xf, "attn.k").view(total, Hkv, dk), lin(xf, "attn.v").view(total, Hkv, dk),
                                                   *(sd[f"attn.canon_{n}.weight"].squeeze(1) for n in "qkv"), *conv_ref,
                                                   maps_cpu.token_seq_starts, maps_cpu.token_seq_ends, maps_cpu.token_seq_slots,
                                                   kc_ref, vc_ref, sm)
    params = {n: sd["attn." + n] for n in ("v_null", "null_base", "null_slope_raw", "len_gain_raw", "mag_beta_raw")}
    mem_ref = mem0.clone()
    out_ref = torch.zeros(total, D)
    pos = 0
    for n, slot in zip(lens, slots):
        sl = slice(pos, pos + n)
        tr = lambda t: t[sl].transpose(0, 1).unsqueeze(0)
        c, mag = oracle.polar_prefill_oracle(tr(q_r), tr(k_r), tr(v_r), torch.arange(1, n + 1, dtype=torch.float32), params)
        content = lin(c[0].transpose(0, 1).reshape(n, H * dk) * torch.sigmoid(q_gate[sl, :, dk:].reshape(n, H * dk)), "attn.proj")
        count = lin(mag[0].transpose(0, 1), "attn.mu_proj")
        glog = F.logsigmoid(lin(xf[sl], "attn.mem.w_gamma") + 3.9)
        beta = torch.sigmoid(lin(xf[sl], "attn.mem.w_beta"))
        r, S = oracle.chunk_gated_delta_rule_oracle(q_r[sl][None], k_r[sl][None], v_r[sl][None], glog[None], beta[None],
                                                    initial_state=mem_ref[slot][None])
        mem_ref[slot] = S[0]
        r = F.rms_norm(r[0], (dk,)).reshape(n, H * dk)
        out_ref[sl] = content + count + lin(r * torch.sigmoid(lin(xf[sl], "attn.mem.gate")), "attn.mem.proj")
        pos += n

    # ---- this library, bf16 ----
    dev = torch.device("cuda", 0)
    sd_g = {n: (t.bfloat16() if t.ndim > 1 else t).to(dev) for n, t in sd.items()}
    conv_g = [c.bfloat16().to(dev) for c in conv0]
    mem_g = mem0.to(dev)
    kc, vc = torch.zeros(n_cache, Hkv, dk, dtype=torch.bfloat16, device=dev), torch.zeros(n_cache, Hkv, dk, dtype=torch.bfloat16, device=dev)
    maps = PackedMaps(lens, slots, dev)
    out = global_attention_prefill_packed(x.to(dev), sd_g, maps, num_heads=H, num_kv_heads=Hkv, head_dim=dk,
                                          conv_states=conv_g, mem_state_table=mem_g, k_cache=kc, v_cache=vc,
                                          slot_mapping=sm.to(dev))
    torch.cuda.synchronize()
    assert max_rel(out, out_ref) < 2e-2
    assert max_rel(mem_g, mem_ref) < 2e-2
    assert torch.equal(mem_g[1].cpu(), mem0[1])                       # a row no sequence owns
    for a, b in zip(conv_g, conv_ref):
        assert max_rel(a, b) < 2e-2
    assert max_rel(kc, kc_ref) < 2e-2 and max_rel(vc, vc_ref) < 2e-2


@pytest.mark.gpu
def test_mixing_steps_issued_back_to_back_with_an_inputs_ready_event():
    """With ``inputs_ready`` the memory branch of a step may run under the previous step's attention
    kernel; four steps on different inputs must still give exactly the results of isolated calls."""
    from atma_b200.mixing import global_layer_mixing
    dev = torch.device("cuda", 0)
    B, T, H, Hkv, dk = 1, 2048, 8, 2, 128
    params = dict(v_null=torch.zeros(H, dk, device=dev), null_base=torch.full((H,), -2.0, device=dev),
                  null_slope_raw=torch.full((H,), -1.0, device=dev), len_gain_raw=torch.full((H,), -2.0, device=dev),
                  mag_beta_raw=torch.full((H,), 0.5, device=dev))
    n_keys = torch.arange(1, T + 1, dtype=torch.float32, device=dev)
    gen = torch.Generator(device=dev).manual_seed(5)
    steps = [dict(q=torch.randn(B, T, H, dk, device=dev, generator=gen).bfloat16(),
                  k=torch.randn(B, T, Hkv, dk, device=dev, generator=gen).bfloat16(),
                  v=torch.randn(B, T, Hkv, dk, device=dev, generator=gen).bfloat16(),
                  g=torch.nn.functional.logsigmoid(torch.randn(B, T, H, device=dev, generator=gen) + 3.9),
                  beta=torch.sigmoid(torch.randn(B, T, H, device=dev, generator=gen))) for _ in range(4)]
    want = [global_layer_mixing(s["q"], s["k"], s["v"], s["g"], s["beta"], n_keys, params) for s in steps]
    torch.cuda.synchronize()
    ready = torch.cuda.Event()
    ready.record()
    got = [global_layer_mixing(s["q"], s["k"], s["v"], s["g"], s["beta"], n_keys, params, inputs_ready=ready) for s in steps]
    torch.cuda.synchronize()
    for a, b in zip(got, want):
        for x, y in zip(a, b):
            assert torch.equal(x, y)
