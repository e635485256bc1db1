"""GPU parity at the sizes that are benchmarked (BASELINE configs 1-3 at their own shapes, the
64K-token prefill launch, the 64K-token scan and the 64 x 32K paged decode), against the fp32
CPU oracle and the golden vectors made from the reference.

Tolerances: fp32 path atol 1e-4; 16-bit path max error relative to the tensor's largest
magnitude <= 2e-2 (fp32 accumulation, fp32 recurrent state)."""

import os
import sys

import pytest
import torch
import torch.nn.functional as F

import atma_b200
import oracle
from atma_b200.block import global_block_forward
from conftest import max_abs, max_rel
from gpu_util import polar_params

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
import seeded_weights as sw  # noqa: E402

pytestmark = pytest.mark.gpu
BF16_REL = 2e-2


def _scan_gpu(q, k, v, g, beta):
    o, S = atma_b200.chunk_gated_delta_rule(q=q.cuda(), k=k.cuda(), v=v.cuda(), g=g.cuda(), beta=beta.cuda(), scale=1.0,
                                            initial_state=None, output_final_state=True, use_qk_l2norm_in_kernel=True)
    return o.cpu(), S.cpu()


# ---- BASELINE config 3: the gated-delta scan at B=8, T=16384, H=8, d=128, chunk 64, seed 2 ----------
def _config3_inputs(B, T, H, seed, decay):
    torch.manual_seed(seed)
    d = 128
    q = F.normalize(torch.randn(B, T, H, d), dim=-1).bfloat16()
    k = F.normalize(torch.randn(B, T, H, d), dim=-1).bfloat16()
    v = torch.randn(B, T, H, d).bfloat16()
    beta = torch.sigmoid(torch.randn(B, T, H))
    g = -F.softplus(torch.randn(B, T, H)) if decay == "config3" else F.logsigmoid(torch.randn(B, T, H) + 3.9)
    return q, k, v, g, beta


def test_config3_scan_full_size_against_oracle():
    """Every output row over the whole 16384-token horizon and the final fp32 state."""
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    q, k, v, g, beta = _config3_inputs(8, 16384, 8, seed=2, decay="config3")
    o, S = _scan_gpu(q, k, v, g, beta)
    assert torch.isfinite(o.float()).all() and torch.isfinite(S).all()
    for b in range(8):                                    # oracle one batch row at a time (memory)
        o_ref, S_ref = oracle.chunk_gated_delta_rule_oracle(q[b:b + 1], k[b:b + 1], v[b:b + 1], g[b:b + 1], beta[b:b + 1])
        assert max_rel(o[b:b + 1], o_ref) < BF16_REL, b
        assert max_rel(S[b:b + 1], S_ref) < BF16_REL, b
        # the error must not grow along the horizon: last 1024 tokens on their own scale
        assert max_rel(o[b:b + 1, -1024:], o_ref[:, -1024:]) < BF16_REL, b


@pytest.mark.parametrize("T", [16384, 65536])
def test_scan_long_horizon_at_the_models_decay(T):
    """The model initialises the decay at gamma ~ 0.98 (g = logsigmoid(N(0,1) + 3.9)), where an error
    in the carried state fades slowly; one batch row, 256 and 1024 chunks.  The 65,536-token case with
    2 KV heads is the benchmark's own scan launch."""
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    torch.manual_seed(20 + T // 16384)
    H, Hkv, d = 8, 2, 128
    q = torch.randn(1, T, H, d).bfloat16()
    k = torch.randn(1, T, Hkv, d).bfloat16()
    v = torch.randn(1, T, Hkv, d).bfloat16()
    g = F.logsigmoid(torch.randn(1, T, H) + 3.9)
    beta = torch.sigmoid(torch.randn(1, T, H))
    o, S = _scan_gpu(q, k, v, g, beta)
    o_ref, S_ref = oracle.chunk_gated_delta_rule_oracle(q, k, v, g, beta)
    assert max_rel(o, o_ref) < BF16_REL and max_rel(S, S_ref) < BF16_REL
    for a in range(0, T, T // 8):                          # every eighth of the horizon on its own scale
        assert max_rel(o[:, a:a + T // 8], o_ref[:, a:a + T // 8]) < BF16_REL, a


# ---- the benchmark's 64K-token Polar launch: sampled query rows -----------------------------------------
def test_polar_64k_launch_sampled_rows_against_oracle():
    torch.manual_seed(4)
    T, H, Hkv, dk = 65536, 8, 2, 128
    q = torch.randn(1, T, H, dk).bfloat16()
    k = torch.randn(1, T, Hkv, dk).bfloat16()
    v = torch.randn(1, T, Hkv, dk).bfloat16()
    pc, pg = polar_params(H, dk, random=False)
    n = torch.arange(1, T + 1, dtype=torch.float32)
    c, m = atma_b200.polar_attention_fwd(q.cuda().transpose(1, 2), k.cuda().transpose(1, 2), v.cuda().transpose(1, 2),
                                         n.cuda(), **pg)
    rows = torch.cat([torch.tensor([0, 127, 128, 32767, 32768, T - 129, T - 128, T - 1]),
                      torch.randint(0, T, (40,), generator=torch.Generator().manual_seed(6))])
    c_ref, m_ref = oracle.polar_prefill_oracle(q[:, rows].transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), n[rows], pc)
    assert max_rel(c[:, :, rows], c_ref) < BF16_REL
    assert max_abs(m[:, :, rows], m_ref) < BF16_REL
    norms = c.float().norm(dim=-1)
    assert norms.max() < 1.01 and norms.min() > 0.98 and torch.isfinite(m.float()).all()


# ---- the benchmark's decode launch: 64 sequences x 32,768 tokens of context, 256-token pages -----------
def test_decode_64x32k_launch_four_sequences_against_oracle():
    dev = torch.device("cuda", 0)
    B, ctx, H, Hkv, dk, bs = 64, 32768, 8, 2, 128, 256
    pages = ctx // bs
    gen = torch.Generator(device=dev).manual_seed(9)
    k_cache = torch.randn(B * pages, bs, Hkv, dk, device=dev, generator=gen, dtype=torch.float32).bfloat16()
    v_cache = torch.randn(B * pages, bs, Hkv, dk, device=dev, generator=gen, dtype=torch.float32).bfloat16()
    bt = torch.randperm(B * pages, generator=torch.Generator().manual_seed(3)).int().view(B, pages)
    lens = torch.full((B,), ctx, dtype=torch.int32)
    lens[1], lens[62] = ctx - 255, ctx - 4097                                  # ragged ends inside the batch
    q = torch.randn(B, H, dk, generator=torch.Generator().manual_seed(5)).bfloat16()
    pc, pg = polar_params(H, dk, random=False)
    c, m = atma_b200.polar_attention_decode(q.cuda(), k_cache, v_cache, bt.cuda(), lens.cuda(), **pg)
    for b in (0, 1, 62, 63):
        phys = bt[b].long()
        kc, vc = k_cache[phys.to(dev)].cpu(), v_cache[phys.to(dev)].cpu()      # this sequence's pages, in order
        c_ref, m_ref = oracle.polar_decode_oracle(q[b:b + 1], kc, vc, torch.arange(pages, dtype=torch.int32)[None],
                                                  lens[b:b + 1], pc)
        assert max_rel(c[b:b + 1], c_ref) < BF16_REL, b
        assert max_abs(m[b:b + 1], m_ref) < BF16_REL, b


# ---- BASELINE config 1 at its own shape: one global block, hidden 1024, 8/2 heads of 128, T=2048 -------
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, BF16_REL)])
def test_config1_block_full_shape_against_reference_rows(golden, dtype, tol):
    """Weights regenerated from their seed; the expected rows come from model/reference.py's Block
    itself (tests/golden/make_golden.py).  fp32 takes the fp32 kernels, bf16 the tcgen05 Polar kernel
    and the tensor-core scan."""
    g = golden["block_cfg1"]
    sd = sw.block_state(seed=int(g["weight_seed"]), dim=1024, head_dim=128, num_kv_heads=2)
    x = torch.randn(1, 2048, 1024, generator=torch.Generator().manual_seed(int(g["x_seed"])))
    polar = ("null_base", "null_slope_raw", "len_gain_raw", "mag_beta_raw", "v_null")
    sd_g = {n: (t if n.split(".")[-1] in polar else t.to(dtype)).cuda() for n, t in sd.items()}
    y = global_block_forward(x.to(dtype).cuda(), sd_g, head_dim=128, num_kv_heads=2)
    rows = g["rows"]
    if dtype == torch.float32:
        assert max_abs(y[0, rows], g["y_rows"]) < tol
    else:
        assert max_rel(y[0, rows], g["y_rows"]) < tol


def test_block_chunked_continuation_carries_the_memory_state(golden):
    """Two calls with the memory state handed over == one call, on the memory branch's own output:
    the state after the first 1024 tokens, used as initial_state for the second half, must reproduce
    the one-pass final state (same kernels: tight tolerance) - config 1's shape, bf16."""
    g = golden["block_cfg1"]
    sd = sw.block_state(seed=int(g["weight_seed"]), dim=1024, head_dim=128, num_kv_heads=2)
    gen = torch.Generator().manual_seed(77)
    T, H, Hkv, dk = 2048, 8, 2, 128
    q = torch.randn(1, T, H, dk, generator=gen).bfloat16().cuda()
    k = torch.randn(1, T, Hkv, dk, generator=gen).bfloat16().cuda()
    v = torch.randn(1, T, Hkv, dk, generator=gen).bfloat16().cuda()
    glog = F.logsigmoid(torch.randn(1, T, H, generator=gen) + 3.9).cuda()
    beta = torch.sigmoid(torch.randn(1, T, H, generator=gen)).cuda()
    kw = dict(scale=1.0, output_final_state=True, use_qk_l2norm_in_kernel=True)
    o_full, S_full = atma_b200.chunk_gated_delta_rule(q=q, k=k, v=v, g=glog, beta=beta, initial_state=None, **kw)
    o_a, S_a = atma_b200.chunk_gated_delta_rule(q=q[:, :1024], k=k[:, :1024], v=v[:, :1024], g=glog[:, :1024],
                                                beta=beta[:, :1024], initial_state=None, **kw)
    o_b, S_b = atma_b200.chunk_gated_delta_rule(q=q[:, 1024:], k=k[:, 1024:], v=v[:, 1024:], g=glog[:, 1024:],
                                                beta=beta[:, 1024:], initial_state=S_a, **kw)
    assert max_rel(torch.cat([o_a, o_b], 1), o_full) < 2e-3 and max_rel(S_b, S_full) < 2e-3
    assert sd["attn.mem.proj.weight"].abs().max() > 0


# ---- golden cases for the local layers' gated conv and the memory read-out ------------------------------
def test_lfm2_kernels_match_the_reference_module(golden):
    """Packed prefill kernel for the first 13 tokens, then the decode-step kernel token by token from
    the carried conv state, between cuBLAS projections == LFM2Conv.forward of the reference (fp32)."""
    from atma_b200.inference_ops import lfm2_conv_decode_step, lfm2_conv_packed
    g = golden["lfm2"]
    sd = {n: t.cuda() for n, t in sw.block_state(seed=int(g["weight_seed"]), dim=96, head_dim=32, num_kv_heads=1,
                                                 attention=False).items()}
    x = g["x"].cuda()
    B, T, D = x.shape
    T0 = 13
    lin = lambda t, n: F.linear(t, sd[n + ".weight"], sd[n + ".bias"])
    w = sd["attn.conv.weight"].squeeze(1).contiguous()
    proj = lin(x, "attn.in_proj")
    starts = (torch.arange(B, device="cuda").repeat_interleave(T0) * T0).int()
    slots = torch.tensor([2, 0], device="cuda")
    table = torch.zeros(B + 1, D, 2, device="cuda")
    y_pre = lfm2_conv_packed(proj[:, :T0].reshape(B * T0, 3 * D).contiguous(), w, table, starts, starts + T0,
                             slots.repeat_interleave(T0).int())
    outs = [lin(y_pre.view(B, T0, D), "attn.out_proj")]
    for t in range(T0, T):
        outs.append(lin(lfm2_conv_decode_step(proj[:, t].contiguous(), w, slots, table), "attn.out_proj")[:, None])
    assert max_abs(torch.cat(outs, 1), g["mix"]) < 1e-4


def test_memory_readout_kernels_match_the_reference_module(golden):
    """Scan kernel + RMSNorm(r) * sigmoid(gate) epilogue kernel between cuBLAS projections ==
    TitansMemory.forward of the reference (fp32 path)."""
    from atma_b200.inference_ops import rms_sigmoid_gate
    g = golden["mem_readout"]
    sd = {k: v.cuda() for k, v in g["state"].items()}
    x, q, k, v = (g[n].cuda() for n in ("x", "q", "k", "v"))
    B, H, T, dk = q.shape
    lin = lambda t, n: F.linear(t, sd[n + ".weight"], sd[n + ".bias"])
    glog = F.logsigmoid(lin(x, "mem.w_gamma") + 3.9)
    beta = torch.sigmoid(lin(x, "mem.w_beta"))
    r, _ = atma_b200.chunk_gated_delta_rule(q=q.transpose(1, 2).contiguous(), k=k.transpose(1, 2).contiguous(),
                                            v=v.transpose(1, 2).contiguous(), g=glog, beta=beta, scale=1.0,
                                            output_final_state=True, use_qk_l2norm_in_kernel=True)
    gated = rms_sigmoid_gate(r.reshape(B * T, H, dk), lin(x, "mem.gate").reshape(B * T, H * dk))
    assert max_abs(lin(gated, "mem.proj").view(B, T, -1), g["out"]) < 1e-4
