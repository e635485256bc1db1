"""CPU: the block- and model-level restatement in oracle/model.py reproduces the reference's own
outputs (golden vectors made by tests/golden/make_golden.py from model/reference.py), with the
weights regenerated from their seed by tests/golden/seeded_weights.py."""

import os
import sys

import torch

import oracle
from conftest import max_abs

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
import seeded_weights as sw  # noqa: E402


def test_local_block_and_lfm2_conv_match_reference(golden):
    g = golden["lfm2"]
    sd = sw.block_state(seed=int(g["weight_seed"]), dim=96, head_dim=32, num_kv_heads=1, attention=False)
    assert max_abs(oracle.lfm2_mix_oracle(g["x"], sd, "attn."), g["mix"]) < 2e-6
    y = oracle.block_oracle(g["x"], sd, "", attention=False, head_dim=32, num_kv_heads=1)
    assert max_abs(y, g["y"]) < 5e-6


def test_lfm2_packed_and_step_oracles_match_the_reference_module(golden):
    """The op-by-op checkers of the fused LFM2 kernels (packed prefill, then single-token steps from
    the carried conv state) against LFM2Conv.forward on the same weights."""
    g = golden["lfm2"]
    sd = sw.block_state(seed=int(g["weight_seed"]), dim=96, head_dim=32, num_kv_heads=1, attention=False)
    x, w = g["x"], sd["attn.conv.weight"].squeeze(1)
    B, T, D = x.shape
    lin = lambda t, n: torch.nn.functional.linear(t, sd[n + ".weight"], sd[n + ".bias"])
    T0 = 13
    proj = lin(x, "attn.in_proj")                                  # (B, T, 3D)
    packed = proj[:, :T0].reshape(B * T0, 3 * D)
    starts = torch.arange(B).repeat_interleave(T0) * T0
    table = torch.zeros(B + 1, D, 2)
    slots = torch.tensor([2, 0])
    y_pre = oracle.lfm2_conv_packed_oracle(packed, w, table, starts.int(), (starts + T0).int(),
                                           slots.repeat_interleave(T0).int())
    outs = [lin(y_pre.view(B, T0, D), "attn.out_proj")]
    for t in range(T0, T):
        outs.append(lin(oracle.lfm2_conv_step_oracle(proj[:, t], w, slots, table), "attn.out_proj")[:, None])
    assert max_abs(torch.cat(outs, 1), g["mix"]) < 2e-6


def test_memory_readout_matches_reference(golden):
    g = golden["mem_readout"]
    sd = {"mem." + k[4:] if k.startswith("mem.") else k: v for k, v in g["state"].items()}
    out, _ = oracle.memory_readout_oracle(g["x"], g["q"], g["k"], g["v"], sd, "mem.")
    assert max_abs(out, g["out"]) < 5e-6
    # the epilogue checker used by the fused kernel's test is the same expression
    B, H, T, dk = g["q"].shape
    qn = torch.nn.functional.normalize(g["q"], dim=-1)
    kn = torch.nn.functional.normalize(g["k"], dim=-1)
    lin = lambda t, n: torch.nn.functional.linear(t, sd[n + ".weight"], sd[n + ".bias"])
    gamma = torch.sigmoid(lin(g["x"], "mem.w_gamma") + 3.9).transpose(1, 2)
    beta = torch.sigmoid(lin(g["x"], "mem.w_beta")).transpose(1, 2)
    r, _ = oracle.gated_delta_chunked(qn, kn, g["v"], gamma, beta, chunk=64)
    gated = oracle.rms_sigmoid_gate_oracle(r.transpose(1, 2).reshape(B * T, H, dk), lin(g["x"], "mem.gate").reshape(B * T, H * dk))
    assert max_abs(lin(gated, "mem.proj").view(B, T, -1), g["out"]) < 5e-6


def test_small_model_logits_match_reference(golden):
    g = golden["model_small"]
    sd = sw.model_state(seed=int(g["weight_seed"]), vocab=640, layers=8, dim=512, head_dim=128, num_kv_heads=1)
    logits = oracle.model_oracle(g["ids"], sd, layers=8, head_dim=128, num_kv_heads=1)
    assert max_abs(logits, g["logits"]) < 1e-4


def test_config1_block_rows_match_reference(golden):
    """BASELINE config 1 at its own shape (hidden 1024, 8/2 heads of 128, T=2048), sampled rows."""
    g = golden["block_cfg1"]
    sd = sw.block_state(seed=int(g["weight_seed"]), dim=1024, head_dim=128, num_kv_heads=2)
    x = torch.randn(1, 2048, 1024, generator=torch.Generator().manual_seed(int(g["x_seed"])))
    torch.set_num_threads(max(1, min(8, os.cpu_count() or 1)))
    y = oracle.block_oracle(x, sd, "", attention=True, head_dim=128, num_kv_heads=2)
    assert max_abs(y[0, g["rows"]], g["y_rows"]) < 1e-4
    assert abs(float(y.abs().max()) - float(g["y_absmax"])) < 1e-3
