"""Generate golden input/output vectors from the UNMODIFIED reference implementation.

Run once, in a container where the reference checkout is mounted:

    python tests/golden/make_golden.py <path to the reference checkout>

It imports the reference's own pure-PyTorch oracle on the CPU (model/blocks.py,
model/reference.py, scripts/titans_proto.py and the CPU branches of
inference/models/atma.py), runs it on small seeded inputs and stores inputs and
outputs in ``tests/golden/golden.pt``.  The reference cannot travel to the GPU box,
so the committed vectors are what pins the CPU restatement in ``oracle/`` (and,
through it, the CUDA kernels) to the reference's results.
"""

import os
import sys
from types import SimpleNamespace

import torch
import torch.nn.functional as F


def main(ref_root):
    sys.path.insert(0, ref_root)
    torch.set_num_threads(4)
    from model.blocks import polar_reduce, gated_delta_chunked, polar_attention_online
    from model import reference as ref
    from scripts.titans_proto import gated_delta_sequential
    from inference.models.atma import prefill_causal_conv1d, _gpu_conv_step

    G = {}

    # ---- Polar: materialised oracle, causal / windowed / arbitrary n_keys ------------
    def polar_case(name, B, H, Hkv, Tq, Tk, dk, seed, window=None, n_keys=None, dtype=torch.float32):
        g = torch.Generator().manual_seed(seed)
        q = torch.randn(B, H, Tq, dk, generator=g).to(dtype)
        k = torch.randn(B, Hkv, Tk, dk, generator=g).to(dtype)
        v = torch.randn(B, Hkv, Tk, dk, generator=g).to(dtype)
        params = dict(v_null=torch.randn(H, dk, generator=g) * 0.5,
                      null_base=2.0 + 0.5 * torch.randn(H, generator=g),
                      null_slope_raw=0.5 + 0.5 * torch.randn(H, generator=g),
                      len_gain_raw=-1.0 + 0.5 * torch.randn(H, generator=g),
                      mag_beta_raw=-1.5 + 0.5 * torch.randn(H, generator=g))
        if n_keys is None:
            n_keys = torch.arange(1, Tq + 1, dtype=torch.float32) + (Tk - Tq)
        groups = H // Hkv
        ke = k.repeat_interleave(groups, dim=1)                       # model/reference.py:155-157
        ve = v.repeat_interleave(groups, dim=1)
        sigma = torch.matmul(q.float(), ke.float().transpose(-2, -1)) / (dk ** 0.5)
        ki = torch.arange(Tk)
        invalid = ki[None, None, None, :] >= n_keys.view(1, 1, -1, 1)  # inference/models/atma.py:237-244
        n_temp = n_keys
        if window is not None:
            invalid = invalid | (ki[None, None, None, :] < (n_keys.view(1, 1, -1, 1) - window))
            n_temp = torch.minimum(n_keys, n_keys.new_tensor(float(window)))
        sigma = sigma.masked_fill(invalid, float("-inf"))
        c, mag = polar_reduce(sigma, ve.float(), n_temp, **params)
        G[name] = dict(q=q, k=k, v=v, n_keys=n_keys, window=-1 if window is None else window,
                       c=c, mag=mag, **params)

    polar_case("polar_causal_small", 2, 4, 2, 48, 48, 32, seed=11)
    polar_case("polar_causal_dk128", 1, 4, 1, 136, 136, 128, seed=12)
    polar_case("polar_window", 1, 4, 1, 96, 96, 64, seed=13, window=16)
    polar_case("polar_offset_prefill", 1, 4, 2, 40, 104, 64, seed=14)            # continuation chunk
    polar_case("polar_padding_queries", 2, 3, 3, 4, 16, 128, seed=15,
               n_keys=torch.tensor([5., 0., 12., 0.]))                            # kernel/test_polar_kernel.py:144-158
    polar_case("polar_causal_bf16", 1, 4, 2, 144, 144, 128, seed=16, dtype=torch.bfloat16)

    # The streaming torch form is recorded too, only to document its known deviation.
    g = G["polar_causal_small"]
    p = {k_: g[k_] for k_ in ("v_null", "null_base", "null_slope_raw", "len_gain_raw", "mag_beta_raw")}
    c_on, m_on = polar_attention_online(g["q"], g["k"].repeat_interleave(2, 1), g["v"].repeat_interleave(2, 1),
                                        g["n_keys"], k_block=16, **p)
    G["polar_causal_small"]["c_online"], G["polar_causal_small"]["mag_online"] = c_on, m_on

    # ---- gated delta: chunked + sequential, with and without carried state ----------
    def delta_case(name, B, H, N, dk, dv, chunk, seed, with_s0, gamma_bias):
        g = torch.Generator().manual_seed(seed)
        q = F.normalize(torch.randn(B, H, N, dk, generator=g), dim=-1)
        k = F.normalize(torch.randn(B, H, N, dk, generator=g), dim=-1)
        v = torch.randn(B, H, N, dv, generator=g)
        gamma = torch.sigmoid(torch.randn(B, H, N, generator=g) + gamma_bias)
        beta = torch.sigmoid(torch.randn(B, H, N, generator=g))
        S0 = torch.randn(B, H, dv, dk, generator=g) * 0.3 if with_s0 else None
        R, S = gated_delta_chunked(q, k, v, gamma, beta, chunk=chunk, S0=S0)
        Rs, Ss = gated_delta_sequential(q, k, v, gamma, beta, S0=S0)
        G[name] = dict(q=q, k=k, v=v, gamma=gamma, beta=beta, chunk=chunk,
                       S0=S0 if with_s0 else torch.zeros(0), R=R, S=S, R_seq=Rs, S_seq=Ss)

    delta_case("delta_small", 2, 2, 100, 16, 24, 32, seed=21, with_s0=False, gamma_bias=0.0)
    delta_case("delta_carry", 1, 3, 130, 32, 32, 64, seed=22, with_s0=True, gamma_bias=3.9)
    delta_case("delta_d128", 1, 1, 136, 128, 128, 64, seed=23, with_s0=True, gamma_bias=3.9)

    # ---- decode step: the torch fallback of inference/models/atma.py:362-371 --------
    g = torch.Generator().manual_seed(31)
    Bd, Hd, d = 3, 2, 32
    q = torch.randn(Bd, Hd, d, generator=g); k = torch.randn(Bd, Hd, d, generator=g)
    v = torch.randn(Bd, Hd, d, generator=g)
    gamma = torch.rand(Bd, Hd, generator=g); beta = torch.rand(Bd, Hd, generator=g)
    table = torch.randn(6, Hd, d, d, generator=g)
    slots = torch.tensor([4, 0, 2])
    S = table[slots]
    qn, kn = F.normalize(q, dim=-1), F.normalize(k, dim=-1)
    St = S.transpose(-1, -2)
    Sd = gamma[..., None, None] * St
    pred = torch.einsum("bhvk,bhk->bhv", Sd, kn)
    u = beta[..., None] * (v - pred)
    S_new = Sd + u.unsqueeze(-1) * kn.unsqueeze(-2)
    table_out = table.clone()
    table_out[slots] = S_new.transpose(-1, -2)
    r = torch.einsum("bhvk,bhk->bhv", S_new, qn)
    G["delta_step"] = dict(q=q, k=k, v=v, gamma=gamma, beta=beta, table=table, slots=slots,
                           r=r, table_out=table_out)

    # ---- depthwise causal conv: fresh prefill, continuation, decode step ------------
    g = torch.Generator().manual_seed(41)
    C, K = 37, 4
    x = torch.randn(19, C, generator=g); w = torch.randn(C, K, generator=g)
    tables = {"x": torch.zeros(3, C, K - 1)}
    fresh = prefill_causal_conv1d("x", SimpleNamespace(num_cached_tokens=0, seq_slot=1), x[:11], w, None, tables)
    st_fresh = tables["x"][1].clone()
    cont = prefill_causal_conv1d("x", SimpleNamespace(num_cached_tokens=11, seq_slot=1), x[11:], w, None, tables)
    st_cont = tables["x"][1].clone()
    xs = torch.randn(2, C, generator=g)
    slots = torch.tensor([1, 2])
    step = _gpu_conv_step("x", slots, tables, xs, w)
    G["conv"] = dict(x=x, w=w, fresh=fresh, st_fresh=st_fresh, cont=cont, st_cont=st_cont,
                     xs=xs, slots=slots, step=step, table_after_step=tables["x"].clone())
    # K = 3 (LFM2 conv) one-token prompt: state shorter than the kernel
    w3 = torch.randn(C, 3, generator=g)
    tables3 = {"x": torch.zeros(1, C, 2)}
    one = prefill_causal_conv1d("x", SimpleNamespace(num_cached_tokens=0, seq_slot=0), x[:1], w3, None, tables3)
    G["conv_k3_T1"] = dict(x=x[:1], w=w3, out=one, st=tables3["x"][0].clone())

    # ---- eager-bf16 elementwise expressions (tests/test_decode_kernels.py:56-66) ----
    g = torch.Generator().manual_seed(5)
    packed = torch.randn(16, 256, generator=g).to(torch.bfloat16)
    xx, gate = packed.chunk(2, dim=-1)
    logits = (4.0 * torch.randn(8, 515, generator=g)).to(torch.bfloat16)
    G["elementwise"] = dict(packed=packed, sq=gate * xx.relu().square(),
                            logits=logits, capped=15.0 * logits * (logits.square() + 225.0).rsqrt(),
                            logits32=logits.float(),
                            capped32=15.0 * logits.float() * (logits.float().square() + 225.0).rsqrt())

    # ---- one global block (tiny shape of BASELINE config 1) ---------------------------
    torch.manual_seed(0)
    blk = ref.Block(128, attention=True, head_dim=32, num_kv_heads=2, attn_window=None,
                    mem_enabled=True, mem_chunk=16, mem_kernel="torch")
    with torch.no_grad():
        blk.attn.mem.proj.weight.normal_(0, 0.05)               # tests/verify.py:363 randomises the zero-init proj
        blk.attn.v_null.normal_(0, 0.2)
        x = torch.randn(2, 40, 128)
        y = blk(x)
    G["block"] = dict(x=x, y=y, state={k_: v_.detach().clone() for k_, v_ in blk.state_dict().items()})

    # ---- seeded-weight cases: weights come from seeded_weights.py on both sides -------
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    import seeded_weights as sw
    from model.config import AtmaConfig

    # BASELINE config 1 at its own shape: one global block, hidden 1024, 8/2 heads of 128, T=2048
    sd = sw.block_state(seed=0, dim=1024, head_dim=128, num_kv_heads=2)
    blk = ref.Block(1024, attention=True, head_dim=128, num_kv_heads=2, attn_window=None,
                    mem_enabled=True, mem_chunk=64, mem_kernel="torch")
    blk.load_state_dict(sd, strict=True)
    x = torch.randn(1, 2048, 1024, generator=torch.Generator().manual_seed(100))
    with torch.no_grad():
        y = blk(x)
    rows = torch.cat([torch.arange(0, 8), torch.arange(60, 70), torch.arange(8, 2048, 29), torch.arange(2040, 2048)]).unique()
    G["block_cfg1"] = dict(weight_seed=0, x_seed=100, rows=rows, y_rows=y[0, rows].clone(),
                           y_absmax=y.abs().max(), y_sum=y.double().sum().float())

    # local (LFM2 gated conv) mixing module and block, model/reference.py:31-49
    sd = sw.block_state(seed=1, dim=96, head_dim=32, num_kv_heads=1, attention=False)
    blk = ref.Block(96, attention=False)
    blk.load_state_dict(sd, strict=True)
    x = torch.randn(2, 21, 96, generator=torch.Generator().manual_seed(101))
    with torch.no_grad():
        G["lfm2"] = dict(weight_seed=1, x=x, mix=blk.attn(x), y=blk(x))

    # memory branch with its read-out, model/blocks.py:463-490 (TitansMemory.forward, torch backend)
    gen = torch.Generator().manual_seed(102)
    dim, H, dk, T = 64, 2, 32, 150
    sd = sw.attention_state(gen, dim, dk, 1, prefix="")
    att = ref.PolarAttention(dim, head_dim=dk, num_kv_heads=1, mem_enabled=True, mem_chunk=64, mem_kernel="torch")
    att.load_state_dict(sd, strict=True)
    x = torch.randn(2, T, dim, generator=gen)
    q_t, k_t, v_t = (torch.randn(2, H, T, dk, generator=gen) for _ in range(3))
    with torch.no_grad():
        out = att.mem(x, q_t, k_t, v_t)
    G["mem_readout"] = dict(x=x, q=q_t, k=k_t, v=v_t, out=out,
                            state={k_: v_.clone() for k_, v_ in sd.items() if k_.startswith("mem.")})

    # a whole small model: 8 layers (2 global), model/reference.py:236-269
    cfg = AtmaConfig(vocab_size=640, num_hidden_layers=8, hidden_size=512, head_dim=128, attn_window=None,
                     mem_enabled=True, mem_chunk=64, mem_kernel="torch", attn_kernel="torch")
    sd = sw.model_state(seed=7, vocab=640, layers=8, dim=512, head_dim=128, num_kv_heads=1)
    model = ref.ReferenceModel(cfg)
    model.load_state_dict(sd, strict=True)
    ids = torch.randint(0, 640, (2, 90), generator=torch.Generator().manual_seed(103))
    with torch.no_grad():
        logits = model(ids)
    G["model_small"] = dict(weight_seed=7, ids=ids, logits=logits)

    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden.pt")
    torch.save(G, out)
    print("wrote", out, os.path.getsize(out), "bytes;", len(G), "cases")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path to the reference checkout>")
    main(sys.argv[1])
