"""GPU parity of the whole model on this package's kernels (atma_b200/model.py) against the reference
model's logits (golden: ReferenceModel of model/reference.py:236-269 on seeded weights), and of the fused
decode-side kernels against the separate ops they replace."""

import os
import sys

import pytest
import torch
import torch.nn.functional as F

import atma_b200
from atma_b200.model import AtmaModel, CapturedDecode
from conftest import max_abs, max_rel
from gpu_util import polar_params, rand

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
import seeded_weights as sw  # noqa: E402

pytestmark = pytest.mark.gpu
CFG = dict(layers=8, hidden=512, head_dim=128, num_kv_heads=1)
BLOCK = 16


def _model(golden, dtype):
    g = golden["model_small"]
    sd = sw.model_state(seed=int(g["weight_seed"]), vocab=640, layers=8, dim=512, head_dim=128, num_kv_heads=1)
    return AtmaModel(sd, dtype=dtype, **CFG), g["ids"], g["logits"]


def _paging(n_seqs, max_len, seed=0):
    """Block tables over a shuffled pool of pages, as the reference's block manager hands them out."""
    per = (max_len + BLOCK - 1) // BLOCK
    perm = torch.randperm(n_seqs * per + 3, generator=torch.Generator().manual_seed(seed))
    bt = perm[:n_seqs * per].view(n_seqs, per).int()
    return bt, n_seqs * per + 3


def _slot_rows(bt, seq, positions):
    return bt[seq, positions // BLOCK].long() * BLOCK + positions % BLOCK


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-4), (torch.bfloat16, 2e-2)])
def test_prefill_logits_match_the_reference_model(golden, dtype, tol):
    """Packed prefill of the two prompts: logits at every position against ReferenceModel."""
    model, ids, want = _model(golden, dtype)
    B, T = ids.shape
    bt, nblk = _paging(B, T)
    state = model.new_state(max_seqs=4, num_blocks=nblk, block_size=BLOCK)
    slots = [2, 0]
    sm = torch.cat([_slot_rows(bt, b, torch.arange(T)) for b in range(B)])
    h = model.prefill(ids.reshape(-1), [T] * B, slots, state, sm)
    logits = model.logits(h).view(B, T, -1)
    if dtype == torch.float32:
        assert max_abs(logits, want) < tol
        return
    # 16-bit: error of every position on the tensor's largest magnitude.  Eight layers of 16-bit projections
    # put the typical position at ~1e-2.  A query with two or three visible keys can be ill-conditioned: its
    # direction c = s / |s| divides by a nearly cancelled sum, which amplifies the rounding of the operands (the
    # fp32 run above is exact at the same positions), so up to 1% of the positions may exceed 2e-2, none 1e-1.
    err = (logits.float().cpu() - want).abs().amax(-1) / want.abs().max()
    assert float((err < tol).float().mean()) >= 0.99 and float(err.max()) < 1e-1, (float(err.max()), err.topk(3))
    assert float(err.median()) < 1.2e-2


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-4), (torch.bfloat16, 2e-2)])
def test_decode_continues_the_prefill(golden, dtype, tol):
    """Prefill 70 tokens of each prompt, then decode the remaining 20 one token per step (conv states, memory
    states and K/V pages carried by the tables): the logits of every decoded position against ReferenceModel."""
    model, ids, want = _model(golden, dtype)
    B, T = ids.shape
    T0 = 70
    bt, nblk = _paging(B, T, seed=1)
    state = model.new_state(max_seqs=4, num_blocks=nblk, block_size=BLOCK)
    slots = torch.tensor([1, 3])
    sm = torch.cat([_slot_rows(bt, b, torch.arange(T0)) for b in range(B)])
    model.prefill(ids[:, :T0].reshape(-1), [T0] * B, slots.tolist(), state, sm)
    dev = model.device
    worst = 0.0
    for t in range(T0, T):
        smap = torch.stack([_slot_rows(bt, b, torch.tensor(t)) for b in range(B)]).int().to(dev)
        logits = model.decode(ids[:, t].to(dev), state, slots.to(dev), smap, bt.to(dev),
                              torch.full((B,), t + 1, dtype=torch.int32, device=dev))
        err = max_abs(logits, want[:, t]) if dtype == torch.float32 else max_rel(logits, want[:, t])
        worst = max(worst, err)
    assert worst < tol, worst


def test_captured_decode_equals_eager(golden):
    """The decode step replayed from a CUDA graph == the same step issued launch by launch, bit for bit, on
    the same starting state (padded batch row included: slot -1, context 0)."""
    model, ids, _ = _model(golden, torch.bfloat16)
    B, T = ids.shape
    T0 = 40
    bt, nblk = _paging(B + 1, T, seed=2)
    state = model.new_state(max_seqs=4, num_blocks=nblk, block_size=BLOCK)
    sm = torch.cat([_slot_rows(bt, b, torch.arange(T0)) for b in range(B)])
    model.prefill(ids[:, :T0].reshape(-1), [T0] * B, [0, 1], state, sm)
    dev = model.device
    cap = CapturedDecode(model, state, batch=B + 1, max_blocks=bt.shape[1])
    cap.ids[:B] = ids[:, T0].to(dev)
    cap.seq_slots.copy_(torch.tensor([0, 1, -1]))
    cap.slot_mapping[:B] = torch.stack([_slot_rows(bt, b, torch.tensor(T0)) for b in range(B)]).int().to(dev)
    cap.block_tables.copy_(bt.to(dev))
    cap.context_lens.copy_(torch.tensor([T0 + 1, T0 + 1, 0]))
    snap = lambda: ({k: v.clone() for k, v in state.conv.items()}, {k: v.clone() for k, v in state.mem.items()},
                    {k: v.clone() for k, v in state.k_cache.items()}, {k: v.clone() for k, v in state.v_cache.items()})

    def restore(s):
        for dst, src in zip((state.conv, state.mem, state.k_cache, state.v_cache), s):
            for k in dst:
                dst[k].copy_(src[k])

    before = snap()
    cap.capture()                                          # its warm-up runs advance the state: put it back
    restore(before)
    eager = cap._run().clone()
    after_eager = snap()
    restore(before)
    replayed = cap.replay().clone()
    torch.cuda.synchronize()
    assert torch.equal(eager[:B], replayed[:B])
    for a, b in zip(after_eager, snap()):
        for k in a:
            assert torch.equal(a[k], b[k]), k


# ---- the fused decode-side kernels against the ops they replace ------------------------------------------
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_qkv_prep_decode_equals_the_separate_ops(dtype):
    B, H, Hkv, dk, K = 5, 8, 2, 128, 4
    q_gate = rand((B, H, 2 * dk), 1, dtype).cuda()
    kv = rand((B, 2 * Hkv * dk + 7), 2, dtype).cuda()                       # k and v as column ranges of a wider row
    k, v = kv[:, :Hkv * dk].view(B, Hkv, dk), kv[:, Hkv * dk:2 * Hkv * dk].view(B, Hkv, dk)
    w = [rand((C, K), 3 + i, dtype, 0.3).cuda() for i, C in enumerate((H * dk, Hkv * dk, Hkv * dk))]
    slots = torch.tensor([3, 0, -1, 5, 1]).cuda()
    tables = [rand((6, C, K - 1), 7 + i, dtype).cuda() for i, C in enumerate((H * dk, Hkv * dk, Hkv * dk))]
    kc, vc = torch.zeros(4, 8, Hkv, dk, dtype=dtype).cuda(), torch.zeros(4, 8, Hkv, dk, dtype=dtype).cuda()
    smap = torch.tensor([9, 31, -1, 0, 17], dtype=torch.int32).cuda()
    # the reference's sequence of ops (inference/models/atma.py:557-572) on copies of the tables
    t_ref = [t.clone() for t in tables]
    kc_ref, vc_ref = kc.clone(), vc.clone()
    live = slots >= 0
    qn, kn = F.rms_norm(q_gate[..., :dk], (dk,)), F.rms_norm(k, (dk,))
    outs = []
    for x, wt, tab in ((qn.reshape(B, -1), w[0], t_ref[0]), (kn.reshape(B, -1), w[1], t_ref[1]), (v.reshape(B, -1), w[2], t_ref[2])):
        conv = torch.zeros_like(x)
        conv[live] = atma_b200.causal_conv1d_decode_step(x[live].contiguous(), wt, slots[live], tab)
        conv[~live] = (x[~live].float() * wt[:, -1].float()).to(dtype)
        outs.append(x + conv)
    q_ref, k_ref, v_ref = outs[0].view(B, H, dk), outs[1].view(B, Hkv, dk), outs[2].view(B, Hkv, dk)
    atma_b200.store_kvcache(k_ref, v_ref, kc_ref, vc_ref, smap)
    q_o, k_o, v_o = atma_b200.qkv_prep_decode(q_gate, k, v, *w, *tables, slots, kc, vc, smap)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    assert max_rel(q_o, q_ref) < tol and max_rel(k_o, k_ref) < tol and max_rel(v_o, v_ref) < tol
    for a, b in zip(tables, t_ref):
        assert max_rel(a, b) < tol
    assert max_rel(kc, kc_ref) < tol and max_rel(vc, vc_ref) < tol
    assert torch.equal(kc.view(-1, Hkv, dk)[1], torch.zeros_like(kc.view(-1, Hkv, dk)[1]))      # an untouched cache row


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_fused_memory_step_equals_the_separate_ops(dtype):
    """Un-expanded KV heads, gates from logits, RMSNorm * sigmoid(gate) epilogue == repeat_interleave + sigmoid +
    gated_delta_decode_step + rms_norm + gate multiply (inference/models/atma.py:352-375, 609-611)."""
    B, H, Hkv, d = 6, 8, 2, 128
    q, k, v = rand((B, H, d), 1, dtype).cuda(), rand((B, Hkv, d), 2, dtype).cuda(), rand((B, Hkv, d), 3, dtype).cuda()
    z = rand((B, 2 * H + H * d), 4, dtype).cuda()
    g_l, b_l, gate = z[:, :H], z[:, H:2 * H], z[:, 2 * H:]
    table = (torch.randn(8, H, d, d, generator=torch.Generator().manual_seed(5)) * 0.2).cuda()
    slots = torch.tensor([4, 0, 7, -1, 2, 1]).cuda()
    t_ref = table.clone()
    live = slots >= 0
    gamma, beta = torch.sigmoid(g_l.float() + 3.9), torch.sigmoid(b_l.float())
    r = atma_b200.gated_delta_decode_step(q[live], k[live].repeat_interleave(H // Hkv, 1), v[live].repeat_interleave(H // Hkv, 1),
                                          gamma[live], beta[live], t_ref, slots[live])
    want = (F.rms_norm(r, (d,)).reshape(-1, H * d).to(dtype) * torch.sigmoid(gate[live]))
    out = torch.full((B, H * d + 5), 7.0, dtype=dtype).cuda()
    got = atma_b200.gated_delta_decode_step_fused(q, k, v, table, slots, gate_logits=(g_l, b_l), gate=gate, out=out[:, :H * d])
    tol = 2e-2 if dtype == torch.bfloat16 else 2e-5
    assert max_rel(got[live], want) < tol
    assert float(got[~live].abs().max()) == 0.0 and float((out[:, H * d:] - 7.0).abs().max()) == 0.0
    assert max_abs(table, t_ref) < 2e-5
    # plain form: fp32 read-out, gamma / beta given
    t2 = t_ref.clone()
    r2 = atma_b200.gated_delta_decode_step_fused(q, k, v, t2, slots, gamma=gamma, beta=beta)
    t3 = t_ref.clone()
    r3 = atma_b200.gated_delta_decode_step(q[live], k[live].repeat_interleave(H // Hkv, 1), v[live].repeat_interleave(H // Hkv, 1),
                                           gamma[live], beta[live], t3, slots[live])
    assert max_abs(r2[live], r3) < 2e-4 and max_abs(t2, t3) < 2e-5


def test_decode_merge_writes_the_gated_direction_in_place():
    """polar_attention_decode(gate=, out=) == c * sigmoid(gate) of the plain call, landing in column ranges of a
    wider activation buffer, other columns untouched."""
    from test_gpu_polar_decode import make_paged
    B, H, Hkv, dk = 4, 8, 2, 128
    kc, vc, bt, cl = make_paged(B, Hkv, dk, 16, [70, 1, 300, 129], torch.bfloat16, seed=4)
    q = rand((B, H, dk), 9, torch.bfloat16).cuda()
    qg = rand((B, H, 2 * dk), 10, torch.bfloat16).cuda()
    _, pg = polar_params(H, dk, 2)
    c, m = atma_b200.polar_attention_decode(q, kc.cuda(), vc.cuda(), bt.cuda(), cl.cuda(), **pg)
    act = torch.full((B, 2 * H * dk + H), 3.0, dtype=torch.bfloat16).cuda()
    atma_b200.polar_attention_decode(q, kc.cuda(), vc.cuda(), bt.cuda(), cl.cuda(), gate=qg[..., dk:],
                                     out=(act[:, :H * dk].view(B, H, dk), act[:, H * dk:H * dk + H]), **pg)
    want = c * torch.sigmoid(qg[..., dk:])
    assert torch.equal(act[:, :H * dk].view(B, H, dk), want) and torch.equal(act[:, H * dk:H * dk + H], m)
    assert float((act[:, H * dk + H:] - 3.0).abs().max()) == 0.0


@pytest.mark.parametrize("dtype,D", [(torch.bfloat16, 1024), (torch.float32, 512), (torch.float16, 100)])
def test_add_rms_norm(dtype, D):
    x, y, w = rand((7, D), 1, dtype).cuda(), rand((7, D), 2, dtype).cuda(), (1 + 0.1 * rand((D,), 3)).to(dtype).cuda()
    xo, h = atma_b200.add_rms_norm(x, y, w, 1e-6)
    x_ref = x + y
    assert torch.equal(xo, x_ref)
    h_ref = F.rms_norm(x_ref.float(), (D,), weight=w.float(), eps=1e-6)
    assert max_rel(h, h_ref) < (1e-2 if dtype != torch.float32 else 1e-6)
    x2, h2 = atma_b200.add_rms_norm(x, None, None, 1e-6)
    assert x2 is x and max_rel(h2, F.rms_norm(x.float(), (D,), eps=1e-6)) < (1e-2 if dtype != torch.float32 else 1e-6)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-4), (torch.bfloat16, 2e-2)])
def test_prefix_hit_from_another_request_equals_full_recompute(golden, dtype, tol):
    """Request A is prefilled with state snapshots at every page boundary and registered in the prefix cache.
    Request B shares A's first two pages and then differs.  B served from the cache - A's K/V pages in its block
    table, conv and memory state from the page-2 snapshot, only the tail prefilled - gives the logits and final
    states of B prefilled from scratch (the reference inherits the K/V but not the state there, docs/inference.md:72-75)."""
    from atma_b200.model import PrefixStateCache
    model, ids, _ = _model(golden, dtype)
    page = 64
    gen = torch.Generator().manual_seed(11)
    a_ids = torch.randint(0, 640, (200,), generator=gen)
    b_ids = torch.cat([a_ids[:2 * page], torch.randint(0, 640, (75,), generator=gen)])
    n_a, n_b = a_ids.numel(), b_ids.numel()
    state = model.new_state(max_seqs=4, num_blocks=16, block_size=page)
    rows_of = lambda table, n: (table[torch.arange(n) // page].long() * page + torch.arange(n) % page)
    bt_a = torch.tensor([5, 2, 9, 0])
    _, snaps = model.prefill(a_ids, [n_a], [0], state, rows_of(bt_a, n_a), snapshot_every=page)
    cache = PrefixStateCache(page)
    cache.register(a_ids.tolist(), snaps, 0, bt_a)
    # B from scratch, in its own pages and slot
    bt_full = torch.tensor([11, 12, 13, 14, 15])
    h_full = model.prefill(b_ids, [n_b], [1], state, rows_of(bt_full, n_b))
    logits_full = model.logits(h_full)
    # B through the cache
    n_pages, phys, hit_snaps, row = cache.lookup(b_ids.tolist())
    assert n_pages == 2 and phys == [5, 2] and hit_snaps is snaps
    bt_b = torch.tensor(phys + [7, 8, 3])
    tail = torch.arange(n_pages * page, n_b)
    sm_tail = bt_b[tail // page].long() * page + tail % page
    h_tail = model.prefill_from_prefix(b_ids[n_pages * page:], n_pages * page, 2, state, sm_tail, bt_b, hit_snaps, row)
    logits_tail = model.logits(h_tail)
    err = max_abs if dtype == torch.float32 else max_rel
    assert err(logits_tail, logits_full[n_pages * page:]) < tol
    for name, tab in state.conv.items():
        assert err(tab[2], tab[1]) < tol, name
    for i, tab in state.mem.items():
        assert err(tab[2], tab[1]) < tol, i
    # and the snapshot itself is the state of a prefill that stops at the page boundary
    st2 = model.new_state(max_seqs=1, num_blocks=4, block_size=page)
    model.prefill(a_ids[:2 * page], [2 * page], [0], st2, torch.arange(2 * page))
    for name, tab in st2.conv.items():
        assert err(snaps.conv[name][1], tab[0]) < tol, name
    for i, tab in st2.mem.items():
        assert err(snaps.mem[i][1], tab[0]) < tol, i
