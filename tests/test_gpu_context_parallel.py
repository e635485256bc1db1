"""GPU (needs >= 2 devices; skipped on a 1-GPU box): the context-parallel prefill over NCCL gives
the single-GPU result - Polar ring with statistics carry, gated-delta state prefix."""

import os
import socket
import time

import pytest
import torch

pytestmark = pytest.mark.gpu
T, H, HKV, DK = 2048, 8, 2, 128


def _inputs():
    g = torch.Generator().manual_seed(0)
    t = dict(q=torch.randn(1, T, H, DK, generator=g).bfloat16(), k=torch.randn(1, T, HKV, DK, generator=g).bfloat16(),
             v=torch.randn(1, T, HKV, DK, generator=g).bfloat16(),
             g=-torch.nn.functional.softplus(torch.randn(1, T, H, generator=g)),
             beta=torch.sigmoid(torch.randn(1, T, H, generator=g)))
    params = dict(v_null=torch.randn(H, DK, generator=g) * 0.3, null_base=torch.full((H,), 2.0),
                  null_slope_raw=torch.full((H,), 0.5), len_gain_raw=torch.full((H,), -1.0),
                  mag_beta_raw=torch.full((H,), -1.5))
    return t, params


def _worker(rank, world, port, ret):
    import torch.distributed as dist
    import atma_b200
    from atma_b200 import context_parallel as cp
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        t, params = _inputs()
        tg = {n: x.to(dev) for n, x in t.items()}
        pg = {n: x.to(dev) for n, x in params.items()}
        shard = cp.shard_sequence(tg, rank, world)
        polar, o, S = cp.cp_global_layer_prefill(shard, pg, polar_mode="ring")   # memory branch beside the ring
        torch.cuda.synchronize()
        pol_g, o_g, S_g = cp.cp_global_layer_prefill(shard, pg, polar_mode="gather")
        torch.cuda.synchronize()
        ret[f"gather{rank}"] = dict(c=[p[0].float().cpu() for p in pol_g], mag=[p[1].float().cpu() for p in pol_g])
        ret[rank] = dict(pos=shard.positions, c=[p[0].float().cpu() for p in polar], mag=[p[1].float().cpu() for p in polar],
                         o=[x.float().cpu() for x in o], S=S.float().cpu())
        # the same step replayed from a CUDA graph, twice, with the inputs reloaded in between,
        # must give exactly what the launch-by-launch step gave
        ret[f"stage{rank}"] = "launch-by-launch step done"
        polar, o, S = pol_g, o_g, S_g
        cap = cp.CapturedPrefill(shard, pg, polar_mode="gather")
        ret[f"stage{rank}"] = f"capture returned (captured={cap.captured}, error={getattr(cap, 'error', None)!r})"
        same = cap.captured
        for _ in range(2):
            for f in ("q", "k", "v", "g", "beta"):
                for x in getattr(cap.static, f):
                    x.zero_()
            cap.load(shard)
            polar2, o2, S2 = cap.replay()
            torch.cuda.synchronize()
            same = same and all(torch.equal(a[0], b[0]) and torch.equal(a[1], b[1]) for a, b in zip(polar, polar2))
            same = same and all(torch.equal(a, b) for a, b in zip(o, o2)) and torch.equal(S, S2)
        ret[f"graph{rank}"] = bool(same)
        ret[f"stage{rank}"] = "replays done"
        del polar2, o2, S2
        cap.close()
        torch.cuda.synchronize()
        ret[f"stage{rank}"] = "graph released"
        # the host-fed pipeline: steps from pinned host memory through the captured steps
        host_shard = cp.GlobalLayerShard(positions=shard.positions,
                                         **{f: [x.cpu().pin_memory() for x in getattr(shard, f)] for f in ("q", "k", "v", "g", "beta")})
        pipe = cp.HostFedCapturedPrefill(shard, pg, polar_mode="gather")
        want = [polar[0][0], polar[0][1], polar[1][0], polar[1][1], o[0], o[1], S]
        fed = True
        for step in range(3):
            ticket = pipe.submit(host_shard)
            got = pipe.results(ticket)
            fed = fed and all(torch.equal(a, b.cpu()) for a, b in zip(got, want))
        packed = pipe.host_shard(0)                       # the single-copy path: views of one pinned buffer
        for f in ("q", "k", "v", "g", "beta"):
            for dst, src in zip(getattr(packed, f), getattr(shard, f)):
                dst.copy_(src.cpu())
        for step in range(2):
            got = pipe.results(pipe.submit(packed))
            fed = fed and all(torch.equal(a, b.cpu()) for a, b in zip(got, want))
        ret[f"fed{rank}"] = bool(fed)
        pipe.close()
        # decode over the context-parallel cache: this rank's K/V rows (its two segments) in its own pages
        Hkv, dk, bs = shard.k[0].shape[2], shard.k[0].shape[3], 64
        rows_k = torch.cat([x[0] for x in shard.k])
        rows_v = torch.cat([x[0] for x in shard.v])
        n_local = rows_k.shape[0]
        pages = (n_local + bs - 1) // bs
        kc = torch.zeros(pages, bs, Hkv, dk, dtype=rows_k.dtype, device=dev)
        vc = torch.zeros_like(kc)
        kc.view(-1, Hkv, dk)[:n_local], vc.view(-1, Hkv, dk)[:n_local] = rows_k, rows_v
        qd = torch.randn(1, shard.q[0].shape[2], dk, generator=torch.Generator().manual_seed(3)).to(dev, rows_k.dtype)
        cd, md = cp.cp_polar_decode(qd, kc, vc, torch.arange(pages, dtype=torch.int32, device=dev)[None],
                                    torch.tensor([n_local], dtype=torch.int32, device=dev),
                                    torch.tensor([n_local * world], dtype=torch.int32, device=dev), pg)
        ret[f"dec{rank}"] = (cd.float().cpu(), md.float().cpu())
        ret[f"stage{rank}"] = "pipeline released"
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_context_parallel_matches_one_gpu():
    import torch.multiprocessing as mp
    import atma_b200
    world = 2
    t, params = _inputs()
    tg = {n: x.cuda() for n, x in t.items()}
    pg = {n: x.cuda() for n, x in params.items()}
    n = torch.arange(1, T + 1, dtype=torch.float32).cuda()
    c_ref, m_ref = atma_b200.polar_attention_fwd(tg["q"].transpose(1, 2), tg["k"].transpose(1, 2), tg["v"].transpose(1, 2), n, **pg)
    o_ref, S_ref = atma_b200.chunk_gated_delta_rule(q=tg["q"], k=tg["k"], v=tg["v"], g=tg["g"], beta=tg["beta"], scale=1.0,
                                                    output_final_state=True, use_qk_l2norm_in_kernel=True)
    c_ref, m_ref, o_ref, S_ref = (x.float().cpu() for x in (c_ref, m_ref, o_ref, S_ref))
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    ret = mp.Manager().dict()
    ctx = mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=False)
    deadline = time.time() + 150
    while not ctx.join(timeout=5):
        if time.time() > deadline:                  # never leave ranks waiting on one another
            for p in ctx.processes:
                p.kill()
            pytest.fail(f"context-parallel ranks did not finish in time; stages: {[ret.get(f'stage{r}') for r in range(world)]}")
    rel = lambda a, b: float((a - b).abs().max() / b.abs().max().clamp_min(1e-12))
    for rank in range(world):
        r = ret[rank]
        for part, (a, b) in enumerate(r["pos"]):
            assert rel(r["c"][part], c_ref[:, :, a:b]) < 2e-2
            assert rel(r["mag"][part], m_ref[:, :, a:b]) < 2e-2
            assert rel(r["o"][part], o_ref[:, a:b]) < 2e-2
            assert rel(ret[f"gather{rank}"]["c"][part], c_ref[:, :, a:b]) < 2e-2
            assert rel(ret[f"gather{rank}"]["mag"][part], m_ref[:, :, a:b]) < 2e-2
        assert rel(r["S"], S_ref[0]) < 2e-2
        assert ret[f"graph{rank}"], "graph replay differs from the launch-by-launch step (or capture failed)"
        assert ret[f"fed{rank}"], "the host-fed pipeline differs from the launch-by-launch step"
    # one decode step over the distributed cache == single-GPU paged decode over the whole sequence's K/V
    qd = torch.randn(1, tg["q"].shape[2], tg["q"].shape[3], generator=torch.Generator().manual_seed(3)).to("cuda", tg["q"].dtype)
    bs = 64
    kc = tg["k"][0].reshape(T // bs, bs, *tg["k"].shape[2:]).contiguous()
    vc = tg["v"][0].reshape(T // bs, bs, *tg["v"].shape[2:]).contiguous()
    c1, m1 = atma_b200.polar_attention_decode(qd, kc, vc, torch.arange(T // bs, dtype=torch.int32, device="cuda")[None],
                                              torch.tensor([T], dtype=torch.int32, device="cuda"), **pg)
    for rank in range(world):
        cd, md = ret[f"dec{rank}"]
        assert rel(cd, c1.float().cpu()) < 2e-2 and rel(md, m1.float().cpu()) < 2e-2


# ---- the whole model over a context-parallel group -----------------------------------------------------------------
MODEL_CFG = dict(layers=8, hidden=512, head_dim=128, num_kv_heads=1)
MODEL_T, MODEL_BLOCK = 1024, 64


def _model_worker(rank, world, port, ret):
    import torch.distributed as dist
    from atma_b200 import context_parallel as cp
    from atma_b200.model import AtmaModel, random_state_dict
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        sd = random_state_dict(vocab=640, seed=5, device=dev, **MODEL_CFG)
        model = AtmaModel(sd, device=dev, **MODEL_CFG)
        ids = torch.randint(0, 640, (MODEL_T,), generator=torch.Generator().manual_seed(9))
        # the single-GPU prefill of the whole prompt (every rank computes it for itself)
        pages = MODEL_T // MODEL_BLOCK + 1
        ref_state = model.new_state(max_seqs=2, num_blocks=pages, block_size=MODEL_BLOCK)
        h_ref = model.prefill(ids, [MODEL_T], [1], ref_state, torch.arange(MODEL_T))
        # context-parallel: this rank's two zig-zag segments, K/V of its own tokens in its own pages
        (a0, a1), (b0, b1) = cp.zigzag_segments(MODEL_T, world)[rank]
        L = a1 - a0
        state = model.new_state(max_seqs=2, num_blocks=2 * L // MODEL_BLOCK + 1, block_size=MODEL_BLOCK)
        h = model.prefill_context_parallel([ids[a0:a1], ids[b0:b1]], [(a0, a1), (b0, b1)], state, 1,
                                           [torch.arange(L), torch.arange(L, 2 * L)])
        torch.cuda.synchronize()
        rel = lambda a, b: float((a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-12))
        out = dict(h=[rel(h[0], h_ref[a0:a1]), rel(h[1], h_ref[b0:b1])])
        out["mem"] = max(rel(state.mem[i][1], ref_state.mem[i][1]) for i in model.global_layers)
        out["conv"] = max(rel(state.conv[n][1], ref_state.conv[n][1]) for n in state.conv)
        # K/V rows of this rank's tokens against the rows the single-GPU prefill cached
        gl = model.global_layers[0]
        mine = state.k_cache[gl].view(-1, model.Hkv, model.dk)
        whole = ref_state.k_cache[gl].view(-1, model.Hkv, model.dk)
        out["kv"] = max(rel(mine[:L], whole[a0:a1]), rel(mine[L:2 * L], whole[b0:b1]))
        # decode three tokens over the distributed cache (every rank the same call; the owner of the last segment stores
        # the new K/V rows behind its own) against the single-GPU decode that continues the single-GPU prefill
        owner = cp.segment_owner(2 * world - 1, world) == rank
        slot1 = torch.tensor([1], device=dev)
        nxt = torch.randint(0, 640, (3,), generator=torch.Generator().manual_seed(11))
        bt_local = torch.arange(state.k_cache[gl].shape[0], dtype=torch.int32, device=dev)[None]
        bt_ref = torch.arange(ref_state.k_cache[gl].shape[0], dtype=torch.int32, device=dev)[None]
        worst = 0.0
        for t in range(3):
            tok = nxt[t:t + 1].to(dev)
            total = torch.tensor([MODEL_T + t + 1], dtype=torch.int32, device=dev)
            lg_ref = model.decode(tok, ref_state, slot1, torch.tensor([MODEL_T + t], dtype=torch.int32, device=dev), bt_ref, total)
            local = torch.tensor([2 * L + (t + 1 if owner else 0)], dtype=torch.int32, device=dev)
            sm_new = torch.tensor([2 * L + t if owner else -1], dtype=torch.int32, device=dev)
            lg = model.decode(tok, state, slot1, sm_new, bt_local, total, local_lens=local)
            worst = max(worst, rel(lg, lg_ref))
        out["decode"] = worst
        ret[rank] = out
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [1, 2])
def test_context_parallel_model_prefill_matches_one_gpu(world):
    """The whole model with one prompt cut over the ranks (conv halos, Polar over gathered K/V, memory state prefix)
    against the packed single-GPU prefill of the same prompt: hidden states of every token, final conv and memory
    states, cached K/V rows.  Same kernels on both sides; the differences are the order of the 16-bit roundings
    around the segment borders."""
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    ret = mp.Manager().dict()
    ctx = mp.spawn(_model_worker, args=(world, port, ret), nprocs=world, join=False)
    deadline = time.time() + 150
    while not ctx.join(timeout=5):
        if time.time() > deadline:
            for p in ctx.processes:
                p.kill()
            pytest.fail("context-parallel model ranks did not finish in time")
    for rank in range(world):
        r = ret[rank]
        assert max(r["h"]) < 2e-2, r
        assert r["mem"] < 2e-2 and r["conv"] < 1e-2 and r["kv"] < 1e-2, r
        assert r["decode"] < 2e-2, r
