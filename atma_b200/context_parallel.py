"""Context-parallel prefill of one global layer's mixing across the GPUs of one box.

The reference runs prefill on one GPU only; its chunked-prefill continuation
(inference/models/atma.py:509-544) is the single-device statement of what a sequence split
must reproduce: queries of a later segment attend to all earlier K/V with absolute key
counts, the memory starts from the previous segment's final state, a conv starts from the
previous segment's last K-1 inputs.  This module shards ONE sequence over the ranks of a
``torch.distributed`` group:

* the sequence is cut into 2N equal segments and rank r owns segments r and 2N-1-r
  ("zig-zag"), which balances the causal triangle;
* **Polar**: every rank keeps its queries; the un-expanded K/V blocks travel a ring
  (NCCL send/recv into local buffers, double-buffered, overlapped with the tile kernel of
  the current block).  Per received block the prefill kernel runs with absolute key offsets
  and carries its running statistics (m, L, Q2, S) to the next step; the null sink is folded
  on the last block a query segment sees;
* **gated-delta memory**: a segment acts on the state as an affine map S_out = P S_in + Qm.
  Each rank builds the per-chunk factors of its two segments once, gets (P, Qm) of both from
  one launch of four recurrences over them (the P recurrences use v = 0 and start from the
  identity), an all-gather shares the 2N pairs (1 MB each at the model's shape), the prefix is
  composed locally in fp32, and a second launch produces the outputs from the true incoming
  states - the factors are not recomputed;
* **depthwise conv**: a K-1 row halo from the previous segment's owner.

The compute kernels are injected through a small backend object so that the routing can be
exercised on CPU ranks (gloo) against the oracle; the default backend is the CUDA library.
"""

from dataclasses import dataclass

import torch
import torch.distributed as dist


def zigzag_segments(total, world):
    """[(start, end)] of the two segments rank r owns, for every r.  ``total`` must divide by 2N."""
    if total % (2 * world) != 0:
        raise ValueError(f"sequence length {total} must be a multiple of 2*world = {2 * world}")
    seg = total // (2 * world)
    return [((r * seg, (r + 1) * seg), ((2 * world - 1 - r) * seg, (2 * world - r) * seg)) for r in range(world)]


def segment_owner(seg_index, world):
    return seg_index if seg_index < world else 2 * world - 1 - seg_index


def ring_plan(rank, world):
    """For each ring step s, the (q_part, kv_part, diagonal) block products rank ``rank`` runs on
    the K/V block that started at rank (rank - s) % world.  Parts: 0 = the low segment of the
    block's owner, 1 = its high segment.  Every step holds two products (three at s = 0)."""
    plan = []
    for s in range(world):
        a = (rank - s) % world
        prods = [(1, 0, False)]                                   # my high segment sees every low segment
        if a < rank:
            prods.append((0, 0, False))
        elif a > rank:
            prods.append((1, 1, False))
        else:
            prods = [(0, 0, True), (1, 0, False), (1, 1, True)]
        plan.append((a, prods))
    return plan


class CudaBackend:
    """The production backend: hand-written sm_100a kernels through the C ABI."""

    def polar_block(self, q, k, v, n_keys, params, key_offset, stats_in, finalize, eps, window):
        from .polar import polar_prefill_raw
        return polar_prefill_raw(q, k, v, n_keys, params, eps=eps, window=window, key_offset=key_offset,
                                 stats_in=stats_in, finalize=finalize)

    def scan(self, q, k, v, g, beta, initial_state):
        from .gated_delta import chunk_gated_delta_rule
        return chunk_gated_delta_rule(q=q, k=k, v=v, g=g, beta=beta, scale=1.0, initial_state=initial_state,
                                      output_final_state=True, use_qk_l2norm_in_kernel=True)

    def scan_factors(self, q, k, v, g, beta):
        from .gated_delta import scan_factors
        return scan_factors(q, k, v, g, beta, scale=1.0, use_qk_l2norm_in_kernel=True)

    def scan_recur(self, factors, rec_of, initial_state, zero_value, want_output):
        from .gated_delta import scan_recur
        return scan_recur(factors, rec_of, initial_state, zero_value, want_output)

    def prepare_params(self, params, device):
        from .polar import _params
        return _params(device=device, **params)

    def decode_partials(self, q, k_cache, v_cache, block_tables, local_lens, total_lens, params, eps):
        from .polar import polar_decode_partials
        return polar_decode_partials(q, k_cache, v_cache, block_tables, local_lens, total_lens, params, eps=eps)

    def decode_merge(self, stats, sums, total_lens, params, dtype, eps):
        from .polar import polar_decode_merge
        return polar_decode_merge(stats, sums, total_lens, params, dtype, eps=eps)


def _exchange(send_buf, recv_buf, rank, world, group):
    """Post the ring hop: my current K/V block goes to rank+1 while rank-1's arrives."""
    ops = [dist.P2POp(dist.isend, send_buf, (rank + 1) % world, group),
           dist.P2POp(dist.irecv, recv_buf, (rank - 1) % world, group)]
    return dist.batch_isend_irecv(ops)


@torch.no_grad()
def ring_polar_prefill(q_parts, k_parts, v_parts, positions, params, *, backend=None, group=None,
                       eps=1e-6, window=None):
    """Polar attention for this rank's two query segments over the whole (sharded) sequence.

    q_parts:  [q_lo, q_hi], each (1, H, L, dk)  - this rank's queries (low / high segment)
    k_parts, v_parts: [lo, hi], each (1, Hkv, L, dk) - this rank's keys / values
    positions: [(start_lo, end_lo), (start_hi, end_hi)] absolute token ranges of the two segments
    params: the five raw Polar parameters (dict of tensors)
    Returns [(c_lo, mag_lo), (c_hi, mag_hi)]."""
    backend = backend or CudaBackend()
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    dev = q_parts[0].device
    L = q_parts[0].shape[2]
    seg = positions[0][1] - positions[0][0]
    prepared = backend.prepare_params(params, dev)
    n_keys = [torch.arange(p0 + 1, p1 + 1, device=dev, dtype=torch.float32) for (p0, p1) in positions]

    # one contiguous buffer per hop: [K_lo, K_hi, V_lo, V_hi]
    cur = torch.stack([k_parts[0], k_parts[1], v_parts[0], v_parts[1]]).contiguous()
    nxt = torch.empty_like(cur)
    plan = ring_plan(rank, world)
    # the last product in which each query part takes part -> that call folds the null sink
    last = {}
    for s, (_, prods) in enumerate(plan):
        for i, (qp, kp, _) in enumerate(prods):
            last[qp] = (s, i)
    stats = [None, None]
    out = [None, None]
    for s, (owner, prods) in enumerate(plan):
        works = _exchange(cur, nxt, rank, world, group) if s + 1 < world else []
        owner_pos = [(owner * seg, (owner + 1) * seg), ((2 * world - 1 - owner) * seg, (2 * world - owner) * seg)]
        for i, (qp, kp, _diag) in enumerate(prods):
            fin = last[qp] == (s, i)
            res = backend.polar_block(q_parts[qp], cur[kp], cur[2 + kp], n_keys[qp], prepared,
                                      owner_pos[kp][0], stats[qp], fin, eps, window)
            if fin:
                out[qp] = res
            else:
                stats[qp] = res
        for w in works:
            w.wait()
        if s + 1 < world:
            cur, nxt = nxt, cur
    return out


@torch.no_grad()
def gathered_polar_prefill(q_parts, k_parts, v_parts, positions, params, *, backend=None, group=None,
                           eps=1e-6, window=None, events=None):
    """Same contract as ``ring_polar_prefill``, for sequences whose K/V fit every GPU: one
    all-gather brings the un-expanded K/V of the whole sequence into local HBM (token order),
    then each query segment is ONE kernel launch over the keys it can see (absolute key counts
    do the masking).  Two launches per rank instead of 2N+1 and no statistics carried through
    memory; the launch of the later (longer) segment is issued first and the other one runs
    beside it on a second stream.  ``events`` = two CUDA timing events recorded on the current
    stream before the first and after the last Polar launch (the all-gather lies before them)."""
    backend = backend or CudaBackend()
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    dev = q_parts[0].device
    Hkv, L, dk = k_parts[0].shape[1], k_parts[0].shape[2], k_parts[0].shape[3]
    prepared = backend.prepare_params(params, dev)
    # token-major send buffer (part, k|v, L, Hkv, dk); the gathered slots (rank, part) are put in
    # sequence order with one index_select per tensor
    mine = torch.stack([torch.stack([k_parts[p][0].transpose(0, 1), v_parts[p][0].transpose(0, 1)]) for p in (0, 1)])
    flat = torch.empty((2 * world, 2, L, Hkv, dk), dtype=mine.dtype, device=dev)    # slot 2*rank + part
    dist.all_gather_into_tensor(flat, mine.contiguous(), group=group)
    slot_of_seg = _slot_index(world, dev)
    k_all = flat[:, 0].index_select(0, slot_of_seg).view(2 * world * L, Hkv, dk)
    v_all = flat[:, 1].index_select(0, slot_of_seg).view(2 * world * L, Hkv, dk)

    def run(part):
        p0, p1 = positions[part]
        n_keys = torch.arange(p0 + 1, p1 + 1, device=dev, dtype=torch.float32)
        kv = lambda x: x[:p1].unsqueeze(0).transpose(1, 2)           # (1, Hkv, visible keys, dk) view
        return backend.polar_block(q_parts[part], kv(k_all), kv(v_all), n_keys, prepared, 0, None, True, eps, window)

    if dev.type != "cuda":
        return [run(0), run(1)]
    cur = torch.cuda.current_stream(dev)
    second = _second_stream(dev)
    kv_ready = torch.cuda.Event()
    kv_ready.record(cur)                                             # k_all, v_all (and the queries) are ready here
    if events:
        events[0].record(cur)
    out_hi = run(1)                                                  # long rows first
    second.wait_event(kv_ready)                                      # ... and the short segment beside them
    with torch.cuda.stream(second):
        out_lo = run(0)
    cur.wait_stream(second)
    if events:
        events[1].record(cur)
    for t in out_lo:
        t.record_stream(cur)
    k_all.record_stream(second)
    v_all.record_stream(second)
    return [out_lo, out_hi]


_second = {}
_slots = {}


def _slot_index(world, device):
    """Gathered slot (2*rank + part) of every segment in sequence order; cached per device so that
    no host-to-device copy happens inside a captured step."""
    key = (world, device)
    if key not in _slots:
        _slots[key] = torch.tensor([2 * segment_owner(i, world) + (0 if i < world else 1) for i in range(2 * world)],
                                   device=device)
    return _slots[key]


def _second_stream(device):
    if device.index not in _second:
        _second[device.index] = torch.cuda.Stream(device=device)
    return _second[device.index]


def compose_state_prefix(P_all, Q_all, S0=None):
    """S_in of every segment from the per-segment affine maps, in time order.
    P_all (n_seg, H, dk, dk) and Q_all (n_seg, H, dk, dv) in the [K,V] state layout:
    S_out = P S_in + Q.  Returns (n_seg, H, dk, dv) incoming states and the final state."""
    n_seg = P_all.shape[0]
    S = torch.zeros_like(Q_all[0]) if S0 is None else S0.clone()
    states = []
    for i in range(n_seg):
        states.append(S)
        S = torch.matmul(P_all[i], S) + Q_all[i]
    return torch.stack(states), S


@torch.no_grad()
def cp_gated_delta_scan(q_parts, k_parts, v_parts, g_parts, beta_parts, *, backend=None, group=None,
                        initial_state=None):
    """Gated-delta scan of this rank's two segments with the state handed across ranks as a
    prefix of affine maps.  q_parts [lo, hi] each (1, L, H, dk); k, v (1, L, Hkv, d); g, beta
    (1, L, H).  Returns ([o_lo, o_hi], final_state_of_the_whole_sequence)."""
    backend = backend or CudaBackend()
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    H, dk = q_parts[0].shape[2], q_parts[0].shape[3]
    dv = v_parts[0].shape[3]
    dev = q_parts[0].device
    if dk != dv:
        raise ValueError("the affine-map pass stores the dk x dk map in the state, so it needs dk == dv")
    # four recurrences over the factors of the two segments: (lo, P), (lo, Q), (hi, P), (hi, Q)
    eye = torch.eye(dk, device=dev, dtype=torch.float32).expand(H, dk, dk)
    zero = torch.zeros(H, dk, dv, device=dev, dtype=torch.float32)
    S0b = torch.stack([eye, zero, eye, zero]).contiguous()
    factors = backend.scan_factors(torch.cat(q_parts), torch.cat(k_parts), torch.cat(v_parts), torch.cat(g_parts),
                                   torch.cat(beta_parts))
    _, Sf = backend.scan_recur(factors, [0, 0, 1, 1], S0b, [True, False, True, False], want_output=False)
    mine = torch.stack([Sf[0], Sf[1], Sf[2], Sf[3]]).contiguous()   # P_lo, Q_lo, P_hi, Q_hi
    gathered = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine, group=group)
    P_all = torch.stack([gathered[segment_owner(i, world)][0 if i < world else 2] for i in range(2 * world)])
    Q_all = torch.stack([gathered[segment_owner(i, world)][1 if i < world else 3] for i in range(2 * world)])
    S_in, S_final = compose_state_prefix(P_all, Q_all, initial_state)
    my_states = torch.stack([S_in[rank], S_in[2 * world - 1 - rank]]).contiguous()
    o, _ = backend.scan_recur(factors, [0, 1], my_states, None, want_output=True)
    return [o[0:1], o[1:2]], S_final


@torch.no_grad()
def cp_polar_decode(q, k_cache, v_cache, block_tables, local_lens, total_lens, params, *, backend=None, group=None, eps=1e-6):
    """One decode step of Polar attention for sequences whose K/V were prefilled context-parallel: every rank
    holds the pages of its own segments and the same query q (B,H,dk).  Each rank reduces the keys of ITS cache
    (``local_lens`` (B,) of them, reached through ``block_tables``) to partial statistics (m, L, sum p^2, sum p v),
    one small all-gather shares them, and every rank merges all partials with the rule of the single-GPU kernel
    (L and the sums scale by e^(m_i - m), the squares by its square; the null sink is folded once, for the whole
    context of ``total_lens`` keys).  The single-device statement of the same computation is the reference's
    paged decode, kernel/polar_triton.py:796-858.  Full-context attention only (no window).
    Returns c (B,H,dk), mag (B,H) on every rank."""
    backend = backend or CudaBackend()
    world = dist.get_world_size(group)
    prepared = backend.prepare_params(params, q.device)
    stats, sums = backend.decode_partials(q, k_cache, v_cache, block_tables, local_lens, total_lens, prepared, eps)
    B, H, P, dk = sums.shape
    mine = torch.cat([stats, sums], dim=-1).contiguous()                        # (B, H, P, 4 + dk)
    gathered = torch.empty((world * B, H, P, 4 + dk), dtype=mine.dtype, device=mine.device)
    dist.all_gather_into_tensor(gathered, mine, group=group)
    allp = gathered.view(world, B, H, P, 4 + dk).permute(1, 2, 0, 3, 4).reshape(B, H, world * P, 4 + dk)     # every rank's partials side by side
    return backend.decode_merge(allp[..., :4].contiguous(), allp[..., 4:].contiguous(), total_lens, prepared, q.dtype, eps)


@torch.no_grad()
def cp_conv_halos(x_parts, kernel_size, *, group=None):
    """The K-1 input rows that precede each of this rank's two segments (zeros for the first
    segment of the sequence).  x_parts [lo, hi] each (L, C).  Returns [halo_lo, halo_hi],
    each (C, K-1) in the conv-state layout (oldest first), ready to be passed as
    ``initial_states`` of the prefill conv."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    Kh = kernel_size - 1
    tails = [x[-Kh:].contiguous() for x in x_parts]                 # what the NEXT segment needs
    my_segs = [rank, 2 * world - 1 - rank]
    halos = [torch.zeros_like(tails[0]), torch.zeros_like(tails[1])]
    ops = []
    for part, seg_idx in enumerate(my_segs):
        nxt_seg = seg_idx + 1
        if nxt_seg < 2 * world:
            dst = segment_owner(nxt_seg, world)
            if dst == rank:                                         # my own two segments are adjacent (seg N-1, N)
                halos[my_segs.index(nxt_seg)] = tails[part].clone()
            else:
                ops.append(dist.P2POp(dist.isend, tails[part], dst, group, tag=nxt_seg))
        prev_seg = seg_idx - 1
        if prev_seg >= 0:
            src = segment_owner(prev_seg, world)
            if src != rank:
                ops.append(dist.P2POp(dist.irecv, halos[part], src, group, tag=seg_idx))
    if ops:
        for w in dist.batch_isend_irecv(ops):
            w.wait()
    return [h.transpose(0, 1).contiguous() for h in halos]


@dataclass
class GlobalLayerShard:
    """One rank's slice of a sequence for the global-layer mixing step (two zig-zag segments)."""
    q: list      # [lo, hi] each (1, L, H, dk)
    k: list      # (1, L, Hkv, dk)
    v: list
    g: list      # (1, L, H) log decay
    beta: list   # (1, L, H)
    positions: list


def shard_sequence(t, rank, world):
    """Cut full-sequence tensors (1, T, ...) into this rank's two zig-zag segments."""
    T = t["q"].shape[1]
    (a0, a1), (b0, b1) = zigzag_segments(T, world)[rank]
    cut = lambda x: [x[:, a0:a1].contiguous(), x[:, b0:b1].contiguous()]
    return GlobalLayerShard(q=cut(t["q"]), k=cut(t["k"]), v=cut(t["v"]), g=cut(t["g"]), beta=cut(t["beta"]),
                            positions=[(a0, a1), (b0, b1)])


_side = {}


def _side_resources(device, group):
    """A high-priority stream for the memory branch and a second communicator for its all-gather,
    so that the gather does not queue behind the ring's send/recv on the first communicator's
    stream.  Created once per (device, group); every rank must reach the first call together."""
    key = (device.index, id(group))
    if key not in _side:
        ranks = dist.get_process_group_ranks(group) if group is not None else None
        _side[key] = (torch.cuda.Stream(device=device, priority=-1), dist.new_group(ranks=ranks, backend="nccl"))
    return _side[key]


GATHER_LIMIT_BYTES = 8 << 30


def default_polar_mode(shard, world):
    """"gather" while the K/V of the whole sequence (what every rank then holds) stay below
    ``GATHER_LIMIT_BYTES``, else "ring" (memory per GPU stays O(T/N))."""
    kv_bytes = world * sum(x.numel() * x.element_size() for x in (*shard.k, *shard.v))
    return "gather" if kv_bytes <= GATHER_LIMIT_BYTES else "ring"


@torch.no_grad()
def cp_global_layer_prefill(shard, params, *, backend=None, group=None, overlap=None, polar_mode=None, window=None):
    """Polar pass + gated-delta prefix scan for one rank's shard.  Returns
    ([(c, mag) lo, hi], [o lo, hi], final memory state).  On CUDA tensors the memory branch runs
    beside the attention on a side stream (``overlap``, default on for CUDA).  ``polar_mode``:
    "gather" (all-gather K/V, one launch per query segment), "ring" (K/V blocks travel a ring,
    2N+1 launches with carried statistics; memory per GPU stays O(T/N)), default: gather while
    the whole sequence's K/V is below ``GATHER_LIMIT_BYTES``.  ``window``: sliding-window attention
    (keys older than ``window`` positions are masked, as in the reference's local Polar layers)."""
    tr = lambda x: x.transpose(1, 2)
    dev = shard.q[0].device
    if overlap is None:
        overlap = dev.type == "cuda"
    if overlap:
        cur = torch.cuda.current_stream(dev)
        side, scan_group = _side_resources(dev, group)
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            o, S = cp_gated_delta_scan(shard.q, shard.k, shard.v, shard.g, shard.beta, backend=backend,
                                       group=scan_group)
    if polar_mode is None:
        polar_mode = default_polar_mode(shard, dist.get_world_size(group))
    if polar_mode not in ("gather", "ring"):
        raise ValueError(f"polar_mode must be 'gather' or 'ring', not {polar_mode!r}")
    polar_fn = gathered_polar_prefill if polar_mode == "gather" else ring_polar_prefill
    polar = polar_fn([tr(x) for x in shard.q], [tr(x) for x in shard.k], [tr(x) for x in shard.v],
                     shard.positions, params, backend=backend, group=group, window=window)
    if overlap:
        cur.wait_stream(side)
        for t in (*o, S):
            t.record_stream(cur)
    else:
        o, S = cp_gated_delta_scan(shard.q, shard.k, shard.v, shard.g, shard.beta, backend=backend, group=group)
    return polar, o, S


class CapturedPrefill:
    """``cp_global_layer_prefill`` for one fixed shard shape, captured into a CUDA graph.

    At 8 ranks a 64K-token step is about forty short launches and a dozen NCCL calls per rank;
    issued one by one from Python the host is slower than the GPU.  Capturing the step (kernels,
    ring send/recv, the state all-gather, both streams) and replaying it removes the host from
    the step.  Every rank must construct the object and call ``replay`` the same number of times.

    ``static`` is the shard the graph reads: fill its tensors (``load``, or copy into them from
    pinned host memory) and call ``replay``; the returned tensors are owned by the graph and are
    overwritten by the next replay.
    """

    def __init__(self, shard, params, *, group=None, warmup=3, polar_mode=None, window=None, static=None):
        dev = shard.q[0].device
        self.group = group
        self.polar_mode = polar_mode
        self.window = window
        if static is None:
            static = GlobalLayerShard(positions=list(shard.positions),
                                      **{f: [x.clone() for x in getattr(shard, f)] for f in ("q", "k", "v", "g", "beta")})
        else:                                              # caller-owned input tensors (e.g. views of one packed buffer)
            for f in ("q", "k", "v", "g", "beta"):
                for dst, src in zip(getattr(static, f), getattr(shard, f)):
                    dst.copy_(src)
        self.static = static
        self.params = params
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):                      # warm up off the default stream: lazy
            for _ in range(warmup):                        # initialisation must not land in the capture
                cp_global_layer_prefill(self.static, params, group=group, polar_mode=polar_mode, window=window)
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        dist.barrier(group=group)
        self.graph = torch.cuda.CUDAGraph()
        ok = 1
        self.error = None
        try:
            with torch.cuda.graph(self.graph, capture_error_mode="thread_local"):
                try:
                    self.outputs = cp_global_layer_prefill(self.static, params, group=group, polar_mode=polar_mode, window=window)
                except Exception as inner:                 # noqa: BLE001 - keep the first error: ending the
                    self.error = inner                     # capture after it reports "unjoined work" instead
                    raise
        except Exception as exc:                           # noqa: BLE001 - reported, then agreed on below
            ok = 0
            self.error = self.error or exc
        flag = torch.tensor([ok], device=dev, dtype=torch.int32)
        torch.cuda.synchronize(dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
        self.captured = bool(flag.item())                  # all ranks replay, or all run eagerly
        if not self.captured:
            self.graph = None

    def close(self):
        """Release the graph (and the NCCL work captured in it).  Call it on every rank before the
        process group is destroyed."""
        self.outputs = None
        if self.graph is not None:
            self.graph.reset()
            self.graph = None
        self.captured = False

    def load(self, shard):
        for f in ("q", "k", "v", "g", "beta"):
            for dst, src in zip(getattr(self.static, f), getattr(shard, f)):
                dst.copy_(src, non_blocking=True)

    def replay(self):
        if self.captured:
            self.graph.replay()
            return self.outputs
        return cp_global_layer_prefill(self.static, self.params, group=self.group, polar_mode=self.polar_mode,
                                       window=self.window)


def _packed_views(buf, templates):
    """Views of one byte buffer with the shapes and dtypes of ``templates`` (256-byte aligned offsets)."""
    views, off = [], 0
    for t in templates:
        n = t.numel() * t.element_size()
        views.append(buf[off:off + n].view(t.dtype).view(t.shape))
        off += (n + 255) // 256 * 256
    return views


def _packed_bytes(templates):
    return sum((t.numel() * t.element_size() + 255) // 256 * 256 for t in templates)


class HostFedCapturedPrefill:
    """Context-parallel steps fed from pinned host memory: ``depth`` captured steps with their own
    input buffers on a three-stream pipeline (copy-in | graph replay | copy-out), so that the PCIe
    copies of neighbouring steps hide behind the replay.  Every rank must construct it, call
    ``submit`` the same number of times and ``close`` it before the process group goes away.

    A step moves ONE buffer in each direction: the inputs of a step are views of one device buffer
    and ``host_shard(slot)`` hands out matching views of one pinned buffer for the producer of the
    activations to fill, the seven results are packed on the device and leave in one copy.  (Ten
    copies in and seven out per step, as separate tensors need, cost more in per-copy latency than
    in bytes once eight ranks share the host.)  The copy-in stream runs up to ``depth`` - 1 steps
    ahead of the replays, so a late copy on one rank does not stall the collectives of all ranks.

    ``submit(host_shard)`` takes a ``GlobalLayerShard`` of pinned tensors - one of ``host_shard(i)``
    for the single-copy path, any other pinned shard is copied tensor by tensor - and returns a
    ticket; ``results(ticket)`` waits for that step's copy and returns the pinned outputs
    [c_lo, mag_lo, c_hi, mag_hi, o_lo, o_hi, S] (reused ``depth`` submits later).  ``copy_only``
    skips the replays: what is left is the host <-> device traffic of the pipeline alone."""

    FIELDS = ("q", "k", "v", "g", "beta")

    def __init__(self, shard, params, *, group=None, polar_mode=None, depth=3, window=None, copy_only=False):
        dev = shard.q[0].device
        torch.cuda.set_device(dev)                       # pinned allocations below belong to this rank's device
        self.device, self.depth, self.copy_only = dev, depth, copy_only
        templates = [x for f in self.FIELDS for x in getattr(shard, f)]
        nbytes = _packed_bytes(templates)
        self.in_dev = [torch.empty(nbytes, dtype=torch.uint8, device=dev) for _ in range(depth)]
        self.in_host = [torch.empty(nbytes, dtype=torch.uint8, pin_memory=True) for _ in range(depth)]
        self._host_shards = [self._as_shard(b, shard) for b in self.in_host]
        self.caps = [CapturedPrefill(shard, params, group=group, polar_mode=polar_mode, window=window,
                                     static=self._as_shard(self.in_dev[i], shard)) for i in range(depth)]
        self.copy_in, self.compute, self.copy_out = (torch.cuda.Stream(device=dev) for _ in range(3))
        self.in_free = [None] * depth
        self.out_done = [None] * depth
        self.out_dev = [None] * depth
        self.out_host = [None] * depth
        self.out_views = [None] * depth
        self.step = 0

    def _as_shard(self, buf, like):
        views = _packed_views(buf, [x for f in self.FIELDS for x in getattr(like, f)])
        it = iter(views)
        return GlobalLayerShard(positions=list(like.positions), **{f: [next(it) for _ in getattr(like, f)] for f in self.FIELDS})

    def host_shard(self, slot):
        """Pinned views (one packed buffer) for the inputs of a step; fill them, then ``submit`` them."""
        return self._host_shards[slot % self.depth]

    @staticmethod
    def _flat(outputs):
        polar, o, S = outputs
        return [polar[0][0], polar[0][1], polar[1][0], polar[1][1], o[0], o[1], S]

    def submit(self, host_shard):
        slot = self.step % self.depth
        self.step += 1
        cap = self.caps[slot]
        packed_src = next((i for i, h in enumerate(self._host_shards) if h is host_shard), None)
        with torch.cuda.stream(self.copy_in):
            if self.in_free[slot] is not None:
                self.copy_in.wait_event(self.in_free[slot])
            if packed_src is not None:
                self.in_dev[slot].copy_(self.in_host[packed_src], non_blocking=True)
            else:
                for f in self.FIELDS:
                    for dst, src in zip(getattr(cap.static, f), getattr(host_shard, f)):
                        dst.copy_(src, non_blocking=True)
            arrived = torch.cuda.Event()
            arrived.record(self.copy_in)
        with torch.cuda.stream(self.compute):
            self.compute.wait_event(arrived)
            if self.out_done[slot] is not None:                 # the slot's packed results were read out
                self.compute.wait_event(self.out_done[slot])
            outs = self._flat(cap.outputs if self.copy_only and cap.outputs is not None else cap.replay())
            if self.out_dev[slot] is None:
                nb = _packed_bytes(outs)
                self.out_dev[slot] = torch.empty(nb, dtype=torch.uint8, device=self.device)
                self.out_host[slot] = torch.empty(nb, dtype=torch.uint8, pin_memory=True)
                self.out_views[slot] = (_packed_views(self.out_dev[slot], outs), _packed_views(self.out_host[slot], outs))
            for dst, src in zip(self.out_views[slot][0], outs):  # pack on the device: seven small device copies
                dst.copy_(src, non_blocking=True)
            computed = torch.cuda.Event()
            computed.record(self.compute)
        self.in_free[slot] = computed
        with torch.cuda.stream(self.copy_out):
            self.copy_out.wait_event(computed)
            self.out_host[slot].copy_(self.out_dev[slot], non_blocking=True)
            done = torch.cuda.Event()
            done.record(self.copy_out)
        self.out_done[slot] = done
        return self.step - 1

    def results(self, ticket):
        if ticket < self.step - self.depth or ticket >= self.step:
            raise ValueError("that step's result slot has been reused (or the step was never submitted)")
        self.out_done[ticket % self.depth].synchronize()
        return self.out_views[ticket % self.depth][1]

    def drain(self, stream=None):
        stream = stream or torch.cuda.current_stream(self.device)
        for s in (self.copy_in, self.compute, self.copy_out):
            stream.wait_stream(s)

    def close(self):
        torch.cuda.synchronize(self.device)
        for cap in self.caps:
            cap.close()
