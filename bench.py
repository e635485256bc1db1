"""Benchmark of ATMA's global-layer mixing hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Metric (BASELINE.json): global-layer prefill tok/s at a 64K-token context, with decode tok/s
at batch 64 x 32K context reported beside it, each against its roofline.

A "step" is one pass of one global layer's mixing over one 65,536-token sequence:
Polar prefill (H=8, Hkv=2, dk=128, bf16, full causal context) followed by the gated-delta
chunked scan (H=8, d=128, chunk 64, fp32 state).  Inputs are seeded synthetic tensors with
the value distributions BASELINE.json names.  `value` times the kernels with the inputs
resident in HBM; `e2e` times the same public API calls with pinned-host inputs copied in and
the results copied out inside the timed region.  With N > 1 ranks the SAME single sequence is
sharded over the ranks (context parallel: NCCL ring of K/V blocks, gated-delta state prefix),
so scaling is strong; the decode leg shards its batch of 64 sequences with no collective.

`--impl reference` times the CPU oracle (a restatement of the reference's pure-PyTorch
implementation, the only implementation of this path the reference can run without a GPU)
on the host cores, on a bounded sample of the same workload.
"""

import argparse
import json
import os
import statistics
import sys
import time

import torch
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

H, HKV, DK, CHUNK = 8, 2, 128, 64
T_PREFILL = 65536
DEC_B, DEC_CTX, DEC_BLOCK = 64, 32768, 256
METRIC = "global_layer_prefill_tok_s_at_64k"
# roofline.traffic is not measured by the run that prints it (that needs a profiler): it is the DRAM
# traffic (dram__bytes_read.sum + dram__bytes_write.sum, one ncu pass) of the same launch at the same
# shape, scaled by the token count / cache bytes where the run uses another size.
PREFILL_TRAFFIC_64K = 336.0e6      # read 231 MB + write 105 MB for the 65,536-token launch
DECODE_TRAFFIC_RATIO = 2155.3 / 2147.5   # read 2147.8 MB + write 5.8-9.3 MB for 2147.5 MB of cache rows (64 x 32K)
REF_SAMPLE_TOKENS = 4096           # what one step of the reference arm times, whatever N, K and W are


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm=d["hbm_gbs"], tf_burst=d["bf16_tflops"], tf_sustained=d["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm=6650.0, tf_burst=1590.0, tf_sustained=1400.0, source="fallback")


def polar_flops(T):
    return 4.0 * H * DK * T * (T + 1) / 2.0          # QK^T + PV over the causal triangle


def scan_flops(T):
    return 155648.0 * H * T                           # per token per head: 4C dk + 6 dk dv + 3C dv


class ClockSampler:
    """SM clock and throttle reasons during the timed region, read through NVML every millisecond
    on a background thread (read-only queries), so that a timed region of a few tens of
    milliseconds still holds samples.  ``mark_begin`` / ``mark_end`` cut the samples to the region."""
    NAMES = (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40), ("sw_thermal_slowdown", 0x20), ("sw_power_cap", 0x4))

    def __init__(self, gpu_index):
        self.gpu, self.rows, self.thread, self.stop_flag = gpu_index, [], None, False
        self.t_begin = self.t_end = None

    def _index(self):
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            try:
                return int(vis.split(",")[self.gpu])
            except (ValueError, IndexError):
                pass
        return self.gpu

    def start(self):
        import threading
        try:
            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(self._index())
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
        except Exception:                                   # noqa: BLE001 - no NVML: no samples
            return

        def loop():
            while not self.stop_flag:
                try:
                    mhz = float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM))
                    reasons = int(pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(h))
                    self.rows.append((time.time(), mhz, reasons))
                except Exception:                           # noqa: BLE001
                    pass
                time.sleep(0.001)

        self.thread = threading.Thread(target=loop, daemon=True)
        self.thread.start()

    def mark_begin(self):
        self.t_begin = time.time()

    def mark_end(self):
        self.t_end = time.time()

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.thread is None:
            return out
        if self.t_end is None:
            self.t_end = time.time()
        self.stop_flag = True
        self.thread.join(timeout=2)
        inside = [r for r in self.rows if self.t_begin is not None and self.t_begin <= r[0] <= self.t_end]
        if inside:
            bits = 0
            for r in inside:
                bits |= r[2]
            out.update(sm_mhz=statistics.median(r[1] for r in inside), sm_max_mhz=self.max_mhz,
                       reasons=[n for n, bit in self.NAMES if bits & bit], samples=len(inside), window="timed region")
        return out


def make_prefill_inputs(seed, device=None, pinned=False):
    """One 64K-token sequence for one global layer: q ~ N(0,1) bf16 (B,T,H,dk), k/v with the
    2 un-expanded KV heads for Polar; the memory branch sees the same q and the expanded k, v
    (inference/models/atma.py:416-420), gates as BASELINE config 3 names them."""
    g = torch.Generator().manual_seed(seed)
    T = T_PREFILL
    t = dict(
        q=torch.randn(1, T, H, DK, generator=g).to(torch.bfloat16),
        k=torch.randn(1, T, HKV, DK, generator=g).to(torch.bfloat16),
        v=torch.randn(1, T, HKV, DK, generator=g).to(torch.bfloat16),
        g=(-F.softplus(torch.randn(1, T, H, generator=g))).float(),
        beta=torch.sigmoid(torch.randn(1, T, H, generator=g)).float(),
    )
    if pinned:
        t = {n: x.pin_memory() for n, x in t.items()}
    if device is not None:
        t = {n: x.to(device) for n, x in t.items()}
    return t


def default_polar_params(device):
    return dict(v_null=torch.zeros(H, DK, device=device), null_base=torch.full((H,), 2.0, device=device),
                null_slope_raw=torch.full((H,), 0.5, device=device), len_gain_raw=torch.full((H,), -1.0, device=device),
                mag_beta_raw=torch.full((H,), -1.5, device=device))


def prefill_step(ab, t, n_keys, params, events=None, ready=None):
    """Polar prefill + gated-delta scan through the public API (the two independent branches
    run on two streams).  ``ready``: the event after which the resident inputs are valid, so that
    the memory branch of a step does not wait for the previous step's attention kernel.
    Returns (c, mag, o, S)."""
    from atma_b200.mixing import global_layer_mixing
    return global_layer_mixing(t["q"], t["k"], t["v"], t["g"], t["beta"], n_keys, params, events=events,
                               inputs_ready=ready)


def bench_decode(ab, device, steps, warmup, peaks):
    """Decode of one global layer's mixing at batch 64 x 32K context: paged Polar decode that first stores the
    new token's K/V rows, gated-delta state step beside it.  Context larger than L2 by 17x."""
    g = torch.Generator().manual_seed(3)
    nblk_seq = DEC_CTX // DEC_BLOCK
    num_blocks = DEC_B * nblk_seq
    k_cache = torch.randn(num_blocks, DEC_BLOCK, HKV, DK, device=device, dtype=torch.bfloat16)
    v_cache = torch.randn(num_blocks, DEC_BLOCK, HKV, DK, device=device, dtype=torch.bfloat16)
    bt = torch.randperm(num_blocks, generator=g).to(torch.int32).view(DEC_B, nblk_seq).to(device)
    cl = torch.full((DEC_B,), DEC_CTX, dtype=torch.int32, device=device)
    q = torch.randn(DEC_B, H, DK, device=device, dtype=torch.bfloat16)
    kn = torch.randn(DEC_B, HKV, DK, device=device, dtype=torch.bfloat16)
    vn = torch.randn(DEC_B, HKV, DK, device=device, dtype=torch.bfloat16)
    slot_map = (bt[:, -1].long() * DEC_BLOCK + DEC_BLOCK - 1).to(torch.int32)
    state = torch.randn(DEC_B, H, DK, DK, device=device) * 0.1
    gamma = torch.rand(DEC_B, H, device=device) * 0.1 + 0.9
    beta = torch.rand(DEC_B, H, device=device)
    slots = torch.arange(DEC_B, device=device)
    params = default_polar_params(device)

    side = torch.cuda.Stream(device=device)

    from atma_b200.polar import DECODE_BESIDE_MAX_ROWS

    def step():
        # the memory branch reads and writes nothing the attention branch touches: it runs beside it, as the two
        # branches of the reference's decode layer may (inference/models/atma.py:572-590) - for small batches beside
        # the merge launch (the decode call's own hook), else beside the whole call (fork / join)
        if DEC_B <= DECODE_BESIDE_MAX_ROWS:
            return ab.polar_attention_decode(
                q, k_cache, v_cache, bt, cl, append=(kn, vn, slot_map),
                beside=lambda: ab.gated_delta_decode_step_fused(q, kn, vn, state, slots, gamma=gamma, beta=beta), **params)
        cur = torch.cuda.current_stream(device)
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            r = ab.gated_delta_decode_step_fused(q, kn, vn, state, slots, gamma=gamma, beta=beta)   # un-expanded KV heads
        # the new token's K/V rows are stored by the decode call itself (the key-range CTA that ends with them)
        c, mag = ab.polar_attention_decode(q, k_cache, v_cache, bt, cl, append=(kn, vn, slot_map), **params)
        cur.wait_stream(side)
        return c, mag, r

    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    pe = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(steps)]
    e0.record()
    for i in range(steps):
        pe[i][0].record()
        ab.polar_attention_decode(q, k_cache, v_cache, bt, cl, append=(kn, vn, slot_map), **params)
        pe[i][1].record()
        pe[i][2].record()
        ab.gated_delta_decode_step_fused(q, kn, vn, state, slots, gamma=gamma, beta=beta)
        pe[i][3].record()
    e1.record()
    torch.cuda.synchronize()
    eager_ms = e0.elapsed_time(e1) / steps
    polar_ms = sum(e[0].elapsed_time(e[1]) for e in pe) / steps
    mem_step_ms = sum(e[2].elapsed_time(e[3]) for e in pe) / steps
    # The memory step is a ~15 us kernel: one launch between two events carries the events' own latency.  Timed
    # again as 8 launches back to back over 4 rotating state tables (together larger than L2), per launch.
    tables = [state] + [torch.randn_like(state) * 0.1 for _ in range(3)]
    for tb in tables:
        ab.gated_delta_decode_step_fused(q, kn, vn, tb, slots, gamma=gamma, beta=beta)
    torch.cuda.synchronize()
    b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda._sleep(2_000_000)                                  # the host gets ahead of the device
    b0.record()
    for i in range(8):
        ab.gated_delta_decode_step_fused(q, kn, vn, tables[i % 4], slots, gamma=gamma, beta=beta)
    b1.record()
    torch.cuda.synchronize()
    mem_step_b2b_ms = b0.elapsed_time(b1) / 8
    del tables
    # the step as the engine runs it: captured once, replayed (inference/engine/model_runner.py:254-310)
    ms, graphed = eager_ms, False
    try:
        warm = torch.cuda.Stream(device=device)
        warm.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(warm):
            step()
        torch.cuda.current_stream(device).wait_stream(warm)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        for _ in range(warmup):
            graph.replay()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(steps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        ms, graphed = e0.elapsed_time(e1) / steps, True
        del graph
    except Exception as exc:                                     # noqa: BLE001 - the eager timing stands
        print(f"[bench] decode step not captured: {exc!r}", file=sys.stderr)
    kv_bytes = 2.0 * DEC_B * DEC_CTX * HKV * DK * 2
    state_bytes = 2.0 * DEC_B * H * DK * DK * 4
    return {
        "metric": "global_layer_decode_tok_s_at_b64_ctx32k", "value": DEC_B / (ms * 1e-3), "unit": "tok/s",
        "ms_per_step": ms, "ms_per_step_eager": eager_ms, "cuda_graph": graphed,
        "config": {"batch": DEC_B, "context": DEC_CTX, "block_size": DEC_BLOCK, "layers": 1},
        "roofline": {"kernel": "polar_decode (split + merge)", "bound": "hbm",
                     "achieved": kv_bytes / (polar_ms * 1e-3) / 1e9, "peak": peaks["hbm"], "unit": "GB/s",
                     "frac": kv_bytes / (polar_ms * 1e-3) / 1e9 / peaks["hbm"],
                     # ncu capture of the 64 x 32K launch (two DRAM counters, one pass): 2155 MB moved for 2147.5 MB
                     # algorithmic; a sharded batch scales it by its cache bytes.
                     "traffic": kv_bytes * DECODE_TRAFFIC_RATIO,
                     "algorithmic_bytes": kv_bytes, "kernel_ms": polar_ms, "peak_source": peaks["source"]},
        "memory_step": {"kernel": "gated_delta_step_wide_kernel", "kernel_ms": mem_step_b2b_ms,
                        "kernel_ms_single_launch_between_events": mem_step_ms, "algorithmic_bytes": state_bytes,
                        "achieved": state_bytes / (mem_step_b2b_ms * 1e-3) / 1e9, "unit": "GB/s",
                        "frac": state_bytes / (mem_step_b2b_ms * 1e-3) / 1e9 / peaks["hbm"],
                        "method": "8 launches back to back over 4 rotating state tables (larger than L2), per launch"},
        "step_bytes": kv_bytes + state_bytes,
        "step_hbm_frac": (kv_bytes + state_bytes) / (ms * 1e-3) / 1e9 / peaks["hbm"],
    }


def cpu_baseline(sample_T, threads):
    """The oracle (restating the reference's polar_reduce + gated_delta_chunked CPU path) on
    one global layer at `sample_T` tokens.  Returns seconds."""
    import oracle
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(0)
    q = torch.randn(1, H, sample_T, DK, generator=g)
    k = torch.randn(1, HKV, sample_T, DK, generator=g)
    v = torch.randn(1, HKV, sample_T, DK, generator=g)
    params = {n: x.cpu() for n, x in default_polar_params("cpu").items()}
    n_keys = torch.arange(1, sample_T + 1, dtype=torch.float32)
    glog = -F.softplus(torch.randn(1, sample_T, H, generator=g))
    beta = torch.sigmoid(torch.randn(1, sample_T, H, generator=g))
    t0 = time.perf_counter()
    oracle.polar_prefill_oracle(q, k, v, n_keys, params)
    ke, ve = k.repeat_interleave(H // HKV, 1), v.repeat_interleave(H // HKV, 1)
    oracle.chunk_gated_delta_rule_oracle(q.transpose(1, 2), ke.transpose(1, 2), ve.transpose(1, 2), glog, beta, chunk=CHUNK)
    return time.perf_counter() - t0


def run_reference(args, rank):
    """The reference arm: the CPU oracle (a restatement of the reference's pure-PyTorch path - the reference
    itself is Python that cannot travel to this box) on all host cores.  Each step times the SAME bounded
    sample of the workload, REF_SAMPLE_TOKENS tokens, whatever N, K and W are."""
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    sample_T = REF_SAMPLE_TOKENS
    for _ in range(args.warmup):
        cpu_baseline(sample_T, threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_baseline(sample_T, threads)
    sec = (time.perf_counter() - t0) / max(1, args.steps)
    val = sample_T / sec
    sample = (f"one global layer (Polar materialised + gated-delta chunked, fp32) at T={sample_T} tokens; "
              f"Polar cost is quadratic, so tok/s at 64K would be ~{T_PREFILL // sample_T}x lower")
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": "tok/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            # the same workload as the GPU arm; each step times a bounded sample of it (see cpu_baseline.sample)
            "config": {"workload": f"global-layer mixing prefill: Polar attention + gated-delta scan, one {T_PREFILL}-token sequence",
                       "tokens": T_PREFILL, "heads": H, "kv_heads": HKV, "head_dim": DK, "chunk": CHUNK, "window": None,
                       "sample_tokens": sample_T},
            "cpu_baseline": {"value": val, "unit": "tok/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    emit(line)


def bench_prep(ab, dev, tokens, n_seqs, iters):
    """The fused q/k/v preparation of a packed prefill (RMSNorm, three residual convs, state rows,
    cache scatter) on `n_seqs` equal sequences.  Algorithmic bytes: the q half of the q|gate
    projection, k, v read; q, k, v and the two cache rows written."""
    from atma_b200.layer import PackedMaps
    g = torch.Generator().manual_seed(1)
    per = tokens // n_seqs
    total = per * n_seqs
    maps = PackedMaps([per] * n_seqs, list(range(n_seqs)), dev)
    q_gate = torch.randn(total, H, 2 * DK, generator=g).bfloat16().to(dev)
    k = torch.randn(total, HKV, DK, generator=g).bfloat16().to(dev)
    v = torch.randn(total, HKV, DK, generator=g).bfloat16().to(dev)
    w = [(torch.randn(C, 4, generator=g) * 0.3).bfloat16().to(dev) for C in (H * DK, HKV * DK, HKV * DK)]
    st = [torch.zeros(n_seqs, C, 3, dtype=torch.bfloat16, device=dev) for C in (H * DK, HKV * DK, HKV * DK)]
    kc = torch.zeros(total, HKV, DK, dtype=torch.bfloat16, device=dev)
    vc = torch.zeros_like(kc)
    # cache slots as the engine hands them out: 256-token pages in random order, rows in order inside a page
    pages = torch.randperm((total + DEC_BLOCK - 1) // DEC_BLOCK, generator=g)
    t_idx = torch.arange(total)
    sm = (pages[t_idx // DEC_BLOCK] * DEC_BLOCK + t_idx % DEC_BLOCK).to(dev)
    kc = torch.zeros(pages.numel() * DEC_BLOCK, HKV, DK, dtype=torch.bfloat16, device=dev)
    vc = torch.zeros_like(kc)
    run = lambda: ab.qkv_prep_prefill(q_gate, k, v, *w, *st, maps.token_seq_starts, maps.token_seq_ends,
                                      maps.token_seq_slots, kc, vc, sm)
    for _ in range(3):
        run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda._sleep(20_000_000)          # keep the GPU busy while the host queues the launches back to back
    e0.record()
    for _ in range(iters):
        run()
    e1.record()
    torch.cuda.synchronize()
    nbytes = total * (2 * H + 5 * HKV) * DK * 2.0
    ms = e0.elapsed_time(e1) / iters
    # the same timing method on a plain device copy of the q|gate projection, as a reference point
    dst = torch.empty_like(q_gate)
    dst.copy_(q_gate)
    torch.cuda.synchronize()
    torch.cuda._sleep(20_000_000)
    e0.record()
    for _ in range(iters):
        dst.copy_(q_gate)
    e1.record()
    torch.cuda.synchronize()
    bench_prep.copy_gbs = 2.0 * q_gate.numel() * 2 / (e0.elapsed_time(e1) / iters * 1e-3) / 1e9
    return ms, nbytes, total


def profile_case(which):
    """A small case of one kernel for an ncu capture: inputs larger than L2, well under 1 GB,
    five launches.  Prints the shape so that per-launch figures can be scaled."""
    import atma_b200 as ab
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(0)
    if which == "prefill":
        B, T = 1, 16384
        q = torch.randn(B, T, H, DK, generator=g).bfloat16().to(dev)
        k = torch.randn(B, T, HKV, DK, generator=g).bfloat16().to(dev)
        v = torch.randn(B, T, HKV, DK, generator=g).bfloat16().to(dev)
        n = torch.arange(1, T + 1, dtype=torch.float32, device=dev)
        P = default_polar_params(dev)
        for _ in range(5):
            ab.polar_attention_fwd(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), n, **P)
        info = {"kernel": "polar_prefill_sm100_kernel", "B": B, "T": T, "flops_per_launch": polar_flops(T)}
    elif which == "decode":
        Bd, ctx = 16, 16384
        nblk = ctx // DEC_BLOCK
        kc = torch.randn(Bd * nblk, DEC_BLOCK, HKV, DK, device=dev, dtype=torch.bfloat16)
        vc = torch.randn(Bd * nblk, DEC_BLOCK, HKV, DK, device=dev, dtype=torch.bfloat16)
        bt = torch.randperm(Bd * nblk, generator=g).int().view(Bd, nblk).to(dev)
        cl = torch.full((Bd,), ctx, dtype=torch.int32, device=dev)
        q = torch.randn(Bd, H, DK, device=dev, dtype=torch.bfloat16)
        P = default_polar_params(dev)
        for _ in range(5):
            ab.polar_attention_decode(q, kc, vc, bt, cl, **P)
        info = {"kernel": "polar_decode_split_mma_kernel", "B": Bd, "context": ctx,
                "bytes_per_launch": 2.0 * Bd * ctx * HKV * DK * 2}
    elif which == "epilogue":
        total = 65536
        q_gate = torch.randn(total, H, 2 * DK, generator=g).bfloat16().to(dev)
        c = torch.randn(total, H, DK, generator=g).bfloat16().to(dev)
        gate2 = torch.randn(total, H * DK, generator=g).bfloat16().to(dev)
        res = {}
        for name, fn, nbytes in (("sigmoid_gate_mul", lambda: ab.sigmoid_gate_mul(c, q_gate[..., DK:]), 3.0 * c.numel() * 2),
                                 ("rms_sigmoid_gate", lambda: ab.rms_sigmoid_gate(c, gate2), 3.0 * c.numel() * 2)):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda._sleep(20_000_000)
            e0.record()
            for _ in range(5):
                fn()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / 5
            res[name] = {"ms": ms, "bytes_per_launch": nbytes, "gbs": nbytes / (ms * 1e-3) / 1e9}
        info = {"kernel": "sigmoid_gate_mul_kernel, rms_sigmoid_gate_kernel", "tokens": total, **res}
    elif which == "linear":
        # the MLP of one layer at decode batch 8 (hidden 1024, 4x): fc + gate (16.8 MB of weights), proj (8.4 MB); the
        # weights cycle through 12 copies (302 MB) so that every launch reads them from HBM, not from L2
        import torch.nn.functional as F
        D, Fh, copies = 1024, 4096, 12
        w_fc = [(torch.randn(2 * Fh, D, generator=g) / 32).bfloat16().to(dev) for _ in range(copies)]
        w_pr = [(torch.randn(D, Fh, generator=g) / 64).bfloat16().to(dev) for _ in range(copies)]

        def timed_ring(fn, nbytes, iters=24):
            for i in range(copies):
                fn(i)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda._sleep(20_000_000)
            e0.record()
            for i in range(iters):
                fn(i % copies)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / iters
            return {"ms": ms, "bytes_per_launch": nbytes, "gbs": nbytes / (ms * 1e-3) / 1e9}

        res = {}
        for Bs in (8, 16, 64):
            x = torch.randn(Bs, D, generator=g).bfloat16().to(dev)
            a_in = torch.randn(Bs, Fh, generator=g).bfloat16().to(dev)

            def eager_fc(i):
                y = F.linear(x, w_fc[i])
                return ab.squared_relu_gate(y[:, :Fh], y[:, Fh:])
            r = {"cublas_fc_then_gate": timed_ring(eager_fc, 2.0 * 2 * Fh * D),
                 "cublas_proj": timed_ring(lambda i: F.linear(a_in, w_pr[i]), 2.0 * Fh * D)}
            if Bs <= 16:
                r["decode_linear_fc_gated"] = timed_ring(lambda i: ab.decode_linear(x, w_fc[i], None, gated=True), 2.0 * 2 * Fh * D)
                r["decode_linear_proj"] = timed_ring(lambda i: ab.decode_linear(a_in, w_pr[i]), 2.0 * Fh * D)
            res[f"rows_{Bs}"] = r
        Bs = "8, 16, 64"
        info = {"kernel": "decode_linear_kernel", "rows": Bs, **res}
    elif which in ("conv", "step", "prep_decode"):
        def timed_gbs(fn, nbytes, iters=10):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda._sleep(20_000_000)                       # the host queues the launches while the GPU is busy
            e0.record()
            for _ in range(iters):
                fn()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / iters
            return {"ms": ms, "bytes_per_launch": nbytes, "gbs": nbytes / (ms * 1e-3) / 1e9}
        res = {}
        if which == "conv":
            # packed prefill convs on 65,536 tokens in 8 sequences: the Canon conv of q (1024 channels, K=4, residual
            # form) and the gated LFM2 conv (hidden 2048: a (tokens, 3*2048) projection in, (tokens, 2048) out)
            from atma_b200.layer import PackedMaps
            n_seqs, per = 8, 8192
            total = n_seqs * per
            maps = PackedMaps([per] * n_seqs, list(range(n_seqs)), dev)
            for C in (H * DK, HKV * DK):
                x = torch.randn(total, C, generator=g).bfloat16().to(dev)
                w = (torch.randn(C, 4, generator=g) * 0.3).bfloat16().to(dev)
                st = torch.zeros(n_seqs, C, 3, dtype=torch.bfloat16, device=dev)
                res[f"packed_causal_conv1d_C{C}"] = timed_gbs(
                    lambda: ab.packed_causal_conv1d(x, w, st, maps.token_seq_starts, maps.token_seq_ends, maps.token_seq_slots),
                    2.0 * x.numel() * 2)
            D = 2048
            proj = torch.randn(total, 3 * D, generator=g).bfloat16().to(dev)
            w = (torch.randn(D, 3, generator=g) * 0.3).bfloat16().to(dev)
            st = torch.zeros(n_seqs, D, 2, dtype=torch.bfloat16, device=dev)
            res["lfm2_conv_packed_D2048"] = timed_gbs(
                lambda: ab.lfm2_conv_packed(proj, w, st, maps.token_seq_starts, maps.token_seq_ends, maps.token_seq_slots),
                4.0 * total * D * 2)
            dst = torch.empty_like(proj)
            res["plain_copy_same_method"] = timed_gbs(lambda: dst.copy_(proj), 2.0 * proj.numel() * 2)
            info = {"kernel": "packed_conv_vec_kernel, lfm2_conv_packed_vec_kernel", "tokens": total, **res}
        elif which == "step":
            # the memory step on a state table larger than L2: 256 sequences x 8 heads x 64 KB = 134 MB read and written
            Bs = 256
            state = torch.randn(Bs, H, DK, DK, device=dev) * 0.1
            q = torch.randn(Bs, H, DK, device=dev, dtype=torch.bfloat16)
            kn = torch.randn(Bs, HKV, DK, device=dev, dtype=torch.bfloat16)
            vn = torch.randn(Bs, HKV, DK, device=dev, dtype=torch.bfloat16)
            gamma = torch.rand(Bs, H, device=dev) * 0.1 + 0.9
            beta = torch.rand(Bs, H, device=dev)
            slots = torch.arange(Bs, device=dev)
            res["gated_delta_step_wide_B256"] = timed_gbs(
                lambda: ab.gated_delta_decode_step_fused(q, kn, vn, state, slots, gamma=gamma, beta=beta), 2.0 * state.numel() * 4)
            dst = torch.empty_like(state)
            res["plain_copy_same_method"] = timed_gbs(lambda: dst.copy_(state), 2.0 * state.numel() * 4)
            info = {"kernel": "gated_delta_step_wide_kernel", "sequences": Bs, **res}
        else:
            # the decode glue of a global layer at 4096 rows (a launch-latency kernel at the decode batch of 64; this
            # size shows its bandwidth): q half of q|gate, k, v read; q, k, v, two cache rows and 3 state rows r/w
            Bs, K = 4096, 4
            q_gate = torch.randn(Bs, H, 2 * DK, generator=g).bfloat16().to(dev)
            k = torch.randn(Bs, HKV, DK, generator=g).bfloat16().to(dev)
            v = torch.randn(Bs, HKV, DK, generator=g).bfloat16().to(dev)
            w = [(torch.randn(C, K, generator=g) * 0.3).bfloat16().to(dev) for C in (H * DK, HKV * DK, HKV * DK)]
            st = [torch.zeros(Bs, C, K - 1, dtype=torch.bfloat16, device=dev) for C in (H * DK, HKV * DK, HKV * DK)]
            kc = torch.zeros(Bs, HKV, DK, dtype=torch.bfloat16, device=dev)
            vc = torch.zeros_like(kc)
            slots = torch.arange(Bs, device=dev)
            sm = torch.randperm(Bs, generator=g).int().to(dev)
            nbytes = Bs * DK * 2.0 * ((2 * H + 5 * HKV) + 2 * (K - 1) * (H + 2 * HKV))
            res["qkv_prep_decode_B4096"] = timed_gbs(lambda: ab.qkv_prep_decode(q_gate, k, v, *w, *st, slots, kc, vc, sm), nbytes)
            info = {"kernel": "qkv_prep_decode_kernel", "rows": Bs, **res}
    elif which == "prep":
        ms, nbytes, total = bench_prep(ab, dev, tokens=65536, n_seqs=8, iters=5)
        info = {"kernel": "qkv_prep_kernel", "tokens": total, "bytes_per_launch": nbytes, "ms": ms,
                "gbs": nbytes / (ms * 1e-3) / 1e9, "plain_copy_gbs_same_method": bench_prep.copy_gbs}
    else:
        B, T = 2, 16384
        q = torch.randn(B, T, H, DK, generator=g).bfloat16().to(dev)
        k = torch.randn(B, T, HKV, DK, generator=g).bfloat16().to(dev)
        v = torch.randn(B, T, HKV, DK, generator=g).bfloat16().to(dev)
        gl = (-F.softplus(torch.randn(B, T, H, generator=g))).to(dev)
        be = torch.sigmoid(torch.randn(B, T, H, generator=g)).to(dev)
        for _ in range(5):
            ab.chunk_gated_delta_rule(q=q, k=k, v=v, g=gl, beta=be, scale=1.0, output_final_state=True,
                                      use_qk_l2norm_in_kernel=True)
        info = {"kernel": "scan_local_sm100_kernel + scan_recur_sm100_kernel", "B": B, "T": T,
                "flops_per_launch": scan_flops(T) * B,
                "algorithmic_bytes": 4.0 * B * T * H * DK * 2 - 2.0 * B * T * (H - HKV) * DK * 2 + 2.0 * B * T * H * 4}
    torch.cuda.synchronize()
    emit({"profile": which, **info})


def bench_decode_sharded(ab, device, steps, warmup, peaks, world, dist):
    """Decode with the batch of 64 sequences split over the ranks (no collective): every rank
    steps its own 64/N sequences; the aggregate is 64 tokens per slowest-rank step."""
    global DEC_B
    full_b = DEC_B
    DEC_B = full_b // world
    try:
        d = bench_decode(ab, device, steps, warmup, peaks)
    finally:
        DEC_B = full_b
    t = torch.tensor([d["ms_per_step"], d["roofline"]["kernel_ms"]], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, kms = t.tolist()
    d["ms_per_step"], d["value"] = ms, full_b / (ms * 1e-3)
    d["config"]["batch"], d["config"]["batch_per_gpu"], d["config"]["sharding"] = full_b, full_b // world, "batch, no collective"
    return d


def run_context_parallel(args, ab, rank, local_rank, world, device, peaks):
    """N > 1: ONE 65,536-token sequence sharded over the ranks (zig-zag segments); Polar K/V
    blocks travel an NCCL ring, the gated-delta state is handed over as an affine-map prefix."""
    import torch.distributed as dist
    from atma_b200 import context_parallel as cp
    dist.init_process_group("nccl", device_id=device)
    full = make_prefill_inputs(seed=4)                       # the same sequence on every rank
    sh = cp.shard_sequence(full, rank, world)
    del full
    fields = ("q", "k", "v", "g", "beta")
    host = {f: [x.pin_memory() for x in getattr(sh, f)] for f in fields}
    params = default_polar_params(device)

    def to_dev():
        return cp.GlobalLayerShard(positions=sh.positions,
                                   **{f: [x.to(device, non_blocking=True) for x in host[f]] for f in fields})

    mode = cp.default_polar_mode(sh, world)
    polar_fn = cp.gathered_polar_prefill if mode == "gather" else cp.ring_polar_prefill

    def step(shard, ev=None):
        tr = lambda x: x.transpose(1, 2)
        kw = {"events": ev[0:2]} if (ev and mode == "gather") else {}
        if ev and mode != "gather":
            ev[0].record()
        polar = polar_fn([tr(x) for x in shard.q], [tr(x) for x in shard.k], [tr(x) for x in shard.v],
                         shard.positions, params, **kw)
        if ev and mode != "gather":
            ev[1].record()
        if ev:
            ev[2].record()
        o, S = cp.cp_gated_delta_scan(shard.q, shard.k, shard.v, shard.g, shard.beta)
        if ev:
            ev[3].record()
        return polar, o, S

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    dev_shard = to_dev()
    # (1) the two branches one after the other, launch by launch, in the mode the timed step uses, for the
    #     per-branch durations: in gather mode the events bracket the two Polar launches (the K/V all-gather
    #     lies before them); in ring mode the whole ring pass
    for _ in range(args.warmup):
        step(dev_shard)
    barrier()
    n_eager = max(3, min(args.steps, 10))
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(n_eager)]
    h0 = time.perf_counter()
    for i in range(n_eager):
        step(dev_shard, ev[i])
    host_enqueue_ms = (time.perf_counter() - h0) * 1e3 / n_eager
    barrier()
    polar_ms = statistics.median(e[0].elapsed_time(e[1]) for e in ev)
    scan_ms = statistics.median(e[2].elapsed_time(e[3]) for e in ev)

    # (2) the timed step: the public entry (memory branch beside the ring), replayed from a CUDA
    #     graph unless --no-graph
    if args.no_graph:
        run_step = lambda: cp.cp_global_layer_prefill(dev_shard, params)
        static, graph_used = dev_shard, False
    else:
        cap = cp.CapturedPrefill(dev_shard, params)
        run_step, static, graph_used = cap.replay, cap.static, cap.captured
        if not cap.captured and rank == 0:
            print(f"[bench] graph capture failed, running eagerly: {getattr(cap, 'error', None)!r}", file=sys.stderr)
    sampler = ClockSampler(local_rank)
    sampler.start()
    for _ in range(max(args.warmup, 20)):
        run_step()
    barrier()
    sampler.mark_begin()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        run_step()
    e1.record()
    barrier()
    sampler.mark_end()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / args.steps

    # (3) end to end: every step copies its pinned host shard in and all results back out.  With the graph:
    #     two captured steps on a three-stream pipeline (copy-in | replay | copy-out); without: one stream.
    host_shard = cp.GlobalLayerShard(positions=sh.positions, **{f: host[f] for f in fields})
    copy_only_ms = None
    if graph_used:
        pipe = cp.HostFedCapturedPrefill(dev_shard, params)
        # the producer of the activations fills the pipeline's own pinned views (one packed buffer per step slot)
        packed = []
        for i in range(pipe.depth):
            hs = pipe.host_shard(i)
            for f in fields:
                for dst, src in zip(getattr(hs, f), host[f]):
                    dst.copy_(src)
            packed.append(hs)

        def run_pipe(n):
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s0.record()
            for s_ in (pipe.copy_in, pipe.compute, pipe.copy_out):
                s_.wait_event(s0)
            tk = None
            for i in range(n):
                tk = pipe.submit(packed[i % pipe.depth])
            pipe.drain()
            s1.record()
            barrier()
            return s0.elapsed_time(s1) / n, tk

        for i in range(3):
            pipe.submit(packed[i % pipe.depth])
        pipe.drain()
        barrier()
        e2e_ms_local, ticket = run_pipe(args.steps)
        out_host = pipe.results(ticket)
        # the same pipeline with the replays left out: what the host <-> device copies alone cost per step
        pipe.copy_only = True
        run_pipe(3)
        copy_only_ms, _ = run_pipe(args.steps)
        pipe.copy_only = False
        e2e_api = ("atma_b200.context_parallel.HostFedCapturedPrefill.submit (one packed pinned buffer per direction, "
                   f"{pipe.depth} steps in flight)")
    else:
        out_host = None

        def e2e_step():
            nonlocal out_host
            for f in fields:
                for dst, src in zip(getattr(static, f), host[f]):
                    dst.copy_(src, non_blocking=True)
            polar, o, S = run_step()
            outs = [polar[0][0], polar[0][1], polar[1][0], polar[1][1], o[0], o[1], S]
            if out_host is None:
                out_host = [torch.empty(x.shape, dtype=x.dtype, pin_memory=True) for x in outs]
            for dst, src in zip(out_host, outs):
                dst.copy_(src, non_blocking=True)

        for _ in range(2):
            e2e_step()
        barrier()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(args.steps):
            e2e_step()
        s1.record()
        barrier()
        e2e_api = "atma_b200.context_parallel.cp_global_layer_prefill"
        e2e_ms_local = s0.elapsed_time(s1) / args.steps
    e2e_ms = e2e_ms_local
    h2d = sum(x.numel() * x.element_size() for f in fields for x in host[f])
    d2h = sum(x.numel() * x.element_size() for x in out_host)
    t = torch.tensor([ms, e2e_ms, polar_ms, scan_ms, copy_only_ms or 0.0], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms, polar_ms, scan_ms, copy_only_ms = t.tolist()
    bytes_t = torch.tensor([h2d, d2h], device=device, dtype=torch.float64)
    dist.all_reduce(bytes_t)
    h2d, d2h = bytes_t.tolist()
    del dev_shard, static, run_step
    if graph_used:
        pipe.close()
        del pipe
    if not args.no_graph:
        cap.close()
        del cap
    torch.cuda.empty_cache()
    decode = None if args.skip_decode else bench_decode_sharded(ab, device, max(args.steps, 10), args.warmup, peaks, world, dist)
    long_leg = None
    if not args.skip_long and T_PREFILL != 262144:
        long_leg = cp_long_prefill(cp, dist, rank, world, device, params, 262144, peaks)
    config4 = config5 = None
    if not args.skip_model and T_PREFILL != 262144:
        config4 = bench_model_decode_sharded(device, peaks, world, dist)
        torch.cuda.empty_cache()
        config5 = cp_model_prefill(cp, dist, rank, world, device, peaks)
    # non-zero on any rank = a bounded wait of a tensor-core kernel ran out during this run
    status = torch.tensor([ab.device_status()], device=device, dtype=torch.int32)
    dist.all_reduce(status, op=dist.ReduceOp.MAX)
    dist.barrier()
    dist.destroy_process_group()
    if rank != 0:
        return
    achieved_tf = polar_flops(T_PREFILL) / (polar_ms * 1e-3) / 1e12
    line = {
        "metric": METRIC, "value": T_PREFILL / (ms * 1e-3), "unit": "tok/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"global-layer mixing prefill: Polar attention + gated-delta scan, ONE {T_PREFILL}-token sequence "
                               "context-parallel over the GPUs (zig-zag segments, K/V all-gathered over NVLink, one Polar launch per "
                               "query segment, gated-delta state handed over as an affine-map prefix)",
                   "tokens": T_PREFILL, "heads": H, "kv_heads": HKV, "head_dim": DK, "chunk": CHUNK, "window": None,
                   "l2": "per-GPU inputs shrink with N; at N=8 they are 34 MB, below L2", "polar_kernel": "tcgen05",
                   "polar_mode": mode},
        "e2e": {"value": T_PREFILL / (e2e_ms * 1e-3), "unit": "tok/s", "ms_per_step": e2e_ms, "api": e2e_api,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                # the pipeline with the replays left out (copies only), max over ranks, and what that is in GB/s over all ranks
                "copies_only_ms_per_step": copy_only_ms or None,
                "copies_only_gbs_all_ranks": ((h2d + d2h) / (copy_only_ms * 1e-3) / 1e9) if copy_only_ms else None},
        # per rank and step: 2 Polar launches (one per query segment), the chunk-factor kernel and
        # 2 recurrence launches of this library; NCCL and torch's small copy kernels are not counted
        "gpu_launches": args.steps * 5 * world,
        "clocks": clocks,
        "roofline": {"kernel": f"polar_prefill ({mode} mode, all ranks)", "bound": "tensor", "achieved": achieved_tf,
                     "peak": peaks["tf_burst"] * world, "unit": "TFLOP/s", "frac": achieved_tf / (peaks["tf_burst"] * world),
                     "traffic": None, "algorithmic_flops": polar_flops(T_PREFILL), "kernel_ms": polar_ms,
                     "note": ("kernel_ms = first Polar launch to the end of the last one (two launches per rank on two "
                              "streams, after the K/V all-gather)" if mode == "gather" else
                              "kernel_ms = the whole ring pass (all block launches and the hops between them)") +
                             ", launch by launch with nothing beside it, median over steps, max over ranks",
                     "peak_source": peaks["source"] + f" burst x {world} GPUs"},
        "scan": {"kernel_ms": scan_ms, "algorithmic_flops": scan_flops(T_PREFILL)},
        "host_enqueue_ms_eager": host_enqueue_ms, "cuda_graph": graph_used,
        "cpu_baseline": None,
        "decode": decode,
        "prefill_256k": long_leg,
        "config4_model_decode": config4,
        "config5_model_prefill": config5,
        "device_status": int(status.item()),
    }
    emit(line)


def cp_model_prefill(cp, dist, rank, world, device, peaks, tokens=262144, steps=2):
    """BASELINE config 5 over the GPUs: the whole 16-layer model, ONE prompt of 262,144 uniform token ids cut into zig-zag
    segments (``AtmaModel.prefill_context_parallel``: conv halos between neighbours, Polar over the all-gathered K/V,
    memory state as an affine-map prefix), last-token logits on the rank that owns the last segment.  Device-timed,
    max over ranks."""
    from atma_b200.model import AtmaModel, random_state_dict
    sd = random_state_dict(vocab=VOCAB, seed=4, device=device, **MODEL)
    model = AtmaModel(sd, device=device, **MODEL)
    del sd
    (a0, a1), (b0, b1) = cp.zigzag_segments(tokens, world)[rank]
    L = a1 - a0
    bs = DEC_BLOCK
    pages = 2 * L // bs
    state = model.new_state(max_seqs=1, num_blocks=pages, block_size=bs)
    ids = torch.randint(0, VOCAB, (tokens,), generator=torch.Generator().manual_seed(4))
    parts = [ids[a0:a1].to(device), ids[b0:b1].to(device)]
    bt = torch.randperm(pages, generator=torch.Generator().manual_seed(4 + rank))
    pos = torch.arange(2 * L)
    sm = (bt[pos // bs] * bs + pos % bs).to(device)
    owns_last = cp.segment_owner(2 * world - 1, world) == rank

    def step():
        h = model.prefill_context_parallel(parts, [(a0, a1), (b0, b1)], state, 0, [sm[:L], sm[L:]])
        return model.logits(h[1][-1:]) if owns_last else None

    logits = step()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        logits = step()
    e1.record()
    dist.barrier()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / steps, 1.0 if (logits is None or bool(torch.isfinite(logits.float()).all())) else 0.0],
                     device=device, dtype=torch.float64)
    dist.all_reduce(t[:1], op=dist.ReduceOp.MAX)
    dist.all_reduce(t[1:], op=dist.ReduceOp.MIN)
    ms = float(t[0].item())
    n_body = sum(x.numel() for n, x in model.sd.items() if n not in ("embed.weight", "proj.weight", "proj.bias"))
    fl = len(model.global_layers) * polar_flops(tokens) + 2.0 * n_body * tokens + len(model.global_layers) * scan_flops(tokens)
    tf = fl / (ms * 1e-3) / 1e12
    del model, state
    torch.cuda.empty_cache()
    return {"workload": f"BASELINE config 5: full model, one {tokens}-token prompt context-parallel over {world} GPUs",
            "ms_per_step": ms, "value": tokens / (ms * 1e-3), "unit": "tok/s", "steps": steps, "algorithmic_flops": fl,
            "logits_finite": bool(t[1].item() > 0.5), "polar_mode": "gather",
            "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["tf_sustained"] * world, "unit": "TFLOP/s",
                         "frac": tf / (peaks["tf_sustained"] * world),
                         "peak_source": peaks["source"] + f" sustained x {world} GPUs"}}


def cp_long_prefill(cp, dist, rank, world, device, params, tokens, peaks, steps=5, warm=3):
    """The long context-parallel case (BASELINE config 5's length, one global layer's mixing): the captured
    step on a 262,144-token sequence, device-timed, max over ranks."""
    global T_PREFILL
    keep, T_PREFILL = T_PREFILL, tokens
    try:
        full = make_prefill_inputs(seed=5)
    finally:
        T_PREFILL = keep
    sh = cp.shard_sequence(full, rank, world)
    del full
    shard = cp.GlobalLayerShard(positions=sh.positions,
                                **{f: [x.to(device) for x in getattr(sh, f)] for f in ("q", "k", "v", "g", "beta")})
    cap = cp.CapturedPrefill(shard, params)
    for _ in range(warm):
        cap.replay()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        cap.replay()
    e1.record()
    dist.barrier()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / steps], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    graph = cap.captured
    cap.close()
    del cap, shard
    torch.cuda.empty_cache()
    tf = polar_flops(tokens) / (ms * 1e-3) / 1e12
    return {"tokens": tokens, "ms_per_step": ms, "value": tokens / (ms * 1e-3), "unit": "tok/s", "steps": steps, "cuda_graph": graph,
            "polar_mode": cp.default_polar_mode(sh, world), "step_tflops": tf, "frac_of_tensor_peak": tf / (peaks["tf_burst"] * world),
            "note": "whole step (K/V all-gather, Polar, memory branch beside it) against the Polar FLOPs alone"}


def timed(fn, iters, warm=3, flush=None):
    """Median CUDA-event duration (ms) of fn(); ``flush``: a buffer larger than L2 rewritten before every call."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    out = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        out.append(a.elapsed_time(b))
    return statistics.median(out)


def bench_config2(ab, device, peaks):
    """BASELINE config 2: Polar prefill alone, q [4,8192,8,128], k/v [4,8192,2,128], bf16, seed 1, full causal context."""
    torch.manual_seed(1)
    B, T = 4, 8192
    q = torch.randn(B, T, H, DK).bfloat16().to(device)
    k = torch.randn(B, T, HKV, DK).bfloat16().to(device)
    v = torch.randn(B, T, HKV, DK).bfloat16().to(device)
    n = torch.arange(1, T + 1, dtype=torch.float32, device=device)
    P = default_polar_params(device)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)       # the inputs (101 MB) fit L2: flush it
    ms = timed(lambda: ab.polar_attention_fwd(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), n, **P), 10, flush=flush)
    fl = B * polar_flops(T)
    tf = fl / (ms * 1e-3) / 1e12
    return {"workload": "BASELINE config 2: Polar prefill B=4 x 8192, H=8, Hkv=2, dk=128, bf16", "ms": ms,
            "value": B * T / (ms * 1e-3), "unit": "tok/s", "algorithmic_flops": fl,
            "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["tf_burst"], "unit": "TFLOP/s", "frac": tf / peaks["tf_burst"]},
            "l2": "L2 flushed (256 MB written) before every timed launch"}


def bench_config3(ab, device, peaks):
    """BASELINE config 3: gated-delta scan alone, B=8, T=16384, H=8, d=128, chunk 64, bf16 inputs, fp32 state, seed 2."""
    torch.manual_seed(2)
    B, T = 8, 16384
    q = F.normalize(torch.randn(B, T, H, DK), dim=-1).bfloat16().to(device)
    k = F.normalize(torch.randn(B, T, H, DK), dim=-1).bfloat16().to(device)
    v = torch.randn(B, T, H, DK).bfloat16().to(device)
    beta = torch.sigmoid(torch.randn(B, T, H)).to(device)
    g = (-F.softplus(torch.randn(B, T, H))).to(device)
    ms = timed(lambda: ab.chunk_gated_delta_rule(q=q, k=k, v=v, g=g, beta=beta, scale=1.0, output_final_state=True,
                                                 use_qk_l2norm_in_kernel=True), 10)
    fl = scan_flops(T) * B
    nbytes = 4.0 * B * T * H * DK * 2 + 2.0 * B * T * H * 4 + B * H * DK * DK * 4.0     # q, k, v, o + g, beta + final state
    tf, gbs = fl / (ms * 1e-3) / 1e12, nbytes / (ms * 1e-3) / 1e9
    return {"workload": "BASELINE config 3: gated-delta scan B=8 x 16384, H=8, d=128, chunk 64", "ms": ms,
            "value": B * T / (ms * 1e-3), "unit": "tok/s", "algorithmic_flops": fl, "algorithmic_bytes": nbytes,
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm"], "unit": "GB/s", "frac": gbs / peaks["hbm"],
                         "tensor_tflops": tf, "tensor_frac": tf / peaks["tf_burst"]},
            "l2": "inputs (805 MB) larger than L2"}


MODEL = dict(layers=16, hidden=1024, head_dim=128, num_kv_heads=2)
VOCAB = 50304


def bench_model_decode(device, peaks, steps=20, batch=None):
    """BASELINE config 4 on one GPU: the whole 16-layer model (12 LFM2 conv + 4 Polar/gated-delta layers, 378M
    random-init bf16 weights, seed 3), one decode step for 64 sequences with 32,768 tokens of context each in the
    paged cache (256-token pages in shuffled order), replayed from one CUDA graph."""
    from atma_b200.model import AtmaModel, CapturedDecode, random_state_dict
    sd = random_state_dict(vocab=VOCAB, seed=3, device=device, **MODEL)
    model = AtmaModel(sd, device=device, **MODEL)
    del sd
    B, ctx, bs = (batch or DEC_B), DEC_CTX, DEC_BLOCK
    pages = ctx // bs
    state = model.new_state(max_seqs=B, num_blocks=B * pages, block_size=bs)
    g = torch.Generator(device=device).manual_seed(3)
    for i in model.global_layers:
        state.k_cache[i].normal_(generator=g)
        state.v_cache[i].normal_(generator=g)
        state.mem[i].normal_(generator=g).mul_(0.1)
    bt = torch.randperm(B * pages, generator=torch.Generator().manual_seed(3)).int().view(B, pages).to(device)
    cap = CapturedDecode(model, state, batch=B, max_blocks=pages)
    cap.ids.copy_(torch.randint(0, VOCAB, (B,), generator=torch.Generator().manual_seed(3)).to(device))
    cap.block_tables.copy_(bt)
    cap.context_lens.fill_(ctx)
    cap.slot_mapping.copy_((bt[:, -1].long() * bs + bs - 1).int())
    cap.capture()
    for _ in range(3):
        cap.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        cap.replay()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    nbytes = float(model.decode_bytes(B, ctx))
    gbs = nbytes / (ms * 1e-3) / 1e9
    finite = bool(torch.isfinite(cap.logits.float()).all())
    return {"workload": f"BASELINE config 4: full model (16 layers, 4 global), decode of {B} sequences x {ctx} tokens of context, "
                        f"pages of {bs}", "ms_per_step": ms, "value": B / (ms * 1e-3), "unit": "tok/s", "steps": steps,
            "cuda_graph": True, "logits_finite": finite, "algorithmic_bytes": nbytes,
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm"], "unit": "GB/s", "frac": gbs / peaks["hbm"]},
            "projections": ("this library's weight-streaming kernel (batches of up to 16 rows) where its shape rules allow, else cuBLAS"
                            if B <= 16 else "cuBLAS (F.linear); everything between them this library")}


def bench_model_decode_sharded(device, peaks, world, dist):
    """BASELINE config 4 with its 64 sequences split over the ranks (no collective): every rank decodes 64/N sequences
    through the whole model; the aggregate is 64 tokens per slowest-rank step."""
    d = bench_model_decode(device, peaks, batch=DEC_B // world)
    t = torch.tensor([d["ms_per_step"]], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    d["ms_per_step"], d["value"] = ms, DEC_B / (ms * 1e-3)
    d["batch_per_gpu"], d["sharding"] = DEC_B // world, "batch, no collective"
    nbytes = d["algorithmic_bytes"]
    d["roofline"]["achieved"] = nbytes / (ms * 1e-3) / 1e9
    d["roofline"]["frac"] = d["roofline"]["achieved"] / peaks["hbm"]
    d["roofline"]["note"] = "per GPU: this rank's bytes (all weights + its sequences' K/V and state) over the slowest rank's step"
    return d


def bench_model_prefill(device, peaks, tokens=262144, steps=2):
    """BASELINE config 5 on one GPU: the whole model, one prompt of 262,144 uniform token ids, prefilled in one pass
    (packed-prefill path with a single sequence); last-token logits computed."""
    from atma_b200.layer import PackedMaps
    from atma_b200.model import AtmaModel, random_state_dict
    sd = random_state_dict(vocab=VOCAB, seed=4, device=device, **MODEL)
    model = AtmaModel(sd, device=device, **MODEL)
    del sd
    bs = DEC_BLOCK
    pages = tokens // bs
    state = model.new_state(max_seqs=1, num_blocks=pages, block_size=bs)
    ids = torch.randint(0, VOCAB, (tokens,), generator=torch.Generator().manual_seed(4)).to(device)
    bt = torch.randperm(pages, generator=torch.Generator().manual_seed(4))
    pos = torch.arange(tokens)
    sm = (bt[pos // bs] * bs + pos % bs).to(device)
    maps = PackedMaps([tokens], [0], device)

    def step():
        h = model.prefill(ids, [tokens], [0], state, sm, maps=maps)
        return model.logits(h[-1:])

    logits = step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        logits = step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    n_body = sum(t.numel() for n, t in model.sd.items() if n not in ("embed.weight", "proj.weight", "proj.bias"))
    fl = len(model.global_layers) * polar_flops(tokens) + 2.0 * n_body * tokens + len(model.global_layers) * scan_flops(tokens)
    tf = fl / (ms * 1e-3) / 1e12
    return {"workload": f"BASELINE config 5 on one GPU: full model, one {tokens}-token prompt", "ms_per_step": ms,
            "value": tokens / (ms * 1e-3), "unit": "tok/s", "steps": steps, "algorithmic_flops": fl,
            "logits_finite": bool(torch.isfinite(logits.float()).all()),
            "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["tf_sustained"], "unit": "TFLOP/s",
                         "frac": tf / peaks["tf_sustained"], "peak_source": peaks["source"] + " sustained (a step is ~0.7 s long)"}}


_REAL_STDOUT = None


def emit(obj):
    """The one JSON line goes to the process's original stdout; everything else that libraries
    write to file descriptor 1 while the bench runs (NCCL's version banner, ...) goes to stderr."""
    data = (json.dumps(obj) + "\n").encode()
    if _REAL_STDOUT is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_REAL_STDOUT, data)


def main():
    global _REAL_STDOUT, T_PREFILL, METRIC
    sys.stdout.flush()
    _REAL_STDOUT = os.dup(1)
    os.dup2(2, 1)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", type=int, default=T_PREFILL,
                    help="prefill length (default: the metric's 65,536; 262,144 is the long context-parallel case)")
    ap.add_argument("--no-graph", action="store_true",
                    help="N > 1: issue the context-parallel step launch by launch instead of replaying a CUDA graph")
    ap.add_argument("--skip-cpu", action="store_true", help="omit the CPU baseline leg (profiling runs)")
    ap.add_argument("--skip-decode", action="store_true", help="omit the decode leg (profiling runs)")
    ap.add_argument("--skip-long", action="store_true", help="N > 1: omit the 262,144-token leg")
    ap.add_argument("--skip-configs", action="store_true", help="N = 1: omit the BASELINE config 2 / config 3 legs")
    ap.add_argument("--skip-model", action="store_true", help="N = 1: omit the full-model legs (BASELINE configs 4 and 5)")
    ap.add_argument("--profile", default=None, choices=["prefill", "decode", "scan", "prep", "epilogue", "conv", "step", "prep_decode", "linear"],
                    help="run a few launches of ONE kernel on a small case (a few hundred MB, larger than L2) "
                         "and exit; meant to be wrapped in ncu")
    args = ap.parse_args()
    if args.tokens != T_PREFILL:
        T_PREFILL = args.tokens
        METRIC = f"global_layer_prefill_tok_s_at_{T_PREFILL}"
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.profile:
        profile_case(args.profile)
        return
    args.warmup = max(args.warmup, 3)

    import atma_b200 as ab
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    peaks = measured_peaks()
    if world > 1:
        run_context_parallel(args, ab, rank, local_rank, world, device, peaks)
        return
    dist = None

    host = make_prefill_inputs(seed=4 + rank, pinned=True)
    dev_in = {n: x.to(device) for n, x in host.items()}
    params = default_polar_params(device)
    n_keys = torch.arange(1, T_PREFILL + 1, dtype=torch.float32, device=device)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- kernel-resident timing ("value") -------------------------------------------------------
    ready = torch.cuda.Event()
    ready.record()                                              # the inputs are resident from here on
    sampler = ClockSampler(local_rank)
    sampler.start()
    for _ in range(max(args.warmup, 10)):                       # also gives the clock sampler time to come up
        prefill_step(ab, dev_in, n_keys, params, ready=ready)
    barrier()
    sampler.mark_begin()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(args.steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        prefill_step(ab, dev_in, n_keys, params, ev[i], ready=ready)
    e1.record()
    barrier()
    sampler.mark_end()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / args.steps
    polar_ms = sum(e[0].elapsed_time(e[1]) for e in ev) / args.steps
    scan_ms = sum(e[2].elapsed_time(e[3]) for e in ev) / args.steps
    # the same kernels one after the other on one stream, for the isolated kernel durations
    from atma_b200.mixing import global_layer_mixing
    iso = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(9)]
    for e in iso:
        global_layer_mixing(dev_in["q"], dev_in["k"], dev_in["v"], dev_in["g"], dev_in["beta"], n_keys, params,
                            overlap=False, events=e)
        torch.cuda.synchronize()                                # one step at a time: nothing queued beside the kernel
    iso = iso[2:]                                               # the first two calls warm the single-stream path up
    polar_iso_all = sorted(e[0].elapsed_time(e[1]) for e in iso)
    polar_iso_ms = polar_iso_all[len(iso) // 2]                     # median
    scan_iso_ms = sorted(e[2].elapsed_time(e[3]) for e in iso)[len(iso) // 2]

    # ---- end to end: pinned host inputs in, results out, inside the timed region ------------------
    # Public API for host-resident activations: a three-stream pipeline (copy in | kernels | copy out);
    # every step copies its own inputs from pinned memory and returns all four results to pinned memory.
    from atma_b200.mixing import HostFedMixing
    hosts = [host, make_prefill_inputs(seed=104 + rank, pinned=True)]
    pipe = HostFedMixing(device)
    for i in range(4):
        pipe.submit(hosts[i % 2], n_keys, params)
    pipe.drain()
    barrier()
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s0.record()
    for s_ in (pipe.copy_in, pipe.compute, pipe.copy_out):
        s_.wait_event(s0)
    for i in range(args.steps):
        ticket = pipe.submit(hosts[i % 2], n_keys, params)
    pipe.drain()
    s1.record()
    barrier()
    out_host = pipe.results(ticket)
    e2e_ms = s0.elapsed_time(s1) / args.steps
    h2d = sum(x.numel() * x.element_size() for x in host.values())
    d2h = sum(x.numel() * x.element_size() for x in out_host)

    times = torch.tensor([ms, e2e_ms, polar_ms, scan_ms], device=device, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, e2e_ms, polar_ms, scan_ms = times.tolist()

    decode = None
    del dev_in
    torch.cuda.empty_cache()
    if rank == 0 and not args.skip_decode:
        decode = bench_decode(ab, device, max(args.steps, 10), args.warmup, peaks)
        torch.cuda.empty_cache()
    config2 = config3 = None
    if rank == 0 and not args.skip_configs and T_PREFILL == 65536:
        config2 = bench_config2(ab, device, peaks)
        torch.cuda.empty_cache()
        config3 = bench_config3(ab, device, peaks)
        torch.cuda.empty_cache()
    config4 = config5 = None
    if rank == 0 and not args.skip_model and T_PREFILL == 65536:
        config4 = bench_model_decode(device, peaks)
        torch.cuda.empty_cache()
        config5 = bench_model_prefill(device, peaks)
        torch.cuda.empty_cache()
    device_status = ab.device_status()       # non-zero = a bounded wait of a tensor-core kernel ran out during this run
    cpu = None
    if rank == 0 and world == 1 and not args.skip_cpu:
        threads = os.cpu_count() or 1
        sample_T = 16384
        sec = cpu_baseline(sample_T, threads)
        cpu = {"value": sample_T / sec, "unit": "tok/s", "cores": threads, "kind": "port",
               "sample": f"one global layer (Polar materialised + gated-delta chunked, fp32) at T={sample_T}: "
                         f"{sec:.2f} s; Polar cost is quadratic, so tok/s at 64K would be ~4x lower"}
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return

    from atma_b200 import _lib
    from ctypes import byref
    probe = _lib.PolarPrefillArgs()
    probe.dtype, probe.dk, probe.H, probe.Hkv, probe.n_tiles, probe.finalize = 1, DK, H, HKV, 0, 1
    tensor_path = bool(_lib.load().atma_polar_prefill_path(byref(probe)))
    peak_tf = peaks["tf_sustained"] if ms > 1000 else peaks["tf_burst"]
    achieved_tf = polar_flops(T_PREFILL) / (polar_ms * 1e-3) / 1e12
    line = {
        "metric": METRIC, "value": world * T_PREFILL / (ms * 1e-3), "unit": "tok/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"global-layer mixing prefill: Polar attention + gated-delta scan, one {T_PREFILL}-token sequence",
                   "tokens": T_PREFILL, "heads": H, "kv_heads": HKV, "head_dim": DK, "chunk": CHUNK,
                   "window": None, "l2": f"inputs ({(2 * H + 2 * HKV) * DK * 2 * T_PREFILL / 1e6:.0f} MB) larger than L2 (126 MB)",
                   "polar_kernel": "tcgen05" if tensor_path else "cuda-core fp32",
                   "step_overlap": "steps are independent; the memory branch of step i+1 (side stream) may run under the "
                                   "tail of step i's attention kernel"},
        "e2e": {"value": world * T_PREFILL / (e2e_ms * 1e-3), "unit": "tok/s", "ms_per_step": e2e_ms,
                "api": "atma_b200.mixing.HostFedMixing.submit (copy-in | kernels | copy-out streams, double buffered)",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": 3 * args.steps,
        "clocks": clocks,
        "roofline": {"kernel": "polar_prefill", "bound": "tensor", "achieved": achieved_tf, "peak": peak_tf,
                     "unit": "TFLOP/s", "frac": achieved_tf / peak_tf,
                     # ncu capture of this very launch (dram__bytes_read.sum + dram__bytes_write.sum, one pass):
                     # 336 MB = the algorithmic input and output bytes; other lengths scale by the token count.
                     "traffic": PREFILL_TRAFFIC_64K * (T_PREFILL / 65536),
                     "algorithmic_flops": polar_flops(T_PREFILL), "kernel_ms": polar_ms,
                     "kernel_ms_alone": polar_iso_ms, "kernel_ms_alone_min_max": [polar_iso_all[0], polar_iso_all[-1]],
                     # the timed region runs under the power cap (see clocks); against the seconds-long cuBLAS figure:
                     "frac_of_sustained_peak": achieved_tf / peaks["tf_sustained"],
                     "frac_alone": polar_flops(T_PREFILL) / (polar_iso_ms * 1e-3) / 1e12 / peak_tf,
                     "note": "kernel_ms is measured inside the timed region, where the gated-delta recurrence runs "
                             "beside this kernel on a second stream and takes some SMs; kernel_ms_alone is the same "
                             "launch with nothing beside it",
                     "peak_source": peaks["source"] + (" sustained" if ms > 1000 else " burst")},
        "scan": {"kernel_ms": scan_ms, "kernel_ms_alone": scan_iso_ms,
                 "tflops": scan_flops(T_PREFILL) / (scan_iso_ms * 1e-3) / 1e12,
                 "algorithmic_flops": scan_flops(T_PREFILL),
                 "note": "kernel_ms: the single-pass scan (chunk-local kernel + one recurrence CTA per head) beside the "
                         "attention kernel; kernel_ms_alone: the library's own choice with nothing beside it "
                         "(the sequence cut into segments that are walked side by side)"},
        "cpu_baseline": cpu,
        "decode": decode,
        "config2": config2,
        "config3": config3,
        "config4_model_decode": config4,
        "config5_model_prefill_1gpu": config5,
        "device_status": device_status,
    }
    emit(line)


if __name__ == "__main__":
    main()
