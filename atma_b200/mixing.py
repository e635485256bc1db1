"""The two mixing branches of a global layer, scheduled side by side.

In the reference the Polar core and the gated-delta memory read the same post-conv q, k, v
and do not depend on each other (model/reference.py:174-194; inference/models/atma.py:422-426
runs them back to back on one stream).  The memory recurrence is latency-bound and occupies
one SM per (sequence, head), so this helper puts it on a side stream: the tensor-core attention
kernel fills the remaining SMs while the recurrence walks its chunks.
"""

import torch

from .gated_delta import chunk_gated_delta_rule
from .polar import polar_attention_fwd

_side_streams = {}


def _side_stream(device):
    key = (device.type, device.index)
    s = _side_streams.get(key)
    if s is None:
        s = torch.cuda.Stream(device=device, priority=-1)      # high priority: its few CTAs get SMs as they free up
        _side_streams[key] = s
    return s


@torch.no_grad()
def global_layer_mixing(q, k, v, g, beta, n_keys, polar_params, *, window=None, initial_state=None,
                        overlap=True, events=None, inputs_ready=None):
    """q (B,T,H,dk); k, v (B,T,Hkv,dk) post-conv, un-expanded KV heads; g (log decay), beta (B,T,H).
    Returns (c (B,H,T,dk), mag (B,H,T), o (B,T,H,dv), S (B,H,dk,dv)).  ``events`` = four CUDA events
    recorded around the Polar kernel (on the current stream) and the scan (on its stream).

    ``inputs_ready``: a CUDA event after which the inputs are valid.  Without it the memory branch
    waits for everything queued on the current stream so far - also for the previous step's
    attention kernel when steps are issued back to back.  With it the branch waits for the event
    only, so the recurrence of step i+1 runs under the tail of step i's attention kernel."""
    cur = torch.cuda.current_stream(q.device)
    side = _side_stream(q.device) if overlap else cur
    if overlap:
        if inputs_ready is not None:
            side.wait_event(inputs_ready)
            cur.wait_event(inputs_ready)
        else:
            side.wait_stream(cur)
    with torch.cuda.stream(side):
        if events:
            events[2].record(side)
        # beside the attention kernel the single-pass recurrence is the right one: it takes the fewest SM-seconds,
        # and its latency hides under the attention anyway; alone, the library cuts the sequence into segments
        o, S = chunk_gated_delta_rule(q=q, k=k, v=v, g=g, beta=beta, scale=1.0, initial_state=initial_state,
                                      output_final_state=True, use_qk_l2norm_in_kernel=True,
                                      segments=1 if overlap else None)
        if events:
            events[3].record(side)
    if events:
        events[0].record(cur)
    c, mag = polar_attention_fwd(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), n_keys, window=window,
                                 **polar_params)
    if events:
        events[1].record(cur)
    if overlap:
        cur.wait_stream(side)
        o.record_stream(cur)
        S.record_stream(cur)
    return c, mag, o, S


class HostFedMixing:
    """The mixing step for callers whose activations live in pinned host memory.

    Three streams work as a pipeline over consecutive steps: a copy-in stream moves step i+1's
    q, k, v, g, beta to the device while the kernels of step i run on the compute stream and a
    copy-out stream returns step i-1's results (PCIe is full duplex, so the two copies do not
    share bandwidth).  Device inputs are double buffered; results are allocated per step by the
    kernels' wrappers and handed to the copy-out stream.

    ``submit`` enqueues one step and returns at once; ``results(ticket)`` waits for that step's
    device-to-host copies and returns the pinned result tensors (c, mag, o, S).  A result slot is
    reused ``depth`` submits later, so read it (or copy it away) before then.
    """

    NAMES = ("q", "k", "v", "g", "beta")

    def __init__(self, device, depth=2):
        self.device = torch.device(device)
        self.depth = depth
        self.copy_in = torch.cuda.Stream(device=self.device)
        self.copy_out = torch.cuda.Stream(device=self.device)
        self.compute = torch.cuda.Stream(device=self.device)
        self.dev_in = [None] * depth
        self.out_host = [None] * depth
        self.in_free = [None] * depth           # compute finished reading the slot's device inputs
        self.out_done = [None] * depth          # the slot's results are in host memory
        self.step = 0

    def submit(self, host_inputs, n_keys, polar_params, *, window=None, initial_state=None):
        slot = self.step % self.depth
        self.step += 1
        for n in self.NAMES:
            if not host_inputs[n].is_pinned():
                raise ValueError(f"host input {n!r} must be in pinned memory for asynchronous copies")
        if self.dev_in[slot] is None or any(self.dev_in[slot][n].shape != host_inputs[n].shape or
                                            self.dev_in[slot][n].dtype != host_inputs[n].dtype for n in self.NAMES):
            torch.cuda.synchronize(self.device)
            self.dev_in[slot] = {n: torch.empty(host_inputs[n].shape, dtype=host_inputs[n].dtype, device=self.device)
                                 for n in self.NAMES}
            self.in_free[slot] = None
        dev = self.dev_in[slot]
        with torch.cuda.stream(self.copy_in):
            if self.in_free[slot] is not None:
                self.copy_in.wait_event(self.in_free[slot])
            for n in self.NAMES:
                dev[n].copy_(host_inputs[n], non_blocking=True)
            arrived = torch.cuda.Event()
            arrived.record(self.copy_in)
        with torch.cuda.stream(self.compute):
            self.compute.wait_event(arrived)
            c, mag, o, S = global_layer_mixing(dev["q"], dev["k"], dev["v"], dev["g"], dev["beta"], n_keys,
                                               polar_params, window=window, initial_state=initial_state,
                                               inputs_ready=arrived)
            computed = torch.cuda.Event()
            computed.record(self.compute)
        self.in_free[slot] = computed
        outs = (c, mag, o, S)
        if self.out_host[slot] is None or any(h.shape != d.shape or h.dtype != d.dtype
                                              for h, d in zip(self.out_host[slot], outs)):
            self.out_host[slot] = [torch.empty(d.shape, dtype=d.dtype, pin_memory=True) for d in outs]
        with torch.cuda.stream(self.copy_out):
            self.copy_out.wait_event(computed)
            for h, d in zip(self.out_host[slot], outs):
                h.copy_(d, non_blocking=True)
                d.record_stream(self.copy_out)
            done = torch.cuda.Event()
            done.record(self.copy_out)
        self.out_done[slot] = done
        return self.step - 1

    def results(self, ticket):
        if ticket < self.step - self.depth or ticket >= self.step:
            raise ValueError("that step's result slot has been reused (or the step was never submitted)")
        slot = ticket % self.depth
        self.out_done[slot].synchronize()
        return tuple(self.out_host[slot])

    def drain(self, stream=None):
        """Make ``stream`` (default: the current stream) wait for everything submitted so far."""
        stream = stream or torch.cuda.current_stream(self.device)
        for s in (self.copy_in, self.compute, self.copy_out):
            stream.wait_stream(s)
