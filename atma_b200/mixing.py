"""The two mixing branches of a global layer, scheduled side by side.

In the reference the Polar core and the gated-delta memory read the same post-conv q, k, v
and do not depend on each other (model/reference.py:174-194; inference/models/atma.py:422-426
runs them back to back on one stream).  The memory recurrence is latency-bound and occupies
only a few dozen SMs, so this helper puts it on a side stream: the tensor-core attention kernel
fills the remaining SMs while the recurrence walks its chunks.
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
                        overlap=True, events=None):
    """q (B,T,H,dk); k, v (B,T,Hkv,dk) post-conv, un-expanded KV heads; g (log decay), beta (B,T,H).
    Returns (c (B,H,T,dk), mag (B,H,T), o (B,T,H,dv), S (B,H,dk,dv)).  ``events`` = four CUDA events
    recorded around the Polar kernel (on the current stream) and the scan (on its stream)."""
    cur = torch.cuda.current_stream(q.device)
    side = _side_stream(q.device) if overlap else cur
    if overlap:
        side.wait_stream(cur)
    with torch.cuda.stream(side):
        if events:
            events[2].record(side)
        o, S = chunk_gated_delta_rule(q=q, k=k, v=v, g=g, beta=beta, scale=1.0, initial_state=initial_state,
                                      output_final_state=True, use_qk_l2norm_in_kernel=True)
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
