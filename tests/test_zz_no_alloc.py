"""GPU: the decode entry point that brings its own scratch gives the same result as the one
that takes caller scratch.

atma_polar_decode_static exists for hosts that cannot allocate device memory when they decode
(an engine whose KV cache already fills the GPU, a runtime with a fixed memory plan).  Both
entry points are called here through the C ABI on the same inputs, twice in a row with
different context lengths, so that whatever the first call leaves in the shared built-in array
is there when the second one runs.  This file sorts last on purpose: a run that stops at the
first failure has then already executed every other test.
"""

from ctypes import byref

import pytest
import torch

from atma_b200 import _lib
from conftest import max_abs

pytestmark = pytest.mark.gpu


def _args(q, kc, vc, bt, cl, P, c, mag, scratch, n_splits):
    a = _lib.PolarDecodeArgs()
    a.q, a.k_cache, a.v_cache = _lib.ptr(q), _lib.ptr(kc), _lib.ptr(vc)
    a.block_tables, a.bt_stride, a.context_lens = _lib.ptr(bt), bt.stride(0), _lib.ptr(cl)
    a.v_null, a.spg, a.null_base, a.sps, a.beta = (_lib.ptr(P[n]) for n in ("v_null", "spg", "null_base", "sps", "beta"))
    a.c, a.mag, a.scratch = _lib.ptr(c), _lib.ptr(mag), _lib.ptr(scratch)
    a.B, a.H, a.Hkv, a.dk = q.shape[0], q.shape[1], kc.shape[2], q.shape[2]
    a.block_size, a.max_blocks, a.num_blocks = kc.shape[1], bt.shape[1], kc.shape[0]
    a.n_splits, a.dtype, a.window, a.eps = n_splits, _lib.dtype_code(q), 0, 1e-6
    return a


def test_static_scratch_entry_matches_caller_scratch_entry():
    lib = _lib.load()
    dev = "cuda"
    B, H, Hkv, dk, bs, nblk = 6, 8, 2, 128, 64, 12
    g = torch.Generator().manual_seed(77)
    kc = torch.randn(B * nblk, bs, Hkv, dk, generator=g).bfloat16().to(dev)
    vc = torch.randn(B * nblk, bs, Hkv, dk, generator=g).bfloat16().to(dev)
    bt = torch.randperm(B * nblk, generator=g).int().view(B, nblk).to(dev)
    P = dict(v_null=torch.randn(H, dk, generator=g) * 0.2, spg=torch.rand(H, generator=g),
             null_base=2 + torch.randn(H, generator=g) * 0.3, sps=torch.rand(H, generator=g) + 0.5,
             beta=torch.rand(H, generator=g) + 0.1)
    P = {n: t.float().contiguous().to(dev) for n, t in P.items()}
    n_splits = 7
    need = lib.atma_polar_decode_scratch_floats(B, H, dk, n_splits)
    assert need <= lib.atma_polar_decode_static_max_floats()
    scratch = torch.empty(need, device=dev)
    stream = _lib.stream_ptr()
    for lens in ([768, 1, 300, 64, 0, 511], [5, 700, 128, 768, 333, 2]):     # two calls in a row
        q = torch.randn(B, H, dk, generator=g).bfloat16().to(dev)
        cl = torch.tensor(lens, dtype=torch.int32, device=dev)
        c1, m1 = torch.empty(B, H, dk, device=dev, dtype=torch.bfloat16), torch.empty(B, H, device=dev, dtype=torch.bfloat16)
        c2, m2 = torch.empty_like(c1), torch.empty_like(m1)
        a1 = _args(q, kc, vc, bt, cl, P, c1, m1, scratch, n_splits)
        a2 = _args(q, kc, vc, bt, cl, P, c2, m2, None, n_splits)
        _lib.check(lib.atma_polar_decode(byref(a1), stream))
        _lib.check(lib.atma_polar_decode_static(byref(a2), stream))
        torch.cuda.synchronize()
        assert max_abs(c2, c1) < 2e-2 and max_abs(m2, m1) < 2e-2       # the suite's 16-bit tolerance
        assert torch.equal(c2, c1) and torch.equal(m2, m1)              # same kernels, same order: identical


def test_static_scratch_entry_rejects_oversize_requests():
    lib = _lib.load()
    a = _lib.PolarDecodeArgs()
    a.B, a.H, a.Hkv, a.dk, a.n_splits, a.dtype = 4096, 8, 2, 128, 64, 1
    assert lib.atma_polar_decode_static(byref(a), None) == _lib.ATMA_ERR_INVALID
    assert b"exceeds the built-in scratch" in lib.atma_last_error()
