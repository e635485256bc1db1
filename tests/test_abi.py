"""CPU: the C-ABI library builds, loads, and exports every symbol include/atma_b200.h declares.
No compute call is made here (there is no GPU in the CPU suite)."""

import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from atma_b200 import _lib
    if not os.path.exists(_lib.LIB_PATH):
        from atma_b200.build import build
        build()
    return _lib.load()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "atma_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(atma_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(lib):
    names = declared_symbols()
    assert len(names) >= 14
    for name in names:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"


def test_binding_table_matches_header(lib):
    from atma_b200 import _lib
    assert sorted(_lib.EXPORTED_SYMBOLS) == declared_symbols()


def test_struct_layout_matches_header(lib):
    """ctypes mirrors must have the size the C compiler gives the header's structs."""
    import subprocess, tempfile, textwrap
    from atma_b200 import _lib
    src = textwrap.dedent("""
        #include <stdio.h>
        #include "atma_b200.h"
        int main(void) { printf("%zu %zu\\n", sizeof(atma_polar_prefill_args), sizeof(atma_polar_decode_args)); return 0; }
    """)
    with tempfile.TemporaryDirectory() as d:
        c = os.path.join(d, "s.c")
        open(c, "w").write(src)
        exe = os.path.join(d, "s")
        subprocess.check_call(["gcc", "-I", os.path.join(ROOT, "include"), c, "-o", exe])
        a, b = map(int, subprocess.check_output([exe]).split())
    assert ctypes.sizeof(_lib.PolarPrefillArgs) == a
    assert ctypes.sizeof(_lib.PolarDecodeArgs) == b


def test_argument_validation_needs_no_gpu(lib):
    from atma_b200 import _lib
    assert lib.atma_abi_version() == 1
    assert lib.atma_polar_prefill(None, None) == _lib.ATMA_ERR_INVALID
    assert b"null args" in lib.atma_last_error()
    a = _lib.PolarDecodeArgs()
    a.dtype, a.H, a.Hkv = 7, 8, 2
    assert lib.atma_polar_decode(ctypes.byref(a), None) == _lib.ATMA_ERR_INVALID
    assert b"dtype" in lib.atma_last_error()
    with pytest.raises(ValueError):
        _lib.check(_lib.ATMA_ERR_INVALID)
    assert lib.atma_polar_decode_scratch_floats(64, 8, 128, 8) == 64 * 8 * 8 * 132
    # the packed scan: fp32 inputs are refused before anything is launched; scratch sizing is pure arithmetic
    rc = lib.atma_gated_delta_scan_varlen(None, None, None, 0, None, None, None, 2, 100, None, None, None, 0, None, None,
                                          None, None, 8, 2, 128, 128, 1, 1.0, None)
    assert rc == _lib.ATMA_ERR_INVALID and b"16-bit" in lib.atma_last_error()
    chunks = 1000 // 64 + 3
    assert lib.atma_gated_delta_scan_varlen_scratch_bytes(1000, 3, 8, 128, 128) >= 8 * chunks * 73728
    assert lib.atma_gated_delta_scan_varlen_scratch_bytes(1000, 3, 8, 64, 64) == 0


def test_ops_refuse_cpu_tensors():
    import torch
    import atma_b200
    x = torch.zeros(2, 8)
    with pytest.raises(RuntimeError):
        atma_b200.softcap_logits(x)
    with pytest.raises(RuntimeError):
        atma_b200.packed_causal_conv1d(x, torch.zeros(8, 4), torch.zeros(1, 8, 3), *[torch.zeros(2, dtype=torch.int32)] * 3)


def test_decode_split_heuristic():
    from atma_b200.polar import decode_num_splits
    n = decode_num_splits(64, 2, 32768)
    ctas = 64 * 2 * n
    assert ctas / (-(-ctas // 296) * 296) > 0.97 and 32768 // n >= 1024     # nearly full last wave
    assert decode_num_splits(1, 2, 32768) == 31                             # under one wave: as many as allowed
    assert decode_num_splits(1, 2, 256) == 1
    assert decode_num_splits(4096, 2, 32768) == 1


def test_compat_shim_resolves_the_reference_import_paths():
    """With the shim installed the reference's own import statements (inference/models/atma.py:31-80,
    model/blocks.py:24) resolve to this library's functions."""
    import importlib
    import sys
    import atma_b200
    from atma_b200 import compat
    saved_path, saved_mods = list(sys.path), {k: v for k, v in sys.modules.items() if k.split(".")[0] in ("kernel", "fla")}
    for k in saved_mods:
        del sys.modules[k]
    try:
        compat.install()
        pt = importlib.import_module("kernel.polar_triton")
        assert pt.polar_attention_fwd is atma_b200.polar_attention_fwd and pt.polar_attention_decode is atma_b200.polar_attention_decode
        assert pt.polar_attention_packed_fwd is atma_b200.polar_attention_packed_fwd and hasattr(pt, "HAS_TRITON")
        assert importlib.import_module("kernel.gated_delta_triton").gated_delta_decode_step is atma_b200.gated_delta_decode_step
        assert importlib.import_module("kernel.causal_conv1d_triton").causal_conv1d_decode_step is atma_b200.causal_conv1d_decode_step
        ops = importlib.import_module("kernel.inference_ops_triton")
        assert ops.squared_relu_gate is atma_b200.squared_relu_gate and ops.softcap_logits is atma_b200.softcap_logits
        assert ops.packed_causal_conv1d is atma_b200.packed_causal_conv1d and ops.linear_head_rms is atma_b200.linear_head_rms
        from fla.ops.gated_delta_rule import chunk_gated_delta_rule
        assert chunk_gated_delta_rule is atma_b200.chunk_gated_delta_rule
    finally:
        sys.path[:] = saved_path
        for k in [m for m in sys.modules if m.split(".")[0] in ("kernel", "fla")]:
            del sys.modules[k]
        sys.modules.update(saved_mods)


def test_prefill_kernel_register_hand_over_fits_the_launch_pool():
    """The tcgen05 prefill kernel re-divides its registers between warpgroups with setmaxnreg.  The counts it
    asks for must add up to no more than the CTA is launched with (registers per thread as compiled x threads),
    or the last warpgroup's request never returns.  Checked against the compiler's own report of the build."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    log = os.path.join(root, "atma_b200", "build", "polar_prefill_sm100.o.log")
    src = open(os.path.join(root, "atma_b200", "csrc", "polar_prefill_sm100.cu")).read()
    if not os.path.exists(log):
        pytest.skip("no compiler report (the library was not built in this tree)")
    used = [int(x) for x in re.findall(r"Used (\d+) registers", open(log).read())]
    threads = int(re.search(r"constexpr int kThreads = (\d+);", src).group(1))
    dec = int(re.search(r"setmaxnreg\.dec\.sync\.aligned\.u32 (\d+);", src).group(1))
    inc = int(re.search(r"setmaxnreg\.inc\.sync\.aligned\.u32 (\d+);", src).group(1))
    assert used and threads % 128 == 0
    asked = dec * 128 + inc * (threads - 128)                     # the first warpgroup shrinks, the others grow
    assert all(asked <= n * threads for n in used), (asked, used, threads)
