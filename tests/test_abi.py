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
