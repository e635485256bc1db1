"""ctypes binding of libatma_b200.so (the C ABI declared in include/atma_b200.h).

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""

import ctypes
import os
from ctypes import (POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_void_p)

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libatma_b200.so")

ATMA_OK, ATMA_ERR_INVALID, ATMA_ERR_CUDA, ATMA_ERR_UNSUPPORTED = 0, -1, -2, -3
DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


class PolarPrefillArgs(Structure):
    """Mirror of atma_polar_prefill_args; field order and types must match the header."""
    _fields_ = [
        ("q", c_void_p), ("k", c_void_p), ("v", c_void_p),
        ("q_sb", c_int64), ("q_sh", c_int64), ("q_st", c_int64),
        ("k_sb", c_int64), ("k_sh", c_int64), ("k_st", c_int64),
        ("v_sb", c_int64), ("v_sh", c_int64), ("v_st", c_int64),
        ("c", c_void_p), ("c_sb", c_int64), ("c_sh", c_int64), ("c_st", c_int64),
        ("mag", c_void_p), ("mag_sb", c_int64), ("mag_sh", c_int64), ("mag_st", c_int64),
        ("n_keys", c_void_p), ("n_base", c_float), ("key_offset", c_int64),
        ("v_null", c_void_p), ("spg", c_void_p), ("null_base", c_void_p), ("sps", c_void_p),
        ("beta", c_void_p),
        ("stats_in_m", c_void_p), ("stats_in_l", c_void_p), ("stats_in_q2", c_void_p),
        ("stats_in_s", c_void_p),
        ("stats_out_m", c_void_p), ("stats_out_l", c_void_p), ("stats_out_q2", c_void_p),
        ("stats_out_s", c_void_p),
        ("finalize", c_int),
        ("B", c_int), ("H", c_int), ("Hkv", c_int), ("Tq", c_int), ("Tk", c_int), ("dk", c_int),
        ("dtype", c_int), ("window", c_int), ("eps", c_float),
        ("tile_seq_start", c_void_p), ("tile_q_start", c_void_p), ("tile_seq_len", c_void_p),
        ("n_tiles", c_int),
    ]


class PolarDecodeArgs(Structure):
    """Mirror of atma_polar_decode_args."""
    _fields_ = [
        ("q", c_void_p), ("k_cache", c_void_p), ("v_cache", c_void_p),
        ("block_tables", c_void_p), ("bt_stride", c_int64), ("context_lens", c_void_p),
        ("v_null", c_void_p), ("spg", c_void_p), ("null_base", c_void_p), ("sps", c_void_p),
        ("beta", c_void_p),
        ("c", c_void_p), ("mag", c_void_p), ("scratch", c_void_p),
        ("B", c_int), ("H", c_int), ("Hkv", c_int), ("dk", c_int), ("block_size", c_int),
        ("max_blocks", c_int), ("num_blocks", c_int), ("n_splits", c_int), ("dtype", c_int),
        ("window", c_int), ("eps", c_float),
        ("gate", c_void_p), ("gate_sb", c_int64), ("gate_sh", c_int64), ("c_sb", c_int64), ("mag_sb", c_int64),
        ("temp_lens", c_void_p), ("skip_merge", c_int),
        ("append_k", c_void_p), ("append_v", c_void_p), ("append_k_stride", c_int64), ("append_v_stride", c_int64),
        ("append_slots", c_void_p),
    ]


_SIGNATURES = {
    "atma_last_error": (c_char_p, []),
    "atma_abi_version": (c_int, []),
    "atma_polar_prefill": (c_int, [POINTER(PolarPrefillArgs), c_void_p]),
    "atma_polar_prefill_path": (c_int, [POINTER(PolarPrefillArgs)]),
    "atma_device_status": (c_int, [POINTER(c_int)]),
    "atma_polar_decode_scratch_floats": (c_int64, [c_int, c_int, c_int, c_int]),
    "atma_polar_decode": (c_int, [POINTER(PolarDecodeArgs), c_void_p]),
    "atma_polar_decode_merge": (c_int, [POINTER(PolarDecodeArgs), c_void_p]),
    "atma_polar_decode_appends": (c_int, [POINTER(PolarDecodeArgs)]),
    "atma_polar_decode_static_max_floats": (c_int64, []),
    "atma_polar_decode_static": (c_int, [POINTER(PolarDecodeArgs), c_void_p]),
    "atma_gated_delta_decode_step": (c_int, [c_void_p] * 3 + [c_int64] * 6 + [c_int, c_void_p, c_void_p,
                                             c_void_p, c_int64, c_int64, c_void_p, c_void_p,
                                             c_int, c_int, c_int, c_int, c_float, c_void_p]),
    "atma_gated_delta_scan_scratch_bytes": (c_int64, [c_int] * 5),
    "atma_gated_delta_scan": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                      c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                      c_int, c_float, c_void_p]),
    "atma_gated_delta_decode_step_fused": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64,
                                                   c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                                   c_float, c_float, c_void_p, c_int64, c_int64, c_void_p, c_void_p,
                                                   c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_int,
                                                   c_float, c_float, c_void_p]),
    "atma_qkv_prep_decode": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p,
                                     c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p,
                                     c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                     c_float, c_int, c_void_p]),
    "atma_add_rms_norm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p]),
    "atma_decode_linear": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int,
                                   c_void_p]),
    "atma_gated_delta_scan_segmented": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                                c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                                c_int, c_float, c_int, c_void_p]),
    "atma_gated_delta_scan_factors": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                              c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p]),
    "atma_gated_delta_scan_recur": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                            POINTER(c_int), POINTER(c_int), c_void_p, c_void_p, c_void_p, c_void_p]),
    "atma_gated_delta_scan_varlen": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                             c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p,
                                             c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p]),
    "atma_gated_delta_scan_varlen_snapshots": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                                       c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p,
                                                       c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_int,
                                                       c_void_p]),
    "atma_gated_delta_scan_varlen_scratch_bytes": (c_int64, [c_int64, c_int, c_int, c_int, c_int]),
    "atma_causal_conv1d_decode_step": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64,
                                               c_void_p, c_int64, c_int, c_int, c_int, c_int, c_void_p]),
    "atma_packed_causal_conv1d": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p,
                                          c_void_p, c_int64, c_void_p, c_void_p, c_void_p,
                                          c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "atma_qkv_prep_prefill": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_int64,
                                      c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                      c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_void_p, c_void_p, c_void_p,
                                      c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p]),
    "atma_sigmoid_gate_mul": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_void_p,
                                      c_int, c_int, c_int, c_int, c_void_p]),
    "atma_rms_sigmoid_gate": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_int, c_int, c_int, c_float, c_int, c_void_p]),
    "atma_lfm2_conv_decode_step": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_int64,
                                           c_int, c_int, c_int, c_int, c_void_p]),
    "atma_lfm2_conv_packed": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int64,
                                      c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "atma_store_kvcache": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p,
                                   c_int, c_int, c_int, c_void_p]),
    "atma_squared_relu_gate": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int, c_int,
                                       c_int, c_void_p]),
    "atma_softcap_logits": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_void_p]),
    "atma_linear_head_rms": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                     c_int, c_float, c_int, c_void_p]),
}

EXPORTED_SYMBOLS = tuple(_SIGNATURES)

_lib = None


def load():
    """Load the shared library (once).  Raises RuntimeError if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m atma_b200.build` "
            "(nvcc, sm_100a).  atma_b200 has no CPU or PyTorch fallback.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError here = header / library mismatch
        fn.restype, fn.argtypes = res, args
    _lib = lib
    return lib


def check(rc):
    """Turn a C status into the exception the reference API would raise."""
    if rc == ATMA_OK:
        return
    msg = load().atma_last_error().decode("utf-8", "replace")
    if rc in (ATMA_ERR_INVALID, ATMA_ERR_UNSUPPORTED):
        raise ValueError(msg)
    raise RuntimeError(msg)


def ptr(t):
    return None if t is None else c_void_p(t.data_ptr())


def stream_ptr():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def dtype_code(t):
    try:
        return DTYPE_CODE[t.dtype]
    except KeyError:
        raise ValueError(f"unsupported dtype {t.dtype}; expected float32, bfloat16 or float16") from None


def require_cuda(t, what):
    if not t.is_cuda:
        raise RuntimeError(f"{what} requires CUDA tensors (atma_b200 has no CPU path)")


def device_status():
    """Synchronise the current device and return the status word of the tensor-core kernels: 0, or non-zero if a
    bounded wait of a tcgen05 kernel (Polar prefill, gated-delta recurrence, chunk-local stage) ran out since the
    last call (the word is cleared).  Results of launches since the last call are then not to be trusted."""
    import ctypes
    status = ctypes.c_int(-1)
    check(load().atma_device_status(ctypes.byref(status)))
    return status.value

