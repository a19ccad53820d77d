"""ctypes binding of ``libflashquant_b200.so`` (the C ABI declared in include/flashquant_b200.h).

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""

from __future__ import annotations

import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libflashquant_b200.so")

FQ_F32, FQ_F16, FQ_BF16 = 0, 1, 2
_DTYPES = {torch.float32: FQ_F32, torch.float16: FQ_F16, torch.bfloat16: FQ_BF16}

FQ_DEV_BAD_BLOCK_INDEX = 1
FQ_DEV_WAIT_TIMEOUT = 2


class FlashQuantNativeError(RuntimeError):
    """A C-ABI call returned a negative status."""

    def __init__(self, code: int, message: str):
        super().__init__(f"flashquant_b200 native call failed ({code}): {message}")
        self.code = code


_p, _i, _i64, _f, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t

# name -> (restype, argtypes); must list every symbol the header declares
SIGNATURES = {
    "fq_version": (_i, []),
    "fq_last_error_string": (C.c_char_p, []),
    "fq_launch_count": (C.c_uint64, []),
    "fq_tq4_compress": (_i, [_p, _i, _p, _p, _p, _i, _p, _p, _i64, _i, _p]),
    "fq_tq_prod_quantize": (_i, [_p, _i, _p, _p, _i, _p, _p, _p, _p, _p, _p, _i64, _i, _p]),
    "fq_tq4_decompress": (_i, [_p, _p, _p, _i, _p, _i, _i64, _i, _p]),
    "fq_tq4_compress_append": (_i, [_p, _p, _i, _i64, _i, _i, _i64, _p, _p, _i, _p, _i, _p,
                                    _i64, _p, _i, _p]),
    "fq_tq4_compress_append_qjl": (_i, [_p, _p, _i, _i64, _i, _i, _i64, _p, _p, _i, _p, _p, _i,
                                        _p, _p, _p, _i64, _p, _i, _p]),
    "fq_paged_decode_workspace_bytes": (_sz, [_i, _i, _i, _i, _i]),
    "fq_split_k_paged_decode": (_i, [_p, _i, _p, _p, _i64, _p, _p, _i, _p, _i, _p, _i, _i, _i,
                                     _i, _i, _i64, _f, _p, _i, _p, _sz, _p]),
    "fq_split_k_paged_decode_static_max_bytes": (_sz, []),
    "fq_split_k_paged_decode_static": (_i, [_p, _i, _p, _p, _i64, _p, _p, _i, _p, _i, _p, _i, _i,
                                            _i, _i, _i, _i64, _f, _p, _i, _p]),
    "fq_split_k_paged_decode_static_status": (_i, [_p, _p]),
    "fq_paged_decode_partials": (_i, [_p, _i, _p, _p, _i64, _p, _p, _i, _p, _i, _p, _i, _i, _i,
                                      _i, _i, _i64, _f, _i, _p, _p, _sz, _p]),
    "fq_paged_decode_partials_rotated": (_i, [_p, _p, _p, _i64, _p, _p, _i, _p, _i, _i, _i, _i,
                                              _i, _i, _i64, _f, _i, _p, _p, _sz, _p]),
    "fq_paged_decode_stream": (_i, [_p, _p, _p, _i64, _p, _p, _i, _p, _i, _i, _i, _i, _i, _i,
                                    _i64, _f, _i, _p, _sz, _p]),
    "fq_split_k_merge": (_i, [_p, _i, _p, _i, _i, _i, _p, _i, _p]),
    "fq_fused_tq_attention_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "fq_fused_tq_attention": (_i, [_p, _i, _p, _p, _p, _p, _p, _i, _p, _i, _p, _i, _i, _i, _i, _i,
                                   _i, _f, _i, _p, _p, _sz, _p]),
    "fq_workspace_status": (_i, [_p, _p, _p]),
    "fq_tq4_compress_into": (_i, [_p, _i, _p, _p, _p, _i, _p, _p, _i64, _i64, _i64, _i64, _i, _p]),
    "fq_split_k_paged_decode_multi_scratch_bytes": (_sz, [_i, _i, _i]),
    "fq_split_k_paged_decode_multi_workspace_bytes": (_sz, [_i, _i, _i, _i, _i, _i]),
    "fq_split_k_paged_decode_multi": (_i, [_p, _i, _p, _p, _i64, _i, _p, _p, _i, _p, _i, _p, _i, _i,
                                           _i, _i, _i, _i, _i64, _f, _p, _i, _p, _sz, _p, _sz, _p]),
    "fq_pack_2bit": (_i, [_p, _p, _i64, _p, _p]),
    "fq_unpack_2bit": (_i, [_p, _p, _i64, _p]),
    "fq_cache_update_workspace_bytes": (_sz, [_i64, _i64, _i]),
    "fq_cache_update": (_i, [_p, _p, _i, _p, _p, _p, _p, _p, _p, _p, _i, _p, _i, _p, _p, _p, _p,
                             _i64, _i64, _i64, _i64, _p, _p, _i64, _i64, _i, _p, _sz, _p]),
    "fq_tq4_decompress_original_workspace_bytes": (_sz, [_i64, _i]),
    "fq_tq4_decompress_original": (_i, [_p, _p, _p, _i, _p, _p, _i, _i64, _i, _p, _sz, _p]),
    "fq_fused_tq_attention_kv": (_i, [_p, _i, _p, _p, _p, _p, _p, _i, _p, _i, _p, _p, _i, _i, _i,
                                      _i, _i, _i64, _i, _f, _i, _p, _p, _sz, _p]),
    "fq_paged_decode_set_single_launch": (None, [_i]),
    "fq_paged_decode_set_fast_path": (None, [_i]),
    "fq_paged_decode_set_weight_split": (None, [_i]),
    "fq_paged_decode_test_expect_extra_segments": (None, [_i]),
    "fq_set_device_wait_limit_ns": (None, [C.c_uint64]),
    "fq_get_device_wait_limit_ns": (C.c_uint64, []),
    "fq_split_k_paged_decode_qjl": (_i, [_p, _i, _p, _p, _p, _i64, _p, _p, _i, _p, _i, _p, _p, _i,
                                         _i, _i, _i, _i, _i64, _f, _p, _i, _p, _sz, _p]),
    "fq_decode_step_host_staging_bytes": (_sz, [_i, _i, _i, _i, _i64, _i]),
    "fq_decode_step_host": (_i, [_p, _p, _p, _i, _p, _i, _p, _i64, _p, _p, _p, _p, _p, _i, _p, _i,
                                 _p, _i, _p, _i, _p, _i, _i, _i, _i, _i, _i64, _f, _i, _p, _p, _sz,
                                 _p, _sz, _p]),
    "fq_paged_tq4_prefill_workspace_bytes": (_sz, [_i, _i, _i]),
    "fq_paged_tq4_prefill": (_i, [_p, _i, _p, _p, _i64, _p, _p, _p, _i, _p, _i, _p, _i, _i, _i, _i,
                                  _i, _i, _i, _i64, _f, _p, _p, _sz, _p]),
    "fq_decode_step_set_graph": (None, [_i]),
    "fq_decode_step_offsets": (_i, [_i, _i, _i, _i, _i64, _i, _p]),
    "fq_decode_step_host_packed": (_i, [_p, _p, _i, _i, _i, _i64, _p, _p, _p, _p, _i, _p, _i, _p,
                                        _i, _p, _i, _p, _i, _i, _i, _i, _i, _i64, _f, _i, _p, _sz,
                                        _p, _sz, _p]),
}

_lib = None


def load() -> C.CDLL:
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FlashQuantNativeError(
                -100, f"{LIB_PATH} not found: run `python -m flashquant_b200.build` first")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPES[dt]
    except KeyError:
        raise TypeError(f"unsupported dtype {dt}; expected float32, float16 or bfloat16") from None


def ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def stream_ptr(device) -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def check(code: int) -> None:
    if code != 0:
        raise FlashQuantNativeError(code, load().fq_last_error_string().decode())


def require_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise FlashQuantNativeError(
                -101, "this package has no CPU path: every tensor must live on a CUDA device")
