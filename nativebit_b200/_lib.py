"""ctypes binding of libnativebit_b200.so — the only route from Python to the kernels.

There is deliberately no fallback: if the shared library is missing or a call returns a
non-zero status, a RuntimeError is raised.
"""
from __future__ import annotations

import ctypes
import os
import re

from .build import LIB_PATH

NB_F32, NB_F16, NB_BF16 = 0, 1, 2

_HEADER = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "include", "nativebit_b200.h")
_lib = None

_c = ctypes
_SIGNATURES = {
    "nb_version": (_c.c_int, []),
    "nb_status_string": (_c.c_char_p, [_c.c_int]),
    "nb_last_cuda_error": (_c.c_char_p, []),
    "nb_selftest_tables": (_c.c_int, []),
    "nb_unpack": (_c.c_int, [_c.c_void_p, _c.c_int, _c.c_int64, _c.c_void_p, _c.c_void_p]),
    "nb_pack": (_c.c_int, [_c.c_void_p, _c.c_int, _c.c_int64, _c.c_void_p, _c.c_void_p]),
    "nb_dequant": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int, _c.c_int, _c.c_int64, _c.c_int64,
                              _c.c_void_p, _c.c_int, _c.c_void_p]),
    "nb_quantize": (_c.c_int, [_c.c_void_p, _c.c_int64, _c.c_void_p, _c.c_int, _c.c_int, _c.c_int, _c.c_void_p, _c.c_void_p]),
    "nb_gemv_workspace_bytes": (_c.c_size_t, [_c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int]),
    "nb_prefill_workspace_bytes": (_c.c_size_t, [_c.c_int, _c.c_int, _c.c_int]),
    "nb_gemm_prefill": (_c.c_int, [_c.c_void_p, _c.c_int, _c.c_int, _c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int, _c.c_int, _c.c_int,
                                   _c.c_int, _c.c_void_p, _c.c_int, _c.c_void_p, _c.c_size_t, _c.c_void_p]),
    "nb_prefill_fused_workspace_bytes": (_c.c_size_t, [_c.c_int, _c.c_int, _c.c_int]),
    "nb_gemm_prefill_fused": (_c.c_int, [_c.c_void_p, _c.c_int, _c.c_int, _c.c_void_p, _c.c_int, _c.c_int, _c.c_int, _c.c_void_p,
                                         _c.c_int, _c.c_void_p, _c.c_size_t, _c.c_void_p]),
    "nb_gemm_bf16": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int, _c.c_int, _c.c_void_p, _c.c_int, _c.c_void_p,
                                _c.c_void_p]),
    "nb_add_rmsnorm": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_float, _c.c_void_p, _c.c_int, _c.c_int, _c.c_void_p]),
    "nb_rope_kv_write": (_c.c_int, [_c.c_void_p, _c.c_int, _c.c_int, _c.c_int, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p,
                                    _c.c_void_p, _c.c_int, _c.c_void_p, _c.c_void_p]),
    "nb_decode_attention": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int, _c.c_int, _c.c_int,
                                       _c.c_void_p, _c.c_int, _c.c_int, _c.c_void_p]),
    "nb_decode_attention_rope": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int,
                                            _c.c_int, _c.c_int, _c.c_int, _c.c_void_p, _c.c_int, _c.c_int, _c.c_void_p]),
    "nb_silu_mul": (_c.c_int, [_c.c_void_p, _c.c_int, _c.c_int, _c.c_void_p, _c.c_void_p]),
    "nb_lm_head_scratch_bytes": (_c.c_size_t, []),
    "nb_lm_head": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_float, _c.c_void_p, _c.c_int, _c.c_int, _c.c_float,
                              _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p]),
    "nb_prefill_attention": (_c.c_int, [_c.c_void_p, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_void_p, _c.c_void_p, _c.c_int,
                                        _c.c_void_p, _c.c_void_p, _c.c_int, _c.c_void_p, _c.c_int, _c.c_int, _c.c_void_p]),
    "nb_allreduce_buffer_bytes": (_c.c_size_t, [_c.c_int, _c.c_int]),
    "nb_allreduce": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_int, _c.c_void_p, _c.c_int, _c.c_int, _c.c_int, _c.c_uint32,
                                _c.c_void_p, _c.c_void_p]),
    "nb_embed_rows": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int, _c.c_int, _c.c_void_p, _c.c_void_p]),
    "nb_softcap_argmax": (_c.c_int, [_c.c_void_p, _c.c_int, _c.c_int, _c.c_int, _c.c_float, _c.c_void_p, _c.c_void_p, _c.c_void_p,
                                     _c.c_void_p]),
    "nb_gemv_fused": (_c.c_int, [_c.c_int, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_float, _c.c_void_p, _c.c_int, _c.c_void_p,
                                 _c.c_void_p, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_void_p, _c.c_int, _c.c_void_p,
                                 _c.c_size_t, _c.c_void_p]),
    "nb_exchange_buffer_bytes": (_c.c_size_t, [_c.c_int, _c.c_int]),
    "nb_exchange_init": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int, _c.c_int]),
    "nb_gemv_tp": (_c.c_int, [_c.c_int, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_float, _c.c_void_p, _c.c_int, _c.c_void_p,
                              _c.c_void_p, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_void_p, _c.c_int, _c.c_void_p,
                              _c.c_size_t, _c.c_void_p, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_uint32, _c.c_void_p]),
    "nb_exchange_gather": (_c.c_int, [_c.c_void_p, _c.c_int, _c.c_void_p, _c.c_int, _c.c_int, _c.c_int, _c.c_uint32, _c.c_void_p,
                                      _c.c_void_p]),
    "nb_gemv_static": (_c.c_int, [_c.c_void_p, _c.c_int, _c.c_int, _c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int, _c.c_int,
                                  _c.c_int, _c.c_int, _c.c_void_p, _c.c_int, _c.c_void_p]),
    "nb_gemv_static_status": (_c.c_int, [_c.c_void_p, _c.c_int]),
    "nb_gemv_ordered": (_c.c_int, [_c.c_void_p, _c.c_int, _c.c_int, _c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int, _c.c_int,
                                   _c.c_int, _c.c_int, _c.c_void_p, _c.c_int, _c.c_void_p, _c.c_size_t, _c.c_void_p]),
    "nb_stream_packed_bytes": (_c.c_size_t, [_c.c_int, _c.c_int, _c.c_int]),
    "nb_stream_pack": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_void_p,
                                  _c.c_void_p]),
    "nb_stream_state_bytes": (_c.c_size_t, []),
    "nb_stream_max_ops": (_c.c_int, []),
    "nb_stream_ctas": (_c.c_int, []),
    "nb_stream_slots": (_c.c_int, [_c.c_int, _c.c_int, _c.c_int]),
    "nb_stream_run": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_int, _c.c_void_p, _c.c_uint32, _c.c_void_p]),
    "nb_gemv_stream": (_c.c_int, [_c.c_int, _c.c_void_p, _c.c_int, _c.c_void_p, _c.c_void_p, _c.c_float, _c.c_void_p, _c.c_void_p,
                                  _c.c_int, _c.c_int, _c.c_int, _c.c_void_p, _c.c_int, _c.c_void_p]),
    "nb_gemv_stream_max_rows": (_c.c_int, [_c.c_int, _c.c_int]),
    "nb_gemv_stream_rows": (_c.c_int, [_c.c_int, _c.c_void_p, _c.c_int, _c.c_void_p, _c.c_void_p, _c.c_float, _c.c_void_p, _c.c_void_p,
                                       _c.c_int, _c.c_int, _c.c_int, _c.c_void_p, _c.c_int, _c.c_void_p]),
    "nb_group_plan_bytes": (_c.c_size_t, [_c.c_void_p, _c.c_int]),
    "nb_group_max_items": (_c.c_int, []),
    "nb_group_build": (_c.c_int, [_c.c_void_p, _c.c_int, _c.c_int, _c.c_void_p, _c.c_size_t]),
    "nb_group_run": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p]),
    "nb_gemv_plan": (_c.c_int, [_c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_void_p]),
    "nb_gemv": (_c.c_int, [_c.c_void_p, _c.c_int, _c.c_int, _c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int, _c.c_int,
                           _c.c_int, _c.c_int, _c.c_void_p, _c.c_int, _c.c_void_p, _c.c_size_t, _c.c_void_p]),
}


def declared_symbols() -> list[str]:
    """Names of the functions the public header declares."""
    text = open(_HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nb_[a-z0-9_]+)\s*\(", text)))


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m nativebit_b200.build` "
                "(nativebit_b200 has no fallback path)")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def check(status: int, what: str) -> None:
    if status != 0:
        l = lib()
        msg = l.nb_status_string(status).decode()
        cuda = l.nb_last_cuda_error().decode()
        raise RuntimeError(f"{what} failed: status {status} ({msg})" + (f" [{cuda}]" if cuda and status == 5 else ""))
