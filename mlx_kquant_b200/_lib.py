"""ctypes loader for libkquant_b200.so, the C-ABI declared in include/kquant_b200.h.

The library is built in-tree by ``csrc/Makefile`` (``__graft_entry__.build()``
runs it). There is no fallback: if the shared object is missing or does not
load, importing an op raises, so a silent CPU path can never stand in for the
CUDA kernels.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "libkquant_b200.so"

KQ_F32, KQ_F16, KQ_BF16 = 0, 1, 2
KQ_ERR_INVALID_ARGUMENT, KQ_ERR_RUNTIME, KQ_ERR_CUDA, KQ_ERR_UNSUPPORTED = 1, 2, 3, 4

# name -> (restype, argtypes); mirrors include/kquant_b200.h one to one.
SIGNATURES = {
    "kq_last_error": (C.c_char_p, []),
    "kq_version": (C.c_char_p, []),
    "kq_codec_count": (C.c_int, []),
    "kq_codec_info": (C.c_int, [C.c_int, C.POINTER(C.c_char_p), C.POINTER(C.c_int), C.POINTER(C.c_int),
                                C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "kq_codec_find": (C.c_int, [C.c_char_p]),
    "kq_dequantize": (C.c_int, [C.c_void_p, C.c_size_t, C.c_char_p, C.c_int, C.c_void_p, C.c_void_p]),
    "kq_quantize_cpu": (C.c_int, [C.c_void_p, C.c_int, C.c_longlong, C.c_longlong, C.c_char_p, C.c_void_p,
                                  C.c_void_p, C.c_int]),
    "kq_quantized_matmul_workspace_bytes": (C.c_size_t, [C.c_int, C.c_longlong, C.c_int]),
    "kq_quantized_matmul": (C.c_int, [C.c_void_p, C.c_int, C.c_longlong, C.c_int, C.c_longlong, C.c_void_p,
                                      C.c_size_t, C.c_int, C.c_char_p, C.c_int, C.c_void_p, C.c_longlong,
                                      C.c_void_p, C.c_size_t, C.c_void_p]),
    "kq_swiglu": (C.c_int, [C.c_void_p, C.c_void_p, C.c_longlong, C.c_longlong, C.c_int, C.c_int, C.c_void_p,
                            C.c_void_p]),
    "kq_moe_combine": (C.c_int, [C.c_void_p, C.c_void_p, C.c_longlong, C.c_int, C.c_int, C.c_int, C.c_void_p,
                                 C.c_void_p]),
    "kq_swiglu_routed": (C.c_int, [C.c_void_p, C.c_void_p, C.c_longlong, C.c_longlong, C.c_int, C.c_int, C.c_void_p,
                                   C.c_void_p, C.c_int, C.c_void_p]),
    "kq_moe_combine_f32": (C.c_int, [C.c_void_p, C.c_void_p, C.c_longlong, C.c_int, C.c_int, C.c_int, C.c_void_p,
                                     C.c_void_p]),
    "kq_quantized_matmul_qmv_bias": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_size_t, C.c_int,
                                               C.c_char_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "kq_expert_tile_map_capacity": (C.c_longlong, [C.c_longlong, C.c_int]),
    "kq_expert_tile_map_workspace_bytes": (C.c_size_t, [C.c_int]),
    "kq_expert_tile_map": (C.c_int, [C.c_void_p, C.c_longlong, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p,
                                     C.c_size_t, C.c_void_p]),
    "kq_gather_qmm_seg_workspace_bytes": (C.c_size_t, [C.c_int, C.c_longlong, C.c_int, C.c_int, C.c_longlong]),
    "kq_gather_qmm_seg": (C.c_int, [C.c_void_p, C.c_int, C.c_longlong, C.c_int, C.c_void_p, C.c_int, C.c_longlong,
                                    C.c_size_t, C.c_int, C.c_char_p, C.c_void_p, C.c_void_p, C.c_longlong,
                                    C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "kq_device_error_flags": (C.c_int, [C.POINTER(C.c_int), C.c_int]),
    "kq_codec_has_moe_glu": (C.c_int, [C.c_char_p]),
    "kq_moe_decode_workspace_bytes": (C.c_size_t, [C.c_longlong, C.c_int, C.c_int]),
    "kq_moe_glu_gather": (C.c_int, [C.c_void_p, C.c_int, C.c_longlong, C.c_int, C.c_void_p, C.c_longlong, C.c_void_p,
                                    C.c_longlong, C.c_size_t, C.c_int, C.c_int, C.c_char_p, C.c_void_p, C.c_int,
                                    C.c_char_p, C.c_float, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "kq_gather_qmv_mix": (C.c_int, [C.c_void_p, C.c_int, C.c_longlong, C.c_int, C.c_int, C.c_void_p, C.c_longlong,
                                    C.c_size_t, C.c_int, C.c_int, C.c_char_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                    C.c_void_p, C.c_size_t, C.c_int, C.c_void_p]),
    "kq_moe_router_topk": (C.c_int, [C.c_void_p, C.c_int, C.c_longlong, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p,
                                     C.c_void_p, C.c_char_p, C.c_float, C.c_void_p, C.c_void_p, C.c_void_p]),
    "kq_moe_block_workspace_bytes": (C.c_size_t, [C.c_longlong, C.c_int, C.c_int, C.c_int, C.c_int]),
    "kq_moe_swiglu_block": (C.c_int, [C.c_void_p, C.c_int, C.c_longlong, C.c_int, C.c_longlong, C.c_void_p, C.c_void_p,
                                      C.c_longlong, C.c_size_t, C.c_int, C.c_void_p, C.c_longlong, C.c_size_t, C.c_int,
                                      C.c_char_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p,
                                      C.c_size_t, C.c_void_p]),
    "kq_moe_swiglu_block_scatter": (C.c_int, [C.c_void_p, C.c_int, C.c_longlong, C.c_int, C.c_longlong, C.c_void_p,
                                              C.c_void_p, C.c_longlong, C.c_size_t, C.c_int, C.c_void_p, C.c_longlong,
                                              C.c_size_t, C.c_int, C.c_char_p, C.c_void_p, C.c_void_p, C.c_int,
                                              C.c_void_p, C.c_int, C.c_int, C.c_longlong, C.c_void_p, C.c_size_t,
                                              C.c_void_p]),
    "kq_moe_sum_slots": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_longlong, C.c_int, C.c_int,
                                   C.c_void_p, C.c_int, C.c_void_p]),
    "kq_peer_buffer_create": (C.c_int, [C.c_size_t, C.c_void_p, C.c_void_p]),
    "kq_peer_buffer_open": (C.c_int, [C.c_void_p, C.c_void_p]),
    "kq_peer_buffer_close": (C.c_int, [C.c_void_p]),
    "kq_peer_buffer_destroy": (C.c_int, [C.c_void_p]),
    "kq_peer_copy_async": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "kq_gather_qmm_workspace_bytes": (C.c_size_t, [C.c_longlong, C.c_int, C.c_int, C.c_int]),
    "kq_gather_qmm": (C.c_int, [C.c_void_p, C.c_int, C.c_longlong, C.c_int, C.c_int, C.c_void_p, C.c_int,
                                C.c_longlong, C.c_size_t, C.c_int, C.c_char_p, C.c_void_p, C.c_void_p,
                                C.c_longlong, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "kq_gather_qmm_noalloc": (C.c_int, [C.c_void_p, C.c_int, C.c_longlong, C.c_int, C.c_int, C.c_void_p, C.c_int,
                                        C.c_longlong, C.c_size_t, C.c_int, C.c_char_p, C.c_void_p, C.c_void_p,
                                        C.c_longlong, C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
}

_lib = None


def lib() -> C.CDLL:
    """Load (once) and return the shared library with typed entry points."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `make -C {HERE / 'csrc'}` "
                "(or __graft_entry__.build()); there is no CPU fallback.")
        handle = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(rc: int) -> None:
    """Map a KQ_ERR_* code to the exception the reference's binding raises."""
    if rc == 0:
        return
    msg = lib().kq_last_error().decode()
    if rc == KQ_ERR_INVALID_ARGUMENT:
        raise ValueError(msg)
    if rc == KQ_ERR_UNSUPPORTED:
        raise NotImplementedError(msg)
    raise RuntimeError(msg)
