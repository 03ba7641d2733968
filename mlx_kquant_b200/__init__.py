"""kquant_b200: the quantized-weight ops of mlx-kquant on B200 (sm_100a).

    import mlx_kquant_b200 as kq
    y = kq.quantized_matmul(x, w, scales, "q4_k")

``dequantize``, ``quantized_matmul``, ``gather_qmm`` and ``codecs`` keep the
reference's names, argument order and defaults (bindings.cpp:40-43, 94-141,
1349-1381). Everything runs in hand-written CUDA kernels behind the C ABI in
``include/kquant_b200.h``; importing this package without the built library
raises at the first op call.
"""
from .ops import (codec_geometry, codecs, dequantize, expert_tile_map, gather_qmm, gather_qmm_seg, quantize,
                  quantized_matmul, quantized_matmul_qmv_bias)

__all__ = ["codecs", "codec_geometry", "dequantize", "quantized_matmul", "gather_qmm", "quantize", "expert_tile_map",
           "gather_qmm_seg", "quantized_matmul_qmv_bias"]
