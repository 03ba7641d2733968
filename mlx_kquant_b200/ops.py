"""The ``kq.*`` ops over torch tensors, mirroring the reference's Python surface.

Names, argument order, defaults and the keyword-only ``stream`` follow the
reference's binding (bindings.cpp:94-141, 1349-1381, 1439-1461); shape and dtype
rules follow its op layer (src/kquant_ops.cpp). Tensors are ``torch`` CUDA
tensors instead of MLX arrays; CPU tensors are accepted for activations and
indices and are copied to the weights' device and back (that is the end-to-end
path the benchmark times). All arithmetic happens in the CUDA library behind
``include/kquant_b200.h``.
"""
from __future__ import annotations

import torch

from . import _lib
from ._lib import KQ_BF16, KQ_F16, KQ_F32, check

_DT = {torch.float32: KQ_F32, torch.float16: KQ_F16, torch.bfloat16: KQ_BF16}


def codecs() -> list[str]:
    """Names of the supported codecs (bindings.cpp:40-43)."""
    import ctypes as C

    L = _lib.lib()
    out = []
    name = C.c_char_p()
    for i in range(L.kq_codec_count()):
        L.kq_codec_info(i, C.byref(name), None, None, None, None)
        out.append(name.value.decode())
    return out


def codec_geometry(kquant_type: str) -> tuple[int, int, int, bool]:
    """(weights_per_block, bytes_per_block, bits, requires_imatrix) or ValueError."""
    import ctypes as C

    L = _lib.lib()
    i = L.kq_codec_find(kquant_type.encode())
    if i < 0:
        raise ValueError(f"[mlx_kquant] Unknown kquant_type: '{kquant_type}'.")
    v = [C.c_int() for _ in range(4)]
    L.kq_codec_info(i, None, *[C.byref(t) for t in v])
    return v[0].value, v[1].value, v[2].value, bool(v[3].value)


def _stream_ptr(stream, device) -> int:
    if stream is None:
        return torch.cuda.current_stream(device).cuda_stream
    return stream.cuda_stream


def _order_on(stream, device, *tensors) -> None:
    """A caller-given stream runs the kernel: it first waits for what the current stream has queued (the
    operands may have been produced or copied there), and every tensor the kernel touches is recorded on it so
    that the caching allocator does not hand its memory out while the kernel may still run."""
    if stream is None:
        return
    stream.wait_stream(torch.cuda.current_stream(device))
    for t in tensors:
        if t is not None and t.is_cuda:
            t.record_stream(stream)


def _require_cuda(w: torch.Tensor, op: str) -> None:
    if not w.is_cuda:
        raise RuntimeError(f"[mlx_kquant.{op}] w must live on a CUDA device; there is no CPU path.")


def dequantize(w, scales, kquant_type, dtype=None, *, stream=None):
    """Wire bytes -> float tensor; default dtype float16 (src/kquant_ops.cpp:55-110)."""
    if w.dtype != torch.uint8:
        raise ValueError("[mlx_kquant.dequantize] w must be uint8 (raw GGUF wire bytes).")
    if w.dim() < 1:
        raise ValueError("[mlx_kquant.dequantize] w must have at least 1 dimension.")
    out_dtype = dtype or torch.float16
    if out_dtype not in _DT:
        raise ValueError("[mlx_kquant.dequantize] Only real floating output dtypes are supported.")
    wpb, bpb, _, _ = codec_geometry(kquant_type)
    if w.shape[-1] % bpb != 0:
        raise ValueError(
            f"[mlx_kquant.dequantize] Last dim ({w.shape[-1]}) must be a multiple of bytes_per_block ({bpb}) "
            f"for codec '{kquant_type}'.")
    _require_cuda(w, "dequantize")
    w_c = w.contiguous()
    out = torch.empty(w.shape[:-1] + (w.shape[-1] // bpb * wpb,), dtype=out_dtype, device=w.device)
    _order_on(stream, w.device, w_c, out)
    with torch.cuda.device(w.device):
        check(_lib.lib().kq_dequantize(w_c.data_ptr(), w_c.numel(), kquant_type.encode(), _DT[out_dtype],
                                       out.data_ptr(), _stream_ptr(stream, w.device)))
    return out


def quantize(w, kquant_type, imatrix=None, *, stream=None):
    """Float weights [..., K] -> (wire bytes uint8 [..., K / wpb * bpb], scales placeholder uint8 [1]) on the
    HOST, like the reference's CPU-only encoder op (src/kquant_ops.cpp:550-631, bindings.cpp:1439-1446).
    Byte-identical with the reference for the thirteen codecs with a host encoder here (the ten of the benchmark
    and q4_1, q5_0, q5_1); iq2_xxs requires an imatrix. The other eight codecs are decode-only in this library."""
    del stream  # host work: there is no stream to order it on
    if w.dtype not in _DT:
        raise ValueError("[mlx_kquant.quantize] w must be a real floating tensor (float32, float16, or bfloat16).")
    if w.dim() < 1:
        raise ValueError("[mlx_kquant.quantize] w must have at least 1 dimension.")
    wpb, bpb, _, _ = codec_geometry(kquant_type)  # raises for an unknown codec
    K = w.shape[-1]
    if K % wpb != 0:
        raise ValueError(f"[mlx_kquant.quantize] Last dim ({K}) must be a multiple of weights_per_block ({wpb}) "
                         f"for codec '{kquant_type}'.")
    im_ptr = None
    if imatrix is not None:
        if imatrix.dtype != torch.float32:
            raise ValueError("[mlx_kquant.quantize] imatrix must be float32.")
        if imatrix.dim() != 1 or imatrix.shape[-1] != K:
            raise ValueError(f"[mlx_kquant.quantize] imatrix shape must be [K]=({K},) but got {tuple(imatrix.shape)}.")
        imatrix = imatrix.detach().cpu().contiguous()
        im_ptr = imatrix.data_ptr()
    w_c = w.detach().cpu().contiguous()
    out = torch.empty(w.shape[:-1] + (K // wpb * bpb,), dtype=torch.uint8)
    check(_lib.lib().kq_quantize_cpu(w_c.data_ptr(), _DT[w.dtype], w_c.numel(), K, kquant_type.encode(), im_ptr,
                                     out.data_ptr(), 0))
    return out, torch.zeros(1, dtype=torch.uint8)


def _prep_x(x: torch.Tensor, device, op: str):
    """Returns (x on device with a dense last dim, was_on_cpu)."""
    if x.dtype not in _DT:
        raise ValueError(f"[mlx_kquant.{op}] Only real floating x dtypes are supported.")
    on_cpu = not x.is_cuda
    if on_cpu:
        x = x.to(device, non_blocking=True)
    return x, on_cpu


def _expanded_inner(w, kquant_type, op):
    wpb, bpb, _, _ = codec_geometry(kquant_type)
    if w.shape[-1] % bpb != 0:
        raise ValueError(
            f"[mlx_kquant.{op}] KQuant weight last dim ({w.shape[-1]} bytes) is not a whole number of "
            f"{bpb}-byte {kquant_type} blocks.")
    return w.shape[-1] // bpb * wpb


def quantized_matmul(x, w, scales, kquant_type, transpose=True, *, stream=None):
    """``x @ dequant(w).T`` (src/kquant_ops.cpp:112-183). Output dtype = x dtype,
    float32 promoted to bfloat16."""
    op = "quantized_matmul"
    if w.dtype != torch.uint8:
        raise ValueError(f"[mlx_kquant.{op}] w must be uint8 (raw GGUF wire bytes).")
    codec_geometry(kquant_type)
    if x.dim() > 2 and w.dim() > 2:
        raise ValueError(f"[mlx_kquant.{op}] batched (>2D) weights are not supported; use gather_qmm for "
                         "mixture-of-experts.")
    wpr = _expanded_inner(w, kquant_type, op)
    inner = wpr if transpose else w.shape[-2]
    outer = w.shape[-2] if transpose else wpr
    if inner != x.shape[-1]:
        raise ValueError(
            f"[mlx_kquant.{op}] x last dim ({x.shape[-1]}) does not match the expanded quantized matrix inner dim "
            f"({inner}) for codec '{kquant_type}' with transpose={'true' if transpose else 'false'}.")
    _require_cuda(w, op)
    x, on_cpu = _prep_x(x, w.device, op)
    out_dtype = torch.bfloat16 if x.dtype == torch.float32 else x.dtype
    w2 = w if w.dim() == 2 else w.reshape(-1, w.shape[-2], w.shape[-1])[0]
    w2 = w2.contiguous()
    K = x.shape[-1]
    x2 = x.reshape(-1, K) if x.dim() != 1 else x.reshape(1, K)
    if x2.stride(-1) != 1 or (x2.stride(0) * x2.element_size()) % 16 != 0 or x2.data_ptr() % 16 != 0:
        x2 = x2.contiguous()
    rows = x2.shape[0]
    y = torch.empty((rows, outer), dtype=out_dtype, device=w.device)
    L = _lib.lib()
    ws_bytes = L.kq_quantized_matmul_workspace_bytes(_DT[x.dtype], rows, K)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=w.device) if ws_bytes else None
    _order_on(stream, w.device, ws, x2, w2, y)
    with torch.cuda.device(w.device):
        check(L.kq_quantized_matmul(x2.data_ptr(), _DT[x.dtype], rows, K, x2.stride(0), w2.data_ptr(),
                                    w2.shape[-1], outer, kquant_type.encode(), int(bool(transpose)),
                                    y.data_ptr(), y.stride(0), ws.data_ptr() if ws is not None else None,
                                    ws_bytes, _stream_ptr(stream, w.device)))
    y = y.reshape(x.shape[:-1] + (outer,))
    return y.cpu() if on_cpu else y


def gather_qmm(x, w, scales, kquant_type, lhs_indices=None, rhs_indices=None, transpose=True,
               sorted_indices=False, *, stream=None):
    """Mixture-of-experts matmul (src/kquant_ops.cpp:293-420): for each index entry,
    ``x[lhs] @ dequant(w[rhs]).T``; output shape ``lhs_indices.shape + [M, N]``."""
    op = "gather_qmm"
    if lhs_indices is None and rhs_indices is None:
        return quantized_matmul(x, w, scales, kquant_type, transpose, stream=stream)
    if w.dtype != torch.uint8:
        raise ValueError(f"[mlx_kquant.{op}] w must be uint8 (raw GGUF wire bytes).")
    codec_geometry(kquant_type)
    if x.dim() < 2:
        raise ValueError(f"[mlx_kquant.{op}] x must have at least two dimensions but got shape {tuple(x.shape)}.")
    wpr = _expanded_inner(w, kquant_type, op)
    inner = wpr if transpose else w.shape[-2]
    outer = w.shape[-2] if transpose else wpr
    if inner != x.shape[-1]:
        raise ValueError(
            f"[mlx_kquant.{op}] x last dim ({x.shape[-1]}) does not match the expanded quantized matrix inner dim "
            f"({inner}) for codec '{kquant_type}' with transpose={'true' if transpose else 'false'}.")
    _require_cuda(w, op)
    x, on_cpu = _prep_x(x, w.device, op)
    out_dtype = torch.bfloat16 if x.dtype == torch.float32 else x.dtype
    dev = w.device

    def default_idx(t):
        shape = t.shape[:-2]
        total = 1
        for d in shape:
            total *= d
        return torch.arange(total, dtype=torch.int64, device=dev).reshape(shape)

    lhs = default_idx(x) if lhs_indices is None else lhs_indices.to(dev)
    rhs = default_idx(w) if rhs_indices is None else rhs_indices.to(dev)
    lhs, rhs = torch.broadcast_tensors(lhs, rhs)
    idx_shape = tuple(lhs.shape)
    # uint32 on the wire; int32 storage holds the same bits for indices < 2^31
    lhs32 = lhs.reshape(-1).to(torch.int32).contiguous()
    rhs32 = rhs.reshape(-1).to(torch.int32).contiguous()
    n_entries = lhs32.numel()

    M, K = x.shape[-2], x.shape[-1]
    x3 = x.reshape(-1, M, K).contiguous()
    if w.dim() == 2:
        w3 = w.unsqueeze(0)
    elif w.dim() == 3:
        w3 = w
    else:
        w3 = w.reshape(-1, w.shape[-2], w.shape[-1])
    # matrix-contiguity is enough: a strided expert dimension is walked in 64-bit
    if w3.stride(2) != 1 or w3.stride(1) != w3.shape[2]:
        w3 = w3.contiguous()
    E = w3.shape[0]
    y = torch.empty((n_entries, M, outer), dtype=out_dtype, device=dev)
    L = _lib.lib()
    ws_bytes = L.kq_gather_qmm_workspace_bytes(n_entries, M, E, K)
    ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device=dev)
    right_sorted = bool(sorted_indices) and lhs_indices is None
    _order_on(stream, dev, ws, y, x3, w3, lhs32, rhs32)
    with torch.cuda.device(dev):
        check(L.kq_gather_qmm(x3.data_ptr(), _DT[x.dtype], x3.shape[0], M, K, w3.data_ptr(), E,
                              w3.stride(0) if E > 1 else w3.shape[1] * w3.shape[2], w3.shape[2], outer,
                              kquant_type.encode(), lhs32.data_ptr(), rhs32.data_ptr(), n_entries,
                              int(bool(transpose)), int(right_sorted), y.data_ptr(), ws.data_ptr(), ws.numel(),
                              _stream_ptr(stream, dev)))
    y = y.reshape(idx_shape + (M, outer))
    return y.cpu() if on_cpu else y


def expert_tile_map(indices, n_experts, *, stream=None):
    """(map uint32-as-int32 [capacity, 3], count [1]) for rows sorted by expert (src/kquant_ops.cpp:422-447):
    map rows are (expert, row_start, num_rows <= 64), the first ``count[0]`` of them valid, in unspecified order.
    Built on the device without a host read. torch has no uint32 arithmetic, so both tensors are int32 holding
    the same bits."""
    op = "expert_tile_map"
    if indices.dim() != 1 or indices.dtype not in (torch.int32, torch.int64, torch.uint32):
        raise ValueError(f"[mlx_kquant.{op}] indices must be 1-D uint32 but got shape {tuple(indices.shape)} "
                         f"dtype {indices.dtype}.")
    rows = indices.shape[0]
    if rows < 1 or n_experts < 1:
        raise ValueError(f"[mlx_kquant.{op}] indices must be non-empty and n_experts positive.")
    if not indices.is_cuda:
        raise RuntimeError(f"[mlx_kquant.{op}] indices must live on a CUDA device; there is no CPU path.")
    dev = indices.device
    idx = indices.to(torch.int32).contiguous()
    L = _lib.lib()
    cap = L.kq_expert_tile_map_capacity(rows, n_experts)
    tile_map = torch.zeros((cap, 3), dtype=torch.int32, device=dev)
    count = torch.zeros(1, dtype=torch.int32, device=dev)
    ws = torch.empty(max(L.kq_expert_tile_map_workspace_bytes(n_experts), 256), dtype=torch.uint8, device=dev)
    _order_on(stream, dev, idx, tile_map, count, ws)
    with torch.cuda.device(dev):
        check(L.kq_expert_tile_map(idx.data_ptr(), rows, n_experts, tile_map.data_ptr(), count.data_ptr(),
                                   ws.data_ptr(), ws.numel(), _stream_ptr(stream, dev)))
    return tile_map, count


def gather_qmm_seg(x, w, scales, kquant_type, map, counts, *, stream=None):  # noqa: A002 - the reference's name
    """Segment product (src/kquant_ops.cpp:466-548): x [rows, K] grouped by expert, w [n_experts, N, bytes],
    ``map`` [n_tiles, 3] = (expert, row_start, num_rows), ``counts`` [1] = valid map rows; returns [rows, N] with
    y[r] = x[r] @ dequant(w[expert covering r]).T. Rows no map entry covers are unspecified."""
    op = "gather_qmm_seg"
    if w.dtype != torch.uint8:
        raise ValueError(f"[mlx_kquant.{op}] w must be uint8 (raw GGUF wire bytes).")
    wpb, bpb, _, _ = codec_geometry(kquant_type)
    if x.dim() != 2:
        raise ValueError(f"[mlx_kquant.{op}] x must be [rows, K] but got shape {tuple(x.shape)}.")
    if w.dim() != 3:
        raise ValueError(f"[mlx_kquant.{op}] w must be (n_experts, N, bytes_per_row) but got shape {tuple(w.shape)}.")
    if map.dim() != 2 or map.shape[1] != 3 or map.shape[0] < 1 or map.dtype not in (torch.int32, torch.uint32):
        raise ValueError(f"[mlx_kquant.{op}] map must be uint32 [n_tiles >= 1, 3] (expert, row_start, num_rows) "
                         f"but got shape {tuple(map.shape)} dtype {map.dtype}.")
    if counts.dim() != 1 or counts.shape[0] != 1 or counts.dtype not in (torch.int32, torch.uint32):
        raise ValueError(f"[mlx_kquant.{op}] counts must be uint32 [1] but got shape {tuple(counts.shape)} "
                         f"dtype {counts.dtype}.")
    if w.shape[-1] % bpb != 0:
        raise ValueError(f"[mlx_kquant.{op}] KQuant weight last dim ({w.shape[-1]} bytes) is not a whole number of "
                         f"{bpb}-byte {kquant_type} blocks.")
    wpr = w.shape[-1] // bpb * wpb
    if wpr != x.shape[-1]:
        raise ValueError(f"[mlx_kquant.{op}] x last dim ({x.shape[-1]}) does not match the expanded quantized row "
                         f"width ({wpr}) for codec '{kquant_type}'.")
    if x.dtype not in _DT:
        raise ValueError(f"[mlx_kquant.{op}] Only real floating x dtypes are supported.")
    _require_cuda(w, op)
    dev = w.device
    xc = x.to(dev).contiguous()
    wc = w if (w.stride(2) == 1 and w.stride(1) == w.shape[2]) else w.contiguous()
    mc = map.to(dev).contiguous()
    cc = counts.to(dev).contiguous()
    rows, K = xc.shape
    E, N = wc.shape[0], wc.shape[1]
    out_dtype = torch.bfloat16 if x.dtype == torch.float32 else x.dtype
    y = torch.empty((rows, N), dtype=out_dtype, device=dev)
    if rows == 0 or N == 0:
        return y
    L = _lib.lib()
    ws = torch.empty(max(L.kq_gather_qmm_seg_workspace_bytes(_DT[x.dtype], rows, K, E, mc.shape[0]), 256),
                     dtype=torch.uint8, device=dev)
    _order_on(stream, dev, xc, wc, mc, cc, ws, y)
    with torch.cuda.device(dev):
        check(L.kq_gather_qmm_seg(xc.data_ptr(), _DT[x.dtype], rows, K, wc.data_ptr(), E, wc.stride(0), wc.shape[2], N,
                                  kquant_type.encode(), mc.data_ptr(), cc.data_ptr(), mc.shape[0], y.data_ptr(),
                                  ws.data_ptr(), ws.numel(), _stream_ptr(stream, dev)))
    return y


def quantized_matmul_qmv_bias(x, w, scales, bias, kquant_type, *, stream=None):
    """Decode-only product with the bias add fused into the kernel's epilogue (src/kquant_ops.cpp:185-283):
    x carries exactly one row, w is 2-D [N, bytes], bias [N]; q8_0 only, like the reference op."""
    op = "quantized_matmul_qmv_bias"
    if kquant_type != "q8_0":
        raise ValueError(f"[mlx_kquant.{op}] only kquant_type 'q8_0' is wired so far, got '{kquant_type}'.")
    if w.dtype != torch.uint8:
        raise ValueError(f"[mlx_kquant.{op}] w must be uint8 (raw GGUF wire bytes).")
    if w.dim() != 2:
        raise ValueError(f"[mlx_kquant.{op}] w must be 2D (this op is not batched); use gather_qmm for "
                         "mixture-of-experts.")
    wpb, bpb, _, _ = codec_geometry(kquant_type)
    if w.shape[-1] % bpb != 0:
        raise ValueError(f"[mlx_kquant.{op}] KQuant weight last dim ({w.shape[-1]} bytes) is not a whole number of "
                         f"{bpb}-byte {kquant_type} blocks.")
    K, N = w.shape[-1] // bpb * wpb, w.shape[0]
    if K != x.shape[-1]:
        raise ValueError(f"[mlx_kquant.{op}] x last dim ({x.shape[-1]}) does not match the expanded quantized matrix "
                         f"inner dim ({K}) for codec '{kquant_type}'.")
    if bias.dim() != 1 or bias.shape[0] != N:
        raise ValueError(f"[mlx_kquant.{op}] bias must be 1D with length {N} (the output dim), got shape "
                         f"{tuple(bias.shape)}.")
    if x.numel() // x.shape[-1] != 1:
        raise ValueError(f"[mlx_kquant.{op}] decode-only: x must carry exactly one row (got "
                         f"{x.numel() // x.shape[-1]}). Use quantized_matmul() + a separate add for prefill/verify "
                         "shapes.")
    if x.dtype not in _DT:
        raise ValueError(f"[mlx_kquant.{op}] Only real floating x dtypes are supported.")
    _require_cuda(w, op)
    dev = w.device
    x, on_cpu = _prep_x(x, dev, op)
    out_dtype = torch.bfloat16 if x.dtype == torch.float32 else x.dtype
    xc = x.reshape(1, K).contiguous()
    wc = w.contiguous()
    bc = bias.to(dev).to(out_dtype).contiguous()
    y = torch.empty(x.shape[:-1] + (N,), dtype=out_dtype, device=dev)
    _order_on(stream, dev, xc, wc, bc, y)
    with torch.cuda.device(dev):
        check(_lib.lib().kq_quantized_matmul_qmv_bias(xc.data_ptr(), _DT[x.dtype], K, wc.data_ptr(), wc.shape[1], N,
                                                      kquant_type.encode(), bc.data_ptr(), y.data_ptr(),
                                                      _stream_ptr(stream, dev)))
    return y.cpu() if on_cpu else y
