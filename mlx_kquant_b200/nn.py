"""torch modules over GGUF wire bytes, the counterparts of the reference's module layer
(mlx_kquant/nn.py:50-268): `KQuantEmbedding`, `KQuantLinear`, `KQuantSwitchLinear`.

Each keeps `weight` as a uint8 buffer of wire bytes (never a float copy) and a one-byte `scales`
placeholder, so that a state dict has the reference's keys and shapes, and calls the `kq.*` ops.
"""
from __future__ import annotations

import os

import torch

from . import ops as kq


def bytes_per_row(codec: str, dims: int) -> int:
    """Wire bytes of one row of `dims` weights (mlx_kquant/codec_geometry.py)."""
    wpb, bpb, _, _ = kq.codec_geometry(codec)
    if dims % wpb != 0:
        raise ValueError(f"[mlx_kquant] {dims} weights per row is not a whole number of {wpb}-weight {codec} blocks.")
    return dims // wpb * bpb


class _KQuantBase(torch.nn.Module):
    def _init_codec(self, codec: str) -> None:
        wpb, _, bits, _ = kq.codec_geometry(codec)
        self.mode = "kquant"
        self.group_size = wpb
        self.bits = bits
        self.kquant_type = codec
        self.register_buffer("scales", torch.zeros(1, dtype=torch.uint8))


class KQuantEmbedding(_KQuantBase):
    """Embedding table in wire bytes (mlx_kquant/nn.py:50-96): a lookup gathers the tokens' wire rows and
    dequantizes only those; `as_linear` is the tied output projection."""

    def __init__(self, num_embeddings: int, dims: int, codec: str, out_dtype: torch.dtype = torch.bfloat16):
        super().__init__()
        self._init_codec(codec)
        self.num_embeddings, self.dims, self.out_dtype = num_embeddings, dims, out_dtype
        self.register_buffer("weight", torch.zeros((num_embeddings, bytes_per_row(codec, dims)), dtype=torch.uint8))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        rows = self.weight[x.to(self.weight.device).reshape(-1)]
        deq = kq.dequantize(rows, self.scales, self.kquant_type, self.out_dtype)
        return deq.reshape(*x.shape, self.dims)

    def as_linear(self, x: torch.Tensor) -> torch.Tensor:
        return kq.quantized_matmul(x, self.weight, self.scales, self.kquant_type, transpose=True)

    def extra_repr(self) -> str:
        return f"{self.num_embeddings}, {self.dims}, kquant_type={self.kquant_type}"


class KQuantLinear(_KQuantBase):
    """Linear layer in wire bytes (mlx_kquant/nn.py:99-158): weight [out_dims, bytes_per_row]."""

    def __init__(self, in_dims: int, out_dims: int, bias: bool, codec: str):
        super().__init__()
        self._init_codec(codec)
        self.register_buffer("weight", torch.zeros((out_dims, bytes_per_row(codec, in_dims)), dtype=torch.uint8))
        if bias:
            self.register_buffer("bias", torch.zeros(out_dims))
        else:
            self.bias = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        # decode (one row) with a bias: the add is fused into the q8_0 decode kernel, as the reference does
        # (mlx_kquant/nn.py:129-146); KQ_DISABLE_QMV_BIAS=1 forces the unfused path, read live
        if (self.bias is not None and self.kquant_type == "q8_0" and x.numel() // x.shape[-1] == 1
                and os.environ.get("KQ_DISABLE_QMV_BIAS") != "1"):
            return kq.quantized_matmul_qmv_bias(x, self.weight, self.scales, self.bias, self.kquant_type)
        y = kq.quantized_matmul(x, self.weight, self.scales, self.kquant_type, transpose=True)
        if self.bias is not None:
            y = y + self.bias.to(y.dtype)
        return y

    def extra_repr(self) -> str:
        out_dims, bpr = self.weight.shape
        return f"output_dims={out_dims}, bytes_per_row={bpr}, kquant_type={self.kquant_type}"


class KQuantSwitchLinear(_KQuantBase):
    """Expert stack in wire bytes (mlx_kquant/nn.py:161-268): weight [n_experts, out_dims, bytes_per_row];
    `forward(x, indices, sorted_indices)` is `gather_qmm` over the stack. Prefill-shaped sorted calls
    (x [B, 1, K], indices [B] ascending, B >= KQ_SWITCH_GEMM_MIN_ROWS, default 512) take the segment product
    with a device-built tile map, which needs no host read of the routing."""

    def __init__(self, num_experts: int, output_dims: int, input_dims: int, bias: bool, codec: str):
        super().__init__()
        self._init_codec(codec)
        self.register_buffer("weight", torch.zeros((num_experts, output_dims, bytes_per_row(codec, input_dims)),
                                                   dtype=torch.uint8))
        if bias:
            self.register_buffer("bias", torch.zeros((num_experts, output_dims)))
        else:
            self.bias = None

    def forward(self, x: torch.Tensor, indices: torch.Tensor, sorted_indices: bool = False) -> torch.Tensor:
        if (sorted_indices and indices.dim() == 1 and x.dim() == 3 and x.shape[0] == indices.numel()
                and x.shape[1] == 1):
            min_rows = int(os.environ.get("KQ_SWITCH_GEMM_MIN_ROWS", "512"))
            if min_rows > 0 and indices.numel() >= min_rows:
                y = self._sorted_expert_gemm(x, indices)
                return self._add_bias(y, indices)
        y = kq.gather_qmm(x, self.weight, self.scales, self.kquant_type, rhs_indices=indices, transpose=True,
                          sorted_indices=sorted_indices)
        return self._add_bias(y, indices)

    def _add_bias(self, y: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
        if self.bias is None:
            return y
        return y + self.bias[indices.to(self.bias.device).long()].unsqueeze(-2).to(y.dtype)

    def _sorted_expert_gemm(self, x: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
        xf = x.reshape(indices.numel(), -1)
        idx = indices.to(self.weight.device)
        maps = kq.expert_tile_map(idx.to(torch.int32), self.weight.shape[0])
        return kq.gather_qmm_seg(xf, self.weight, self.scales, self.kquant_type, *maps)[:, None, :]

    def extra_repr(self) -> str:
        n, m, b = self.weight.shape
        return f"num_experts={n}, output_dims={m}, bytes_per_row={b}, kquant_type={self.kquant_type}"


class KQuantMultiLinear(_KQuantBase):
    """Per-head batched linear in wire bytes (mlx_kquant/nn.py:271-352), the absorbed-attention up-projections of
    the deepseek_v3 family: weight [num_heads, out_dims, bytes_per_row], dispatched through `gather_qmm` with the
    head as the expert index. `forward(x, transpose)`: x is [B, Hx, L, D] with Hx = num_heads (per-head
    activations) or 1 (one activation shared by all heads); `transpose=True` computes x[..., h, :, :] @ W[h].T,
    `transpose=False` computes x @ W[h] (contraction over the axis that is not quantized)."""

    def __init__(self, input_dims: int, output_dims: int, num_heads: int, codec: str):
        super().__init__()
        self._init_codec(codec)
        self.num_heads = num_heads
        self.register_buffer("weight", torch.zeros((num_heads, output_dims, bytes_per_row(codec, input_dims)),
                                                   dtype=torch.uint8))
        self._gather_idx = None

    def forward(self, x: torch.Tensor, transpose: bool = True) -> torch.Tensor:
        nh = self.num_heads
        B, Hx = x.shape[0], x.shape[1]
        dev = self.weight.device
        cached = self._gather_idx
        if cached is not None and cached[0] == (B, Hx, dev):
            lhs, rhs = cached[1], cached[2]
        else:
            rhs = torch.arange(nh, device=dev).reshape(1, nh).expand(B, nh).contiguous()
            if Hx == nh:
                lhs = torch.arange(B * nh, device=dev).reshape(B, nh)
            elif Hx == 1:
                lhs = torch.arange(B, device=dev).reshape(B, 1).expand(B, nh).contiguous()
            else:
                raise ValueError(f"KQuantMultiLinear: head axis {Hx} is neither 1 nor num_heads={nh} "
                                 f"(x.shape={tuple(x.shape)})")
            self._gather_idx = ((B, Hx, dev), lhs, rhs)
        return kq.gather_qmm(x, self.weight, self.scales, self.kquant_type, lhs_indices=lhs, rhs_indices=rhs,
                             transpose=transpose)

    def extra_repr(self) -> str:
        nh, out_dims, bpr = self.weight.shape
        return f"num_heads={nh}, output_dims={out_dims}, bytes_per_row={bpr}, kquant_type={self.kquant_type}"
