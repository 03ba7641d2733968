"""Synthetic wire bytes for timing runs.

Encoding a large matrix with the CPU encoder takes seconds to minutes (iq2_xxs:
about a quarter of a million weights per second per core), so throughput runs
use random but VALID wire bytes instead: uniform random quants and sub-scales
with every fp16 super-scale field overwritten by a small finite value. This is
the reference's own recipe for timing-only cells
(benchmarks/bench_qmm_bm128_ab.py:13-16, tests/test_cpu_decode.py:70-87).
Parity tests never use these bytes as a stand-in for encoded weights.
"""
from __future__ import annotations

import torch

from .ops import codec_geometry

# byte offsets of the fp16 fields inside one block
_F16_FIELDS = {"q2_k": (80, 82), "q3_k": (108,), "q4_k": (0, 2), "q5_k": (0, 2), "q6_k": (208,), "q4_0": (0,),
               "q8_0": (0,), "iq4_nl": (0,), "iq4_xs": (0,), "iq2_xxs": (0,), "q4_1": (0, 2), "q5_0": (0,),
               "q5_1": (0, 2), "iq3_xxs": (0,), "iq3_s": (0,), "iq2_xs": (0,), "iq2_s": (0,), "iq1_s": (0,),
               "iq1_m": (), "mxfp4": (), "nvfp4": ()}


def random_wire(kquant_type: str, rows: int, K: int, *, seed: int = 0, device="cuda", lead: tuple = ()) -> torch.Tensor:
    """uint8 tensor ``lead + (rows, K / wpb * bpb)`` of valid wire bytes."""
    wpb, bpb, _, _ = codec_geometry(kquant_type)
    if K % wpb:
        raise ValueError(f"K={K} is not a multiple of weights_per_block={wpb}")
    nb = K // wpb
    g = torch.Generator(device=device).manual_seed(seed)
    shape = tuple(lead) + (rows, nb, bpb)
    w = torch.randint(0, 256, shape, dtype=torch.uint8, device=device, generator=g)
    d = torch.empty(tuple(lead) + (rows, nb), dtype=torch.float32, device=device).uniform_(0.001, 0.02, generator=g)
    dbits = d.to(torch.float16).view(torch.int16).to(torch.int32) & 0xFFFF
    for off in _F16_FIELDS[kquant_type]:
        w[..., off] = (dbits & 0xFF).to(torch.uint8)
        w[..., off + 1] = (dbits >> 8).to(torch.uint8)
    if kquant_type == "iq1_m":      # fp16 super-scale = the top nibbles of the four scale words
        for k in range(4):
            hi = w[..., 48 + 2 * k + 1]
            w[..., 48 + 2 * k + 1] = (hi & 0x0F) | (((dbits >> (4 * k)) & 0xF) << 4).to(torch.uint8)
    elif kquant_type == "mxfp4":    # E8M0 exponent byte
        w[..., 0] = torch.randint(116, 123, w.shape[:-1], dtype=torch.uint8, device=device, generator=g)
    elif kquant_type == "nvfp4":    # four unsigned E4M3 scale bytes
        w[..., 0:4] = torch.randint(0x08, 0x30, w.shape[:-1] + (4,), dtype=torch.uint8, device=device, generator=g)
    return w.reshape(tuple(lead) + (rows, nb * bpb))
