"""Run one op a few times on synthetic inputs - the small driver that profiler
captures are taken from.

    python -m mlx_kquant_b200.profile_case matmul  q4_k 4096 4096 1 40
    python -m mlx_kquant_b200.profile_case dequant q6_k 14336 4096 f16 2
    python -m mlx_kquant_b200.profile_case gather  q4_k 768 2048 64 8

matmul  <codec> N K M launches [f16|bf16]: quantized_matmul of x [M, K] against
        `launches` distinct weight matrices [N, K] (distinct so that no launch
        finds its weights in L2).
dequant <codec> rows K dtype launches
gather  <codec> N K tokens top_k: one gather_qmm over 128 experts.
"""
from __future__ import annotations

import sys

import torch

from . import dequantize, gather_qmm, quantized_matmul
from .synth import random_wire

_DT = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}


def main(argv: list[str]) -> int:
    what, codec = argv[0], argv[1]
    if what == "matmul":
        N, K, M, launches = (int(v) for v in argv[2:6])
        dt = _DT[argv[6]] if len(argv) > 6 else torch.float16
        W = random_wire(codec, N, K, seed=1, lead=(launches,))
        x = torch.randn(M, K, device="cuda").to(dt)
        for i in range(launches):
            y = quantized_matmul(x, W[i], None, codec)
    elif what == "dequant":
        rows, K = int(argv[2]), int(argv[3])
        dt, launches = _DT[argv[4]], int(argv[5])
        W = random_wire(codec, rows, K, seed=2, lead=(launches,))
        for i in range(launches):
            y = dequantize(W[i], None, codec, dt)
    elif what == "gather":
        N, K, T, top_k = (int(v) for v in argv[2:6])
        W = random_wire(codec, N, K, seed=3, lead=(128,))
        x = torch.randn(T, 1, K, device="cuda").to(torch.bfloat16)
        idx = torch.randint(0, 128, (T, top_k), device="cuda")
        y = gather_qmm(x, W, None, codec, lhs_indices=torch.arange(T, device="cuda")[:, None].expand(T, top_k),
                       rhs_indices=idx)
    else:
        print(__doc__)
        return 2
    torch.cuda.synchronize()
    print("ok", tuple(y.shape), float(y.float().abs().mean()))
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
