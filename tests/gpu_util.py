"""Helpers shared by the GPU parity tests (torch <-> numpy bit views, wire minting)."""
from __future__ import annotations

import numpy as np
import torch

from oracle import kq_oracle
from oracle.kq_oracle import GEOMETRY

TORCH_DT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def t2np_bits(t: torch.Tensor) -> np.ndarray:
    """Device tensor -> numpy array of raw bit patterns (uint32 / uint16)."""
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.float32:
        return t.view(torch.int32).numpy().view(np.uint32)
    return t.view(torch.int16).numpy().view(np.uint16)


def np_bits(a: np.ndarray) -> np.ndarray:
    return a.view(np.uint32) if a.dtype == np.float32 else a.view(np.uint16)


def x_to_torch(x_f32: np.ndarray, dt: str, device="cuda") -> tuple[torch.Tensor, np.ndarray]:
    """float32 numpy -> (torch tensor of dtype dt on device, the oracle-side storage array)."""
    t = torch.from_numpy(x_f32).to(TORCH_DT[dt])
    if dt == "f32":
        store = x_f32.copy()
    elif dt == "f16":
        store = t.numpy().copy()
    else:
        store = t.view(torch.int16).numpy().view(np.uint16).copy()
    return t.to(device), store


def y_to_f32(y: torch.Tensor) -> np.ndarray:
    return y.detach().float().cpu().numpy()


def synthetic_wire(codec: str, rows: int, K: int, seed: int) -> np.ndarray:
    """Random but valid wire bytes: uniform bytes with every fp16 scale field set
    to a small finite value - the reference's own recipe for codecs without an
    encoder at hand (tests/test_cpu_decode.py:70-87)."""
    wpb, bpb, _, _ = GEOMETRY[codec]
    rng = np.random.default_rng(seed)
    nb = K // wpb
    w = rng.integers(0, 256, (rows, nb, bpb), dtype=np.uint8)
    d = rng.uniform(0.001, 0.02, (rows, nb)).astype(np.float16).view(np.uint16)
    f16_at = {"q2_k": (80, 82), "q3_k": (108,), "q4_k": (0, 2), "q5_k": (0, 2), "q6_k": (208,), "q4_0": (0,),
              "q8_0": (0,), "iq4_nl": (0,), "iq4_xs": (0,), "iq2_xxs": (0,), "q4_1": (0, 2), "q5_0": (0,),
              "q5_1": (0, 2)}[codec]
    for off in f16_at:
        w[:, :, off] = (d & 0xFF).astype(np.uint8)
        w[:, :, off + 1] = (d >> 8).astype(np.uint8)
    return w.reshape(rows, nb * bpb)


def mint_wire(codec: str, W: np.ndarray, imatrix=None) -> np.ndarray:
    """Really-encoded wire bytes from the reference encoder when its library is
    present, else synthetic valid bytes of the same shape."""
    if kq_oracle.Ref.available():
        if imatrix is None and GEOMETRY[codec][3]:
            imatrix = np.ones(W.shape[-1], np.float32)
        return kq_oracle.Ref().quantize(W, codec, imatrix)
    return synthetic_wire(codec, W.shape[0], W.shape[1], seed=int(abs(W[0, 0]) * 1e6) % 9973)
