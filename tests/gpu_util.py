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


synthetic_wire = kq_oracle.synthetic_wire


def mint_wire(codec: str, W: np.ndarray, imatrix=None) -> np.ndarray:
    """Really-encoded wire bytes from the reference encoder when its library is
    present (and the codec has an encoder: mxfp4 / nvfp4 are decode-only in the
    reference, src/kquant_codec.cpp:33-34), else synthetic valid bytes of the same shape."""
    if kq_oracle.Ref.available() and codec not in kq_oracle.DECODE_ONLY:
        if imatrix is None and GEOMETRY[codec][3]:
            imatrix = np.ones(W.shape[-1], np.float32)
        return kq_oracle.Ref().quantize(W, codec, imatrix)
    return synthetic_wire(codec, W.shape[0], W.shape[1], seed=int(abs(W[0, 0]) * 1e6) % 9973)
