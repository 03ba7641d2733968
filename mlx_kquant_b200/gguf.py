"""Minimal GGUF (v2 / v3, little-endian) reader and writer for tensor wire bytes and KV metadata — the job
of the reference's C++ loader (src/kquant_gguf.h:1-81: tensors as raw wire bytes, every KV value decoded to
a plain Python form) without a third-party GGUF package.

`read_gguf(path)` returns `(metadata, tensors)`: `tensors[name]` is a `GGUFTensor` whose `data` is
* a uint8 tensor `[*outer_dims, bytes_per_row]` of wire bytes for a block codec (`codec` names it as
  the `kq.*` ops do, e.g. "q4_k"), ready to be a `KQuant*` module's `weight`;
* a float32 / float16 / bfloat16 tensor of the logical shape for unquantized tensors (`codec` None).
GGUF lists dimensions innermost first; shapes here are outermost first, as torch has them.
"""
from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass
from pathlib import Path

import numpy as np
import torch

_MAGIC = b"GGUF"
# ggml tensor type ids of the codecs the ops know, and of the float types
GGML_TYPES = {0: "f32", 1: "f16", 2: "q4_0", 3: "q4_1", 6: "q5_0", 7: "q5_1", 8: "q8_0", 10: "q2_k", 11: "q3_k", 12: "q4_k", 13: "q5_k", 14: "q6_k",
              16: "iq2_xxs", 17: "iq2_xs", 18: "iq3_xxs", 19: "iq1_s", 20: "iq4_nl", 21: "iq3_s", 22: "iq2_s", 23: "iq4_xs",
              29: "iq1_m", 30: "bf16", 39: "mxfp4", 40: "nvfp4"}
_TYPE_IDS = {v: k for k, v in GGML_TYPES.items()}
_FLOATS = {"f32": (torch.float32, 4), "f16": (torch.float16, 2), "bf16": (torch.bfloat16, 2)}
# (weights per block, bytes per block); must agree with the library's registry (checked in the tests)
BLOCKS = {"q4_0": (32, 18), "q4_1": (32, 20), "q5_0": (32, 22), "q5_1": (32, 24), "q8_0": (32, 34), "q2_k": (256, 84), "q3_k": (256, 110), "q4_k": (256, 144),
          "q5_k": (256, 176), "q6_k": (256, 210), "iq2_xxs": (256, 66), "iq4_nl": (32, 18), "iq4_xs": (256, 136),
          "iq3_xxs": (256, 98), "iq3_s": (256, 110), "iq2_xs": (256, 74), "iq2_s": (256, 82), "iq1_s": (256, 50),
          "iq1_m": (256, 56), "mxfp4": (32, 17), "nvfp4": (64, 36)}

_SCALARS = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
_T_STRING, _T_ARRAY = 8, 9


@dataclass
class GGUFTensor:
    name: str
    codec: str | None          # block codec name, or None for float tensors
    dtype: str                 # ggml type name ("q4_k", "f16", ...)
    shape: tuple[int, ...]     # logical shape, outermost first
    data: torch.Tensor


class _Cursor:
    def __init__(self, buf):
        self.buf, self.pos = buf, 0

    def unpack(self, fmt):
        v = struct.unpack_from(fmt, self.buf, self.pos)[0]
        self.pos += struct.calcsize(fmt)
        return v

    def string(self):
        n = self.unpack("<Q")
        s = bytes(self.buf[self.pos:self.pos + n]).decode("utf-8", errors="replace")
        self.pos += n
        return s

    def value(self, t):
        if t in _SCALARS:
            return self.unpack(_SCALARS[t])
        if t == _T_STRING:
            return self.string()
        if t == _T_ARRAY:
            et, n = self.unpack("<I"), self.unpack("<Q")
            return [self.value(et) for _ in range(n)]
        raise ValueError(f"[mlx_kquant.gguf] unknown metadata value type {t}")


def read_gguf(path: str | Path, device: torch.device | str | None = None):
    """Parse a GGUF file. Tensor bytes are copied out of a memory map (the file is not kept open)."""
    with open(path, "rb") as f:
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
    try:
        cur = _Cursor(mm)
        if bytes(mm[:4]) != _MAGIC:
            raise ValueError(f"[mlx_kquant.gguf] {path}: not a GGUF file")
        cur.pos = 4
        version = cur.unpack("<I")
        if version not in (2, 3):
            raise ValueError(f"[mlx_kquant.gguf] {path}: unsupported GGUF version {version}")
        n_tensors, n_kv = cur.unpack("<Q"), cur.unpack("<Q")
        meta = {}
        for _ in range(n_kv):
            key = cur.string()
            meta[key] = cur.value(cur.unpack("<I"))
        infos = []
        for _ in range(n_tensors):
            name = cur.string()
            nd = cur.unpack("<I")
            ne = [cur.unpack("<Q") for _ in range(nd)]      # innermost first
            tid, off = cur.unpack("<I"), cur.unpack("<Q")
            infos.append((name, ne, tid, off))
        align = int(meta.get("general.alignment", 32))
        base = (cur.pos + align - 1) // align * align
        tensors = {}
        for name, ne, tid, off in infos:
            tname = GGML_TYPES.get(tid)
            if tname is None:
                raise ValueError(f"[mlx_kquant.gguf] tensor '{name}': ggml type {tid} is not supported")
            shape = tuple(reversed(ne)) if ne else ()
            n_el = int(np.prod(ne)) if ne else 1
            if tname in _FLOATS:
                dt, sz = _FLOATS[tname]
                raw = np.frombuffer(mm, dtype=np.uint8, count=n_el * sz, offset=base + off).copy()
                data = torch.from_numpy(raw).view(dt).reshape(shape)
                codec = None
            else:
                wpb, bpb = BLOCKS[tname]
                if not ne or ne[0] % wpb != 0:
                    raise ValueError(f"[mlx_kquant.gguf] tensor '{name}': row of {ne[0] if ne else 0} weights is not a "
                                     f"whole number of {wpb}-weight {tname} blocks")
                bpr = ne[0] // wpb * bpb
                rows = n_el // ne[0]
                raw = np.frombuffer(mm, dtype=np.uint8, count=rows * bpr, offset=base + off).copy()
                data = torch.from_numpy(raw).reshape(*shape[:-1], bpr)
                codec = tname
            if device is not None:
                data = data.to(device)
            tensors[name] = GGUFTensor(name, codec, tname, shape, data)
        return meta, tensors
    finally:
        mm.close()


def _pack_value(v) -> bytes:
    if isinstance(v, bool):
        return struct.pack("<I?", 7, v)
    if isinstance(v, int):  # the narrowest of u32 / i32 / u64 / i64: readers expect u32 for the common keys
        if 0 <= v < 2**32:
            return struct.pack("<II", 4, v)
        if -2**31 <= v < 0:
            return struct.pack("<Ii", 5, v)
        return struct.pack("<Iq", 11, v) if v < 0 else struct.pack("<IQ", 10, v)
    if isinstance(v, float):
        return struct.pack("<Id", 12, v)
    if isinstance(v, str):
        b = v.encode()
        return struct.pack("<IQ", _T_STRING, len(b)) + b
    if isinstance(v, (list, tuple)):
        if not v:
            return struct.pack("<IIQ", _T_ARRAY, 4, 0)
        items = [_pack_value(x) for x in v]
        if len({it[:4] for it in items}) != 1:
            raise ValueError("[mlx_kquant.gguf] metadata arrays must hold one value type")
        return struct.pack("<I", _T_ARRAY) + items[0][:4] + struct.pack("<Q", len(v)) + b"".join(it[4:] for it in items)
    raise TypeError(f"[mlx_kquant.gguf] cannot store metadata value of type {type(v).__name__}")


def _pack_string(s: str) -> bytes:
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def write_gguf(path: str | Path, metadata: dict, tensors: dict[str, tuple[str, tuple[int, ...], torch.Tensor]],
               alignment: int = 32) -> None:
    """Write a GGUF v3 file. `tensors[name] = (ggml type name, logical shape outermost first, data)`, data being
    the wire bytes (uint8, any shape with the right byte count) or the float tensor itself."""
    meta = dict(metadata)
    meta.setdefault("general.alignment", alignment)
    alignment = int(meta["general.alignment"])  # what readers pad with: a value in `metadata` wins over the argument
    head = _MAGIC + struct.pack("<IQQ", 3, len(tensors), len(meta))
    for k, v in meta.items():
        head += _pack_string(k) + _pack_value(v)
    blobs, infos, off = [], b"", 0
    for name, (tname, shape, data) in tensors.items():
        raw = data.detach().cpu().contiguous().view(torch.uint8).reshape(-1).numpy().tobytes()
        ne = list(reversed(shape))
        infos += _pack_string(name) + struct.pack("<I", len(ne)) + b"".join(struct.pack("<Q", d) for d in ne)
        infos += struct.pack("<IQ", _TYPE_IDS[tname], off)
        pad = (-len(raw)) % alignment
        blobs.append(raw + b"\0" * pad)
        off += len(raw) + pad
    body = head + infos
    body += b"\0" * ((-len(body)) % alignment)
    with open(path, "wb") as f:
        f.write(body)
        for b in blobs:
            f.write(b)
