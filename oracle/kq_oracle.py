"""TEST INFRASTRUCTURE - ctypes front-end for the two CPU checkers.

``Oracle``  wraps oracle/libkq_oracle.so, the plain-C restatement of the
            reference's decode / matmul / gather arithmetic (kq_oracle.c).
``Ref``     wraps oracle/_ref/libkqref.so, the reference's own CPU codec
            library compiled in place (ref_wrap.cpp); also the only encoder, so
            it mints the wire bytes every parity test runs on.

Only tests, the smoke check and the benchmark's CPU-baseline leg import this
module; the shipped package never does.

Arrays are numpy. bfloat16 has no numpy dtype, so bf16 tensors travel as
``uint16`` bit patterns; ``DT`` maps the three dtype names to the integer codes
of the C entry points (0 f32, 1 f16, 2 bf16).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
DT = {"f32": 0, "f16": 1, "bf16": 2}
NP_OF = {"f32": np.float32, "f16": np.float16, "bf16": np.uint16}

# (weights_per_block, bytes_per_block, bits, requires_imatrix): the ten in-scope
# rows of the reference registry, src/kquant_codec.cpp:12-37, then the other eleven in the order of this
# library's registry.
GEOMETRY = {
    "q2_k": (256, 84, 2, False), "q3_k": (256, 110, 3, False), "q4_k": (256, 144, 4, False),
    "q5_k": (256, 176, 5, False), "q6_k": (256, 210, 6, False), "q4_0": (32, 18, 4, False),
    "q8_0": (32, 34, 8, False), "iq4_nl": (32, 18, 4, False), "iq4_xs": (256, 136, 4, False),
    "iq2_xxs": (256, 66, 2, True), "q4_1": (32, 20, 4, False), "q5_0": (32, 22, 5, False),
    "q5_1": (32, 24, 5, False), "iq3_xxs": (256, 98, 3, False), "iq3_s": (256, 110, 3, False),
    "iq2_xs": (256, 74, 2, True), "iq2_s": (256, 82, 2, False), "iq1_s": (256, 50, 1, True),
    "iq1_m": (256, 56, 1, False), "mxfp4": (32, 17, 4, False), "nvfp4": (64, 36, 4, False),
}
# codecs the reference can decode but not encode (src/kquant_codec.cpp:33-34)
DECODE_ONLY = ("mxfp4", "nvfp4")
CODECS = list(GEOMETRY)


# byte offsets of the fp16 fields inside one block (iq1_m, mxfp4 and nvfp4 carry their scales differently)
F16_FIELDS = {"q2_k": (80, 82), "q3_k": (108,), "q4_k": (0, 2), "q5_k": (0, 2), "q6_k": (208,), "q4_0": (0,),
              "q8_0": (0,), "iq4_nl": (0,), "iq4_xs": (0,), "iq2_xxs": (0,), "q4_1": (0, 2), "q5_0": (0,),
              "q5_1": (0, 2), "iq3_xxs": (0,), "iq3_s": (0,), "iq2_xs": (0,), "iq2_s": (0,), "iq1_s": (0,),
              "iq1_m": (), "mxfp4": (), "nvfp4": ()}


def synthetic_wire(codec: str, rows: int, K: int, seed: int) -> np.ndarray:
    """Random but valid wire bytes: uniform bytes with every scale field set to a small finite value - the
    reference's own recipe for codecs without an encoder at hand (tests/test_cpu_decode.py:70-87). iq1_m keeps
    its fp16 super-scale in the top nibbles of its four scale words; mxfp4 has an E8M0 exponent byte and nvfp4
    four unsigned E4M3 bytes."""
    wpb, bpb, _, _ = GEOMETRY[codec]
    rng = np.random.default_rng(seed)
    nb = K // wpb
    w = rng.integers(0, 256, (rows, nb, bpb), dtype=np.uint8)
    d = rng.uniform(0.001, 0.02, (rows, nb)).astype(np.float16).view(np.uint16)
    for off in F16_FIELDS[codec]:
        w[:, :, off] = (d & 0xFF).astype(np.uint8)
        w[:, :, off + 1] = (d >> 8).astype(np.uint8)
    if codec == "iq1_m":
        for k in range(4):   # nibble k of d goes to the top nibble of little-endian scale word k (bytes 48 + 2k + 1)
            hi = w[:, :, 48 + 2 * k + 1]
            w[:, :, 48 + 2 * k + 1] = (hi & 0x0F) | ((((d >> (4 * k)) & 0xF) << 4).astype(np.uint8))
    elif codec == "mxfp4":
        w[:, :, 0] = rng.integers(116, 123, (rows, nb), dtype=np.uint8)      # 2^-12 .. 2^-6 after the halving
    elif codec == "nvfp4":
        w[:, :, 0:4] = rng.integers(0x08, 0x30, (rows, nb, 4), dtype=np.uint8)
    return w.reshape(rows, nb * bpb)


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """IEEE round-to-nearest-even float32 -> bfloat16 bit patterns (uint16)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    r = np.where(nan, (u >> 16) | 0x40, r)
    return r.astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def to_f32(a: np.ndarray, dtype: str) -> np.ndarray:
    return bf16_bits_to_f32(a) if dtype == "bf16" else np.asarray(a, dtype=np.float32)


def from_f32(a: np.ndarray, dtype: str) -> np.ndarray:
    if dtype == "bf16":
        return f32_to_bf16_bits(a)
    return np.asarray(a, dtype=np.float32).astype(NP_OF[dtype])


def build(ref_dir: str | None = None) -> None:
    """Compile both checkers with the Makefile beside this file."""
    cmd = ["make", "-s", "-C", str(HERE), "all"]
    ref_dir = ref_dir or os.environ.get("KQ_REFERENCE_DIR") or str(HERE.parent.parent / "reference")
    cmd.append(f"REF={ref_dir}")
    subprocess.run(cmd, check=True)


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


class Oracle:
    """The C restatement (always available once built)."""

    def __init__(self):
        path = HERE / "libkq_oracle.so"
        if not path.exists():
            build()
        self.lib = C.CDLL(str(path))
        self.lib.kqo_dequantize.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_char_p, C.c_int]
        self.lib.kqo_qmm.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                     C.c_int, C.c_char_p, C.c_int]
        self.lib.kqo_gather_qmm.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                            C.c_longlong, C.c_int, C.c_int, C.c_int, C.c_int,
                                            C.c_longlong, C.c_int, C.c_char_p, C.c_int]

    def threads(self) -> int:
        return int(self.lib.kqo_threads())

    def dequantize(self, wire: np.ndarray, codec: str, dtype: str = "f32") -> np.ndarray:
        wpb, bpb, _, _ = GEOMETRY[codec]
        wire = np.ascontiguousarray(wire, dtype=np.uint8)
        assert wire.shape[-1] % bpb == 0
        shape = wire.shape[:-1] + (wire.shape[-1] // bpb * wpb,)
        out = np.empty(shape, dtype=NP_OF[dtype])
        rc = self.lib.kqo_dequantize(_p(wire), _p(out), out.size, codec.encode(), DT[dtype])
        if rc:
            raise RuntimeError(f"kqo_dequantize rc={rc}")
        return out

    def qmm(self, x: np.ndarray, wire: np.ndarray, codec: str, dtype: str, transpose: bool = True) -> np.ndarray:
        """x [M, K] in `dtype` storage, wire [N, bytes] (or [K, bytes] if not transpose)."""
        wpb, bpb, _, _ = GEOMETRY[codec]
        x = np.ascontiguousarray(x)
        wire = np.ascontiguousarray(wire, dtype=np.uint8)
        M, K = x.shape
        wpr = wire.shape[-1] // bpb * wpb
        N = wire.shape[0] if transpose else wpr
        assert (wpr if transpose else wire.shape[0]) == K
        out = np.empty((M, N), dtype=NP_OF[dtype])
        rc = self.lib.kqo_qmm(_p(out), _p(x), _p(wire), M, N, K, int(transpose), codec.encode(), DT[dtype])
        if rc:
            raise RuntimeError(f"kqo_qmm rc={rc}")
        return out

    def gather_qmm(self, x, wire, lhs, rhs, codec, dtype, transpose=True):
        """x [B, M, K], wire [E, N, bytes], lhs/rhs flat uint32 [n]; out [n, M, N]."""
        wpb, bpb, _, _ = GEOMETRY[codec]
        x = np.ascontiguousarray(x)
        wire = np.ascontiguousarray(wire, dtype=np.uint8)
        lhs = np.ascontiguousarray(lhs, dtype=np.uint32).ravel()
        rhs = np.ascontiguousarray(rhs, dtype=np.uint32).ravel()
        _, M, K = x.shape
        E = wire.shape[0]
        wpr = wire.shape[-1] // bpb * wpb
        N = wire.shape[1] if transpose else wpr
        out = np.empty((lhs.size, M, N), dtype=NP_OF[dtype])
        rc = self.lib.kqo_gather_qmm(_p(out), _p(x), _p(wire), _p(lhs), _p(rhs), lhs.size, M, N, K, E,
                                     wire.shape[1] * wire.shape[2], int(transpose), codec.encode(), DT[dtype])
        if rc:
            raise RuntimeError(f"kqo_gather_qmm rc={rc}")
        return out


class Ref:
    """The reference's compiled CPU library; `Ref.available()` says if it was built."""

    PATH = HERE / "_ref" / "libkqref.so"

    @classmethod
    def available(cls) -> bool:
        return cls.PATH.exists()

    def __init__(self):
        if not self.available():
            raise RuntimeError("oracle/_ref/libkqref.so has not been built (make -C oracle ref)")
        self.lib = C.CDLL(str(self.PATH))
        self.lib.kqref_last_error.restype = C.c_char_p
        self.lib.kqref_quantize_f32.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_char_p, C.c_void_p, C.c_size_t]
        self.lib.kqref_dequantize.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_char_p, C.c_int]
        self.lib.kqref_qmm.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                       C.c_int, C.c_char_p, C.c_int]

    def _check(self, rc):
        if rc:
            raise RuntimeError(self.lib.kqref_last_error().decode())

    def threads(self) -> int:
        return int(self.lib.kqref_threads())

    def codecs(self):
        out = []
        name = C.create_string_buffer(32)
        v = [C.c_int() for _ in range(5)]
        for i in range(self.lib.kqref_codec_count()):
            self.lib.kqref_codec_info(i, name, 32, *[C.byref(t) for t in v])
            out.append((name.value.decode(), v[0].value, v[1].value, v[2].value, bool(v[3].value), bool(v[4].value)))
        return out

    def quantize(self, w: np.ndarray, codec: str, imatrix: np.ndarray | None = None, threads: int | None = None) -> np.ndarray:
        """float32 [..., K] -> uint8 [..., K/wpb*bpb] with the reference encoder.

        Rows are encoded by independent calls spread over `threads` Python threads
        (the encoder is single-threaded; a whole-matrix call and per-row calls give
        the same bytes because blocks are independent and the imatrix offset is
        (block*wpb) % K, src/kquant_cpu_encode.cpp:471).
        """
        wpb, bpb, _, req = GEOMETRY[codec]
        w = np.ascontiguousarray(w, dtype=np.float32)
        K = w.shape[-1]
        assert K % wpb == 0
        rows = w.size // K
        w2 = w.reshape(rows, K)
        out = np.empty((rows, K // wpb * bpb), dtype=np.uint8)
        im = None
        if imatrix is not None:
            im = np.ascontiguousarray(imatrix, dtype=np.float32)
            assert im.shape == (K,)
        elif req:
            raise ValueError(f"codec '{codec}' requires an importance matrix (imatrix)")
        nt = max(1, min(threads or os.cpu_count() or 1, rows))
        bounds = np.linspace(0, rows, nt + 1).astype(int)

        def job(i):
            a, b = bounds[i], bounds[i + 1]
            if a == b:
                return 0
            return self.lib.kqref_quantize_f32(_p(w2[a:b]), _p(out[a:b]), (b - a) * K, codec.encode(),
                                               _p(im) if im is not None else None, K)

        if nt == 1:
            self._check(job(0))
        else:
            with ThreadPoolExecutor(nt) as ex:
                for rc in ex.map(job, range(nt)):
                    self._check(rc)
        return out.reshape(w.shape[:-1] + (out.shape[-1],))

    def dequantize(self, wire: np.ndarray, codec: str, dtype: str = "f32") -> np.ndarray:
        wpb, bpb, _, _ = GEOMETRY[codec]
        wire = np.ascontiguousarray(wire, dtype=np.uint8)
        shape = wire.shape[:-1] + (wire.shape[-1] // bpb * wpb,)
        out = np.empty(shape, dtype=NP_OF[dtype])
        self._check(self.lib.kqref_dequantize(_p(wire), _p(out), out.size, codec.encode(), DT[dtype]))
        return out

    def qmm(self, x: np.ndarray, wire: np.ndarray, codec: str, dtype: str, transpose: bool = True) -> np.ndarray:
        wpb, bpb, _, _ = GEOMETRY[codec]
        x = np.ascontiguousarray(x)
        wire = np.ascontiguousarray(wire, dtype=np.uint8)
        M, K = x.shape
        wpr = wire.shape[-1] // bpb * wpb
        N = wire.shape[0] if transpose else wpr
        out = np.empty((M, N), dtype=NP_OF[dtype])
        self._check(self.lib.kqref_qmm(_p(out), _p(x), _p(wire), M, N, K, int(transpose), codec.encode(), DT[dtype]))
        return out
