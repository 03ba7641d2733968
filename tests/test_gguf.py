"""GGUF reader / writer: wire bytes and metadata survive a file round trip, block geometry agrees with the
library's codec registry, and a tensor read from a file drives a KQuantLinear (GPU)."""
from __future__ import annotations

import pytest
import torch

import mlx_kquant_b200 as kq
from mlx_kquant_b200 import gguf
from mlx_kquant_b200.nn import KQuantLinear


def test_block_table_matches_registry():
    assert set(gguf.BLOCKS) == set(kq.codecs())
    for codec, (wpb, bpb) in gguf.BLOCKS.items():
        assert kq.codec_geometry(codec)[:2] == (wpb, bpb), codec
        assert codec in gguf.GGML_TYPES.values()


def _tensors():
    g = torch.Generator().manual_seed(0)
    w = torch.randn(64, 512, generator=g) * 0.05
    wire, _ = kq.quantize(w, "q4_k")
    stack = torch.randn(2 * 32, 256, generator=g) * 0.05
    swire, _ = kq.quantize(stack, "q6_k")
    return w, {
        "blk.0.ffn_up.weight": ("q4_k", (64, 512), wire),
        "blk.0.ffn_gate_exps.weight": ("q6_k", (2, 32, 256), swire.reshape(2, 32, -1)),
        "blk.0.attn_norm.weight": ("f32", (512,), torch.randn(512, generator=g)),
        "token_embd.weight": ("f16", (10, 32), torch.randn(10, 32, generator=g).half()),
        "output_norm.weight": ("bf16", (32,), torch.randn(32, generator=g).bfloat16()),
    }


def test_round_trip(tmp_path):
    _, tensors = _tensors()
    meta = {"general.architecture": "llama", "llama.block_count": 1, "llama.rope.freq_base": 10000.5,
            "general.offset": -3, "tokenizer.ggml.add_bos_token": True, "tokenizer.ggml.tokens": ["<s>", "a", "b"],
            "llama.rope.dimension_sections": [1, 2, 3]}
    path = tmp_path / "tiny.gguf"
    gguf.write_gguf(path, meta, tensors)
    got_meta, got = gguf.read_gguf(path)
    for k, v in meta.items():
        assert got_meta[k] == v, k
    assert got_meta["general.alignment"] == 32
    assert list(got) == list(tensors)                      # file order kept
    for name, (tname, shape, data) in tensors.items():
        t = got[name]
        assert t.dtype == tname and t.shape == tuple(shape)
        assert t.codec == (tname if tname in gguf.BLOCKS else None)
        assert torch.equal(t.data, data.reshape(t.data.shape)), name
    assert tuple(got["blk.0.ffn_gate_exps.weight"].data.shape) == (2, 32, 210)
    assert tuple(got["blk.0.ffn_up.weight"].data.shape) == (64, 288)


def test_alignment_in_metadata_wins_over_the_argument(tmp_path):
    """Readers pad tensor offsets with general.alignment from the file: the writer must use that value too."""
    _, tensors = _tensors()
    path = tmp_path / "aligned64.gguf"
    gguf.write_gguf(path, {"general.alignment": 64}, tensors, alignment=32)
    got_meta, got = gguf.read_gguf(path)
    assert got_meta["general.alignment"] == 64
    for name, (_, _, data) in tensors.items():
        assert torch.equal(got[name].data, data.reshape(got[name].data.shape)), name


def test_rejects_foreign_files(tmp_path):
    p = tmp_path / "x.bin"
    p.write_bytes(b"NOPE" + b"\0" * 64)
    with pytest.raises(ValueError):
        gguf.read_gguf(p)


@pytest.mark.gpu
def test_tensor_from_file_drives_a_linear(tmp_path):
    w, tensors = _tensors()
    path = tmp_path / "tiny.gguf"
    gguf.write_gguf(path, {"general.architecture": "llama"}, tensors)
    _, got = gguf.read_gguf(path, device="cuda")
    t = got["blk.0.ffn_up.weight"]
    lin = KQuantLinear(t.shape[1], t.shape[0], bias=False, codec=t.codec).cuda()
    lin.weight.copy_(t.data)
    x = torch.randn(3, 512, device="cuda").half()
    want = x.float() @ kq.dequantize(t.data, None, "q4_k", torch.float32).T
    assert float((lin(x).float() - want).norm() / want.norm()) < 2e-3
    # and the dequantized weights are the encoder's view of w
    assert float((kq.dequantize(t.data, None, "q4_k", torch.float32).cpu() - w).norm() / w.norm()) < 0.1


def test_interoperates_with_gguf_py(tmp_path):
    # files written by the gguf package are read here, and files written here are read by it
    ggpy = pytest.importorskip("gguf")
    import numpy as np
    w = torch.randn(8, 512, generator=torch.Generator().manual_seed(3)) * 0.05
    wire, _ = kq.quantize(w, "q4_k")
    theirs = tmp_path / "theirs.gguf"
    wr = ggpy.GGUFWriter(str(theirs), "llama")
    wr.add_uint32("llama.block_count", 2)
    wr.add_string("general.name", "tiny")
    wr.add_array("tokenizer.ggml.tokens", ["a", "b"])
    wr.add_tensor("blk.0.ffn_up.weight", wire.numpy(), raw_dtype=ggpy.GGMLQuantizationType.Q4_K)
    wr.add_tensor("norm.weight", np.ones(512, np.float32))
    wr.write_header_to_file()
    wr.write_kv_data_to_file()
    wr.write_tensors_to_file()
    wr.close()
    meta, tensors = gguf.read_gguf(theirs)
    assert meta["general.architecture"] == "llama" and meta["llama.block_count"] == 2
    assert meta["tokenizer.ggml.tokens"] == ["a", "b"]
    t = tensors["blk.0.ffn_up.weight"]
    assert t.codec == "q4_k" and t.shape == (8, 512) and torch.equal(t.data, wire)
    assert tensors["norm.weight"].codec is None and float(tensors["norm.weight"].data.sum()) == 512.0
    ours = tmp_path / "ours.gguf"
    gguf.write_gguf(ours, {"general.architecture": "llama", "llama.block_count": 2}, {"a.weight": ("q4_k", (8, 512), wire)})
    r = ggpy.GGUFReader(str(ours))
    assert r.tensors[0].name == "a.weight" and r.tensors[0].tensor_type.name == "Q4_K"
    assert np.array_equal(np.asarray(r.tensors[0].data).reshape(-1), wire.numpy().reshape(-1))
