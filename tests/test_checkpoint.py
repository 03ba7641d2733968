"""kquant checkpoint directory (config.json per_tensor map + safetensors wire bytes) and the module-swap
seam, as the reference's tests/test_loader.py / test_convert.py exercise mlx_kquant/loader.py and convert.py."""
from __future__ import annotations

import json

import pytest
import torch

import mlx_kquant_b200 as kq
from mlx_kquant_b200 import checkpoint
from mlx_kquant_b200.nn import KQuantEmbedding, KQuantLinear, KQuantSwitchLinear


class Experts(torch.nn.Module):
    def __init__(self, n, out_dims, in_dims):
        super().__init__()
        self.weight = torch.nn.Parameter(torch.randn(n, out_dims, in_dims) * 0.05)


class Tiny(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.embed = torch.nn.Embedding(64, 256)
        self.up = torch.nn.Linear(256, 512, bias=True)
        self.down = torch.nn.Linear(512, 256, bias=False)
        self.experts = Experts(4, 128, 256)
        self.norm = torch.nn.LayerNorm(256)
        self.head = torch.nn.Linear(256, 64, bias=False)   # kept in float

    def forward(self, tok):
        h = self.embed(tok).to(torch.bfloat16)
        h = h + self.down(torch.nn.functional.silu(self.up(h)))
        return self.head(self.norm(h.float()))


def _codec_for(path, module):
    return {"embed": "q8_0", "up": "q4_k", "down": "q6_k", "experts": "q4_k"}.get(path)


def test_quantize_save_load_roundtrip(tmp_path):
    torch.manual_seed(0)
    model = Tiny()
    ref_up = model.up.weight.detach().clone()
    per_tensor = checkpoint.quantize_model(model, _codec_for)
    assert per_tensor == {"embed": "q8_0", "up": "q4_k", "down": "q6_k", "experts": "q4_k"}
    assert isinstance(model.up, KQuantLinear) and isinstance(model.embed, KQuantEmbedding)
    assert isinstance(model.experts, KQuantSwitchLinear) and isinstance(model.head, torch.nn.Linear)
    # the wire bytes are the encoder's: same as quantizing the float weight directly
    wire, _ = kq.quantize(ref_up, "q4_k")
    assert torch.equal(model.up.weight, wire)
    checkpoint.save(model, per_tensor, tmp_path / "ckpt", config={"model_type": "tiny"})
    cfg = json.loads((tmp_path / "ckpt" / "config.json").read_text())
    assert cfg["quantization"] == {"mode": "kquant", "per_tensor": per_tensor} and cfg["model_type"] == "tiny"
    fresh = checkpoint.load(Tiny(), tmp_path / "ckpt")
    want, got = model.state_dict(), fresh.state_dict()
    assert set(want) == set(got) and {"up.weight", "up.scales", "up.bias", "experts.weight"} <= set(got)
    for k in want:
        assert torch.equal(want[k], got[k]), k
    assert got["up.weight"].dtype == torch.uint8 and tuple(got["up.weight"].shape) == (512, 144)
    assert tuple(got["experts.weight"].shape) == (4, 128, 144)


def test_load_rejects_plain_checkpoint(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps({"model_type": "tiny"}))
    with pytest.raises(ValueError):
        checkpoint.load(Tiny(), tmp_path)


@pytest.mark.gpu
def test_loaded_model_runs_and_matches_dequantized_float_model(tmp_path):
    torch.manual_seed(1)
    model = Tiny()
    per_tensor = checkpoint.quantize_model(model, _codec_for)
    checkpoint.save(model, per_tensor, tmp_path / "ckpt")
    q = checkpoint.load(Tiny(), tmp_path / "ckpt", device="cuda")
    # float twin holding the dequantized weights
    f = Tiny().cuda()
    f.load_state_dict({k: v for k, v in q.state_dict().items() if v.dtype != torch.uint8 and not k.endswith("scales")},
                      strict=False)
    with torch.no_grad():
        f.embed.weight.copy_(kq.dequantize(q.embed.weight, None, "q8_0", torch.float32))
        f.up.weight.copy_(kq.dequantize(q.up.weight, None, "q4_k", torch.float32))
        f.down.weight.copy_(kq.dequantize(q.down.weight, None, "q6_k", torch.float32))
    tok = torch.randint(0, 64, (2, 9), device="cuda")
    with torch.no_grad():
        got = q(tok).float()
        h = f.embed(tok).to(torch.bfloat16).float()
        h = h + (torch.nn.functional.silu((h @ f.up.weight.T + f.up.bias).to(torch.bfloat16).float())
                 @ f.down.weight.T).to(torch.bfloat16).float()
        want = f.head(f.norm(h.to(torch.bfloat16).float()))
    assert float((got - want).norm() / want.norm()) < 2e-2
