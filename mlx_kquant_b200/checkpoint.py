"""The kquant checkpoint format and the module-swap seam, for torch models.

On-disk format is the reference's (mlx_kquant/convert.py:1-30, mlx_kquant/loader.py:1-20): `config.json`
carries `{"quantization": {"mode": "kquant", "per_tensor": {bare_module_path: codec}}}` and the safetensors
hold `<path>.weight` (uint8 wire bytes), `<path>.scales` (uint8 [1] placeholder) and an optional
`<path>.bias`; tensors that are not quantized keep their float dtype.

* `install_kquant_modules(model, per_tensor)` — mlx_kquant/_install.py:27-83: replace every
  `torch.nn.Linear` / `torch.nn.Embedding` (and any module exposing a 3-D `weight`, the expert-stack
  shape) whose `<path>.weight` has a codec by the matching `KQuant*` module.
* `quantize_model(model, codec_for)` — mlx_kquant/convert.py:78-205: encode the chosen weights with
  `kq.quantize` (host code, as in the reference), swap the modules, return the `per_tensor` map.
* `save(model, per_tensor, path)` / `load(model, path)` — write and read the directory.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Callable

import torch

from . import ops as kq
from .nn import KQuantEmbedding, KQuantLinear, KQuantSwitchLinear

_WEIGHTS = "model.safetensors"


def _set_module(model: torch.nn.Module, path: str, new: torch.nn.Module) -> None:
    parent = model
    parts = path.split(".")
    for p in parts[:-1]:
        parent = getattr(parent, p)
    setattr(parent, parts[-1], new)


def _kquant_twin(module: torch.nn.Module, codec: str):
    """The KQuant* module that takes the place of `module`, or None when its kind is not quantizable."""
    w = getattr(module, "weight", None)
    if isinstance(module, torch.nn.Linear):
        out_dims, in_dims = w.shape
        return KQuantLinear(in_dims, out_dims, module.bias is not None, codec)
    if isinstance(module, torch.nn.Embedding):
        num_emb, dims = w.shape
        return KQuantEmbedding(num_emb, dims, codec, out_dtype=w.dtype if w.dtype != torch.float32 else torch.bfloat16)
    if isinstance(w, torch.Tensor) and w.dim() == 3 and not isinstance(module, KQuantSwitchLinear):
        n_experts, out_dims, in_dims = w.shape
        return KQuantSwitchLinear(n_experts, out_dims, in_dims, getattr(module, "bias", None) is not None, codec)
    return None


def install_kquant_modules(model: torch.nn.Module, per_tensor: dict[str, str]) -> int:
    """Swap leaf modules for their kquant equivalents. `per_tensor` maps `<path>.weight` -> codec name.
    Returns the number of modules replaced."""
    n = 0
    for path, module in list(model.named_modules()):
        codec = per_tensor.get(f"{path}.weight")
        if codec is None or isinstance(module, (KQuantLinear, KQuantEmbedding, KQuantSwitchLinear)):
            continue
        twin = _kquant_twin(module, codec)
        if twin is None:
            continue
        w = module.weight
        _set_module(model, path, twin.to(w.device))
        n += 1
    return n


def quantize_model(model: torch.nn.Module, codec_for: Callable[[str, torch.nn.Module], str | None],
                   imatrix: dict[str, torch.Tensor] | None = None) -> dict[str, str]:
    """Encode in place. `codec_for(path, module)` names the codec of a module's weight or returns None to keep
    it in float. Returns the bare-path `per_tensor` map of the checkpoint format."""
    per_tensor: dict[str, str] = {}
    for path, module in list(model.named_modules()):
        w = getattr(module, "weight", None)
        if not isinstance(w, torch.Tensor) or not w.is_floating_point():
            continue
        codec = codec_for(path, module)
        if codec is None:
            continue
        twin = _kquant_twin(module, codec)
        if twin is None:
            continue
        imat = None if imatrix is None else imatrix.get(path)
        flat = w.detach().reshape(-1, w.shape[-1]).float().cpu()
        wire, _ = kq.quantize(flat, codec, imat)
        twin.weight.copy_(wire.reshape(*w.shape[:-1], wire.shape[-1]))
        bias = getattr(module, "bias", None)
        if bias is not None:
            twin.bias.copy_(bias.detach().float().cpu())
        _set_module(model, path, twin.to(w.device))
        per_tensor[path] = codec
    return per_tensor


def save(model: torch.nn.Module, per_tensor: dict[str, str], path: str | Path, config: dict | None = None) -> None:
    """Write `config.json` and `model.safetensors` in the kquant checkpoint format."""
    from safetensors.torch import save_file

    out = Path(path)
    out.mkdir(parents=True, exist_ok=True)
    cfg = dict(config or {})
    block = {"mode": "kquant", "per_tensor": dict(per_tensor)}
    cfg["quantization"] = block
    cfg["quantization_config"] = block
    (out / "config.json").write_text(json.dumps(cfg, indent=2, sort_keys=True))
    state = {k: v.detach().cpu().contiguous() for k, v in model.state_dict().items()}
    save_file(state, str(out / _WEIGHTS))


def read_per_tensor(path: str | Path) -> dict[str, str]:
    cfg = json.loads((Path(path) / "config.json").read_text())
    block = cfg.get("quantization") or cfg.get("quantization_config") or {}
    if block.get("mode") != "kquant":
        raise ValueError(f"[mlx_kquant] {path}: config.json has no quantization block with mode 'kquant'.")
    return dict(block.get("per_tensor", {}))


def load(model: torch.nn.Module, path: str | Path, device: torch.device | str | None = None) -> torch.nn.Module:
    """Swap in the KQuant* modules the checkpoint's `per_tensor` map names, then load its tensors.
    `model` is the constructed float model (weights may be uninitialised)."""
    from safetensors.torch import load_file

    per_tensor = read_per_tensor(path)
    # the map's keys are bare module paths; the install seam keys on `<path>.weight` (mlx_kquant/loader.py:10-14)
    weight_keyed = {(k if k.endswith(".weight") else f"{k}.weight"): v for k, v in per_tensor.items()}
    install_kquant_modules(model, weight_keyed)
    files = sorted(Path(path).glob("model*.safetensors"))
    if not files:
        raise FileNotFoundError(f"[mlx_kquant] no model*.safetensors under {path}")
    state: dict[str, torch.Tensor] = {}
    for f in files:
        state.update(load_file(str(f)))
    model.load_state_dict(state, strict=True)
    return model.to(device) if device is not None else model
