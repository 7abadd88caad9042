"""Model registry for checkpoints on disk: config.json's "architecture" names the class; `load_model` builds it from a
folder holding config.json and model.safetensors. Classes register a `from_pretrained(path, dtype=..., device=...)`."""
from __future__ import annotations

import json
import os
from typing import Callable, Dict

import torch

_REGISTRY: Dict[str, Callable] = {}


def register_model(architecture: str, loader: Callable) -> None:
    _REGISTRY[architecture] = loader


def architectures():
    return sorted(_REGISTRY)


def load_model(path: str, dtype: torch.dtype = torch.bfloat16, device=None, **kw):
    with open(os.path.join(path, "config.json")) as f:
        arch = json.load(f).get("architecture")
    if arch not in _REGISTRY:
        raise KeyError(f"config.json names architecture {arch!r}; registered: {architectures()}")
    return _REGISTRY[arch](path, dtype=dtype, device=device, **kw)


def _gelutar(path, **kw):
    from .models.gelutar import GelutarForCausalLM
    return GelutarForCausalLM.from_pretrained(path, **kw)


def _zugunex(path, **kw):
    from .models.zugunex import ZugunexForCausalLM
    return ZugunexForCausalLM.from_pretrained(path, **kw)


def _vazepel(path, **kw):
    from .models.vazepel import VazepelForCausalLM
    return VazepelForCausalLM.from_pretrained(path, **kw)


def _fubinex(path, **kw):
    from .models.fubinex import FubinexForCausalLM
    return FubinexForCausalLM.from_pretrained(path, **kw)


def _custom_lm(path, dtype=torch.bfloat16, device=None, **kw):
    """The RMSNorm / SwiGLU / RoPE decoder (models/custom_transformer.py): config.json holds its Config fields, the checkpoint
    its state_dict."""
    from .checkpoint import load_safetensors
    from .models.custom_transformer import Config, ModelForCausalLM
    with open(os.path.join(path, "config.json")) as f:
        d = json.load(f)
    d.pop("architecture", None)
    m = ModelForCausalLM(Config(**d))
    m.load_state_dict(load_safetensors(os.path.join(path, "model.safetensors")), strict=False)
    return m.to(device=device or "cuda", dtype=dtype).eval()


register_model("Gelutar", _gelutar)
register_model("Zugunex", _zugunex)
register_model("Vazepel", _vazepel)
register_model("Fubinex", _fubinex)
register_model("ModelForCausalLM", _custom_lm)
