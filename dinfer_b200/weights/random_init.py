"""Random weights: a model folder (``config.json`` + ``model.safetensors``) from a configuration and
a seed, or the same tensors made directly on the device (for benchmarks at sizes one does not
want on disk).

Matrices and the embedding are ``N(0, std)``, norm weights ``1 + U(-jitter, jitter)``.  Each tensor
has its own generator seeded from ``(seed, name)``, so a tensor's values do not depend on which
other tensors exist or in which order they are made.  The reference has no such mode for Qwen3;
its other models use one-off fixture scripts (scripts/verify/gen_tiny_glm.py).
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Any, Dict, List

import torch

from ..config.registry import resolve_architecture
from ..parts.base import BuildEnv
from ..parts.spec import TensorDecl
from .loader import WeightSource
from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensor(decl: TensorDecl, seed: int, std: float, jitter: float, dtype: torch.dtype,
                  device="cpu") -> torch.Tensor:
    gen = torch.Generator(device=device)
    gen.manual_seed(_tensor_seed(seed, decl.name))
    if decl.kind == "int":
        raise ValueError(f"{decl.name}: integer tables have no random rule")
    if decl.init == "ones":
        t = torch.rand(decl.shape, generator=gen, device=device, dtype=torch.float32)
        t = 1.0 + (2.0 * t - 1.0) * jitter
    else:
        t = torch.randn(decl.shape, generator=gen, device=device, dtype=torch.float32) * std
    return t.to(dtype)


def model_declarations(config_dict: Dict[str, Any]) -> List[TensorDecl]:
    """The tensors the architecture of ``config_dict`` takes from its file (no optional ones that
    the configuration makes redundant: a tied head is left out)."""
    from ..models.decoder import DecoderModel
    arch = resolve_architecture(config_dict)
    cfg = arch.parse_config(config_dict)
    spec = arch.build_spec(cfg)
    env = BuildEnv(torch.device("cpu"), torch.float32, spec.hidden_size, spec.max_positions)
    model = DecoderModel(spec, env)
    seen, out = set(), []
    for d in model.declarations():
        if d.optional or d.name in seen:
            continue
        seen.add(d.name)
        out.append(d)
    return out


def write_random_model(model_dir: str, config_dict: Dict[str, Any], seed: int, std: float = 0.02,
                       norm_jitter: float = 0.0, dtype: torch.dtype = torch.bfloat16, device="cpu") -> str:
    """Write ``config.json`` and ``model.safetensors`` into ``model_dir``.  ``device``: where the values are drawn
    (a large model is made much faster on a CUDA device; the values depend on the kind of device)."""
    decls = model_declarations(config_dict)
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config_dict, f, indent=1)
    write_safetensors(os.path.join(model_dir, "model.safetensors"),
                      ((d.name, random_tensor(d, seed, std, norm_jitter, dtype, device).cpu()) for d in decls),
                      metadata={"format": "pt", "seed": str(seed)})
    return model_dir


class RandomSource(WeightSource):
    """The tensors ``write_random_model`` would write, generated on ``device`` when asked for."""

    def __init__(self, config_dict: Dict[str, Any], seed: int, std: float = 0.02, norm_jitter: float = 0.0,
                 dtype: torch.dtype = torch.bfloat16, device="cuda"):
        self.where = f"random weights (seed {seed})"
        self.decls = {d.name: d for d in model_declarations(config_dict)}
        self.seed, self.std, self.jitter, self.dt, self.device = seed, std, norm_jitter, dtype, device

    def names(self):
        return list(self.decls)

    def shape(self, name):
        return tuple(self.decls[name].shape)

    def dtype(self, name):
        return self.dt

    def get(self, name):
        return random_tensor(self.decls[name], self.seed, self.std, self.jitter, self.dt, self.device)
