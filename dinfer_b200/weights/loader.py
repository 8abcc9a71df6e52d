"""From tensor names to tensors on the device.

The model's parts declare what they take (name, shape, kind); the loader holds that list against
what the source has and raises ONE error that lists every missing tensor, every tensor of the
wrong shape and every tensor the model does not use.  Then each tensor is placed:

  * integer tables -> int32;
  * float32 engine -> float32 (the whole model runs in true 32-bit);
  * bfloat16 engine -> bfloat16, except that a tensor the file stores in 32-bit stays 32-bit
    (F64 narrows to F32, F16 goes to bfloat16).

The reference reads by name the same way and converts everything to bf16
(crates/layers/src/weights.rs:142-226); its errors come one at a time (weights.rs:143,
models/qwen3/src/model.rs:147-153,494).
"""
from __future__ import annotations

from typing import Dict, List, Sequence, Tuple

import torch

from ..parts.spec import TensorDecl
from .safetensors_io import SafetensorsFiles


class WeightError(ValueError):
    """Missing, unexpected or wrongly shaped tensors; ``missing``, ``unexpected`` and ``wrong_shape``
    hold the lists that the message prints."""

    def __init__(self, where: str, missing, unexpected, wrong_shape, wrong_dtype=()):
        self.missing, self.unexpected = list(missing), list(unexpected)
        self.wrong_shape, self.wrong_dtype = list(wrong_shape), list(wrong_dtype)
        lines = [f"{where}: the weights do not fit the model"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + "; ".join(
                f"{n} is {list(got)}, expected {list(want)}" for n, got, want in self.wrong_shape))
        if self.wrong_dtype:
            lines.append(f"  wrong dtype ({len(self.wrong_dtype)}): " + "; ".join(
                f"{n} is {got}, expected {want}" for n, got, want in self.wrong_dtype))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        super().__init__("\n".join(lines))


class WeightSource:
    """Where tensors come from: names, shapes, and one tensor at a time."""
    where = "weights"

    def names(self) -> List[str]:
        raise NotImplementedError

    def shape(self, name: str) -> Tuple[int, ...]:
        raise NotImplementedError

    def dtype(self, name: str) -> torch.dtype:
        raise NotImplementedError

    def get(self, name: str) -> torch.Tensor:
        raise NotImplementedError

    def close(self) -> None:
        pass


class SafetensorsSource(WeightSource):
    def __init__(self, model_dir: str):
        self.where = model_dir
        self.files = SafetensorsFiles(model_dir)

    def names(self):
        return self.files.names()

    def shape(self, name):
        return self.files.entries[name].shape

    def dtype(self, name):
        return self.files.torch_dtype(name)

    def get(self, name):
        return self.files.tensor(name)

    def close(self):
        self.files.close()


class DictSource(WeightSource):
    def __init__(self, tensors: Dict[str, torch.Tensor], where: str = "tensors"):
        self.tensors, self.where = tensors, where

    def names(self):
        return list(self.tensors)

    def shape(self, name):
        return tuple(self.tensors[name].shape)

    def dtype(self, name):
        return self.tensors[name].dtype

    def get(self, name):
        return self.tensors[name]


_FLOATS = (torch.float32, torch.float64, torch.float16, torch.bfloat16)
_INTS = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)


def verify(source: WeightSource, decls: Sequence[TensorDecl], allow_unexpected: bool = False) -> List[str]:
    """Hold what the source has against what the model declares; ONE error for everything that does not fit.
    Returns the tensors the model does not use: an error like the rest by default; with ``allow_unexpected`` (a
    checkpoint that carries buffers of its training code, say) they are only reported."""
    have = set(source.names())
    wanted = {}
    for d in decls:
        wanted.setdefault(d.name, d)
    missing, wrong_shape, wrong_dtype = [], [], []
    for name, d in wanted.items():
        if name not in have:
            if not d.optional:
                missing.append(name)
            continue
        got = tuple(source.shape(name))
        if got != tuple(d.shape):
            wrong_shape.append((name, got, tuple(d.shape)))
        dt = source.dtype(name)
        if d.kind == "float" and dt not in _FLOATS:
            wrong_dtype.append((name, str(dt).replace("torch.", ""), "a floating type"))
        if d.kind == "int" and dt not in _INTS:
            wrong_dtype.append((name, str(dt).replace("torch.", ""), "an integer type"))
    unexpected = sorted(have - set(wanted))
    if missing or wrong_shape or wrong_dtype or (unexpected and not allow_unexpected):
        raise WeightError(source.where, missing, unexpected, wrong_shape, wrong_dtype)
    return unexpected


def placed_dtype(stored: torch.dtype, kind: str, act_dtype: torch.dtype) -> torch.dtype:
    if kind == "int":
        return torch.int32
    if act_dtype == torch.float32:
        return torch.float32
    if stored in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


def load_tensors(source: WeightSource, decls: Sequence[TensorDecl], act_dtype: torch.dtype,
                 device, allow_unexpected: bool = False, unused: List[str] | None = None) -> Dict[str, torch.Tensor]:
    """Verify, then bring every declared tensor the source has to ``device`` in its placed dtype.  ``unused``:
    a list that receives the names of tensors the model does not use (only reachable with ``allow_unexpected``)."""
    extra = verify(source, decls, allow_unexpected)
    if unused is not None:
        unused.extend(extra)
    have = set(source.names())
    out: Dict[str, torch.Tensor] = {}
    for d in decls:
        if d.name in out or d.name not in have:
            continue
        t = source.get(d.name)
        dt = placed_dtype(t.dtype, d.kind, act_dtype)
        out[d.name] = t.to(device=device).to(dtype=dt).contiguous()
    return out
