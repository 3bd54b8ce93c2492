"""Weights from safetensors, by tensor name.

The reference borrows tensors from a model that another library loaded
(engine/model.py:190-229: twelve names per layer, the embedding, the final norm and
an optional head) and fails with a bare KeyError when one is absent. This loader
opens the files itself, asks every part of the `ModelSpec` which tensors it reads,
and raises ONE `WeightsError` that lists all missing tensors, all unexpected ones
and all wrong shapes before anything is copied.

Storage on the device:
  matrices     the engine's dtype (bfloat16 or float32); in a bfloat16 engine a matrix
               that the file stores in 32-bit stays in 32-bit and runs on the slower
               kernel that takes such a weight;
  biases and norm weights   float32 (widening bfloat16 is exact);
  integer tables            int32.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Iterable

import torch

from ..config.model_spec import ModelSpec, PartSpec
from ..parts.base import REGISTRIES, TensorSpec, layer_part_specs, with_sub_parts


class WeightsError(ValueError):
    """The checkpoint does not hold what the model reads; the message lists every fault."""


def _part_specs(registry: str, spec: PartSpec) -> list[TensorSpec]:
    """The tensors of a part and of the parts nested inside it."""
    out: list[TensorSpec] = []
    for sub_registry, sub in with_sub_parts(registry, spec):
        out += list(REGISTRIES[sub_registry].get(sub.kind).tensor_specs(sub))
    return out


def collect_tensor_specs(spec: ModelSpec) -> dict[str, TensorSpec]:
    """Every tensor the model reads, by full name, in the order the parts name them."""
    found: list[TensorSpec] = []
    found += _part_specs("embedding", spec.embedding)
    for layer in spec.layers:
        # an unknown arrangement, or a layer without the parts its arrangement declares, fails
        # here, before any file is opened
        for _role, registry, part in layer_part_specs(layer):
            found += _part_specs(registry, part)
    found += _part_specs("norm", spec.final_norm)
    found += _part_specs("head", spec.head)
    out: dict[str, TensorSpec] = {}
    for t in found:
        if t.name in out and out[t.name].shape != t.shape:
            raise WeightsError(f"two parts read tensor '{t.name}' with shapes {out[t.name].shape} and {t.shape}")
        out[t.name] = t
    return out


def _checkpoint_files(folder: Path) -> list[Path]:
    index = folder / "model.safetensors.index.json"
    if index.is_file():
        names = sorted(set(json.loads(index.read_text())["weight_map"].values()))
        return [folder / n for n in names]
    single = folder / "model.safetensors"
    if single.is_file():
        return [single]
    raise WeightsError(f"{folder}: neither model.safetensors nor model.safetensors.index.json is there")


def check_against_specs(
    expected: dict[str, TensorSpec], present: dict[str, tuple[int, ...]], where: str
) -> None:
    """Raises one error that lists missing and unexpected tensors and wrong shapes."""
    missing = [n for n in expected if n not in present]
    unexpected = [n for n in present if n not in expected]
    wrong = [
        f"{n}: file has {tuple(present[n])}, the model reads {tuple(expected[n].shape)}"
        for n in expected
        if n in present and tuple(present[n]) != tuple(expected[n].shape)
    ]
    if not (missing or unexpected or wrong):
        return
    lines = [f"{where}: the tensors do not fit the model"]
    if missing:
        lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
    if unexpected:
        lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
    if wrong:
        lines.append(f"  wrong shape ({len(wrong)}): " + "; ".join(wrong))
    raise WeightsError("\n".join(lines))


def place(tensor: torch.Tensor, spec: TensorSpec, dtype: torch.dtype, device) -> torch.Tensor:
    """Storage class of one tensor on the device (see the module's header)."""
    if spec.kind == "index":
        if tensor.dtype.is_floating_point:
            raise WeightsError(f"{spec.name}: an integer table is stored as {tensor.dtype}")
        return tensor.to(device=device, dtype=torch.int32).contiguous()
    if not tensor.dtype.is_floating_point:
        raise WeightsError(f"{spec.name}: stored as {tensor.dtype}, a floating-point tensor is read")
    if spec.kind in ("vector", "scale"):
        return tensor.to(device=device, dtype=torch.float32).contiguous()
    if dtype == torch.bfloat16 and tensor.dtype in (torch.float32, torch.float64):
        return tensor.to(device=device, dtype=torch.float32).contiguous()
    return tensor.to(device=device, dtype=dtype).contiguous()


def load_tensors(folder: str | Path, spec: ModelSpec, dtype: torch.dtype, device) -> dict[str, torch.Tensor]:
    """name -> tensor on `device` for every tensor the model reads; raises WeightsError."""
    from safetensors import safe_open

    folder = Path(folder)
    expected = collect_tensor_specs(spec)
    files = _checkpoint_files(folder)
    present: dict[str, tuple[int, ...]] = {}
    owner: dict[str, Path] = {}
    for path in files:
        if not path.is_file():
            raise WeightsError(f"{path}: the index names this file, it is not there")
        with safe_open(str(path), framework="pt", device="cpu") as f:
            for name in f.keys():
                present[name] = tuple(f.get_slice(name).get_shape())
                owner[name] = path
    check_against_specs(expected, present, str(folder))
    out: dict[str, torch.Tensor] = {}
    for path in files:
        with safe_open(str(path), framework="pt", device="cpu") as f:
            for name in f.keys():
                if owner[name] == path:
                    out[name] = place(f.get_tensor(name), expected[name], dtype, device)
    return out


def place_tensors(
    tensors: dict[str, torch.Tensor], spec: ModelSpec, dtype: torch.dtype, device, where: str = "tensors"
) -> dict[str, torch.Tensor]:
    """The same validation and placement for tensors that are already in memory."""
    expected = collect_tensor_specs(spec)
    check_against_specs(expected, {n: tuple(t.shape) for n, t in tensors.items()}, where)
    return {n: place(t, expected[n], dtype, device) for n, t in tensors.items()}


def names_in(files: Iterable[Path]) -> list[str]:
    from safetensors import safe_open

    out = []
    for path in files:
        with safe_open(str(path), framework="pt", device="cpu") as f:
            out += list(f.keys())
    return out
