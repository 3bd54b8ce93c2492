"""Random-weights mode: a model folder (config.json, model.safetensors) from a
configuration and a seed.

The draw follows the tensor's kind: matrices and biases N(0, 0.02), norm weights
1 + N(0, 0.02), integer tables uniform. Tensors are drawn in the order of their
sorted names from one seeded CPU generator, so a folder is the same wherever it is
written. (The reference's only random model is a test fixture: tests/tiny_model.py:21-50.)
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Mapping

import torch

from ..config.registry import resolve
from .loader import collect_tensor_specs

STD = 0.02


def draw(spec, generator: torch.Generator, device="cpu") -> torch.Tensor:
    if spec.kind == "index":
        return torch.randint(0, max(1, spec.shape[0]), spec.shape, generator=generator, device=device, dtype=torch.int32)
    t = torch.randn(spec.shape, generator=generator, device=device, dtype=torch.float32) * STD
    return t + 1.0 if spec.kind == "scale" else t


def random_tensors(raw_config: Mapping[str, Any], seed: int, dtype: torch.dtype, device="cpu") -> dict[str, torch.Tensor]:
    """name -> tensor for the architecture that `raw_config` names, drawn on `device`.
    Floating-point tensors are rounded to `dtype`, as a checkpoint of that dtype would hold them."""
    _, spec = resolve(raw_config)
    generator = torch.Generator(device=device).manual_seed(int(seed))
    out = {}
    for name, tensor_spec in sorted(collect_tensor_specs(spec).items()):
        t = draw(tensor_spec, generator, device)
        out[name] = t if tensor_spec.kind == "index" else t.to(dtype)
    return out


def write_random_model(folder: str | Path, raw_config: Mapping[str, Any], seed: int, dtype: torch.dtype = torch.bfloat16) -> Path:
    """Writes config.json and model.safetensors into `folder` and returns it."""
    from safetensors.torch import save_file

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    config, _ = resolve(raw_config)
    tensors = random_tensors(raw_config, seed, dtype, "cpu")
    written = config.to_dict()
    written["torch_dtype"] = str(dtype).replace("torch.", "")
    (folder / "config.json").write_text(json.dumps(written, indent=2) + "\n")
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(folder / "model.safetensors"))
    return folder
