"""From a model folder to something that steps: configuration, weights, parts, cache.

`Engine` owns the model (parts built from the folder's config.json through the
architecture registry, tensors read from its safetensors) and hands out paged caches
and runners for it, in the manner of the reference's `Qwen2Engine.from_hf_model` /
`new_paged_cache` (engine/model.py:190-229,257-272), but from files, for any registered
architecture, and with no code path that runs without the CUDA kernels.
"""

from __future__ import annotations

from pathlib import Path
from typing import Any, Mapping

import torch

from ..cache import CacheManager, PagedKVCache, plan_cache
from ..config import ModelSpec, resolve, resolve_folder
from ..parts import Runtime
from ..weights import load_tensors, place_tensors, random_tensors
from .model import DecoderModel
from .runner import ModelRunner

DTYPES = {
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
    "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32,
}


def as_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"dtype {dtype} is not supported (bfloat16 or float32)")
        return dtype
    try:
        return DTYPES[str(dtype)]
    except KeyError:
        raise ValueError(f"dtype '{dtype}' is not supported (bfloat16 or float32)") from None


def _default_ops():
    from ..kernels import ops

    ops.require_cuda()
    return ops


class Engine:
    def __init__(self, config: Any, spec: ModelSpec, tensors: dict[str, torch.Tensor], runtime: Runtime) -> None:
        self.config = config
        self.spec = spec
        self.runtime = runtime
        self.dtype = runtime.dtype
        self.device = runtime.device
        self.cache_plan = plan_cache(spec)
        self.model = DecoderModel(spec, tensors, runtime)

    # -- construction ------------------------------------------------------ #

    @classmethod
    def from_pretrained(cls, folder: str | Path, dtype="bfloat16", device="cuda:0", ops=None) -> "Engine":
        """Reads config.json and the safetensors of `folder`; the architecture named in
        config.json chooses the model."""
        dtype = as_dtype(dtype)
        config, spec = resolve_folder(folder)
        runtime = Runtime(ops or _default_ops(), dtype, torch.device(device))
        tensors = load_tensors(folder, spec, dtype, runtime.device)
        return cls(config, spec, tensors, runtime)

    @classmethod
    def from_random(cls, raw_config: Mapping[str, Any], seed: int = 0, dtype="bfloat16", device="cuda:0", ops=None,
                    as_written: bool = False) -> "Engine":
        """Random weights without a folder. They are drawn on the device (quick at large shapes);
        with `as_written` on the CPU instead, which gives the very tensors that
        `write_random_model` writes for this configuration, seed and dtype."""
        dtype = as_dtype(dtype)
        config, spec = resolve(raw_config)
        runtime = Runtime(ops or _default_ops(), dtype, torch.device(device))
        tensors = random_tensors(raw_config, seed, dtype, "cpu" if as_written else runtime.device)
        tensors = place_tensors(tensors, spec, dtype, runtime.device, "random weights")
        return cls(config, spec, tensors, runtime)

    # -- caches and runners ------------------------------------------------ #

    def new_paged_cache(self, num_blocks: int, block_size: int = 16, max_num_seqs: int = 256) -> PagedKVCache:
        """A pool of `num_blocks` pages of `block_size` tokens for every page group of the model."""
        manager = CacheManager(self.cache_plan.groups, num_blocks, block_size, max_num_seqs)
        return PagedKVCache(self.cache_plan, manager, self.dtype, self.device)

    def bytes_per_block(self, block_size: int = 16) -> int:
        """Device bytes behind one page id (the reference: 2 x layers x kv heads x head size x
        element size per token, bench/baseline.py:78-90)."""
        return self.cache_plan.bytes_per_block(block_size, torch.empty((), dtype=self.dtype).element_size())

    def new_runner(self, cache: PagedKVCache, use_graphs: bool = True) -> ModelRunner:
        return ModelRunner(self.model, cache, use_graphs)

    @property
    def vocab_size(self) -> int:
        return self.spec.vocab_size

    def weight_bytes(self, num_tokens: int = 1) -> int:
        """Bytes of the weights that a step of `num_tokens` tokens reads: every distinct tensor
        that a part holds, once. A part that reads only some of what it holds (experts chosen by
        a router) says so itself with `step_weight_bytes(num_tokens)`."""
        seen: dict[int, int] = {}
        extra = 0

        def visit(obj: Any) -> None:
            nonlocal extra
            own = getattr(obj, "step_weight_bytes", None)
            if own is not None:
                extra += int(own(num_tokens))
                return
            for value in vars(obj).values():
                if isinstance(value, torch.Tensor):
                    seen[value.data_ptr()] = value.numel() * value.element_size()
                elif hasattr(value, "runtime") and value is not obj:
                    visit(value)

        for part in self.model.parts():
            visit(part)
        return sum(seen.values()) + extra
