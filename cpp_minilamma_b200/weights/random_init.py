"""Seeded random weights: a model folder from a configuration, or tensors on a device.

The reference's exporter (model/tinymodel/export_model.py:27,55-75) draws every matrix
as randn * 0.02 and sets norms to one.  Here each tensor has a generator of its own,
seeded by (seed, position in the model's tensor list), so a tensor's values do not
depend on which other tensors exist; matrices and biases are N(0, matrix_std), norm
weights 1 + N(0, norm_std) (norm_std > 0 in tests, so that a dropped norm weight shows).
Values are rounded once to the storage dtype; a float32 run of a bfloat16 folder widens
those same values.
"""
from __future__ import annotations

from pathlib import Path
from typing import Dict, Sequence

import torch

from ..config.base import ModelConfig, lookup_architecture, save_config
from ..parts.base import WeightSpec
from .safetensors_io import write_safetensors


def _fill(spec: WeightSpec, index: int, seed: int, matrix_std: float, norm_std: float, device) -> torch.Tensor:
    gen = torch.Generator(device=device)
    gen.manual_seed((int(seed) * 1000003 + index * 7919 + 12345) % (2 ** 63 - 1))
    shape = tuple(spec.shape)
    if spec.init == "zeros":
        return torch.zeros(shape, dtype=torch.float32, device=device)
    if spec.init == "ones":
        return torch.ones(shape, dtype=torch.float32, device=device)
    noise = torch.randn(shape, generator=gen, dtype=torch.float32, device=device)
    if spec.init == "norm":
        return 1.0 + norm_std * noise
    if spec.init == "normal":
        return matrix_std * noise
    raise ValueError(f"unknown init {spec.init!r} for tensor {spec.name}")


def random_tensors(specs: Sequence[WeightSpec], seed: int, storage_dtype: torch.dtype, device="cpu",
                   matrix_std: float = 0.02, norm_std: float = 0.1) -> Dict[str, torch.Tensor]:
    """Tensors in spec order.  Matrices take `storage_dtype`; vectors are float32 when
    the storage is float32 and `storage_dtype` otherwise (as a checkpoint stores them)."""
    out: Dict[str, torch.Tensor] = {}
    for index, spec in enumerate(specs):
        if spec.kind == "int_table":
            raise ValueError(f"no random fill for the integer table {spec.name}")
        out[spec.name] = _fill(spec, index, seed, matrix_std, norm_std, device).to(storage_dtype)
    return out


def write_random_model(config: ModelConfig, folder, seed: int, matrix_std: float = 0.02,
                       norm_std: float = 0.1) -> Path:
    """Write `config.json` and `model.safetensors` for `config` with seeded random weights.
    The storage dtype is the configuration's `torch_dtype`."""
    from ..engine.model import Model  # late: engine imports weights
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    _, builder = lookup_architecture(config.architecture)
    model = Model(builder(config), torch.float32, "cpu", max_positions=1)
    storage = {"bfloat16": torch.bfloat16, "float32": torch.float32,
               "float16": torch.float16}[getattr(config, "torch_dtype", "bfloat16")]
    tensors = random_tensors(model.weight_specs(), seed, storage, "cpu", matrix_std, norm_std)
    save_config(config, folder)
    write_safetensors(folder / "model.safetensors", tensors, {"format": "pt", "seed": str(seed)})
    return folder
