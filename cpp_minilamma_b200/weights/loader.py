"""Binding a model folder's tensors to a model's `WeightSpec`s by name.

Checks come first and are reported together: one `WeightError` lists every missing
tensor, every unexpected one and every wrong shape or kind of dtype.  (The reference
fails at the first fault, e.g. "missing tensor: " + name, src/load.cc:483, and skips
unknown tensors silently, src/gguf_load.cc:339-342; here an unexpected tensor is an
error.)

Where each tensor ends up:
  * matrix, stored BF16:  bfloat16 in a bfloat16 run, widened to float32 in a float32 run;
  * matrix, stored F16:   rounded to bfloat16 in a bfloat16 run (the kernels have no float16 instance),
                          widened exactly in a float32 run;
  * matrix, stored F32:   stays float32 in either run (its product then runs in float32);
  * vector (norm weights, biases): float32 always - every stored value is kept exactly;
  * int_table: int32.
"""
from __future__ import annotations

from typing import Dict, List, Sequence

import torch

from ..parts.base import WeightSpec
from .safetensors_io import ModelFiles


class WeightError(ValueError):
    """The folder's tensors do not match what the model loads."""

    def __init__(self, missing, unexpected, wrong):
        self.missing, self.unexpected, self.wrong = list(missing), list(unexpected), list(wrong)
        lines = ["model tensors do not match the architecture:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong:
            lines.append(f"  wrong shape or dtype ({len(self.wrong)}): " + "; ".join(self.wrong))
        super().__init__("\n".join(lines))


_FLOATS = (torch.float32, torch.bfloat16, torch.float16)
_INTS = (torch.int32, torch.int64)


def check_tensors(found: Dict[str, tuple], specs: Sequence[WeightSpec]) -> None:
    """found: name -> (dtype, shape).  Raises one WeightError for all faults."""
    wanted = {s.name: s for s in specs}
    missing = [n for n in wanted if n not in found]
    unexpected = sorted(n for n in found if n not in wanted)
    wrong = []
    for name, spec in wanted.items():
        if name not in found:
            continue
        dtype, shape = found[name]
        if tuple(shape) != tuple(spec.shape):
            wrong.append(f"{name}: shape {tuple(shape)}, expected {tuple(spec.shape)}")
        elif spec.kind == "int_table" and dtype not in _INTS:
            wrong.append(f"{name}: dtype {dtype}, expected an integer table")
        elif spec.kind != "int_table" and dtype not in _FLOATS:
            wrong.append(f"{name}: dtype {dtype}, expected a floating-point tensor")
    if missing or unexpected or wrong:
        raise WeightError(missing, unexpected, wrong)


def placement_dtype(spec: WeightSpec, stored: torch.dtype, run_dtype: torch.dtype) -> torch.dtype:
    if spec.kind == "int_table":
        return torch.int32
    if spec.kind == "vector" or stored == torch.float32:
        return torch.float32
    return run_dtype


def load_tensors(folder, specs: Sequence[WeightSpec], run_dtype: torch.dtype, device) -> Dict[str, torch.Tensor]:
    files = ModelFiles(folder)
    try:
        check_tensors({n: (e.dtype, e.shape) for n, e in files.entries.items()}, specs)
        out: Dict[str, torch.Tensor] = {}
        for spec in specs:
            host = files.read(spec.name)
            out[spec.name] = host.to(device=device, dtype=placement_dtype(spec, host.dtype, run_dtype)).contiguous()
        return out
    finally:
        files.close()
