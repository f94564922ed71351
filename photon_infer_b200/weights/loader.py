"""Loads the tensors a model declares, by name, and reports everything that does not
fit in ONE error: missing tensors, unexpected tensors, wrong shapes.

Storage rule: matrices (operands of products, lookup tables) are held in the run
dtype, bfloat16 for serving; integer tables as int32; a ``vector`` tensor (norm
weights) stored in 32-bit stays 32-bit.  In the float32 run everything is widened to
float32, which is exact for bfloat16 and float16 files.
"""
from __future__ import annotations

import fnmatch
import sys
from typing import Dict, Sequence

import torch

from ..errors import ErrorCode, PhotonError
from ..parts.base import TensorSpec
from .safetensors_io import open_model_files

_FLOATS = (torch.float32, torch.bfloat16, torch.float16, torch.float64)


def target_dtype(spec: TensorSpec, stored: torch.dtype, run_dtype: torch.dtype) -> torch.dtype:
    if spec.role == "int":
        return torch.int32
    if run_dtype == torch.float32:
        return torch.float32
    if spec.role == "vector" and stored in (torch.float32, torch.float64):
        return torch.float32
    return run_dtype


def check_names_and_shapes(declared: Dict[str, TensorSpec], found: Dict[str, tuple], dtypes: Dict[str, torch.dtype],
                           where: str, ignorable: Sequence[str] = ()) -> None:
    """``ignorable``: name patterns (``fnmatch``) of tensors that some exports of the architecture carry
    and the model has no use for (buffers that are recomputed from the configuration); they are named
    in one line on stderr instead of counting as unexpected."""
    missing = sorted(n for n in declared if n not in found)
    unexpected = sorted(n for n in found if n not in declared)
    ignored = [n for n in unexpected if any(fnmatch.fnmatchcase(n, pat) for pat in ignorable)]
    if ignored:
        unexpected = [n for n in unexpected if n not in ignored]
        print(f"[photon] warning: {len(ignored)} tensors in {where} are not used and were skipped: "
              + ", ".join(ignored[:4]) + (", ..." if len(ignored) > 4 else ""), file=sys.stderr, flush=True)
    wrong = []
    for n, spec in declared.items():
        if n in found:
            if tuple(found[n]) != tuple(spec.shape):
                wrong.append(f"{n}: expected {list(spec.shape)}, file has {list(found[n])}")
            elif spec.role == "int" and dtypes[n] in _FLOATS:
                wrong.append(f"{n}: expected an integer table, file has {dtypes[n]}")
            elif spec.role != "int" and dtypes[n] not in _FLOATS:
                wrong.append(f"{n}: expected floating point, file has {dtypes[n]}")
    if missing or unexpected or wrong:
        lines = [f"the weights in {where} do not fit the model:"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shape or type ({len(wrong)}): " + "; ".join(wrong))
        raise PhotonError(ErrorCode.WEIGHTS_MISMATCH, "\n".join(lines))


def load_tensors(folder: str, declared: Dict[str, TensorSpec], run_dtype: torch.dtype,
                 device, ignorable: Sequence[str] = ()) -> Dict[str, torch.Tensor]:
    """``declared`` maps full tensor names to their specs; returns device tensors by name."""
    entries, files = open_model_files(folder)
    try:
        check_names_and_shapes(declared, {n: e.shape for n, e in entries.items()},
                               {n: e.dtype for n, e in entries.items()}, folder, ignorable)
        out: Dict[str, torch.Tensor] = {}
        for name, spec in declared.items():
            e = entries[name]
            t = e.file.read(name)
            out[name] = t.to(device=device, dtype=target_dtype(spec, e.dtype, run_dtype)).contiguous()
        return out
    finally:
        for f in files:
            f.close()
