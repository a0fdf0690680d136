"""Bind the tensors of a model folder to the names a model declares.

One pass compares what the model declares with what the files hold and raises a single
``WeightsError`` listing every missing tensor, every unexpected tensor and every wrong
shape.  (The reference stops at the first missing name, crates/safetensors/src/lib.rs:541-544,
and checks shapes separately, crates/model/src/weights.rs:1348-1460.)

Precision policy.  ``bfloat16``: a tensor stored as BF16 stays bf16, F16 is widened through
float32 and rounded to bf16 (the reference narrows BF16 to F16 instead,
crates/safetensors/src/lib.rs:197-254), a tensor stored in 32-bit stays 32-bit, integer
tables become int32.  ``float32``: every floating tensor becomes float32.
"""
from __future__ import annotations

from typing import Dict, Iterable, List

import torch

from ..parts.base import TensorDecl
from .safetensors_io import SafetensorsDir, SafetensorsError


class WeightsError(ValueError):
    def __init__(self, message: str, missing=(), unexpected=(), wrong_shape=()):
        super().__init__(message)
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)


def check_names(decls: Iterable[TensorDecl], found: Dict[str, tuple], where: str) -> None:
    """``found`` maps name -> shape.  Raises one WeightsError naming all disagreements."""
    decls = list(decls)
    wanted = {d.name: d for d in decls}
    missing = [d.name for d in decls if d.name not in found and not d.optional]
    unexpected = [n for n in found if n not in wanted]
    wrong = [(n, tuple(wanted[n].shape), tuple(found[n])) for n in found
             if n in wanted and tuple(found[n]) != tuple(wanted[n].shape)]
    if not (missing or unexpected or wrong):
        return
    lines = [f"{where}: the tensors do not match the model"]
    if missing:
        lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
    if unexpected:
        lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
    if wrong:
        lines.append(f"  wrong shape ({len(wrong)}): " + ", ".join(
            f"{n} expected {list(e)} found {list(f)}" for n, e, f in wrong))
    raise WeightsError("\n".join(lines), missing, unexpected, wrong)


def convert(t: torch.Tensor, mode: str) -> torch.Tensor:
    """Apply the precision policy to one CPU tensor."""
    if not t.is_floating_point():
        return t.to(torch.int32)
    if mode == "float32":
        return t.to(torch.float32)
    if t.dtype == torch.float32:
        return t
    if t.dtype == torch.float16:
        return t.to(torch.float32).to(torch.bfloat16)
    return t


def load_tensors(model_dir: str, decls: List[TensorDecl], mode: str, device) -> Dict[str, torch.Tensor]:
    try:
        files = SafetensorsDir(model_dir)
    except SafetensorsError as e:
        raise WeightsError(str(e)) from None
    check_names(decls, {n: e.shape for n, e in files.entries.items()}, model_dir)
    out: Dict[str, torch.Tensor] = {}
    for d in decls:
        if d.name not in files.entries:
            continue
        out[d.name] = convert(files.tensor(d.name), mode).to(device)
    return out
