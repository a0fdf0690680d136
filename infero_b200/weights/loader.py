"""Bind the tensors of a model folder to the names a model declares.

One pass compares what the model declares with what the files hold and raises a single
``WeightsError`` listing every missing tensor, every unexpected tensor and every wrong
shape.  (The reference stops at the first missing name, crates/safetensors/src/lib.rs:541-544,
and checks shapes separately, crates/model/src/weights.rs:1348-1460.)

Precision policy.  ``bfloat16``: a tensor stored as BF16 stays bf16, F16 is widened through
float32 and rounded to bf16 (the reference narrows BF16 to F16 instead,
crates/safetensors/src/lib.rs:197-254), integer tables become int32.  A tensor stored in
32-bit stays 32-bit where the arithmetic is 32-bit anyway (norm weights, biases, and any role a
part invents for itself); the operands of matrix products (roles ``matrix`` and ``embedding``)
are rounded to bf16 once, here, because that is what the tensor-core kernels of a bfloat16
engine multiply: a checkpoint stored in float32 then runs the same kernels as one stored in
bf16 (the reference likewise narrows matrices and widens norms and biases to f32,
crates/model/src/weights.rs:2063-2077).  ``float32``: every floating tensor becomes float32.
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


PRODUCT_ROLES = ("matrix", "embedding")


def convert(t: torch.Tensor, mode: str, role: str = "matrix") -> torch.Tensor:
    """Apply the precision policy to one CPU tensor."""
    if not t.is_floating_point():
        return t.to(torch.int32)
    if mode == "float32":
        return t.to(torch.float32)
    if t.dtype in (torch.float32, torch.float64):
        return t.to(torch.bfloat16) if role in PRODUCT_ROLES else t.to(torch.float32)
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
        out[d.name] = convert(files.tensor(d.name), mode, d.role).to(device)
    return out
