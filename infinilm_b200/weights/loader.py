"""Loads a model's tensors by name and hands each part its own.

Every tensor the model's parts list is looked up by its checkpoint name; names and shapes are
checked for the whole model first, and one error lists everything that is missing, unexpected,
of the wrong shape, or of the wrong kind (integers offered for a matrix or a vector). Storage precision is kept: bfloat16 stays bfloat16 (float16 is converted
to bfloat16), a tensor stored in 32-bit stays 32-bit, integer tables become int32. Operands of
matrix products are then brought to the compute dtype by the parts themselves.

Parity with InfiniLM: `python/infinilm/modeling_utils.py:71-100` (missing and unexpected keys in
one RuntimeError), `:131-136` (dtype cast on load), `:192-359` (file by file), `:342-351`
(lm_head.weight absent: the embedding table is used).
"""
from __future__ import annotations

from typing import Callable, Dict, Iterable, List, Mapping, Optional, Tuple

import torch

from .safetensors_io import SafetensorsFile, checkpoint_files


class WeightError(RuntimeError):
    """Lists every missing, unexpected and mis-shaped tensor of a checkpoint."""

    def __init__(self, missing: List[str], unexpected: List[str], wrong_shape: List[Tuple[str, tuple, tuple]],
                 other: Optional[List[str]] = None):
        self.missing, self.unexpected, self.wrong_shape, self.other = missing, unexpected, wrong_shape, other or []
        lines = ["Error(s) in loading weights:"]
        if missing:
            lines.append(f"  missing tensor(s) ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensor(s) ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong_shape:
            lines.append(f"  wrong shape ({len(wrong_shape)}): " + ", ".join(
                f"{n} is {list(got)}, expected {list(exp)}" for n, got, exp in wrong_shape))
        for o in self.other:
            lines.append("  " + o)
        super().__init__("\n".join(lines))


class TensorSource:
    """Where tensors come from: `names()`, `info(name) -> (dtype, shape)`, `get(name) -> tensor`."""

    def names(self) -> List[str]:
        raise NotImplementedError

    def info(self, name: str):
        raise NotImplementedError

    def get(self, name: str) -> torch.Tensor:
        raise NotImplementedError

    def close(self) -> None:
        pass


class FolderSource(TensorSource):
    def __init__(self, model_dir: str):
        self.files = [SafetensorsFile(p) for p in checkpoint_files(model_dir)]
        self.where: Dict[str, SafetensorsFile] = {}
        for f in self.files:
            for n in f.names():
                self.where[n] = f

    def names(self):
        return list(self.where)

    def info(self, name):
        return self.where[name].info(name)

    def get(self, name):
        return self.where[name].tensor(name)

    def close(self):
        for f in self.files:
            f.close()


class DictSource(TensorSource):
    def __init__(self, tensors: Mapping[str, torch.Tensor]):
        self.tensors = tensors

    def names(self):
        return list(self.tensors)

    def info(self, name):
        t = self.tensors[name]
        return t.dtype, tuple(t.shape)

    def get(self, name):
        return self.tensors[name]


def stored_precision(t: torch.Tensor, role: str) -> torch.Tensor:
    """bfloat16 stays, float16 -> bfloat16, 32-bit floats stay, wider floats -> float32,
    integer tables -> int32."""
    if role == "table" or not t.dtype.is_floating_point:
        return t.to(torch.int32)
    if t.dtype in (torch.bfloat16, torch.float32):
        return t
    if t.dtype == torch.float16:
        return t.to(torch.bfloat16)
    return t.to(torch.float32)


def check_against(model, source: TensorSource) -> None:
    """Compares the model's wanted tensors with what the source holds; raises one `WeightError`."""
    have = set(source.names())
    wanted = set()
    missing, wrong, kind = [], [], []
    for part, ws in model.weight_specs():
        full = part.full_name(ws.name)
        wanted.add(full)
        if full not in have:
            if ws.fallback is not None and ws.fallback in have:
                full_fb = ws.fallback
                _, shape = source.info(full_fb)
                if tuple(shape) != tuple(ws.shape):
                    wrong.append((f"{full} (taken from {full_fb})", tuple(shape), tuple(ws.shape)))
                continue
            missing.append(full)
            continue
        dt, shape = source.info(full)
        if tuple(shape) != tuple(ws.shape):
            wrong.append((full, tuple(shape), tuple(ws.shape)))
        floating = getattr(dt, "is_floating_point", None)
        if floating is not None and floating != (ws.role != "table"):
            kind.append(f"wrong kind of numbers: {full} is stored as {dt}, a {ws.role} needs "
                        + ("integers" if ws.role == "table" else "floating point"))
    unexpected = sorted(have - wanted)
    if missing or unexpected or wrong or kind:
        raise WeightError(sorted(missing), unexpected, wrong, kind)


def load_into(model, source: TensorSource, device: torch.device,
              progress: Optional[Callable[[str], None]] = None) -> None:
    """Checks, then moves each part's tensors to `device` and gives them to the part."""
    check_against(model, source)
    have = set(source.names())
    shared: Dict[str, torch.Tensor] = {}         # device copies that a fallback may share
    fallback_names = {ws.fallback for _, ws in model.weight_specs() if ws.fallback}
    for part in model.parts():
        tensors: Dict[str, torch.Tensor] = {}
        for ws in part.weight_specs():
            full = part.full_name(ws.name)
            src_name = full if full in have else ws.fallback
            if src_name in shared:
                tensors[ws.name] = shared[src_name]
                continue
            t = stored_precision(source.get(src_name), ws.role)
            if ws.role == "matrix":
                t = t.to(device=device, dtype=model.dtype, non_blocking=False)
            else:
                t = t.to(device=device)
            tensors[ws.name] = t
            if src_name in fallback_names:
                shared[src_name] = t
        part.set_weights(tensors)
        if progress is not None:
            progress(part.prefix)
