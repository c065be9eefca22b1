"""Reading and writing safetensors files (8-byte little-endian header length, JSON header,
raw tensor bytes), by tensor name, without loading what is not asked for.

Parity with InfiniLM: `python/infinilm/modeling_utils.py:103-138` (open a checkpoint file, check
the `format` metadata), `:222-236` (index file lists the shards, else every *.safetensors).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Optional, Tuple

import torch

_ST2TORCH = {
    "F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "F64": torch.float64,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
_TORCH2ST = {v: k for k, v in _ST2TORCH.items()}


class SafetensorsError(IOError):
    pass


class SafetensorsFile:
    """One .safetensors file, memory-mapped; tensors are read on demand."""

    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        head = self._f.read(8)
        if len(head) != 8:
            raise SafetensorsError(f"{path}: not a safetensors file (too short)")
        (n,) = struct.unpack("<Q", head)
        size = os.path.getsize(path)
        if n <= 0 or 8 + n > size:
            raise SafetensorsError(f"{path}: bad header length {n}")
        try:
            header = json.loads(self._f.read(n).decode("utf-8"))
        except Exception as e:
            raise SafetensorsError(f"{path}: header is not JSON: {e}") from e
        self.metadata = header.pop("__metadata__", None) or {}
        fmt = self.metadata.get("format")
        if fmt is not None and fmt not in ("pt", "tf", "flax", "mlx"):
            raise SafetensorsError(f"{path}: metadata format {fmt!r} is not one of pt, tf, flax, mlx")
        self._base = 8 + n
        self.entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        for name, e in header.items():
            b, en = e["data_offsets"]
            if e["dtype"] not in _ST2TORCH:
                raise SafetensorsError(f"{path}: tensor {name} has unsupported dtype {e['dtype']}")
            if self._base + en > size or b > en:
                raise SafetensorsError(f"{path}: tensor {name} lies outside the file")
            self.entries[name] = (e["dtype"], tuple(int(x) for x in e["shape"]), int(b), int(en))
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def names(self) -> List[str]:
        return list(self.entries)

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        d, shape, _, _ = self.entries[name]
        return _ST2TORCH[d], shape

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that views the mapped file (read-only memory: copy before writing)."""
        d, shape, b, e = self.entries[name]
        dt = _ST2TORCH[d]
        numel = 1
        for s in shape:
            numel *= s
        if numel == 0:
            return torch.empty(shape, dtype=dt)
        if (e - b) != numel * torch.empty((), dtype=dt).element_size():
            raise SafetensorsError(f"{self.path}: tensor {name}: byte size does not match its shape")
        buf = memoryview(self._mm)[self._base + b: self._base + e]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")     # torch warns that the buffer is not writable
            t = torch.frombuffer(buf, dtype=dt, count=numel)
        return t.reshape(shape)

    def close(self) -> None:
        try:
            if self._mm is not None:
                self._mm.close()
        except BufferError:
            pass                                 # tensors still view the map; the OS frees it at exit
        self._f.close()


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Optional[Dict[str, str]] = None) -> None:
    header = {"__metadata__": dict(metadata or {"format": "pt"})}
    off = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _TORCH2ST:
            raise SafetensorsError(f"cannot store dtype {t.dtype}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _TORCH2ST[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + nbytes]}
        off += nbytes
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * ((8 - len(hj) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            f.write(t.view(torch.uint8).reshape(-1).numpy().tobytes() if t.numel() else b"")
    os.replace(tmp, path)


def checkpoint_files(model_dir: str) -> List[str]:
    """The safetensors files of a model folder: those the index names, else all, sorted."""
    idx = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(idx):
        with open(idx, "r") as f:
            wm = json.load(f).get("weight_map", {})
        files = sorted(set(wm.values()))
        return [os.path.join(model_dir, fn) for fn in files]
    files = sorted(fn for fn in os.listdir(model_dir) if fn.endswith(".safetensors"))
    if not files:
        raise SafetensorsError(f"no .safetensors file in {model_dir}")
    return [os.path.join(model_dir, fn) for fn in files]
