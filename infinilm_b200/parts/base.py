"""Interfaces of the parts a layer is put together from, and the registries that name them.

A part is built from its parameters alone (`PartSpec.params`); it never learns which model it is
in. Five kinds of part exist, each with its own registry:

  norm              `add_norm(resid, branch, branch_scale, out, rows=None)`
  position          rotation tables for a mixer (`inv_freq`, `mscale`, `rot_dim`)
  mixer             `forward(x, ctx, cache) -> y`, `cache_need()`
  feed_forward      `forward(x, ctx) -> y`
  arrangement       a block of two norms, a mixer and a feed-forward: `run(resid, pending, ctx, cache)`

Every part lists the checkpoint tensors it wants (`weight_specs`) and receives them, already on
the device, through `set_weights`.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional

import torch

from .spec import CacheNeed, PartSpec, WeightSpec


class Part:
    """Common base: parameters in, list of wanted tensors out, tensors in."""

    # True: a step of single tokens through this part may be captured once and replayed as a CUDA graph - the part
    # launches the same kernels on the same buffers whatever the step's lengths and slots, reads what changes from the
    # step's device arrays only, and never waits for the device. A part says so itself; by default it is not replayed.
    graph_safe = False

    def __init__(self, params: Dict[str, Any], prefix: str, dtype: torch.dtype):
        self.params = dict(params)
        self.prefix = prefix
        self.dtype = dtype                       # compute dtype: torch.float32 or torch.bfloat16

    def weight_specs(self) -> List[WeightSpec]:
        return []

    def set_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        """`tensors` maps local names to device tensors (matrices already in the compute dtype)."""

    def full_name(self, local: str) -> str:
        return f"{self.prefix}.{local}" if self.prefix else local


class ResidualTail:
    """Handed to a branch (mixer or feed-forward) whose last matrix product can finish the branch itself: add
    `scale` * result into `resid` (float32 [T,H], in place) and prepare `norm` of the sum for the next product, which
    then gets an `ops.NormedInput` instead of normalised rows. Saves the add+norm kernel between two products."""
    __slots__ = ("resid", "scale", "norm")

    def __init__(self, resid: torch.Tensor, scale: float, norm: "Norm"):
        self.resid, self.scale, self.norm = resid, float(scale), norm


class Norm(Part):
    fusable_rms = False                          # True: an RMSNorm with `.weight` and `.eps` that a ResidualTail may name

    def add_norm(self, resid: torch.Tensor, branch: Optional[torch.Tensor], branch_scale: float,
                 out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """resid (f32 [T,H]) += branch_scale * branch; out = norm(resid). With `rows`, only those
        rows are normalised into out[0:len(rows)] and resid is left alone."""
        raise NotImplementedError


class PositionEncoding(Part):
    """A position encoding that a mixer applies to its queries and keys. Two forms:

    rotary: `rot_dim`, `inv_freq`, `mscale` - a table that the mixer's fused rotate-and-store kernel applies
      (angle = position * inv_freq[i], pairs (i, i + rot_dim/2), cos and sin times mscale);
    any other function of (q, k, position): `has_transform = True` and `transform(qkv, ctx, ...)`, which changes the
      q and k columns of the projected rows in place before the keys are written to the cache (rot_dim stays 0). The
      mixer then leaves its fused projection-and-rotation kernel for the plain sequence projection, transform, store.
    An encoding that acts on the scores (a bias per distance) is neither: it needs the attention kernels themselves."""
    rot_dim: int = 0
    mscale: float = 1.0
    inv_freq: Optional[torch.Tensor] = None     # float32 [rot_dim/2] on the device
    has_transform = False

    def to_device(self, device: torch.device) -> None:
        pass

    def transform(self, qkv: torch.Tensor, ctx, n_heads: int, n_kv_heads: int, head_dim: int) -> None:
        """qkv [T, (n_heads + 2 n_kv_heads) * head_dim] in the compute dtype: change q (the first n_heads heads) and k
        (the next n_kv_heads) in place; `ctx.tok_pos` holds each row's position (int32 on the device)."""


class Mixer(Part):
    def cache_need(self) -> Optional[CacheNeed]:
        return None

    # A part that can read an `ops.NormedInput` as `x`, or take a `tail=ResidualTail` in `forward` and return the
    # `ops.NormedInput` of the next norm, says so here for a step of T rows; by default it can do neither.
    def accepts_normed(self, T: int) -> bool:
        return False

    def fuses_tail(self, T: int) -> bool:
        return False

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        """x [T,H] in the compute dtype -> y [T,H]. `cache` is this run entry's view of the cache
        (`PagedKVView`, `StateView` or None); `cache.writable` is False when the entry reads
        another entry's cache."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        raise NotImplementedError

    def accepts_normed(self, T: int) -> bool:     # see Mixer
        return False

    def fuses_tail(self, T: int) -> bool:
        return False


class Arrangement:
    """How the parts of one layer are wired around the residual stream."""

    def __init__(self, mixer_norm: Norm, mixer: Mixer, ffn_norm: Norm, ffn: FeedForward, params: Dict[str, Any]):
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = mixer_norm, mixer, ffn_norm, ffn
        self.params = dict(params)

    def parts(self) -> List[Part]:
        return [self.mixer_norm, self.mixer, self.ffn_norm, self.ffn]

    def run(self, resid: torch.Tensor, pending, ctx, cache):
        """`pending` is (branch, scale) not yet added to `resid`, or None, or an `ops.NormedInput` (the add is done and
        this block's first norm prepared; only given if `accepts_normed_input`). Returns the new pending. An arrangement
        with `takes_next_norm` has one more argument, `next_norm=None`: the first norm of the block that runs next, if that
        block accepts a normed input; it may then return an `ops.NormedInput` for it."""
        raise NotImplementedError

    takes_next_norm = False                      # True: `run` has the `next_norm` argument and may use it

    def accepts_normed_input(self, T: int) -> bool:
        return False


_REGISTRIES: Dict[str, Dict[str, Callable]] = {
    "norm": {}, "position": {}, "mixer": {}, "feed_forward": {}, "arrangement": {}, "embedding": {}, "head": {},
}


def register_part(family: str, kind: str, cls: Callable) -> None:
    """Register `cls` under `kind` in one of the families above. A test or a new architecture
    calls this for its own parts; nothing else in the framework has to change."""
    if family not in _REGISTRIES:
        raise KeyError(f"unknown part family {family!r} ({', '.join(_REGISTRIES)})")
    _REGISTRIES[family][kind] = cls


def unregister_part(family: str, kind: str) -> None:
    _REGISTRIES[family].pop(kind, None)


def part_class(family: str, kind: str) -> Callable:
    _ensure_builtin()
    try:
        return _REGISTRIES[family][kind]
    except KeyError:
        raise KeyError(f"no {family} part of kind {kind!r} is registered "
                       f"(known: {', '.join(sorted(_REGISTRIES[family]))})") from None


def build_part(family: str, spec: PartSpec, dtype: torch.dtype):
    return part_class(family, spec.kind)(spec.params, spec.prefix, dtype)


_builtin_done = False


def _ensure_builtin() -> None:
    global _builtin_done
    if not _builtin_done:
        _builtin_done = True
        from . import attention, blocks, embedding, feed_forward, norms, position  # noqa: F401
