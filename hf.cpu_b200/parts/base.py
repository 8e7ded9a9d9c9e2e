"""Interfaces of the parts a layer is put together from, and their registries.

Five categories: ``norm``, ``position``, ``mixer``, ``ffn`` and ``block``.  A part
is chosen by the ``kind`` of a :class:`PartSpec` and receives every size and
constant through the spec's arguments; no part knows which model it is in.

The reference runs one fixed layer with ``if`` switches for its variants
(src/model.c:574-624); the same steps are separate parts here so that a layer
can pick a different mixer or feed-forward than its neighbour.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch

from ..config.base import ConfigError, PartSpec
from ..weights.loader import TensorSpec

CATEGORIES = ("norm", "position", "mixer", "ffn", "block", "embedding", "head")
_REGISTRY: Dict[str, Dict[str, Callable[..., "Part"]]] = {c: {} for c in CATEGORIES}


def register_part(category: str, kind: str, factory: Callable[..., "Part"]) -> None:
    """Register ``factory(**spec.args, **context)`` under ``kind`` in ``category``."""
    if category not in _REGISTRY:
        raise ConfigError(f"unknown part category '{category}' (known: {', '.join(CATEGORIES)})")
    _REGISTRY[category][kind] = factory


def unregister_part(category: str, kind: str) -> None:
    _REGISTRY[category].pop(kind, None)


def make_part(category: str, spec: PartSpec, **context: Any) -> "Part":
    try:
        factory = _REGISTRY[category][spec.kind]
    except KeyError:
        raise ConfigError(f"no {category} part of kind '{spec.kind}' is registered "
                          f"(known: {', '.join(sorted(_REGISTRY[category]))})") from None
    return factory(**spec.args, **context)


@dataclass(frozen=True)
class CacheSpec:
    """What a mixer asks of the paged cache: per token ``2 * num_kv_heads * head_dim`` values
    (keys then values); ``window`` = 0 keeps every key, else only the most recent ``window``."""
    num_kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class StateSpec:
    """Per-request state of fixed size: one tensor of ``shape`` per live request."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class Part:
    # True when forward() only launches kernels on tensors at stable addresses and reads nothing of the step
    # on the host, so that a decode step may be captured once as a CUDA graph and replayed
    graph_safe = False

    def tensor_specs(self) -> List[TensorSpec]:
        """The checkpoint tensors this part needs."""
        return []

    def bind(self, tensors: Dict[str, torch.Tensor], run_dtype: torch.dtype, device: torch.device) -> None:
        """Take ownership of the loaded tensors (and fuse or lay them out for the kernels)."""

    def weight_bytes(self) -> int:
        """Bytes of weights a step reads from this part (for roofline accounting)."""
        return 0

    def flops(self, *a) -> float:
        """Floating-point operations of this part in one step (a multiply-add counts two), for the reported
        fraction of the tensor-core peak.  Mixers are asked with (q_lens, kv_lens): the tokens each request brings
        and holds afterwards; feed-forwards and the head with the number of rows they transform."""
        return 0.0


class Norm(Part):
    def fused_args(self):
        """(weight, eps) when this norm is an RMSNorm that a product's tail may apply itself, else None."""
        return None

    def forward(self, x: torch.Tensor, out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Normalise rows of the float32 residual ``x`` into ``out`` (run dtype).  With ``rows``
        (int32 indices) only those rows are read, in that order."""
        raise NotImplementedError


class PositionEncoding(Part):
    def prepare(self, max_positions: int, device: torch.device) -> None:
        """Build whatever tables are needed for positions ``0 .. max_positions-1``."""


class Mixer(Part):
    def cache_spec(self) -> Optional[CacheSpec]:
        return None

    def state_spec(self) -> Optional[StateSpec]:
        return None

    def step_arrays_key(self) -> Optional[Any]:
        """A hashable name for the int32 index arrays this mixer wants built for every step, or None.  Mixers that
        return equal keys share one set (the layers of a model usually do)."""
        return None

    def step_arrays(self, batch) -> Dict[str, Any]:
        """Called once per step and key with the host's view of the step (``batch.q_lens``, ``.kv_lens``, ``.starts``,
        ``.block_size``): returns named integer arrays (numpy), which the engine appends to the step's one
        host-to-device copy.  ``forward`` finds them on the device as ``ctx.arrays(key)[name]``.  For a step of
        single tokens the sizes must depend on the number of requests only (such steps are replayed as a graph)."""
        return {}

    def forward(self, ctx, xn: torch.Tensor, residual: torch.Tensor, cache, state, write_cache: bool) -> None:
        """Mix ``xn`` ([T, hidden], run dtype) across tokens and add the result into the float32
        ``residual``.  ``cache`` is the entry's :class:`LayerCache` (or None), ``state`` the entry's
        per-request state tensor ``[max_requests, *shape]`` (or None); ``write_cache`` is False when
        the entry reads another entry's cache."""
        raise NotImplementedError

    # Optional: ``forward_then_norm(ctx, xn, residual, cache, state, write_cache, norm, out) -> bool`` does the same
    # and, if it returns True, has also written ``out = norm(residual)`` (the block then skips that norm).


class FeedForward(Part):
    def forward(self, ctx, xn: torch.Tensor, residual: torch.Tensor) -> None:
        """Token-wise transform of ``xn`` added into the float32 ``residual``."""
        raise NotImplementedError

    # Optional: ``forward_then_norm(ctx, xn, residual, norm, out) -> bool``, as for mixers.


class Block(Part):
    def forward(self, ctx, x: torch.Tensor, norm1: Norm, mixer: Mixer, norm2: Norm, ffn: FeedForward,
                cache, state, write_cache: bool, xn_ready: Optional[torch.Tensor] = None,
                next_norm: Optional[Norm] = None) -> Optional[torch.Tensor]:
        """Run one layer on the float32 residual stream ``x`` in place.  ``xn_ready`` is ``norm1(x)`` if the
        previous block already computed it.  If ``next_norm`` is given the block may return ``next_norm(x)`` of
        its result (computed in the tail of its last product); returning None leaves that norm to the next block."""
        raise NotImplementedError
