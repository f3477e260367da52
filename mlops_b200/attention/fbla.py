"""The `mlops.attention` Python interface over the CUDA library.

The public surface is the reference's (attention/python/mlops/attention/fbla.py:43-150): the ``FBLACache`` record and
``empty / encode / append / prefill / decode`` with the same argument names, defaults and exception types, so code
written against `mlops.attention` runs unchanged. Shapes: K / V chunks ``[B, Hkv, n, 128]``, prefill queries
``[B, Hq, n, 128]``, decode queries ``[B, Hq, 128]``, all BF16 on one CUDA device. Everything that touches cache bytes
or computes attention happens inside libmlops_attention.so; this module only allocates tensors and forwards.
"""
from dataclasses import dataclass
from typing import Optional

import torch

from . import _C

GROUP = 128      # tokens per quantisation group
HEAD_DIM = 128
# mode string -> (coarse bits, fine bits, value of mlops_fbla_format)
_PLANES = {"3+3": (3, 3, 0), "4+2": (4, 2, 1)}


@dataclass
class FBLACache:
    coarse: torch.Tensor  # uint8  [B, Hkv, 8 * groups, 512 * coarse bits]: the coarse plane's records
    fine: torch.Tensor    # uint8  [B, Hkv, 8 * groups, 512 * fine bits]
    meta: torch.Tensor    # bf16   [B, Hkv, groups, 512]: per-channel base / step of K and V
    sink_k: torch.Tensor  # bf16   [B, Hkv, 128, 128]: the first group, kept exact
    sink_v: torch.Tensor
    open_k: torch.Tensor  # bf16   [B, Hkv, 128, 128]: the group still being filled
    open_v: torch.Tensor
    tokens: int
    capacity: int
    format: int
    images: Optional[torch.Tensor] = None  # the reference's persistent prefill images; this library has none


def _require_kv(k, v):
    """K and V of one chunk: equal 4-D shapes with a head dimension of 128, on one CUDA device."""
    same = k.ndim == 4 and tuple(k.shape) == tuple(v.shape) and k.shape[-1] == HEAD_DIM
    if not same:
        raise ValueError(f"expected k and v of one shape [B, Hkv, n, {HEAD_DIM}]; k is {tuple(k.shape)}, v is {tuple(v.shape)}")
    if not (k.is_cuda and v.is_cuda and k.device == v.device):
        raise ValueError(f"k and v have to live on the same CUDA device (k: {k.device}, v: {v.device})")


def empty(batch: int, kv_heads: int, capacity: int, mode: str = "3+3", device="cuda") -> FBLACache:
    """A cache with room for ``capacity`` tokens and none stored. All arrays start as zeros."""
    planes = _PLANES.get(mode)
    if planes is None:
        raise ValueError(f"unknown mode {mode!r}: choose '3+3' or '4+2'")
    coarse_bits, fine_bits, fmt = planes
    groups = -(-capacity // GROUP)

    def zeros(shape, dtype):
        return torch.zeros(shape, dtype=dtype, device=device)

    records = 8 * groups
    windows = [zeros((batch, kv_heads, GROUP, HEAD_DIM), torch.bfloat16) for _ in ("sink_k", "sink_v", "open_k", "open_v")]
    with torch.cuda.device(torch.device(device)):
        image_bytes = _C.images_bytes(batch, kv_heads, groups * GROUP)
    return FBLACache(coarse=zeros((batch, kv_heads, records, 512 * coarse_bits), torch.uint8),
                     fine=zeros((batch, kv_heads, records, 512 * fine_bits), torch.uint8),
                     meta=zeros((batch, kv_heads, groups, 512), torch.bfloat16),
                     sink_k=windows[0], sink_v=windows[1], open_k=windows[2], open_v=windows[3],
                     tokens=0, capacity=capacity, format=fmt,
                     images=zeros((image_bytes,), torch.uint8) if image_bytes > 0 else None)


def _extend(cache, k, v, q=None, scale=0.0):
    """One library call: store the chunk (k, v) behind the cache's tokens and, given q, attend from its positions."""
    _require_kv(k, v)
    held = tuple(cache.meta.shape[:2])
    if tuple(k.shape[:2]) != held:
        raise ValueError(f"the chunk is [batch, kv_heads] = {tuple(k.shape[:2])} but the cache was built for {held}")
    added = int(k.shape[2])
    if cache.tokens + added > cache.capacity:
        raise ValueError(f"{added} more tokens do not fit: the cache holds {cache.tokens} of {cache.capacity}")
    q_heads = int(q.shape[1]) if q is not None else int(k.shape[1])
    result = _C.prefill(q, k.to(torch.bfloat16).contiguous(), v.to(torch.bfloat16).contiguous(),
                        cache.coarse, cache.fine, cache.meta, cache.sink_k, cache.sink_v, cache.open_k, cache.open_v,
                        cache.tokens, cache.capacity, q_heads, cache.format, scale, cache.images)
    cache.tokens += added
    return result


@torch.no_grad()
def encode(k: torch.Tensor, v: torch.Tensor, mode: str = "3+3", capacity: Optional[int] = None) -> FBLACache:
    """Quantise dense K / V ``[B, Hkv, N, 128]`` into a new cache (room for ``capacity`` tokens, default N)."""
    _require_kv(k, v)
    batch, kv_heads, n = (int(x) for x in k.shape[:3])
    room = n if capacity is None else int(capacity)
    if room < n:
        raise ValueError(f"a capacity of {room} tokens cannot hold the {n} given")
    cache = empty(batch, kv_heads, room, mode, k.device)
    _extend(cache, k, v)
    return cache


@torch.no_grad()
def append(cache: FBLACache, k: torch.Tensor, v: torch.Tensor) -> FBLACache:
    """Store ``[B, Hkv, n, 128]`` more K / V in ``cache`` (in place; also returned). Tokens land in the BF16 open
    group; once a group is full it is quantised when the following token arrives, so growing a cache token by token
    ends in the same bytes as :func:`encode` of the whole sequence."""
    _extend(cache, k, v)
    return cache


@torch.no_grad()
def prefill(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cache: FBLACache, *, scale: float = 0.0) -> torch.Tensor:
    """Causal attention of a chunk. ``k, v [B, Hkv, n, 128]`` are stored in ``cache`` first; the query of chunk
    position i (absolute position ``tokens + i``) sees every token up to its own. Returns ``[B, Hq, n, 128]`` BF16."""
    fits = q.dtype == torch.bfloat16 and q.ndim == 4 and q.shape[0] == k.shape[0] and q.shape[2] == k.shape[2]
    if not fits:
        raise ValueError(f"q has to be a bfloat16 [B, Hq, n, {HEAD_DIM}] tensor with the batch and length of k {tuple(k.shape)}; "
                         f"it is {q.dtype} {tuple(q.shape)}")
    return _extend(cache, k, v, q.contiguous(), scale)


class _ScratchPool:
    """Decode scratch, one buffer per (device, batch x KV heads), grown on demand and kept for later calls."""

    def __init__(self):
        self._buffers = {}

    def get(self, device, heads, nbytes):
        held = self._buffers.get((device, heads))
        if held is not None and held.numel() >= nbytes:
            return held
        fresh = torch.empty((nbytes,), dtype=torch.uint8, device=device)  # the library needs no initial contents
        self._buffers[(device, heads)] = fresh
        return fresh


_pool = _ScratchPool()


def decode(q: torch.Tensor, cache: FBLACache, *, scale: float = 0.0, tau: float = 0.0) -> torch.Tensor:
    """Attention of one new query per head, ``q [B, Hq, 128]`` BF16, over everything in ``cache``.
    ``scale`` 0 selects 1/sqrt(128); ``tau`` 0 selects the format's refinement threshold."""
    if q.dtype != torch.bfloat16:
        raise TypeError(f"decode takes bfloat16 queries, not {q.dtype}")
    batch, q_heads = int(q.shape[0]), int(q.shape[1])
    kv_heads = int(cache.meta.shape[1])
    with torch.cuda.device(q.device):
        need = _C.scratch_bytes(batch, q_heads, kv_heads, cache.tokens, cache.format, cache.capacity)
    scratch = _pool.get(q.device, batch * kv_heads, need)
    return _C.decode(q.contiguous(), cache.coarse, cache.fine, cache.meta, cache.sink_k, cache.sink_v, cache.open_k,
                     cache.open_v, scratch, cache.tokens, cache.capacity, kv_heads, cache.format, scale, tau)
