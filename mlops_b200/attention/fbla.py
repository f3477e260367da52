"""The `mlops.attention` Python interface (reference: attention/python/mlops/attention/fbla.py:43-150), same names,
signatures and error behaviour: ``empty(batch, kv_heads, capacity, "4+2")`` or ``encode(k, v, "4+2", capacity)``,
``prefill(q, k, v, cache)`` (a chunk: q [B, Hq, n, 128], k / v [B, Hkv, n, 128] BF16; appends), ``append(cache, k, v)``,
``decode(q, cache)`` (one query per head). Every cache write and every attention runs in the CUDA library."""
from dataclasses import dataclass
from typing import Optional

import torch

from . import _C

_MODES = {"3+3": (3, 3, 0), "4+2": (4, 2, 1)}


@dataclass
class FBLACache:
    coarse: torch.Tensor  # [B, H, capacity_groups * 8, 2 CB 256] uint8
    fine: torch.Tensor    # [B, H, capacity_groups * 8, 2 FB 256] uint8
    meta: torch.Tensor    # [B, H, capacity_groups, 512] bfloat16
    sink_k: torch.Tensor
    sink_v: torch.Tensor
    open_k: torch.Tensor
    open_v: torch.Tensor
    tokens: int
    capacity: int
    format: int
    images: Optional[torch.Tensor] = None  # always None here: this library keeps no prefill images


def _check_kv(k, v):
    if k.shape != v.shape or k.ndim != 4 or k.shape[-1] != 128:
        raise ValueError(f"k and v must have the same [B, H, N, 128] shape, got {tuple(k.shape)} and {tuple(v.shape)}")
    if not k.is_cuda or k.device != v.device:
        raise ValueError("k and v must be CUDA tensors on the same device")


def empty(batch: int, kv_heads: int, capacity: int, mode: str = "3+3", device="cuda") -> FBLACache:
    """An empty cache laid out for ``capacity`` tokens (zero-filled: 0 tokens)."""
    if mode not in _MODES:
        raise ValueError(f"mode must be '3+3' or '4+2', got {mode!r}")
    cb, fb, fmt = _MODES[mode]
    cg = (capacity + 127) // 128
    u8 = dict(device=device, dtype=torch.uint8)
    bf = dict(device=device, dtype=torch.bfloat16)
    ex = [torch.zeros((batch, kv_heads, 128, 128), **bf) for _ in range(4)]
    with torch.cuda.device(torch.device(device)):
        nimg = _C.images_bytes(batch, kv_heads, cg * 128)
    images = torch.zeros(nimg, **u8) if nimg else None
    return FBLACache(torch.zeros((batch, kv_heads, cg * 8, 2 * cb * 256), **u8),
                     torch.zeros((batch, kv_heads, cg * 8, 2 * fb * 256), **u8),
                     torch.zeros((batch, kv_heads, cg, 512), **bf), ex[0], ex[1], ex[2], ex[3], 0, capacity, fmt, images)


def _prefill(q, cache, k, v, scale):
    _check_kv(k, v)
    c = cache
    if k.shape[:2] != c.meta.shape[:2]:
        raise ValueError(f"k / v heads {tuple(k.shape[:2])} do not match the cache's {tuple(c.meta.shape[:2])}")
    n = k.shape[2]
    if c.tokens + n > c.capacity:
        raise ValueError(f"cache full: {c.tokens} + {n} tokens > capacity {c.capacity}")
    out = _C.prefill(q, k.to(torch.bfloat16).contiguous(), v.to(torch.bfloat16).contiguous(), c.coarse, c.fine,
                     c.meta, c.sink_k, c.sink_v, c.open_k, c.open_v, c.tokens, c.capacity,
                     q.shape[1] if q is not None else k.shape[1], c.format, scale, c.images)
    c.tokens += n
    return out


@torch.no_grad()
def encode(k: torch.Tensor, v: torch.Tensor, mode: str = "3+3", capacity: Optional[int] = None) -> FBLACache:
    """Encode dense ``[B, Hkv, N, 128]`` K / V into an :class:`FBLACache` laid out for ``capacity`` tokens."""
    _check_kv(k, v)
    B, H, N, _ = k.shape
    capacity = N if capacity is None else capacity
    if capacity < N:
        raise ValueError(f"capacity {capacity} < tokens {N}")
    cache = empty(B, H, capacity, mode, k.device)
    _prefill(None, cache, k, v, 0.0)
    return cache


@torch.no_grad()
def append(cache: FBLACache, k: torch.Tensor, v: torch.Tensor) -> FBLACache:
    """Append ``[B, Hkv, n, 128]`` K / V to ``cache`` in place. New tokens go to the open group (BF16); a full open
    group is quantized into its records and metadata when the next token arrives, exactly as :func:`encode` would."""
    _prefill(None, cache, k, v, 0.0)
    return cache


@torch.no_grad()
def prefill(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cache: FBLACache, *, scale: float = 0.0) -> torch.Tensor:
    """Append a chunk ``k, v [B, Hkv, n, 128]`` to ``cache`` and return the attention of its queries
    ``q [B, Hq, n, 128]`` (BF16): position ``cache.tokens + i`` attends to the tokens up to itself."""
    if q.dtype != torch.bfloat16 or q.ndim != 4 or q.shape[0] != k.shape[0] or q.shape[2] != k.shape[2]:
        raise ValueError(f"q must be BF16 [B, Hq, n, 128] matching k {tuple(k.shape)}, got {q.dtype} {tuple(q.shape)}")
    return _prefill(q.contiguous(), cache, k, v, scale)


_SCRATCH = {}  # (device, batch * kv_heads) -> allocated once, reused


def _scratch(device, heads, nbytes):
    key = (device, heads)
    s = _SCRATCH.get(key)
    if s is None or s.numel() < nbytes:
        s = torch.full((nbytes,), 0xFF, dtype=torch.uint8, device=device)
        _SCRATCH[key] = s
    return s


def decode(q: torch.Tensor, cache: FBLACache, *, scale: float = 0.0, tau: float = 0.0) -> torch.Tensor:
    """One decode query per q head ``[B, Hq, 128]`` BF16 against ``cache``; scale 0 = 1/sqrt(128), tau 0 = the
    format's default."""
    if q.dtype != torch.bfloat16:
        raise TypeError(f"q must be bfloat16, got {q.dtype}")
    c = cache
    kv_heads = c.meta.shape[1]
    with torch.cuda.device(q.device):
        nbytes = _C.scratch_bytes(q.shape[0], q.shape[1], kv_heads, c.tokens, c.format, c.capacity)
    scratch = _scratch(q.device, q.shape[0] * kv_heads, nbytes)
    return _C.decode(q.contiguous(), c.coarse, c.fine, c.meta, c.sink_k, c.sink_v, c.open_k, c.open_v, scratch,
                     c.tokens, c.capacity, kv_heads, c.format, scale, tau)
