"""Binding of the C library (include/mlops_fbla.h) for PyTorch tensors: the four functions of the reference's compiled
`mlops.attention._C` module (attention/python/csrc/mlops_attention_torch.cpp:99-111), same names, argument orders,
checks and exceptions -- scratch_bytes, images_bytes, decode, prefill. PyTorch supplies device memory and the current
stream only; every computation happens inside libmlops_attention.so. There is no CPU fallback: importing this module
without the built library raises."""
import ctypes
import os

import torch

_LIB_PATH = os.environ.get("MLOPS_FBLA_LIBRARY") or os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "lib",
                                                                  "libmlops_attention.so")
if not os.path.exists(_LIB_PATH):
    raise ImportError(f"{_LIB_PATH} is missing: build it with `make -C mlops_b200/csrc` (or __graft_entry__.build()); "
                      "this package has no fallback path")
_lib = ctypes.CDLL(_LIB_PATH)

__version__ = "0.4.0"
OK, INVALID_VALUE, CUDA_ERROR = 0, 1, 2


class Config(ctypes.Structure):
    """mlops_fbla_config (64 bytes)."""
    _fields_ = [("batch", ctypes.c_int), ("q_heads", ctypes.c_int), ("kv_heads", ctypes.c_int), ("tokens", ctypes.c_int),
                ("scale", ctypes.c_float), ("tau", ctypes.c_float), ("format", ctypes.c_int), ("capacity", ctypes.c_int),
                ("head_stride", ctypes.c_int), ("group_stride", ctypes.c_int),
                ("out_head_stride", ctypes.c_int64), ("out_token_stride", ctypes.c_int64),
                ("length_stride", ctypes.c_int)]


class Cache(ctypes.Structure):
    """mlops_fbla_cache (64 bytes)."""
    _fields_ = [(n, ctypes.c_void_p) for n in ("coarse", "fine", "meta", "exact_sink_k", "exact_sink_v", "exact_open_k",
                                               "exact_open_v", "tc_images")]


class Sizes(ctypes.Structure):
    _fields_ = [(n, ctypes.c_size_t) for n in ("coarse", "fine", "meta", "exact", "images")]


_vp, _cp = ctypes.c_void_p, ctypes.POINTER(Config)
_lib.mlops_fbla_decode_scratch_bytes.restype = ctypes.c_size_t
_lib.mlops_fbla_decode_scratch_bytes.argtypes = [_cp]
_lib.mlops_fbla_decode_scratch_bytes_for.restype = ctypes.c_size_t
_lib.mlops_fbla_decode_scratch_bytes_for.argtypes = [_cp, ctypes.c_int]
_lib.mlops_fbla_images_bytes.restype = ctypes.c_size_t
_lib.mlops_fbla_images_bytes.argtypes = [_cp]
_lib.mlops_fbla_cache_sizes.restype = ctypes.c_int
_lib.mlops_fbla_cache_sizes.argtypes = [_cp, ctypes.POINTER(Sizes)]
_lib.mlops_fbla_decode.restype = ctypes.c_int
_lib.mlops_fbla_decode.argtypes = [_cp, _vp, ctypes.POINTER(Cache), _vp, _vp, ctypes.c_size_t, _vp]
_lib.mlops_fbla_decode_at.restype = ctypes.c_int
_lib.mlops_fbla_decode_at.argtypes = [_cp, _vp, _vp, ctypes.POINTER(Cache), _vp, _vp, ctypes.c_size_t, _vp]
_lib.mlops_fbla_prefill.restype = ctypes.c_int
_lib.mlops_fbla_prefill.argtypes = [_cp, ctypes.c_int, _vp, _vp, _vp, ctypes.POINTER(Cache), _vp, _vp]
_lib.mlops_fbla_prefill_at.restype = ctypes.c_int
_lib.mlops_fbla_prefill_at.argtypes = [_cp, _vp, _vp, ctypes.c_int, _vp, _vp, _vp, ctypes.POINTER(Cache), _vp, _vp]
_lib.mlops_fbla_append_at.restype = ctypes.c_int
_lib.mlops_fbla_append_at.argtypes = [_cp, _vp, _vp, _vp, ctypes.POINTER(Cache), _vp]
_lib.mlops_fbla_last_error.restype = ctypes.c_char_p
_lib.mlops_fbla_status_string.restype = ctypes.c_char_p
_lib.mlops_fbla_status_string.argtypes = [ctypes.c_int]

lib = _lib  # the raw C ABI, for callers that drive it directly (tests, the bench)


def last_error():
    return _lib.mlops_fbla_last_error().decode()


def _raise(status, what):
    if status == INVALID_VALUE:
        raise ValueError(last_error())
    if status != OK:
        raise RuntimeError(f"{what} failed: {last_error()}")


def _config(batch, q_heads, kv_heads, tokens, fmt, capacity, scale, tau):
    if fmt not in (0, 1):
        raise ValueError("format must be 0 (3+3) or 1 (4+2)")
    return Config(int(batch), int(q_heads), int(kv_heads), int(tokens), float(scale), float(tau), int(fmt), int(capacity), 0, 0, 0, 0, 0)


def _tensor(x, dev, dtype, what):
    if not x.is_cuda or x.device != dev:
        raise ValueError(f"{what}: expected a CUDA tensor on {dev}")
    if x.dtype != dtype or not x.is_contiguous():
        raise ValueError(f"{what}: expected a contiguous {dtype} tensor")


def _cache(coarse, fine, meta, sk, sv, ok, ov, images=None):
    return Cache(coarse.data_ptr(), fine.data_ptr(), meta.data_ptr(), sk.data_ptr(), sv.data_ptr(), ok.data_ptr(), ov.data_ptr(),
                 images.data_ptr() if images is not None else None)


def _stream(dev):
    return ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


def scratch_bytes(batch, q_heads, kv_heads, tokens, format, capacity):
    """Bytes of scratch one decode needs on the current device."""
    cfg = _config(batch, q_heads, kv_heads, tokens, format, capacity, 0.0, 0.0)
    n = int(_lib.mlops_fbla_decode_scratch_bytes(ctypes.byref(cfg)))
    if n <= 0:
        raise ValueError(f"invalid FBLA configuration: batch {batch}, heads {q_heads} / {kv_heads}, tokens {tokens}, capacity {capacity}")
    return n


def images_bytes(batch, kv_heads, capacity):
    """Bytes of persistent prefill images on the current device (this library keeps none: 0)."""
    cfg = _config(batch, kv_heads, kv_heads, 0, 0, capacity, 0.0, 0.0)
    return int(_lib.mlops_fbla_images_bytes(ctypes.byref(cfg)))


def decode(q, coarse, fine, meta, sink_k, sink_v, open_k, open_v, scratch, tokens, capacity, kv_heads, format, scale=0.0, tau=0.0):
    if q.dim() != 3 or q.size(2) != 128:
        raise ValueError(f"q must be [batch, q_heads, 128], got {tuple(q.shape)}")
    dev = q.device
    _tensor(q, dev, torch.bfloat16, "q")
    for x in (coarse, fine):
        _tensor(x, dev, torch.uint8, "packed cache records")
    for x in (meta, sink_k, sink_v, open_k, open_v):
        _tensor(x, dev, torch.bfloat16, "cache metadata / exact group")
    _tensor(scratch, dev, torch.uint8, "scratch")
    cfg = _config(q.size(0), q.size(1), kv_heads, tokens, format, capacity, scale, tau)
    cache = _cache(coarse, fine, meta, sink_k, sink_v, open_k, open_v)
    out = torch.empty_like(q)
    with torch.cuda.device(dev):
        st = _lib.mlops_fbla_decode(ctypes.byref(cfg), q.data_ptr(), ctypes.byref(cache), out.data_ptr(), scratch.data_ptr(),
                                    scratch.numel(), _stream(dev))
    _raise(st, "mlops_fbla_decode")
    return out


def prefill(q, k, v, coarse, fine, meta, sink_k, sink_v, open_k, open_v, tokens, capacity, q_heads, format, scale=0.0, images=None):
    """Appends k / v [B, Hkv, n, 128] to the cache holding `tokens`; with q [B, Hq, n, 128] returns the attention of
    every new position (None for q None: append only)."""
    if k.dim() != 4 or k.size(3) != 128 or v.shape != k.shape:
        raise ValueError(f"k and v must be [batch, kv_heads, n, 128], got {tuple(k.shape)} and {tuple(v.shape)}")
    dev = k.device
    _tensor(k, dev, torch.bfloat16, "k")
    _tensor(v, dev, torch.bfloat16, "v")
    for x in (coarse, fine):
        _tensor(x, dev, torch.uint8, "packed cache records")
    for x in (meta, sink_k, sink_v, open_k, open_v):
        _tensor(x, dev, torch.bfloat16, "cache metadata / exact group")
    B, Hkv, n = k.size(0), k.size(1), k.size(2)
    if q is not None:
        if q.dim() != 4 or q.size(0) != B or q.size(1) != q_heads or q.size(2) != n or q.size(3) != 128:
            raise ValueError(f"q must be [batch, q_heads, n, 128] matching k, got {tuple(q.shape)}")
        _tensor(q, dev, torch.bfloat16, "q")
    cfg = _config(B, q_heads, Hkv, tokens, format, capacity, scale, 0.0)
    cache = _cache(coarse, fine, meta, sink_k, sink_v, open_k, open_v, images)
    out = torch.empty_like(q) if q is not None else None
    with torch.cuda.device(dev):
        st = _lib.mlops_fbla_prefill(ctypes.byref(cfg), int(n), q.data_ptr() if q is not None else None, k.data_ptr(), v.data_ptr(),
                                     ctypes.byref(cache), out.data_ptr() if out is not None else None, _stream(dev))
    _raise(st, "mlops_fbla_prefill")
    return out
