"""Helpers of the GPU parity tests: drive a library that exports the mlops_fbla C ABI (the product, or the reference
build under oracle/_ref) on torch device tensors, and move caches between numpy (oracle side) and the device."""
import ctypes
import os

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
OURS = os.path.join(ROOT, "mlops_b200", "lib", "libmlops_attention.so")
REF = os.path.join(ROOT, "oracle", "_ref", "libmlops_attention_ref.so")
FORMATS = {"3+3": (3, 3, 0), "4+2": (4, 2, 1)}


class Config(ctypes.Structure):
    _fields_ = [("batch", ctypes.c_int), ("q_heads", ctypes.c_int), ("kv_heads", ctypes.c_int), ("tokens", ctypes.c_int),
                ("scale", ctypes.c_float), ("tau", ctypes.c_float), ("format", ctypes.c_int), ("capacity", ctypes.c_int),
                ("head_stride", ctypes.c_int), ("group_stride", ctypes.c_int),
                ("out_head_stride", ctypes.c_int64), ("out_token_stride", ctypes.c_int64), ("length_stride", ctypes.c_int)]


class Cache(ctypes.Structure):
    _fields_ = [(n, ctypes.c_void_p) for n in ("coarse", "fine", "meta", "sink_k", "sink_v", "open_k", "open_v", "images")]


class Token(ctypes.Structure):
    _fields_ = [("q", ctypes.c_void_p), ("k", ctypes.c_void_p), ("v", ctypes.c_void_p), ("batch_stride", ctypes.c_int64),
                ("q_group_stride", ctypes.c_int64), ("kv_group_stride", ctypes.c_int64), ("q_norm", ctypes.c_void_p), ("k_norm", ctypes.c_void_p),
                ("eps", ctypes.c_float), ("freq", ctypes.c_void_p), ("attention_factor", ctypes.c_float), ("q_out", ctypes.c_void_p)]


def bf16_tensor(bits, device="cuda"):
    """numpy uint16 BF16 bit patterns -> torch bfloat16 tensor on the device"""
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).to(device).view(torch.bfloat16)


def bits_of(t):
    """torch bfloat16 tensor -> numpy uint16 bit patterns"""
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def bf16_ulp(x):
    """spacing of BF16 numbers at |x| (numpy float64 array)"""
    e = np.floor(np.log2(np.maximum(np.abs(x), 1e-38)))
    return np.exp2(e - 7)


class CLib:
    """One loaded library exporting the mlops_fbla C ABI."""

    def __init__(self, path):
        self.path = path
        self.lib = ctypes.CDLL(path)  # RTLD_LOCAL: the product and the reference export the same symbol names
        L = self.lib
        vp, cp, kp = ctypes.c_void_p, ctypes.POINTER(Config), ctypes.POINTER(Cache)
        L.mlops_fbla_decode_scratch_bytes.restype = ctypes.c_size_t
        L.mlops_fbla_decode_scratch_bytes.argtypes = [cp]
        L.mlops_fbla_decode.restype = ctypes.c_int
        L.mlops_fbla_decode.argtypes = [cp, vp, kp, vp, vp, ctypes.c_size_t, vp]
        L.mlops_fbla_decode_at.restype = ctypes.c_int
        L.mlops_fbla_decode_at.argtypes = [cp, vp, vp, kp, vp, vp, ctypes.c_size_t, vp]
        L.mlops_fbla_prefill.restype = ctypes.c_int
        L.mlops_fbla_prefill.argtypes = [cp, ctypes.c_int, vp, vp, vp, kp, vp, vp]
        L.mlops_fbla_prefill_at.restype = ctypes.c_int
        L.mlops_fbla_prefill_at.argtypes = [cp, vp, vp, ctypes.c_int, vp, vp, vp, kp, vp, vp]
        L.mlops_fbla_append_at.restype = ctypes.c_int
        L.mlops_fbla_append_at.argtypes = [cp, vp, vp, vp, kp, vp]
        L.mlops_fbla_last_error.restype = ctypes.c_char_p
        tp = ctypes.POINTER(Token)
        L.mlops_fbla_qkv_at.restype = ctypes.c_int
        L.mlops_fbla_qkv_at.argtypes = [cp, vp, tp, kp, vp]
        L.mlops_fbla_qkv_prefill_at.restype = ctypes.c_int
        L.mlops_fbla_qkv_prefill_at.argtypes = [cp, vp, vp, ctypes.c_int, tp, vp, vp, vp, vp]

    def error(self):
        return self.lib.mlops_fbla_last_error().decode()

    @staticmethod
    def empty(batch, kv_heads, capacity, mode, device="cuda"):
        cb, fb, fmt = FORMATS[mode]
        cg = (capacity + 127) // 128
        z = lambda shape, dt: torch.zeros(shape, dtype=dt, device=device)
        c = dict(coarse=z((batch, kv_heads, cg * 8, 2 * cb * 256), torch.uint8), fine=z((batch, kv_heads, cg * 8, 2 * fb * 256), torch.uint8),
                 meta=z((batch, kv_heads, cg, 512), torch.bfloat16), tokens=0, capacity=capacity, mode=mode, batch=batch, kv_heads=kv_heads)
        for n in ("sink_k", "sink_v", "open_k", "open_v"):
            c[n] = z((batch, kv_heads, 128, 128), torch.bfloat16)
        return c

    @staticmethod
    def _cache(c):
        return Cache(*[c[n].data_ptr() for n in ("coarse", "fine", "meta", "sink_k", "sink_v", "open_k", "open_v")], None)

    def _stream(self):
        return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def prefill(self, c, k, v, q=None, scale=0.0, q_heads=None):
        """k, v [B, Hkv, n, 128] bf16 device tensors appended in place; with q returns [B, Hq, n, 128] bf16."""
        n = k.shape[2]
        qh = q.shape[1] if q is not None else (q_heads or c["kv_heads"])
        cfg = Config(c["batch"], qh, c["kv_heads"], c["tokens"], scale, 0.0, FORMATS[c["mode"]][2], c["capacity"], 0, 0, 0, 0, 0)
        out = torch.empty_like(q) if q is not None else None
        kc = self._cache(c)
        st = self.lib.mlops_fbla_prefill(ctypes.byref(cfg), n, q.data_ptr() if q is not None else None, k.data_ptr(), v.data_ptr(),
                                         ctypes.byref(kc), out.data_ptr() if out is not None else None, self._stream())
        if st:
            raise RuntimeError(f"prefill status {st}: {self.error()}")
        c["tokens"] += n
        return out

    def encode(self, k, v, mode, capacity=None):
        B, H, N, _ = k.shape
        c = self.empty(B, H, N if capacity is None else capacity, mode, k.device)
        self.prefill(c, k, v)
        return c

    def scratch(self, c, q_heads, poison=0xFF):
        cfg = Config(c["batch"], q_heads, c["kv_heads"], c["tokens"], 0, 0, FORMATS[c["mode"]][2], c["capacity"], 0, 0, 0, 0, 0)
        n = self.lib.mlops_fbla_decode_scratch_bytes(ctypes.byref(cfg))
        assert n > 0, self.error()
        return torch.full((n,), poison, dtype=torch.uint8, device=c["coarse"].device)

    def decode(self, c, q, scale=0.0, tau=0.0, scratch=None):
        """q [B, Hq, 128] bf16 -> [B, Hq, 128] bf16"""
        cfg = Config(c["batch"], q.shape[1], c["kv_heads"], c["tokens"], scale, tau, FORMATS[c["mode"]][2], c["capacity"], 0, 0, 0, 0, 0)
        if scratch is None:
            scratch = self.scratch(c, q.shape[1])
        out = torch.empty_like(q)
        kc = self._cache(c)
        st = self.lib.mlops_fbla_decode(ctypes.byref(cfg), q.data_ptr(), ctypes.byref(kc), out.data_ptr(), scratch.data_ptr(),
                                        scratch.numel(), self._stream())
        if st:
            raise RuntimeError(f"decode status {st}: {self.error()}")
        self.last_scratch = scratch
        return out


    # ---- device-length calls ----------------------------------------------------------------------------------------
    def decode_at(self, c, q, length, tokens_offset=0, scale=0.0, tau=0.0, scratch=None, length_stride=0, out=None):
        """length: int32 device tensor (one entry, or one per batch row with length_stride 1); the cache length is
        length + tokens_offset; c['capacity'] sets the layout."""
        cfg = Config(c["batch"], q.shape[1], c["kv_heads"], tokens_offset, scale, tau, FORMATS[c["mode"]][2], c["capacity"], 0, 0, 0, 0, length_stride)
        if scratch is None:
            cap = Config(c["batch"], q.shape[1], c["kv_heads"], c["capacity"], 0, 0, FORMATS[c["mode"]][2], c["capacity"], 0, 0, 0, 0, 0)
            n = self.lib.mlops_fbla_decode_scratch_bytes(ctypes.byref(cap))
            scratch = torch.full((n,), 0xFF, dtype=torch.uint8, device=q.device)
        out = torch.empty_like(q) if out is None else out
        kc = self._cache(c)
        st = self.lib.mlops_fbla_decode_at(ctypes.byref(cfg), length.data_ptr(), q.data_ptr(), ctypes.byref(kc), out.data_ptr(),
                                           scratch.data_ptr(), scratch.numel(), self._stream())
        if st:
            raise RuntimeError(f"decode_at status {st}: {self.error()}")
        self.last_scratch = scratch
        return out

    def append_at(self, c, k, v, length, tokens_offset=0, length_stride=0):
        """k, v [B, Hkv, 128]: one token per KV head at position length + tokens_offset (the caller advances length)."""
        cfg = Config(c["batch"], c["kv_heads"], c["kv_heads"], tokens_offset, 0, 0, FORMATS[c["mode"]][2], c["capacity"], 0, 0, 0, 0, length_stride)
        kc = self._cache(c)
        st = self.lib.mlops_fbla_append_at(ctypes.byref(cfg), length.data_ptr(), k.data_ptr(), v.data_ptr(), ctypes.byref(kc), self._stream())
        if st:
            raise RuntimeError(f"append_at status {st}: {self.error()}")

    @staticmethod
    def _token(proj, q_heads, kv_heads, row_stride, q_norm, k_norm, eps, freq, att, q_out):
        """proj: the projection's rows, per row [kv_heads][(qg + 2) * 128] = a KV head's q heads, then k, then v"""
        qg = q_heads // kv_heads
        base = proj.data_ptr()
        return Token(base, base + 2 * qg * 128, base + 2 * (qg + 1) * 128, row_stride, (qg + 2) * 128, (qg + 2) * 128,
                     q_norm.data_ptr() if q_norm is not None else None, k_norm.data_ptr() if k_norm is not None else None, eps, freq.data_ptr(),
                     att, q_out.data_ptr() if q_out is not None else None)

    def qkv_at(self, c, proj, q_heads, length, freq, q_norm=None, k_norm=None, eps=1e-6, att=0.0, tokens_offset=0, length_stride=0):
        """proj [B, kv_heads * (qg + 2) * 128] bf16 (one token per sequence); returns q_out [B, q_heads, 128]; appends k, v."""
        B, kvh = c["batch"], c["kv_heads"]
        q_out = torch.empty((B, q_heads, 128), dtype=torch.bfloat16, device=proj.device)
        cfg = Config(B, q_heads, kvh, tokens_offset, 0, 0, FORMATS[c["mode"]][2], c["capacity"], 0, 0, 0, 0, length_stride)
        tok = self._token(proj, q_heads, kvh, proj.shape[1], q_norm, k_norm, eps, freq, att, q_out)
        kc = self._cache(c)
        st = self.lib.mlops_fbla_qkv_at(ctypes.byref(cfg), length.data_ptr(), ctypes.byref(tok), ctypes.byref(kc), self._stream())
        if st:
            raise RuntimeError(f"qkv_at status {st}: {self.error()}")
        return q_out

    def qkv_prefill_at(self, proj, q_heads, kv_heads, length, count, max_count, capacity, freq, q_norm=None, k_norm=None, eps=1e-6, att=0.0,
                       tokens_offset=0, fill=None):
        """proj [rows, kv_heads * (qg + 2) * 128] bf16; returns (q [q_heads, max_count, 128], k, v [kv_heads, max_count, 128])."""
        def mk(h):
            shape, kw = (h, max_count, 128), dict(dtype=torch.bfloat16, device=proj.device)
            return torch.empty(shape, **kw) if fill is None else torch.full(shape, fill, **kw)
        q_out, k_out, v_out = mk(q_heads), mk(kv_heads), mk(kv_heads)
        cfg = Config(1, q_heads, kv_heads, tokens_offset, 0, 0, 0, capacity, 0, 0, 0, 0, 0)
        tok = self._token(proj, q_heads, kv_heads, proj.shape[1], q_norm, k_norm, eps, freq, att, None)
        st = self.lib.mlops_fbla_qkv_prefill_at(ctypes.byref(cfg), length.data_ptr(), count.data_ptr(), max_count, ctypes.byref(tok),
                                                q_out.data_ptr(), k_out.data_ptr(), v_out.data_ptr(), self._stream())
        if st:
            raise RuntimeError(f"qkv_prefill_at status {st}: {self.error()}")
        return q_out, k_out, v_out

    def prefill_at(self, c, k, v, q, length, count, max_count, tokens_offset=0, out=None):
        """k, v [B, Hkv, max_count, 128], q [B, Hq, max_count, 128] or None; the chunk is their first *count positions."""
        qh = q.shape[1] if q is not None else c["kv_heads"]
        cfg = Config(c["batch"], qh, c["kv_heads"], tokens_offset, 0, 0, FORMATS[c["mode"]][2], c["capacity"], 0, 0, 0, 0, 0)
        if q is not None and out is None:
            out = torch.empty_like(q)
        kc = self._cache(c)
        st = self.lib.mlops_fbla_prefill_at(ctypes.byref(cfg), length.data_ptr(), count.data_ptr(), max_count,
                                            q.data_ptr() if q is not None else None, k.data_ptr(), v.data_ptr(), ctypes.byref(kc),
                                            out.data_ptr() if out is not None else None, self._stream())
        if st:
            raise RuntimeError(f"prefill_at status {st}: {self.error()}")
        return out


def cache_to_numpy(c):
    """device cache -> the oracle's numpy layout (heads flattened)"""
    B, H = c["batch"], c["kv_heads"]
    out = dict(tokens=c["tokens"], capacity=c["capacity"], mode=c["mode"], batch=B, kv_heads=H)
    out["coarse"] = c["coarse"].cpu().numpy().reshape(B * H, -1, c["coarse"].shape[-1])
    out["fine"] = c["fine"].cpu().numpy().reshape(B * H, -1, c["fine"].shape[-1])
    out["meta"] = bits_of(c["meta"]).reshape(B * H, -1, 512)
    for n in ("sink_k", "sink_v", "open_k", "open_v"):
        out[n] = bits_of(c[n]).reshape(B * H, 128, 128)
    return out


def assert_cache_equal(dev_cache, np_cache, what=""):
    got = cache_to_numpy(dev_cache)
    for key in ("meta", "coarse", "fine", "sink_k", "sink_v", "open_k", "open_v"):
        a, b = got[key], np_cache[key].reshape(got[key].shape)
        if not np.array_equal(a, b):
            bad = np.argwhere(a != b)
            raise AssertionError(f"{what} {key}: {len(bad)} differing elements, first at {bad[0].tolist()}: {a[tuple(bad[0])]} vs {b[tuple(bad[0])]}")


def check_close(got_bf16_bits, want64, what="", tol=2e-3):
    """The acceptance rule for attention outputs: |bf16(ours) - oracle| <= tol * max|oracle| + the output's own rounding,
    half a BF16 ulp of the element (of the larger of the two magnitudes: a value that rounds up across a power of two
    is rounded on the coarser grid), where the oracle value is the unrounded float64 model."""
    from tests import datagen
    got = datagen.bf16_to_f32(got_bf16_bits).astype(np.float64).reshape(want64.shape)
    scale = np.abs(want64).max()
    err = np.abs(got - want64)
    bound = tol * scale + 0.5 * bf16_ulp(np.maximum(np.abs(want64), np.abs(got)))
    worst = (err - bound).max()
    rel = err.max() / scale
    if worst > 0:
        i = np.unravel_index(np.argmax(err - bound), err.shape)
        raise AssertionError(f"{what}: max|err| / max|ref| = {rel:.3e} exceeds {tol:g} (+ half ulp) by {worst:.3e} at {i}: got {got[i]!r}, want {want64[i]!r}, "
                             f"scale {scale!r}")
    return rel
