"""ctypes front end of the CPU oracle (oracle/fbla_oracle.c). TEST INFRASTRUCTURE: imported only by tests/, by
__graft_entry__.smoke() and by bench.py's cpu_baseline / reference legs; the product never imports it.

Arrays are numpy: BF16 tensors as uint16 bit patterns, packed planes as uint8. A cache is a dict with the keys
coarse, fine, meta, sink_k, sink_v, open_k, open_v (+ tokens, capacity, format, batch, kv_heads).
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

FORMATS = {"3+3": (3, 3, 0), "4+2": (4, 2, 1)}


class Config(ctypes.Structure):
    """Mirror of mlops_fbla_config (include/mlops_fbla.h), 64 bytes."""
    _fields_ = [("batch", ctypes.c_int), ("q_heads", ctypes.c_int), ("kv_heads", ctypes.c_int), ("tokens", ctypes.c_int),
                ("scale", ctypes.c_float), ("tau", ctypes.c_float), ("format", ctypes.c_int), ("capacity", ctypes.c_int),
                ("head_stride", ctypes.c_int), ("group_stride", ctypes.c_int),
                ("out_head_stride", ctypes.c_int64), ("out_token_stride", ctypes.c_int64),
                ("length_stride", ctypes.c_int)]


def build():
    """Compile the oracle with the Makefile beside it (gcc, a few seconds)."""
    subprocess.run(["make", "-C", _HERE, "libfbla_oracle.so"], check=True, stdout=subprocess.DEVNULL)


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "libfbla_oracle.so")
        if not os.path.exists(path):
            build()
        _LIB = ctypes.CDLL(path)
        _LIB.fbla_oracle_threads.restype = ctypes.c_int
    return _LIB


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def threads():
    return lib().fbla_oracle_threads()


def set_threads(n):
    """Let the oracle's parallel loops use n threads (overrides an inherited OMP_NUM_THREADS)."""
    lib().fbla_oracle_set_threads(ctypes.c_int(int(n)))


def quantize_group(x_bits):
    """x_bits [n, 128] uint16 (BF16) -> base, step [128] uint16, code [n, 128] uint8."""
    x = np.ascontiguousarray(x_bits, dtype=np.uint16)
    n = x.shape[0]
    base, step = np.zeros(128, np.uint16), np.zeros(128, np.uint16)
    code = np.zeros((n, 128), np.uint8)
    lib().fbla_oracle_quantize_group(_p(x), ctypes.c_int(n), ctypes.c_int(128), _p(base), _p(step), _p(code))
    return base, step, code


def pack_record(bits, kpart, vpart):
    """kpart, vpart [16, 128] uint8 plane values -> record bytes [2 * bits * 256]."""
    rec = np.zeros(2 * bits * 256, np.uint8)
    lib().fbla_oracle_pack_record(ctypes.c_int(bits), _p(np.ascontiguousarray(kpart, np.uint8)),
                                  _p(np.ascontiguousarray(vpart, np.uint8)), _p(rec))
    return rec


def unpack_record(bits, rec):
    k, v = np.zeros((16, 128), np.uint8), np.zeros((16, 128), np.uint8)
    lib().fbla_oracle_unpack_record(ctypes.c_int(bits), _p(np.ascontiguousarray(rec, np.uint8)), _p(k), _p(v))
    return k, v


def config(batch, q_heads, kv_heads, tokens, mode, capacity=0, scale=0.0, tau=0.0, head_stride=0, group_stride=0):
    return Config(batch, q_heads, kv_heads, tokens, scale, tau, FORMATS[mode][2], capacity, head_stride, group_stride, 0, 0, 0)


def empty(batch, kv_heads, capacity, mode):
    cb, fb, fmt = FORMATS[mode]
    cg = (capacity + 127) // 128
    heads = batch * kv_heads
    ex = lambda: np.zeros((heads, 128, 128), np.uint16)
    return dict(coarse=np.zeros((heads, cg * 8, 2 * cb * 256), np.uint8), fine=np.zeros((heads, cg * 8, 2 * fb * 256), np.uint8),
                meta=np.zeros((heads, cg, 512), np.uint16), sink_k=ex(), sink_v=ex(), open_k=ex(), open_v=ex(),
                tokens=0, capacity=capacity, mode=mode, batch=batch, kv_heads=kv_heads)


def append(cache, k_bits, v_bits):
    """k_bits, v_bits [batch, kv_heads, n, 128] uint16: appended in place (groups closed on the way)."""
    k = np.ascontiguousarray(k_bits, np.uint16)
    v = np.ascontiguousarray(v_bits, np.uint16)
    n = k.shape[2]
    c = cache
    cfg = config(c["batch"], c["kv_heads"], c["kv_heads"], c["tokens"], c["mode"], c["capacity"])
    rc = lib().fbla_oracle_append(ctypes.byref(cfg), ctypes.c_int(n), _p(k), _p(v), _p(c["coarse"]), _p(c["fine"]), _p(c["meta"]),
                                  _p(c["sink_k"]), _p(c["sink_v"]), _p(c["open_k"]), _p(c["open_v"]))
    if rc:
        raise RuntimeError("fbla_oracle_append failed")
    c["tokens"] += n
    return c


def encode(k_bits, v_bits, mode, capacity=None):
    B, H, N, _ = k_bits.shape
    c = empty(B, H, N if capacity is None else capacity, mode)
    return append(c, k_bits, v_bits)


def decode(q_bits, cache, scale=0.0, tau=0.0, lengths=None, stats=False):
    """q_bits [batch, q_heads, 128] uint16 -> float64 [batch, q_heads, 128] (unrounded)."""
    q = np.ascontiguousarray(q_bits, np.uint16)
    c = cache
    cfg = config(q.shape[0], q.shape[1], c["kv_heads"], c["tokens"], c["mode"], c["capacity"], scale, tau)
    out = np.zeros(q.shape, np.float64)
    st = np.zeros(4, np.int64)
    ln = None if lengths is None else np.ascontiguousarray(lengths, np.int32)
    rc = lib().fbla_oracle_decode(ctypes.byref(cfg), _p(ln), _p(q), _p(c["coarse"]), _p(c["fine"]), _p(c["meta"]), _p(c["sink_k"]),
                                  _p(c["sink_v"]), _p(c["open_k"]), _p(c["open_v"]), _p(out), _p(st))
    if rc:
        raise RuntimeError("fbla_oracle_decode failed")
    return (out, st) if stats else out


def prefill(q_bits, k_bits, v_bits, cache, scale=0.0, pos_first=0, pos_step=1):
    """Appends the chunk and returns the float64 attention of its sampled positions [batch, q_heads, n, 128]
    (positions not sampled are NaN). Order as the kernels': close the chunk's groups, attend, update the windows."""
    q = np.ascontiguousarray(q_bits, np.uint16)
    k = np.ascontiguousarray(k_bits, np.uint16)
    v = np.ascontiguousarray(v_bits, np.uint16)
    c = cache
    n = k.shape[2]
    old = {x: c[x].copy() for x in ("sink_k", "sink_v", "open_k", "open_v")}
    tokens0 = c["tokens"]
    append(c, k, v)
    cfg = config(q.shape[0], q.shape[1], c["kv_heads"], tokens0, c["mode"], c["capacity"], scale)
    out = np.full(q.shape, np.nan, np.float64)
    rc = lib().fbla_oracle_prefill(ctypes.byref(cfg), ctypes.c_int(n), _p(q), _p(k), _p(v), _p(c["coarse"]), _p(c["fine"]), _p(c["meta"]),
                                   _p(old["sink_k"]), _p(old["sink_v"]), _p(old["open_k"]), _p(old["open_v"]),
                                   ctypes.c_int(pos_first), ctypes.c_int(pos_step), _p(out))
    if rc:
        raise RuntimeError("fbla_oracle_prefill failed")
    return out


def exact_decode(q_bits, k_bits, v_bits, scale=None):
    """float64 softmax attention of the last position over BF16 K/V: q [B, Hq, 128], k/v [B, Hkv, N, 128]."""
    B, Hq, _ = q_bits.shape
    _, Hk, N, _ = k_bits.shape
    out = np.zeros((B, Hq, 128), np.float64)
    sc = ctypes.c_float(1.0 / np.sqrt(128.0) if scale is None else scale)
    for b in range(B):
        lib().fbla_oracle_exact_decode(ctypes.c_int(Hq), ctypes.c_int(Hq // Hk), ctypes.c_int(N), sc,
                                       _p(np.ascontiguousarray(q_bits[b])), _p(np.ascontiguousarray(k_bits[b])),
                                       _p(np.ascontiguousarray(v_bits[b])), _p(out[b]))
    return out


def rope_freq(theta=1e6, n=64):
    """The 64 x 4 float table of the rotary frequencies inv_freq = theta^(-2 i / 128), split as the kernels take them."""
    inv = np.asarray([theta ** (-2.0 * i / (2 * n)) for i in range(n)], np.float64)
    out = np.zeros((n, 4), np.float32)
    lib().fbla_oracle_rope_freq(_p(inv), ctypes.c_int(n), _p(out))
    return out


def norm_rope(x_bits, w_bits, eps, pos, freq, att=1.0):
    """x_bits [..., 128] uint16 (BF16) -> the head after the optional RMSNorm (w_bits 128 BF16 or None) and the rotation at
    position pos (an int, or an array broadcastable to x's leading shape)."""
    x = np.ascontiguousarray(x_bits, np.uint16)
    out = np.zeros_like(x)
    flat_x, flat_o = x.reshape(-1, 128), out.reshape(-1, 128)
    posv = np.broadcast_to(np.asarray(pos, np.int64), x.shape[:-1]).reshape(-1)
    w = None if w_bits is None else np.ascontiguousarray(w_bits, np.uint16)
    f = np.ascontiguousarray(freq, np.float32)
    fn = lib().fbla_oracle_norm_rope
    fn.restype = None
    for i in range(flat_x.shape[0]):
        fn(_p(flat_x[i]), _p(w), ctypes.c_float(eps), ctypes.c_int(int(posv[i])), _p(f), ctypes.c_float(att), _p(flat_o[i]))
    return out
