"""CPU-side checks of the drop-in boundary: the shared library loads, exports every function include/mlops_fbla.h
declares, the structs have the ABI sizes of the reference interface, and argument validation answers as the
reference's host code does (attention/fbla/src/fbla.cu:62-80,193-221,408-430) -- all without a GPU."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "mlops_b200", "lib", "libmlops_attention.so")


@pytest.fixture(scope="module")
def C():
    if not os.path.exists(LIB):
        import __graft_entry__
        __graft_entry__.build()
    from mlops_b200.attention import _C
    return _C


def declared_functions():
    names = set()
    for fn in os.listdir(os.path.join(ROOT, "include")):
        text = open(os.path.join(ROOT, "include", fn)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b(mlops_fbla_\w+)\s*\(", text))
    return sorted(names)


def test_exports_every_declared_function(C):
    names = declared_functions()
    assert len(names) >= 11
    for n in names:
        assert hasattr(C.lib, n), f"{n} is declared in include/ but not exported"


def test_struct_sizes(C):
    assert ctypes.sizeof(C.Config) == 64 and ctypes.sizeof(C.Cache) == 64 and ctypes.sizeof(C.Sizes) == 40
    assert C.Config.scale.offset == 16 and C.Config.format.offset == 24 and C.Config.capacity.offset == 28
    assert C.Config.out_head_stride.offset == 40 and C.Config.length_stride.offset == 56
    from tests import gpu_util
    assert ctypes.sizeof(gpu_util.Token) == 96 and gpu_util.Token.eps.offset == 64 and gpu_util.Token.freq.offset == 72
    assert gpu_util.Token.attention_factor.offset == 80 and gpu_util.Token.q_out.offset == 88


def cfg(C, **kw):
    base = dict(batch=1, q_heads=4, kv_heads=2, tokens=1000, scale=0.0, tau=0.0, format=1, capacity=0, head_stride=0, group_stride=0,
                out_head_stride=0, out_token_stride=0, length_stride=0)
    base.update(kw)
    return C.Config(**base)


def test_cache_sizes(C):
    s = C.Sizes()
    assert C.lib.mlops_fbla_cache_sizes(ctypes.byref(cfg(C)), ctypes.byref(s)) == 1
    assert (s.coarse, s.fine, s.meta, s.exact, s.images) == (2 * 8 * 8 * 2048, 2 * 8 * 8 * 1024, 2 * 8 * 1024, 2 * 128 * 128 * 2, 0)
    assert C.lib.mlops_fbla_cache_sizes(ctypes.byref(cfg(C, format=0, capacity=8192)), ctypes.byref(s)) == 1
    assert (s.coarse, s.fine, s.meta) == (2 * 64 * 8 * 1536, 2 * 64 * 8 * 1536, 2 * 64 * 1024)
    # strided units: 3 layers side by side (head_stride 1, group_stride 3 * heads)
    assert C.lib.mlops_fbla_cache_sizes(ctypes.byref(cfg(C, head_stride=1, group_stride=6)), ctypes.byref(s)) == 1
    assert s.meta == ((2 - 1) * 1 + (8 - 1) * 6 + 1) * 1024
    before = (s.coarse, s.fine)
    for bad in (dict(q_heads=3), dict(format=2), dict(batch=0), dict(tokens=0), dict(capacity=500), dict(head_stride=1)):
        assert C.lib.mlops_fbla_cache_sizes(ctypes.byref(cfg(C, **bad)), ctypes.byref(s)) == 0, bad
    assert (s.coarse, s.fine) == before  # untouched on failure


def test_validation_without_a_device(C):
    """Invalid arguments are rejected before anything touches CUDA, with INVALID_VALUE and a message; the message is
    empty again after a successful call."""
    lib = C.lib
    cache = C.Cache(*([0x1000] * 7), None)
    st = lib.mlops_fbla_decode(ctypes.byref(cfg(C)), None, ctypes.byref(cache), 0x1000, 0x1000, 1 << 30, None)
    assert st == C.INVALID_VALUE and "null" in C.last_error()
    st = lib.mlops_fbla_decode(ctypes.byref(cfg(C, q_heads=3)), 0x1000, ctypes.byref(cache), 0x1000, 0x1000, 1 << 30, None)
    assert st == C.INVALID_VALUE
    st = lib.mlops_fbla_decode(ctypes.byref(cfg(C, tau=-1.0)), 0x1000, ctypes.byref(cache), 0x1000, 0x1000, 1 << 30, None)
    assert st == C.INVALID_VALUE and "tau" in C.last_error()
    st = lib.mlops_fbla_decode(ctypes.byref(cfg(C)), 0x1008, ctypes.byref(cache), 0x1000, 0x1000, 1 << 30, None)
    assert st == C.INVALID_VALUE and "boundar" in C.last_error()
    missing = C.Cache(0x1000, None, *([0x1000] * 5), None)
    st = lib.mlops_fbla_decode(ctypes.byref(cfg(C)), 0x1000, ctypes.byref(missing), 0x1000, 0x1000, 1 << 30, None)
    assert st == C.INVALID_VALUE and "seven arrays" in C.last_error()
    st = lib.mlops_fbla_decode(ctypes.byref(cfg(C, length_stride=1)), 0x1000, ctypes.byref(cache), 0x1000, 0x1000, 1 << 30, None)
    assert st == C.INVALID_VALUE
    # prefill
    p = lambda c, count, q, out: lib.mlops_fbla_prefill(ctypes.byref(c), count, q, 0x1000, 0x1000, ctypes.byref(cache), out, None)
    assert p(cfg(C), 0, None, None) == C.INVALID_VALUE
    assert p(cfg(C, capacity=1001), 2, None, None) == C.INVALID_VALUE          # tokens + count > capacity
    assert p(cfg(C), 1, 0x1000, None) == C.INVALID_VALUE and "output" in C.last_error()
    assert p(cfg(C, out_head_stride=128, out_token_stride=4), 1, 0x1000, 0x1000) == C.INVALID_VALUE
    assert p(cfg(C, batch=2, out_head_stride=128, out_token_stride=512), 1, 0x1000, 0x1000) == C.INVALID_VALUE
    # device-length calls
    st = lib.mlops_fbla_decode_at(ctypes.byref(cfg(C, capacity=2048)), None, 0x1000, ctypes.byref(cache), 0x1000, 0x1000, 1 << 30, None)
    assert st == C.INVALID_VALUE
    st = lib.mlops_fbla_append_at(ctypes.byref(cfg(C)), 0x1000, 0x1000, 0x1000, ctypes.byref(cache), None)
    assert st == C.INVALID_VALUE                                                 # capacity must be positive
    st = lib.mlops_fbla_prefill_at(ctypes.byref(cfg(C, capacity=1003)), 0x1000, 0x1000, 4, None, 0x1000, 0x1000, ctypes.byref(cache), None, None)
    assert st == C.INVALID_VALUE                                                 # tokens + max_count > capacity
    assert lib.mlops_fbla_status_string(1) == b"invalid value"
    # size queries answer 0 for invalid input
    assert lib.mlops_fbla_decode_scratch_bytes(ctypes.byref(cfg(C, q_heads=3))) == 0
    assert lib.mlops_fbla_decode_scratch_bytes_for(ctypes.byref(cfg(C)), 0) == 0  # capacity 0
    assert lib.mlops_fbla_images_bytes(ctypes.byref(cfg(C))) == 0


def test_python_interface_rejects_without_cuda(C):
    import torch
    from mlops_b200 import attention
    k = torch.zeros(1, 2, 10, 128, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        attention.encode(k, k[:, :, :5])
    with pytest.raises(ValueError):
        attention.encode(k, k, "5+1")
    if not torch.cuda.is_available():
        with pytest.raises(ValueError):
            attention.encode(k, k)  # not CUDA tensors


def test_qkv_validation_without_a_device(C):
    from tests import gpu_util
    lib = C.lib
    lib.mlops_fbla_qkv_at.restype = ctypes.c_int
    lib.mlops_fbla_qkv_prefill_at.restype = ctypes.c_int
    cache = C.Cache(*([0x1000] * 7), None)
    tok = gpu_util.Token(0x1000, 0x1000, 0x1000, 1024, 768, 768, None, None, 1e-6, 0x1000, 0.0, 0x1000)
    c = cfg(C, capacity=4096, tokens=0)
    vp = ctypes.c_void_p
    assert lib.mlops_fbla_qkv_at(ctypes.byref(c), None, ctypes.byref(tok), ctypes.byref(cache), None) == C.INVALID_VALUE and "null" in C.last_error()
    tok.q_norm = 0x1000  # one norm weight without the other
    assert lib.mlops_fbla_qkv_at(ctypes.byref(c), vp(0x1000), ctypes.byref(tok), ctypes.byref(cache), None) == C.INVALID_VALUE
    assert "both or neither" in C.last_error()
    tok.q_norm = None
    tok.batch_stride = 1023  # odd stride
    assert lib.mlops_fbla_qkv_at(ctypes.byref(c), vp(0x1000), ctypes.byref(tok), ctypes.byref(cache), None) == C.INVALID_VALUE
    tok.batch_stride = 64  # a chunk row shorter than one head
    st = lib.mlops_fbla_qkv_prefill_at(ctypes.byref(c), vp(0x1000), vp(0x1000), ctypes.c_int(8), ctypes.byref(tok), vp(0x1000), vp(0x1000), vp(0x1000), None)
    assert st == C.INVALID_VALUE and "row" in C.last_error()
    st = lib.mlops_fbla_qkv_prefill_at(ctypes.byref(cfg(C, batch=2, capacity=4096, tokens=0)), vp(0x1000), vp(0x1000), ctypes.c_int(8), ctypes.byref(tok),
                                       vp(0x1000), vp(0x1000), vp(0x1000), None)
    assert st == C.INVALID_VALUE and "batch 1" in C.last_error()
