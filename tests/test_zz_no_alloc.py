"""mlops_fbla_decode_static: the decode entry point for callers that cannot allocate device memory (an engine whose
allocator is closed after start-up, a plugin host that forbids cudaMalloc, a real-time loop that must stay out of the
allocator). It runs the usual decode passes on a 32 MiB scratch array that is part of the library image instead of a
caller-provided buffer. Checked here through the C ABI against mlops_fbla_decode on the same cache and queries, on two
calls in a row (the array keeps the previous call's contents, which must not matter: the outputs are compared bit for
bit), that a warmed-up call leaves the device's free memory unchanged, and the size limit.
This file is collected last on purpose: a run that stops at the first failure has then already run every other test."""
import ctypes

import numpy as np
import pytest
import torch

from tests import datagen
from tests import gpu_util as gu

pytestmark = pytest.mark.gpu


def _static_decode(lib, c, q, tau=0.0):
    L = lib.lib
    L.mlops_fbla_decode_static.restype = ctypes.c_int
    L.mlops_fbla_decode_static.argtypes = [ctypes.POINTER(gu.Config), ctypes.c_void_p, ctypes.POINTER(gu.Cache), ctypes.c_void_p, ctypes.c_void_p]
    L.mlops_fbla_decode_static_error.restype = ctypes.c_char_p
    cfg = gu.Config(c["batch"], q.shape[1], c["kv_heads"], c["tokens"], 0.0, tau, gu.FORMATS[c["mode"]][2], c["capacity"], 0, 0, 0, 0, 0)
    out = torch.empty_like(q)
    kc = lib._cache(c)
    st = L.mlops_fbla_decode_static(ctypes.byref(cfg), q.data_ptr(), ctypes.byref(kc), out.data_ptr(),
                                    ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return st, out, L.mlops_fbla_decode_static_error().decode()


@pytest.mark.parametrize("mode", ["3+3", "4+2"])
def test_static_scratch_decode_matches_decode(mode):
    lib = gu.CLib(gu.OURS)
    lib.lib.mlops_fbla_decode_static_prepare.restype = ctypes.c_int
    assert lib.lib.mlops_fbla_decode_static_prepare() == 0  # (the start-up call: module load and address look-up, no launch)
    q, k, v = datagen.baseline_case(1001, 1, 16, 8, 4096)
    qd, kd, vd = gu.bf16_tensor(q), gu.bf16_tensor(k), gu.bf16_tensor(v)
    c = lib.encode(kd, vd, mode)
    want = lib.decode(c, qd)
    # a second, different decode in between leaves other contents in the shared array
    q2, k2, v2 = datagen.uneven_case(3, 2, 8, 2, 3000)
    qd2 = gu.bf16_tensor(q2)
    c2 = lib.encode(gu.bf16_tensor(k2), gu.bf16_tensor(v2), mode)
    want2 = lib.decode(c2, qd2, tau=1e-3)
    for call in range(2):
        st, out, err = _static_decode(lib, c, qd)
        assert st == 0, err
        st2, out2, err2 = _static_decode(lib, c2, qd2, tau=1e-3)
        assert st2 == 0, err2
        torch.cuda.synchronize()
        # Same kernels, same layout, and every scratch word is written before it is read: the bits must be those of
        # mlops_fbla_decode. A looser bound would let a read of the previous call's leftovers slip through.
        assert torch.equal(out, want) and torch.equal(out2, want2), call
    # the property the entry point exists for: a warmed-up call takes no device memory
    L = lib.lib
    cfg = gu.Config(c["batch"], qd.shape[1], c["kv_heads"], c["tokens"], 0.0, 0.0, gu.FORMATS[c["mode"]][2], c["capacity"], 0, 0, 0, 0, 0)
    kc = lib._cache(c)
    free_before = torch.cuda.mem_get_info()[0]
    st = L.mlops_fbla_decode_static(ctypes.byref(cfg), qd.data_ptr(), ctypes.byref(kc), out.data_ptr(), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert st == 0 and torch.cuda.mem_get_info()[0] == free_before, "the static-scratch decode changed the device's free memory"
    assert torch.equal(out, want)


def test_static_scratch_rejects_large_configurations():
    lib = gu.CLib(gu.OURS)
    lib.lib.mlops_fbla_decode_static_scratch_limit.restype = ctypes.c_size_t
    limit = lib.lib.mlops_fbla_decode_static_scratch_limit()
    assert limit == 32 << 20
    q, k, v = datagen.baseline_case(5, 1, 4, 2, 300)
    c = lib.encode(gu.bf16_tensor(k), gu.bf16_tensor(v), "4+2")
    # batch 8 x 8 KV heads at 2^26 tokens: the sub-block masses alone take 4 GiB, far beyond the array; the call must
    # refuse before launching anything (the pointers below are never dereferenced)
    L = lib.lib
    L.mlops_fbla_decode_static.restype = ctypes.c_int
    L.mlops_fbla_decode_static.argtypes = [ctypes.POINTER(gu.Config), ctypes.c_void_p, ctypes.POINTER(gu.Cache), ctypes.c_void_p, ctypes.c_void_p]
    L.mlops_fbla_decode_static_error.restype = ctypes.c_char_p
    cfg = gu.Config(8, 32, 8, 1 << 26, 0.0, 0.0, 1, 0, 0, 0, 0, 0, 0)
    kc = lib._cache(c)
    qd = gu.bf16_tensor(q)
    st = L.mlops_fbla_decode_static(ctypes.byref(cfg), qd.data_ptr(), ctypes.byref(kc), qd.data_ptr(), None)
    err = L.mlops_fbla_decode_static_error().decode()
    assert st == 1 and "scratch" in err and str(limit) in err, (st, err)
    st, _, err = _static_decode(lib, c, gu.bf16_tensor(q))
    assert st == 0 and err == ""
