"""Parity at BASELINE's full sizes, and the layout options of the C API (strided units, strided outputs).

Full sizes: decode configs[1] (batch 8, 32q/8kv, ctx 16 384, 4+2) against the CPU oracle on every row and against the
reference's CUDA library; prefill with configs[3]'s shape (one of its four sequences: 32q/8kv, 8 192 tokens, 4+2)
against the oracle on sampled positions and through a size-independent property (one 8 192-token chunk == four
2 048-token chunks: the same cache bytes, outputs within tolerance of each other).
Layout options follow attention/fbla/tests/test_fbla.cu:874-957 (units of several layers side by side; token-major
prefill output)."""
import ctypes
import os

import numpy as np
import pytest
import torch

from tests import datagen
from tests import gpu_util as gu

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ours():
    assert os.path.exists(gu.OURS)
    return gu.CLib(gu.OURS)


@pytest.fixture(scope="module")
def ref():
    return gu.CLib(gu.REF) if os.path.exists(gu.REF) else None


def test_decode_configs1_full_size(ours, ref, oracle):
    B, QH, KH, N, mode = 8, 32, 8, 16384, "4+2"
    q, k, v = datagen.baseline_case(1002, B, QH, KH, N, outliers=True)
    qd, kd, vd = gu.bf16_tensor(q), gu.bf16_tensor(k), gu.bf16_tensor(v)
    c = ours.encode(kd, vd, mode)
    out = ours.decode(c, qd)
    torch.cuda.synchronize()
    o = oracle.encode(k, v, mode)
    gu.assert_cache_equal(c, o, "configs[1] cache")
    want, stats = oracle.decode(q, o, stats=True)
    gu.check_close(gu.bits_of(out), want, "configs[1] decode")
    assert 0.5 < stats[3] / stats[2] < 0.95  # the refined share of this input (0.776): both passes are exercised at scale
    if ref is not None:
        a = datagen.bf16_to_f32(gu.bits_of(out)).astype(np.float64)
        b = datagen.bf16_to_f32(gu.bits_of(ref.decode(c, qd))).astype(np.float64)
        assert (np.abs(a - b) <= 2e-3 * np.abs(b).max() + gu.bf16_ulp(b)).all()


def test_prefill_configs3_shape(ours, oracle):
    B, QH, KH, S, mode = 1, 32, 8, 8192, "4+2"
    q, k, v = datagen.baseline_case(1004, B, QH, KH, S, q_rows=S, outliers=True)
    qd, kd, vd = gu.bf16_tensor(q), gu.bf16_tensor(k), gu.bf16_tensor(v)
    one = ours.empty(B, KH, S, mode)
    out1 = ours.prefill(one, kd, vd, qd)
    four = ours.empty(B, KH, S, mode)
    outs = [ours.prefill(four, kd[:, :, t:t + 2048].contiguous(), vd[:, :, t:t + 2048].contiguous(), qd[:, :, t:t + 2048].contiguous())
            for t in range(0, S, 2048)]
    torch.cuda.synchronize()
    assert ctypes.CDLL(gu.OURS).fbla_k_attend_tc_status() == 0
    gu.assert_cache_equal(one, gu.cache_to_numpy(four), "one chunk == four chunks")
    a = datagen.bf16_to_f32(gu.bits_of(out1)).astype(np.float64)
    b = datagen.bf16_to_f32(gu.bits_of(torch.cat(outs, 2))).astype(np.float64)
    for pos in range(0, S, 97):  # per position: the output scale shrinks along the sequence
        assert (np.abs(a[:, :, pos] - b[:, :, pos]) <= 2e-3 * np.abs(b[:, :, pos]).max() + gu.bf16_ulp(b[:, :, pos])).all(), pos
    step = 683  # 12 sampled positions through the oracle's float64 model
    want = oracle.prefill(q, k, v, oracle.empty(B, KH, S, mode), pos_step=step)
    idx = np.arange(0, S, step)
    for i in idx:
        gu.check_close(gu.bits_of(out1)[:, :, i], want[:, :, i], f"configs[3] prefill position {i}")


@pytest.mark.parametrize("mode", ["3+3", "4+2"])
def test_units_of_three_layers_side_by_side(ours, mode):
    """head_stride 1, group_stride 3 * heads: the units of three layers interleaved in one allocation; layer 1 is used.
    Records, metadata and outputs equal the dense layout's."""
    B, QH, KH, N, cap, layers, layer = 2, 8, 2, 700, 1024, 3, 1
    cb, fb, fmt = gu.FORMATS[mode]
    heads, cg = B * KH, cap // 128
    q, k, v = datagen.uneven_case(71, B, QH, KH, N, q_rows=N)
    qd, kd, vd = gu.bf16_tensor(q), gu.bf16_tensor(k), gu.bf16_tensor(v)
    dense = ours.empty(B, KH, cap, mode)
    want_pre = ours.prefill(dense, kd, vd, qd)
    want_dec = ours.decode(dense, qd[:, :, -1].contiguous())
    units = cg * layers * heads
    big = dict(coarse=torch.zeros((units, 8, 2 * cb * 256), dtype=torch.uint8, device="cuda"),
               fine=torch.zeros((units, 8, 2 * fb * 256), dtype=torch.uint8, device="cuda"),
               meta=torch.zeros((units, 512), dtype=torch.bfloat16, device="cuda"))
    win = {n: torch.zeros((B, KH, 128, 128), dtype=torch.bfloat16, device="cuda") for n in ("sink_k", "sink_v", "open_k", "open_v")}
    first = layer * heads  # unit of (head 0, group 0) of the layer: (g * layers + layer) * heads + h
    kc = gu.Cache(big["coarse"][first:].data_ptr(), big["fine"][first:].data_ptr(), big["meta"][first:].data_ptr(), win["sink_k"].data_ptr(),
                  win["sink_v"].data_ptr(), win["open_k"].data_ptr(), win["open_v"].data_ptr(), None)
    cfg = gu.Config(B, QH, KH, 0, 0, 0, fmt, cap, 1, layers * heads, 0, 0, 0)
    out = torch.empty_like(qd)
    st = ours.lib.mlops_fbla_prefill(ctypes.byref(cfg), N, qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), ctypes.byref(kc), out.data_ptr(), None)
    assert st == 0, ours.error()
    cfg.tokens = N
    nbytes = ours.lib.mlops_fbla_decode_scratch_bytes(ctypes.byref(cfg))
    scratch = torch.full((nbytes,), 0xFF, dtype=torch.uint8, device="cuda")
    dec = torch.empty((B, QH, 128), dtype=torch.bfloat16, device="cuda")
    st = ours.lib.mlops_fbla_decode(ctypes.byref(cfg), qd[:, :, -1].contiguous().data_ptr(), ctypes.byref(kc), dec.data_ptr(), scratch.data_ptr(),
                                    ctypes.c_size_t(nbytes), None)
    assert st == 0, ours.error()
    torch.cuda.synchronize()
    assert torch.equal(out, want_pre) and torch.equal(dec, want_dec)
    closed = (N - 1) // 128  # groups 0 .. closed - 1 hold records
    for h in range(heads):
        for g in range(closed):
            u = (g * layers + layer) * heads + h
            assert torch.equal(big["coarse"][u], dense["coarse"].reshape(heads, cg, 8, -1)[h, g])
            assert torch.equal(big["fine"][u], dense["fine"].reshape(heads, cg, 8, -1)[h, g])
            assert torch.equal(big["meta"][u], dense["meta"].reshape(heads, cg, 512)[h, g])
    other = torch.ones(units, dtype=torch.bool)
    other[[(g * layers + layer) * heads + h for g in range(cg) for h in range(heads)]] = False
    assert not big["coarse"][other.cuda()].any() and not big["meta"][other.cuda()].view(torch.int16).any()  # the other layers' units are untouched


@pytest.mark.parametrize("count", [300, 7])
def test_token_major_prefill_output(ours, count):
    """out_head_stride 128, out_token_stride q_heads * 128: [token][head][128], the layout the next projection reads
    (count 300: the tensor-core kernel; 7: the warp-per-row kernel)"""
    QH, KH, cap, mode = 8, 2, 1024, "3+3"
    q, k, v = datagen.uneven_case(72, 1, QH, KH, count, q_rows=count)
    qd, kd, vd = gu.bf16_tensor(q), gu.bf16_tensor(k), gu.bf16_tensor(v)
    want = ours.prefill(ours.empty(1, KH, cap, mode), kd, vd, qd)  # [1, QH, count, 128]
    c = ours.empty(1, KH, cap, mode)
    cfg = gu.Config(1, QH, KH, 0, 0, 0, gu.FORMATS[mode][2], cap, 0, 0, 128, QH * 128, 0)
    out = torch.full((count, QH, 128), -2.0, dtype=torch.bfloat16, device="cuda")
    kc = ours._cache(c)
    st = ours.lib.mlops_fbla_prefill(ctypes.byref(cfg), count, qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), ctypes.byref(kc), out.data_ptr(), None)
    assert st == 0, ours.error()
    torch.cuda.synchronize()
    assert torch.equal(out.permute(1, 0, 2), want[0])
    cfg = gu.Config(2, QH, KH, 0, 0, 0, gu.FORMATS[mode][2], cap, 0, 0, 128, QH * 128, 0)  # strided outputs are for batch 1
    assert ours.lib.mlops_fbla_prefill(ctypes.byref(cfg), count, qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), ctypes.byref(kc), out.data_ptr(), None) == 1
