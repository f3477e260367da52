"""GPU parity tests (run with -m gpu on a B200): the CUDA library, called through its C ABI, against the CPU oracle on
the same seeded inputs -- packed bytes bit-exact, attention outputs within 2e-3 of the output scale -- and, when the
reference's own CUDA library was built into oracle/_ref, against that library on the same device buffers.
The case list follows the reference's own matrix (attention/fbla/tests/test_fbla.cu:1181-1282,
attention/python/tests/test_attention.py)."""
import ctypes
import os

import numpy as np
import pytest
import torch

from tests import datagen
from tests import gpu_util as gu

pytestmark = pytest.mark.gpu
MODES = ["3+3", "4+2"]


@pytest.fixture(scope="module")
def ours():
    assert os.path.exists(gu.OURS), "build the library first (python -c 'import __graft_entry__ as g; g.build()')"
    return gu.CLib(gu.OURS)


@pytest.fixture(scope="module")
def ref():
    if not os.path.exists(gu.REF):
        pytest.skip("reference CUDA library not built (oracle/build_ref.sh)")
    return gu.CLib(gu.REF)


def _dev(*arrs):
    return [gu.bf16_tensor(a) for a in arrs]


# ---- quantize-on-write ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("B,H,N,cap,chunks,gen,seed", [
    (1, 1, 512, None, [512], "baseline_case", 21),
    (1, 2, 100, None, [100], "uneven_case", 22),
    (2, 2, 2048, None, [300, 212, 128, 1, 1407], "uneven_case", 23),
    (1, 8, 4096, None, [1024, 1024, 2048], "baseline_case", 1001),
    (1, 2, 3000, 8192, [1500, 1500], "uneven_case", 25),
    (1, 2, 8177, None, [6000, 2100, 77], "baseline_case", 28),
    (1, 2, 2000, 2048, [1, 1, 254, 1744], "uneven_case", 27),
    (1, 2, 1280, None, [128, 128, 1024], "baseline_case", 29),
])
def test_cache_bytes_bit_exact(ours, oracle, mode, B, H, N, cap, chunks, gen, seed):
    """Chunked append: every array of the cache equals the oracle's bit for bit after every chunk."""
    _, k, v = getattr(datagen, gen)(seed, B, H, H, N)
    kd, vd = _dev(k, v)
    capacity = N if cap is None else cap
    c = ours.empty(B, H, capacity, mode)
    o = oracle.empty(B, H, capacity, mode)
    t = 0
    for n in chunks:
        ours.prefill(c, kd[:, :, t:t + n].contiguous(), vd[:, :, t:t + n].contiguous())
        oracle.append(o, k[:, :, t:t + n], v[:, :, t:t + n])
        t += n
        torch.cuda.synchronize()
        gu.assert_cache_equal(c, o, f"{mode} after {t} tokens")


def _edge_kv(seed):
    x = datagen.edge_group(seed).copy()
    x[7, 5] = 0x8000                                          # a -0 among +0: the minimum is -0 on the GPU (min.f32 orders signed zeros)
    k = np.concatenate([x, x[:1]])[None, None]                # 129 tokens: the group closes
    v = np.concatenate([x[::-1], x[:1]])[None, None]
    return k, v


def test_quantizer_edge_channels(ours, oracle):
    """Constant, all-negative, zero-minimum, huge, tiny, signed-zero and two-valued channels."""
    for seed in (3, 4):
        k, v = _edge_kv(seed)
        for mode in MODES:
            c = ours.encode(*_dev(k, v), mode)
            gu.assert_cache_equal(c, oracle.encode(k, v, mode), f"edge {seed} {mode}")


def test_quantizer_edge_channels_reference_library(ours, ref):
    for seed in (3, 4):
        k, v = _edge_kv(seed)
        for mode in MODES:
            a, b = ours.encode(*_dev(k, v), mode), ref.encode(*_dev(k, v), mode)
            gu.assert_cache_equal(a, gu.cache_to_numpy(b), f"edge {seed} {mode} vs reference library")


@pytest.mark.parametrize("mode", MODES)
def test_cache_bytes_match_reference_library(ours, ref, mode):
    """The same chunks through the reference's CUDA library on the same device: identical bytes."""
    _, k, v = datagen.baseline_case(1004, 2, 8, 4, 3000)
    kd, vd = _dev(k, v)
    a, b = ours.empty(2, 4, 4096, mode), ref.empty(2, 4, 4096, mode)
    t = 0
    for n in (700, 1, 1299, 1000):
        for lib, c in ((ours, a), (ref, b)):
            lib.prefill(c, kd[:, :, t:t + n].contiguous(), vd[:, :, t:t + n].contiguous())
        t += n
    torch.cuda.synchronize()
    gu.assert_cache_equal(a, gu.cache_to_numpy(b), mode)


@pytest.mark.parametrize("mode", MODES)
def test_append_matches_encode(ours, mode):
    """Token-by-token growth equals a one-shot encode (attention/python/tests/test_attention.py:195-207)."""
    _, k, v = datagen.uneven_case(7, 1, 4, 2, 700)
    kd, vd = _dev(k, v)
    c = ours.encode(kd[:, :, :100].contiguous(), vd[:, :, :100].contiguous(), mode, capacity=1024)
    for t in range(100, 700):
        ours.prefill(c, kd[:, :, t:t + 1].contiguous(), vd[:, :, t:t + 1].contiguous())
        if t in (127, 128, 255, 256, 699):
            e = ours.encode(kd[:, :, :t + 1].contiguous(), vd[:, :, :t + 1].contiguous(), mode, capacity=1024)
            gu.assert_cache_equal(c, gu.cache_to_numpy(e), f"{mode} t={t}")


# ---- decode ----------------------------------------------------------------------------------------------------------------
DECODE_CASES = [  # (batch, q_heads, kv_heads, tokens, tau, seed, capacity, generator)
    (1, 2, 2, 100, 1e-2, 0, None, "uneven_case"),
    (1, 2, 2, 384, 1e-2, 1, None, "uneven_case"),
    (1, 4, 2, 1000, 3e-3, 2, None, "uneven_case"),
    (2, 8, 2, 4096, 1e-3, 3, None, "uneven_case"),
    (1, 4, 2, 2048, 0.0, 5, None, "uneven_case"),
    (1, 4, 2, 2048, 1e30, 6, None, "uneven_case"),
    (1, 4, 2, 2048, 1e-30, 7, None, "uneven_case"),
    (1, 4, 2, 3000, 1e-3, 8, 8192, "uneven_case"),
    (1, 8, 2, 2048, 1e-30, 11, None, "uneven_case"),
    (1, 16, 2, 3000, 1e-3, 13, None, "uneven_case"),     # 8 queries per KV head: two virtual heads
    (1, 10, 2, 3000, 1e-3, 15, None, "uneven_case"),     # 5: five virtual heads of one query
    (1, 12, 2, 2048, 1e-3, 17, None, "uneven_case"),     # 6: three virtual heads of two
    (1, 16, 8, 4096, 0.0, 1001, None, "baseline_case"),  # the benchmark's first configuration
    (1, 16, 8, 20000, 3e-4, 4, None, "uneven_case"),
    (1, 32, 8, 20000, 3e-4, 12, None, "baseline_case"),
]


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("B,QH,KH,N,tau,seed,cap,gen", DECODE_CASES)
def test_decode_matches_oracle(ours, oracle, mode, B, QH, KH, N, tau, seed, cap, gen):
    """Outputs within 2e-3 x max|out| (+ half a BF16 ulp for the output's own rounding) of the float64 oracle on the
    cache the library itself wrote; two runs on 0xFF-poisoned scratch are bitwise identical."""
    q, k, v = getattr(datagen, gen)(seed, B, QH, KH, N)
    qd, kd, vd = _dev(q, k, v)
    c = ours.encode(kd, vd, mode, cap)
    out1 = ours.decode(c, qd, tau=tau)
    out2 = ours.decode(c, qd, tau=tau)
    torch.cuda.synchronize()
    assert torch.equal(out1, out2), "decode is not bit-reproducible"
    want = oracle.decode(q, gu.cache_to_numpy(c), tau=tau)
    gu.check_close(gu.bits_of(out1), want, f"{mode} decode {B}x{QH}/{KH}x{N}")


@pytest.mark.parametrize("mode", MODES)
def test_decode_matches_reference_library(ours, ref, mode):
    """Ours against the reference's CUDA decode on the same cache and queries: both are BF16 roundings of nearly the
    same FP32 value, so the bound is 2e-3 x max|out| plus one BF16 ulp."""
    q, k, v = datagen.baseline_case(1002, 2, 32, 8, 6000)
    qd, kd, vd = _dev(q, k, v)
    c = ours.encode(kd, vd, mode)
    a = datagen.bf16_to_f32(gu.bits_of(ours.decode(c, qd))).astype(np.float64)
    b = datagen.bf16_to_f32(gu.bits_of(ref.decode(c, qd))).astype(np.float64)
    err = np.abs(a - b)
    assert (err <= 2e-3 * np.abs(b).max() + gu.bf16_ulp(b)).all(), err.max() / np.abs(b).max()


@pytest.mark.parametrize("mode", MODES)
def test_capacity_layout(ours, mode):
    q, k, v = datagen.uneven_case(3, 1, 4, 2, 3000)
    qd, kd, vd = _dev(q, k, v)
    a = ours.decode(ours.encode(kd, vd, mode), qd, tau=1e-3)
    b = ours.decode(ours.encode(kd, vd, mode, capacity=8192), qd, tau=1e-3)
    assert torch.equal(a, b)


def test_decode_status_word_clear(ours):
    """No bounded wait gave up: the status word at the end of the scratch is 0 after a decode."""
    q, k, v = datagen.baseline_case(5, 1, 8, 2, 5000)
    qd, kd, vd = _dev(q, k, v)
    c = ours.encode(kd, vd, "4+2")
    ours.decode(c, qd)
    torch.cuda.synchronize()
    status = ours.last_scratch[-256:].view(torch.int32)[:2].cpu().numpy()
    assert status[0] == 0, status


# ---- prefill ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("B,QH,KH,N,chunks,seed", [
    (1, 2, 2, 100, [100], 21),
    (1, 4, 2, 900, [300, 84, 516], 11),
    (2, 8, 2, 1500, [300, 212, 128, 1, 859], 23),
    (1, 16, 8, 1024, [512, 512], 24),
    (1, 6, 2, 700, [260, 440], 30),
    (1, 2, 2, 1000, [1000], 31),      # one query per KV head: a 256-row CTA spans three groups
    (1, 8, 1, 600, [37, 563], 32),    # eight queries per KV head
])
def test_prefill_matches_oracle(ours, oracle, mode, B, QH, KH, N, chunks, seed):
    q, k, v = datagen.uneven_case(seed, B, QH, KH, N, q_rows=N)
    qd, kd, vd = _dev(q, k, v)
    c = ours.empty(B, KH, 2048, mode)
    o = oracle.empty(B, KH, 2048, mode)
    t = 0
    for n in chunks:
        sl = slice(t, t + n)
        out = ours.prefill(c, kd[:, :, sl].contiguous(), vd[:, :, sl].contiguous(), qd[:, :, sl].contiguous())
        step = max(1, n // 40)
        want = oracle.prefill(q[:, :, sl], k[:, :, sl], v[:, :, sl], o, pos_step=step)
        torch.cuda.synchronize()
        got = gu.bits_of(out)
        idx = np.arange(0, n, step)
        gu.check_close(got[:, :, idx], want[:, :, idx], f"{mode} prefill chunk at {t}")
        gu.assert_cache_equal(c, o, f"{mode} after chunk at {t}")
        t += n
    # no bounded wait of the tensor-core kernel gave up
    assert ctypes.CDLL(gu.OURS).fbla_k_attend_tc_status() == 0


@pytest.mark.parametrize("mode", MODES)
def test_prefill_matches_reference_library(ours, ref, mode):
    q, k, v = datagen.baseline_case(1004, 1, 8, 2, 1100, q_rows=1100)
    qd, kd, vd = _dev(q, k, v)
    ca, cb = ours.empty(1, 2, 2048, mode), ref.empty(1, 2, 2048, mode)
    t = 0
    for n in (500, 600):
        sl = slice(t, t + n)
        args = (kd[:, :, sl].contiguous(), vd[:, :, sl].contiguous(), qd[:, :, sl].contiguous())
        a = datagen.bf16_to_f32(gu.bits_of(ours.prefill(ca, *args))).astype(np.float64)
        b = datagen.bf16_to_f32(gu.bits_of(ref.prefill(cb, *args))).astype(np.float64)
        for pos in range(n):  # per position: the output scale differs along the sequence
            err = np.abs(a[:, :, pos] - b[:, :, pos])
            assert (err <= 2e-3 * np.abs(b[:, :, pos]).max() + gu.bf16_ulp(b[:, :, pos])).all(), (t + pos, err.max())
        t += n


# ---- the Python interface -------------------------------------------------------------------------------------------------
def test_python_interface(oracle):
    from mlops_b200.attention import append, decode, empty, encode, prefill
    q, k, v = datagen.uneven_case(0, 1, 4, 2, 1000)
    qd, kd, vd = _dev(q, k, v)
    for mode in MODES:
        c = encode(kd, vd, mode)
        got = decode(qd, c, tau=3e-3)
        gu.check_close(gu.bits_of(got), oracle.decode(q, oracle.encode(k, v, mode), tau=3e-3), mode)
        d = encode(kd[:, :, :100], vd[:, :, :100], mode, capacity=1024)
        append(d, kd[:, :, 100:], vd[:, :, 100:])
        assert d.tokens == 1000 and torch.equal(decode(qd, d, tau=3e-3), got)
        with pytest.raises(ValueError):
            append(d, kd[:, :, :400], vd[:, :, :400])
        e = empty(1, 2, 1024, mode)
        qq = gu.bf16_tensor(datagen.uneven_case(1, 1, 4, 2, 300, q_rows=300)[0])
        assert prefill(qq, kd[:, :, :300], vd[:, :, :300], e).shape == (1, 4, 300, 128)
    with pytest.raises(TypeError):
        decode(qd.float(), c)
