"""GPU parity of the fused QKV step (mlops_fbla_qkv_at, mlops_fbla_qkv_prefill_at) through the C ABI: against the
reference's own CUDA library on the same device buffers (bit-exact: q, windows, records) and against the CPU oracle
(rotated values within one BF16 ulp -- the oracle's cos / sin come from the double library --, everything else exact).
Cases follow attention/fbla/tests/test_fbla.cu:765-900 (positions around group boundaries, with and without the norm,
per-row lengths, chunk tails)."""
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
    """the reference's own CUDA library when it was built into oracle/_ref, else None (those comparisons are skipped)"""
    return gu.CLib(gu.REF) if os.path.exists(gu.REF) else None


def _i32(*v):
    return torch.tensor(list(v), dtype=torch.int32, device="cuda")


def _rows(seed, rows, q_heads, kv_heads):
    qg = q_heads // kv_heads
    rng = np.random.default_rng(seed)
    return datagen.to_bf16_bits(rng.standard_normal((rows, kv_heads * (qg + 2) * 128), dtype=np.float32) * 1.5)


def _weights(seed):
    rng = np.random.default_rng(seed)
    return datagen.to_bf16_bits(rng.standard_normal(128, dtype=np.float32) * 0.5 + 1.0), datagen.to_bf16_bits(rng.standard_normal(128, dtype=np.float32) * 0.5 + 1.0)


def _split(row_bits, q_heads, kv_heads):
    """one projection row -> q [q_heads, 128], k [kv_heads, 128], v [kv_heads, 128] (bits)"""
    qg = q_heads // kv_heads
    r = row_bits.reshape(kv_heads, qg + 2, 128)
    return r[:, :qg].reshape(q_heads, 128), r[:, qg], r[:, qg + 1]


def _close_ulp(got_bits, want_bits, what):
    g, w = datagen.bf16_to_f32(got_bits).astype(np.float64), datagen.bf16_to_f32(want_bits).astype(np.float64)
    assert (np.abs(g - w) <= gu.bf16_ulp(w)).all(), what
    assert (got_bits != want_bits).mean() < 0.02, what  # and nearly all of them equal


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("norm", [False, True])
def test_qkv_at_steps_match_oracle_and_reference(ours, ref, oracle, mode, norm):
    B, QH, KH, cap, n0 = 2, 8, 2, 1024, 250
    steps = 12  # crosses position 256: a group closes on the way
    _, k, v = datagen.uneven_case(91, B, QH, KH, n0)
    kd, vd = gu.bf16_tensor(k), gu.bf16_tensor(v)
    freq_np = oracle.rope_freq(1e6)
    freq = torch.from_numpy(freq_np).cuda()
    wq, wk = _weights(5)
    wqd, wkd = (gu.bf16_tensor(wq), gu.bf16_tensor(wk)) if norm else (None, None)
    libs = [ours] + ([ref] if ref is not None else [])
    caches = [lib.encode(kd, vd, mode, capacity=cap) for lib in libs]
    o = oracle.encode(k, v, mode, capacity=cap)
    length = _i32(n0)
    for s in range(steps):
        rows = _rows(1000 + s, B, QH, KH)
        proj = gu.bf16_tensor(rows)
        pos = n0 + s
        qs = [lib.qkv_at(c, proj, QH, length, freq, wqd, wkd, 1e-6) for lib, c in zip(libs, caches)]
        torch.cuda.synchronize()
        want_q = np.zeros((B, QH, 128), np.uint16)
        knew, vnew = np.zeros((B, KH, 1, 128), np.uint16), np.zeros((B, KH, 1, 128), np.uint16)
        for b in range(B):
            q, kk, vv = _split(rows[b], QH, KH)
            want_q[b] = oracle.norm_rope(q, wq if norm else None, 1e-6, pos, freq_np)
            knew[b, :, 0] = oracle.norm_rope(kk, wk if norm else None, 1e-6, pos, freq_np)
            vnew[b, :, 0] = vv
        _close_ulp(gu.bits_of(qs[0]), want_q, f"q at {pos}")
        if len(libs) == 2:
            assert torch.equal(qs[0], qs[1]), f"q at {pos} differs from the reference library"
        # the cache: the oracle appends ITS k (possibly an ulp off), so windows are compared within an ulp against the
        # oracle and bit for bit against the reference library; records exactly once the device's own k rows are used
        oracle.append(o, knew, vnew)
        got = gu.cache_to_numpy(caches[0])
        for key in ("open_v", "sink_v"):
            assert np.array_equal(got[key], o[key]), (pos, key)
        _close_ulp(got["open_k"], o["open_k"], f"open_k at {pos}")
        length.add_(1)
    for c in caches:
        c["tokens"] = n0 + steps
    if len(libs) == 2:
        gu.assert_cache_equal(caches[0], gu.cache_to_numpy(caches[1]), f"{mode} norm={norm} against the reference library")


@pytest.mark.parametrize("mode", MODES)
def test_qkv_at_equals_append_at_of_the_rotated_token(ours, oracle, mode):
    """Per-row lengths, positions below 128 (sink window) and on a group boundary: the cache after qkv_at is bit-identical to
    append_at of the k this library rotated itself."""
    B, QH, KH, cap = 3, 4, 2, 512
    lens = [5, 128, 300]
    _, k, v = datagen.uneven_case(92, B, QH, KH, max(lens))
    kd, vd = gu.bf16_tensor(k), gu.bf16_tensor(v)
    a, b = ours.empty(B, KH, cap, mode), ours.empty(B, KH, cap, mode)
    for c in (a, b):
        for bi, n in enumerate(lens):
            row = {key: (val[bi:bi + 1] if torch.is_tensor(val) else val) for key, val in c.items()}
            row["batch"], row["tokens"] = 1, 0
            ours.prefill(row, kd[bi:bi + 1, :, :n].contiguous(), vd[bi:bi + 1, :, :n].contiguous())
    freq_np = oracle.rope_freq(1e4)
    freq = torch.from_numpy(freq_np).cuda()
    length = _i32(*lens)
    rows = _rows(7, B, QH, KH)
    q_out = ours.qkv_at(a, gu.bf16_tensor(rows), QH, length, freq, length_stride=1)
    # the same token through the chunk form (one row at a time: batch 1), then append_at
    ktok, vtok = torch.empty((B, KH, 128), dtype=torch.bfloat16, device="cuda"), torch.empty((B, KH, 128), dtype=torch.bfloat16, device="cuda")
    for bi, n in enumerate(lens):
        qo, ko, vo = ours.qkv_prefill_at(gu.bf16_tensor(rows[bi:bi + 1]), QH, KH, _i32(n), _i32(1), 1, cap, freq)
        ktok[bi], vtok[bi] = ko[:, 0], vo[:, 0]
        assert torch.equal(qo[:, 0], q_out[bi])
    ours.append_at(b, ktok, vtok, length, length_stride=1)
    torch.cuda.synchronize()
    a["tokens"] = b["tokens"] = max(lens) + 1
    gu.assert_cache_equal(a, gu.cache_to_numpy(b), mode)


@pytest.mark.parametrize("norm", [False, True])
def test_qkv_prefill_at_matches_oracle_and_reference(ours, ref, oracle, norm):
    QH, KH, cap, n0, count, max_count = 8, 4, 70000, 65530, 21, 32  # positions across 2^16: both halves of the phase split
    rows = _rows(33, count, QH, KH)
    proj = gu.bf16_tensor(rows)
    freq_np = oracle.rope_freq(1e6)
    freq = torch.from_numpy(freq_np).cuda()
    wq, wk = _weights(6)
    wqd, wkd = (gu.bf16_tensor(wq), gu.bf16_tensor(wk)) if norm else (None, None)
    outs = [lib.qkv_prefill_at(proj, QH, KH, _i32(n0), _i32(count), max_count, cap, freq, wqd, wkd, 1e-6, att=0.75, fill=-3.0)
            for lib in [ours] + ([ref] if ref is not None else [])]
    torch.cuda.synchronize()
    q, k, v = [gu.bits_of(t) for t in outs[0]]
    for i in range(count):
        qi, ki, vi = _split(rows[i], QH, KH)
        _close_ulp(q[:, i], oracle.norm_rope(qi, wq if norm else None, 1e-6, n0 + i, freq_np, 0.75), f"q row {i}")
        _close_ulp(k[:, i], oracle.norm_rope(ki, wk if norm else None, 1e-6, n0 + i, freq_np, 0.75), f"k row {i}")
        assert np.array_equal(v[:, i], vi)
    for t in outs[0]:
        assert (t[:, count:] == -3.0).all()  # rows past the count are not written
    if len(outs) == 2:
        for a, b in zip(outs[0], outs[1]):
            assert torch.equal(a, b)


def test_qkv_argument_checks(ours):
    c = ours.empty(1, 2, 256, "3+3")
    freq = torch.zeros((64, 4), dtype=torch.float32, device="cuda")
    proj = torch.zeros((1, 2 * 4 * 128), dtype=torch.bfloat16, device="cuda")
    w = torch.ones(128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="both or neither"):
        ours.qkv_at(c, proj, 4, _i32(0), freq, q_norm=w)
    with pytest.raises(RuntimeError, match="batch 1"):
        cfg = gu.Config(2, 4, 2, 0, 0, 0, 0, 256, 0, 0, 0, 0, 0)
        tok = ours._token(proj, 4, 2, proj.shape[1], None, None, 0.0, freq, 0.0, None)
        import ctypes
        st = ours.lib.mlops_fbla_qkv_prefill_at(ctypes.byref(cfg), _i32(0).data_ptr(), _i32(1).data_ptr(), 1, ctypes.byref(tok), proj.data_ptr(),
                                                proj.data_ptr(), proj.data_ptr(), None)
        raise RuntimeError(ours.error()) if st else AssertionError("accepted")
