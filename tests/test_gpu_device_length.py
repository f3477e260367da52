"""Device-length entry points (decode_at, append_at, prefill_at): lengths and counts live in device memory and are read
when the kernels run, so the same launches serve any length -- checked against the host-length calls, per-row lengths
against each row alone, and a CUDA graph of (append_at, decode_at) replayed token by token, as the reference's
run_device_length / run_prefill_at / run_batch_lengths do (attention/fbla/tests/test_fbla.cu:482-738, 1056-1179)."""
import numpy as np
import pytest
import torch

from tests import datagen
from tests import gpu_util as gu

pytestmark = pytest.mark.gpu
MODES = ["3+3", "4+2"]


@pytest.fixture(scope="module")
def ours():
    return gu.CLib(gu.OURS)


def _i32(*vals):
    return torch.tensor(list(vals), dtype=torch.int32, device="cuda")


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("B,QH,KH,N,tau,seed", [(1, 16, 8, 400, 3e-4, 41), (2, 8, 2, 1301, 1e-3, 42), (1, 2, 2, 1150, 1e-2, 43), (1, 10, 2, 270, 1e-3, 46)])
def test_decode_at_equals_decode(ours, mode, B, QH, KH, N, tau, seed):
    """The same cache (laid out for a capacity) decoded with a host length and with the length on the device, also
    split as *length + cfg->tokens: bit-identical outputs."""
    q, k, v = datagen.uneven_case(seed, B, QH, KH, N)
    qd, kd, vd = gu.bf16_tensor(q), gu.bf16_tensor(k), gu.bf16_tensor(v)
    c = ours.encode(kd, vd, mode, capacity=2048)
    want = ours.decode(c, qd, tau=tau)
    got = ours.decode_at(c, qd, _i32(N), tau=tau)
    got2 = ours.decode_at(c, qd, _i32(N - 1), tokens_offset=1, tau=tau)
    torch.cuda.synchronize()
    assert torch.equal(want, got) and torch.equal(want, got2)


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("capacity", [8192, 40000])
def test_decode_at_equals_decode_under_a_large_capacity(ours, mode, capacity):
    """Rows far shorter than the cache's capacity: the coarse pass picks how its warps share the work from the capacity
    for both calls (8192: split by the lengths, 40000: windows and groups dealt to every warp by cost -- here with far
    fewer units than warps), so host-length and device-length decodes still run the same kernels and agree bit for bit."""
    B, QH, KH, N = 2, 8, 2, 700
    q, k, v = datagen.uneven_case(47, B, QH, KH, N)
    qd, kd, vd = gu.bf16_tensor(q), gu.bf16_tensor(k), gu.bf16_tensor(v)
    c = ours.encode(kd, vd, mode, capacity=capacity)
    want = ours.decode(c, qd, tau=1e-3)
    got = ours.decode_at(c, qd, _i32(N), tau=1e-3)
    small = ours.decode(ours.encode(kd, vd, mode, capacity=1024), qd, tau=1e-3)  # (the split by the lengths)
    torch.cuda.synchronize()
    assert torch.equal(want, got)
    scale = float(want.float().abs().max())
    assert float((want.float() - small.float()).abs().max()) <= 2e-3 * scale


@pytest.mark.parametrize("mode", MODES)
def test_append_at_graph_replay(ours, oracle, mode):
    """One CUDA graph holding (append_at, decode_at), replayed per token while the device length advances; the cache
    ends bit-identical to a one-shot encode and every step's output equals the host-length decode of that prefix."""
    B, QH, KH, n0, steps = 1, 8, 2, 120, 280
    q, k, v = datagen.uneven_case(45, B, QH, KH, n0 + steps)
    qd, kd, vd = gu.bf16_tensor(q), gu.bf16_tensor(k), gu.bf16_tensor(v)
    cap = 512
    c = ours.encode(kd[:, :, :n0].contiguous(), vd[:, :, :n0].contiguous(), mode, capacity=cap)
    length = _i32(n0)
    ktok, vtok = torch.empty(B, KH, 128, dtype=torch.bfloat16, device="cuda"), torch.empty(B, KH, 128, dtype=torch.bfloat16, device="cuda")
    out = torch.empty_like(qd)
    capcfg = gu.Config(B, QH, KH, cap, 0, 0, gu.FORMATS[mode][2], cap, 0, 0, 0, 0, 0)
    import ctypes
    scratch = torch.full((ours.lib.mlops_fbla_decode_scratch_bytes(ctypes.byref(capcfg)),), 0xFF, dtype=torch.uint8, device="cuda")
    # warm up outside capture (the first call configures kernel attributes), on a copy of the cache
    warm = {key: (val.clone() if torch.is_tensor(val) else val) for key, val in c.items()}
    ktok.copy_(kd[:, :, n0]); vtok.copy_(vd[:, :, n0])
    ours.append_at(warm, ktok, vtok, length)
    ours.decode_at(warm, qd, length, tokens_offset=1, tau=1e-3, scratch=scratch, out=out)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(g, stream=stream):
            ours.append_at(c, ktok, vtok, length)                       # token at position *length
            ours.decode_at(c, qd, length, tokens_offset=1, tau=1e-3, scratch=scratch, out=out)
            length.add_(1)
    checks = {n0, n0 + 7, 127, 128, 255, 256, 383, 384, n0 + steps - 1}
    for t in range(n0, n0 + steps):
        ktok.copy_(kd[:, :, t]); vtok.copy_(vd[:, :, t])
        g.replay()
        if t in checks:
            torch.cuda.synchronize()
            ref = ours.encode(kd[:, :, :t + 1].contiguous(), vd[:, :, :t + 1].contiguous(), mode, capacity=cap)
            assert torch.equal(out, ours.decode(ref, qd, tau=1e-3)), t
    torch.cuda.synchronize()
    c["tokens"] = n0 + steps
    gu.assert_cache_equal(c, oracle.encode(k, v, mode, capacity=cap), f"{mode} after graph replay")


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("QH,KH,lens", [(8, 2, [127, 255, 1000]), (2, 2, [1, 300]), (16, 2, [2000, 129, 4000, 63])])
def test_per_row_lengths(ours, oracle, mode, QH, KH, lens):
    """length_stride 1: every batch row has its own device length. Outputs against the oracle with the same per-row
    lengths; the one-token append at per-row positions against row-wise appends."""
    B, cap = len(lens), 4096
    q, k, v = datagen.uneven_case(51, B, QH, KH, max(lens) + 1)
    qd = gu.bf16_tensor(q)
    c = ours.empty(B, KH, cap, mode)
    o = oracle.empty(B, KH, cap, mode)
    # build row b with lens[b] tokens: encode each row alone into its slice of the batched cache
    for b, n in enumerate(lens):
        row = ours.encode(gu.bf16_tensor(k[b:b + 1, :, :n]), gu.bf16_tensor(v[b:b + 1, :, :n]), mode, capacity=cap)
        orow = oracle.encode(k[b:b + 1, :, :n], v[b:b + 1, :, :n], mode, capacity=cap)
        for key in ("coarse", "fine", "meta", "sink_k", "sink_v", "open_k", "open_v"):
            c[key][b].copy_(row[key][0])
            o[key][b * KH:(b + 1) * KH] = orow[key]
    length = _i32(*lens)
    got = ours.decode_at(c, qd, length, tau=1e-3, length_stride=1)
    torch.cuda.synchronize()
    o["tokens"] = max(lens)
    want = oracle.decode(q, o, tau=1e-3, lengths=np.array(lens, np.int32))
    for b in range(B):
        gu.check_close(gu.bits_of(got)[b], want[b], f"{mode} row {b} of lengths {lens}")
    # append one token per row at its own position, then compare every row with a row-wise encode of n + 1 tokens
    ktok = gu.bf16_tensor(np.stack([k[b, :, n] for b, n in enumerate(lens)]))
    vtok = gu.bf16_tensor(np.stack([v[b, :, n] for b, n in enumerate(lens)]))
    ours.append_at(c, ktok, vtok, length, length_stride=1)
    torch.cuda.synchronize()
    got_np = gu.cache_to_numpy(c)
    for b, n in enumerate(lens):
        orow = oracle.encode(k[b:b + 1, :, :n + 1], v[b:b + 1, :, :n + 1], mode, capacity=cap)
        for key in ("coarse", "fine", "meta", "sink_k", "sink_v", "open_k", "open_v"):
            assert np.array_equal(got_np[key][b * KH:(b + 1) * KH], orow[key]), (b, key)


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("B,QH,KH,n0,counts", [(1, 2, 2, 100, [100, 100]), (1, 4, 2, 1000, [300, 212, 128, 1, 1407]), (2, 8, 2, 2048, [512, 512, 700, 330])])
def test_prefill_at_equals_prefill(ours, mode, B, QH, KH, n0, counts):
    """Chunks with the start and count on the device (launches sized by the ceiling alone) against the host-length
    calls: outputs of the chunk's positions (bit-identical whenever both calls run the same attention kernel) and the whole
    cache bit-identical; rows past the count stay untouched."""
    total = n0 + sum(counts)
    q, k, v = datagen.uneven_case(62, B, QH, KH, total, q_rows=total)
    qd, kd, vd = gu.bf16_tensor(q), gu.bf16_tensor(k), gu.bf16_tensor(v)
    cap = 8192
    a = ours.encode(kd[:, :, :n0].contiguous(), vd[:, :, :n0].contiguous(), mode, capacity=cap)
    b = ours.encode(kd[:, :, :n0].contiguous(), vd[:, :, :n0].contiguous(), mode, capacity=cap)
    max_count = max(counts) + 13
    length, count = _i32(n0), _i32(0)
    t = n0
    for n in counts:
        sl = slice(t, t + n)
        want = ours.prefill(a, kd[:, :, sl].contiguous(), vd[:, :, sl].contiguous(), qd[:, :, sl].contiguous())
        pad = lambda x: torch.nn.functional.pad(x[:, :, sl], (0, 0, 0, max_count - n)).contiguous()
        count.fill_(n)
        out = torch.full((B, QH, max_count, 128), -7.0, dtype=torch.bfloat16, device="cuda")
        ours.prefill_at(b, pad(kd), pad(vd), pad(qd), length, count, max_count, out=out)
        length.add_(n)
        torch.cuda.synchronize()
        qg = QH // KH
        if (n * qg >= 64) == (max_count * qg >= 64):  # the same kernel serves both calls: bit-identical
            assert torch.equal(out[:, :, :n], want), (t, n)
        else:  # the host-length call of a tiny chunk takes the warp-per-row kernel, the ceiling-sized launch the tensor-core one
            w = datagen.bf16_to_f32(gu.bits_of(want)).astype(np.float64)
            g = datagen.bf16_to_f32(gu.bits_of(out[:, :, :n].contiguous())).astype(np.float64)
            assert (np.abs(g - w) <= 2e-3 * np.abs(w).max() + gu.bf16_ulp(w)).all(), (t, n)
        assert (out[:, :, n:] == -7.0).all()
        t += n
    b["tokens"] = a["tokens"]
    gu.assert_cache_equal(b, gu.cache_to_numpy(a), mode)
