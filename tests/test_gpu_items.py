"""The work-item interface on a GPU: every plan, run by an emulated executor (kernels generated from mlops_fbla_item_call,
compiled by NVRTC, one CTA per item, passes in stream order), gives bit for bit what the equally named stream call gives;
and every byte a call changes lies inside the write ranges that mlops_fbla_item_access declares.
Modelled on attention/fbla/tests/test_items.cu:489-496 (items == stream API) and :300-420 (ranges)."""
import ctypes
import os

import numpy as np
import pytest
import torch

from tests import datagen
from tests import gpu_util as gu
from tests import items_util as iu

pytestmark = pytest.mark.gpu
pytest.importorskip("cuda.bindings.nvrtc")


@pytest.fixture(scope="module")
def ours():
    assert os.path.exists(gu.OURS)
    return gu.CLib(gu.OURS)


def _i32(*v):
    return torch.tensor(list(v), dtype=torch.int32, device="cuda")


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _cfg(c, q_heads, tokens_offset=0, length_stride=0):
    return gu.Config(c["batch"], q_heads, c["kv_heads"], tokens_offset, 0, 0, gu.FORMATS[c["mode"]][2], c["capacity"], 0, 0, 0, 0, length_stride)


def _clone(c):
    return {k: (v.clone() if torch.is_tensor(v) else v) for k, v in c.items()}


def _covered(changed, ranges, what):
    """changed: bool array over an argument's bytes; ranges: its write ranges"""
    ok = np.zeros_like(changed)
    for r in ranges:
        for i in range(r.rows):
            ok[r.offset + i * r.stride: r.offset + i * r.stride + r.bytes] = True
    assert not (changed & ~ok).any(), f"{what}: bytes written outside the declared ranges at {np.flatnonzero(changed & ~ok)[:5]}"


def _write_ranges(lib, passes, n, arg):
    out = []
    for p in range(n):
        for item in range(passes[p].items):
            out += [r for r in iu.access(lib, passes, n, p, item) if r.write and iu.ARGS[r.arg] == arg]
    return out


@pytest.mark.parametrize("mode,QH,KH,N,cap,ctas", [("4+2", 8, 2, 3000, 4096, None), ("3+3", 4, 4, 3000, 4096, None),
                                                     # capacities beyond ~34 000 tokens take the coarse kernel that deals windows and groups
                                                     # to every warp by cost; ctas = 3: every pass as a persistent loop of three CTAs
                                                     # walking its items back to back
                                                     ("4+2", 8, 2, 9000, 16384, None), ("3+3", 8, 2, 9000, 16384, 3), ("4+2", 4, 4, 3000, 4096, 3),
                                                     ("4+2", 8, 2, 9000, 40960, 3), ("3+3", 8, 2, 9000, 32768, None)])
def test_decode_plan_equals_decode_at(ours, mode, QH, KH, N, cap, ctas):
    B = 2
    q, k, v = datagen.baseline_case(41, B, QH, KH, N)
    qd = gu.bf16_tensor(q)
    c = ours.encode(gu.bf16_tensor(k), gu.bf16_tensor(v), mode, capacity=cap)
    length = _i32(N)
    want = ours.decode_at(c, qd, length)
    cfg = _cfg(c, QH)
    lib = ours.lib
    nbytes = lib.mlops_fbla_decode_scratch_bytes(ctypes.byref(gu.Config(B, QH, KH, cap, 0, 0, gu.FORMATS[mode][2], cap, 0, 0, 0, 0, 0)))
    scratch = torch.full((nbytes,), 0xA5, dtype=torch.uint8, device="cuda")
    out = torch.full_like(qd, -9.0)
    passes = (iu.Items * 4)()
    kc = ours._cache(c)
    vp = ctypes.c_void_p
    n = lib.mlops_fbla_decode_at_items(ctypes.byref(cfg), vp(length.data_ptr()), vp(qd.data_ptr()), ctypes.byref(kc), vp(out.data_ptr()),
                                       vp(scratch.data_ptr()), ctypes.c_size_t(nbytes), 0, passes, 4)
    assert n == 4, ours.error()
    assert [passes[i].kind for i in range(4)] == [iu.KINDS[x] for x in ("COARSE", "SELECT", "REFINE", "MERGE")]
    assert lib.mlops_fbla_decode_at_items(ctypes.byref(cfg), vp(length.data_ptr()), vp(qd.data_ptr()), ctypes.byref(kc), vp(out.data_ptr()),
                                          vp(scratch.data_ptr()), ctypes.c_size_t(nbytes), 0, None, 0) == 4  # max = 0 only counts
    before = scratch.cpu().numpy().copy()
    iu.run_plan(lib, passes, n, _stream(), ctas)
    assert torch.equal(out, want), "the plan's items differ from mlops_fbla_decode_at"
    changed = scratch.cpu().numpy() != before
    _covered(changed, _write_ranges(lib, passes, n, "SCRATCH"), "decode scratch")
    _covered(np.ones(out.numel() * 2, bool), _write_ranges(lib, passes, n, "OUT"), "decode output")


@pytest.mark.parametrize("mode,count,ctas", [("4+2", 300, None), ("3+3", 5, None), ("3+3", 700, 3)])
def test_prefill_plan_equals_prefill_at(ours, mode, count, ctas):
    """count 300 / 700: the tensor-core pass (TC) -- with ctas = 3 as a persistent loop, so that one CTA runs several
    tensor-core items back to back, each allocating and freeing tensor memory and its barriers; count 5: the
    warp-per-row pass (STREAM)"""
    B, QH, KH, n0, cap = 1, 8, 2, 200, 1024
    max_count = count + 3
    q, k, v = datagen.uneven_case(43, B, QH, KH, n0 + count, q_rows=n0 + count)
    qd, kd, vd = gu.bf16_tensor(q), gu.bf16_tensor(k), gu.bf16_tensor(v)
    a = ours.encode(kd[:, :, :n0].contiguous(), vd[:, :, :n0].contiguous(), mode, capacity=cap)
    b = _clone(a)
    pad = lambda x: torch.nn.functional.pad(x[:, :, n0:n0 + count], (0, 0, 0, max_count - count)).contiguous()
    qp, kp, vp_ = pad(qd), pad(kd), pad(vd)
    length, cnt = _i32(n0), _i32(count)
    want = torch.full((B, QH, max_count, 128), -7.0, dtype=torch.bfloat16, device="cuda")
    ours.prefill_at(a, kp, vp_, qp, length, cnt, max_count, out=want)
    out = torch.full_like(want, -7.0)
    cfg = _cfg(b, QH)
    kc = ours._cache(b)
    lib, vp = ours.lib, ctypes.c_void_p
    passes = (iu.Items * 4)()
    n = lib.mlops_fbla_prefill_at_items(ctypes.byref(cfg), vp(length.data_ptr()), vp(cnt.data_ptr()), max_count, vp(qp.data_ptr()), vp(kp.data_ptr()),
                                        vp(vp_.data_ptr()), ctypes.byref(kc), vp(out.data_ptr()), passes, 4)
    # a count on the device whose ceiling reaches the tensor-core kernel: both attention passes are planned and the count
    # decides on the device which of them works (the other returns at once)
    kinds = ["CLOSE", "TC", "STREAM", "FINISH"] if max_count * (QH // KH) >= 64 else ["CLOSE", "STREAM", "FINISH"]
    assert n == len(kinds), ours.error()
    assert [passes[i].kind for i in range(n)] == [iu.KINDS[x] for x in kinds]
    as_bytes = lambda t: t.contiguous().view(torch.uint8).cpu().numpy().reshape(-1).copy()
    before = {key: as_bytes(b[key]) for key in ("coarse", "fine", "meta", "sink_k", "sink_v", "open_k", "open_v")}
    iu.run_plan(lib, passes, n, _stream(), ctas)
    assert torch.equal(out, want)
    a["tokens"] = b["tokens"] = n0 + count
    gu.assert_cache_equal(a, gu.cache_to_numpy(b), mode)
    names = dict(coarse="COARSE", fine="FINE", meta="META", sink_k="SINK_K", sink_v="SINK_V", open_k="OPEN_K", open_v="OPEN_V")
    for key, arg in names.items():
        _covered(as_bytes(b[key]) != before[key], _write_ranges(lib, passes, n, arg), key)
    changed_out = (out.view(torch.int16) != torch.full_like(want, -7.0).view(torch.int16)).cpu().numpy().reshape(-1)
    _covered(np.repeat(changed_out, 2), _write_ranges(lib, passes, n, "OUT"), "prefill output")


def test_append_and_qkv_plans_equal_their_calls(ours, oracle):
    mode, B, QH, KH, cap = "4+2", 2, 8, 2, 512
    lens = [255, 256]  # the second row closes a group with this token
    _, k, v = datagen.uneven_case(44, B, QH, KH, 256)
    kd, vd = gu.bf16_tensor(k), gu.bf16_tensor(v)
    base = ours.empty(B, KH, cap, mode)
    for bi, nn in enumerate(lens):
        row = {key: (val[bi:bi + 1] if torch.is_tensor(val) else val) for key, val in base.items()}
        row["batch"], row["tokens"] = 1, 0
        ours.prefill(row, kd[bi:bi + 1, :, :nn].contiguous(), vd[bi:bi + 1, :, :nn].contiguous())
    length = _i32(*lens)
    lib, vp = ours.lib, ctypes.c_void_p
    # append_at
    a, b = _clone(base), _clone(base)
    ktok, vtok = kd[:, :, 0].contiguous(), vd[:, :, 1].contiguous()
    ours.append_at(a, ktok, vtok, length, length_stride=1)
    cfg = gu.Config(B, KH, KH, 0, 0, 0, gu.FORMATS[mode][2], cap, 0, 0, 0, 0, 1)
    kc = ours._cache(b)
    passes = (iu.Items * 2)()
    n = lib.mlops_fbla_append_at_items(ctypes.byref(cfg), vp(length.data_ptr()), vp(ktok.data_ptr()), vp(vtok.data_ptr()), ctypes.byref(kc), passes, 2)
    assert n == 2 and [passes[i].kind for i in range(2)] == [iu.KINDS["CLOSE"], iu.KINDS["FINISH"]], ours.error()
    iu.run_plan(lib, passes, n, _stream())
    a["tokens"] = b["tokens"] = 257
    gu.assert_cache_equal(a, gu.cache_to_numpy(b), "append_at items")
    # qkv_at
    a, b = _clone(base), _clone(base)
    rng = np.random.default_rng(3)
    proj = gu.bf16_tensor(datagen.to_bf16_bits(rng.standard_normal((B, KH * (QH // KH + 2) * 128), dtype=np.float32)))
    freq = torch.from_numpy(oracle.rope_freq(1e6)).cuda()
    w = gu.bf16_tensor(datagen.to_bf16_bits(rng.standard_normal(128, dtype=np.float32) * 0.3 + 1.0))
    want_q = ours.qkv_at(a, proj, QH, length, freq, w, w, 1e-6, length_stride=1)
    q_out = torch.full_like(want_q, -5.0)
    cfg = gu.Config(B, QH, KH, 0, 0, 0, gu.FORMATS[mode][2], cap, 0, 0, 0, 0, 1)
    tok = ours._token(proj, QH, KH, proj.shape[1], w, w, 1e-6, freq, 0.0, q_out)
    kc = ours._cache(b)
    n = lib.mlops_fbla_qkv_at_items(ctypes.byref(cfg), vp(length.data_ptr()), ctypes.byref(tok), ctypes.byref(kc), passes, 2)
    assert n == 2 and [passes[i].kind for i in range(2)] == [iu.KINDS["CLOSE"], iu.KINDS["QKV"]], ours.error()
    iu.run_plan(lib, passes, n, _stream())
    assert torch.equal(q_out, want_q)
    gu.assert_cache_equal(a, gu.cache_to_numpy(b), "qkv_at items")
    # qkv_prefill_at
    count, max_count = 19, 24
    rows = gu.bf16_tensor(datagen.to_bf16_bits(rng.standard_normal((count, KH * (QH // KH + 2) * 128), dtype=np.float32)))
    ln, cn = _i32(777), _i32(count)
    want = ours.qkv_prefill_at(rows, QH, KH, ln, cn, max_count, 2048, freq, w, w, 1e-6, fill=-3.0)
    outs = [torch.full_like(t, -3.0) for t in want]
    cfg = gu.Config(1, QH, KH, 0, 0, 0, 0, 2048, 0, 0, 0, 0, 0)
    tok = ours._token(rows, QH, KH, rows.shape[1], w, w, 1e-6, freq, 0.0, None)
    one = (iu.Items * 1)()
    n = lib.mlops_fbla_qkv_prefill_at_items(ctypes.byref(cfg), vp(ln.data_ptr()), vp(cn.data_ptr()), max_count, ctypes.byref(tok), vp(outs[0].data_ptr()),
                                            vp(outs[1].data_ptr()), vp(outs[2].data_ptr()), one, 1)
    assert n == 1 and one[0].kind == iu.KINDS["QKV_CHUNK"], ours.error()
    iu.run_plan(lib, one, n, _stream())
    for x, y in zip(outs, want):
        assert torch.equal(x, y)
    for arg, t in zip(("Q", "K", "V"), outs):
        changed = (t.view(torch.int16) != torch.full_like(t, -3.0).view(torch.int16)).cpu().numpy().reshape(-1)
        _covered(np.repeat(changed, 2), _write_ranges(lib, one, 1, arg), f"qkv chunk {arg}")


def test_plan_argument_checks(ours):
    lib, vp = ours.lib, ctypes.c_void_p
    c = ours.empty(1, 2, 256, "3+3")
    kc = ours._cache(c)
    cfg = _cfg(c, 4)
    passes = (iu.Items * 4)()
    assert lib.mlops_fbla_decode_at_items(ctypes.byref(cfg), None, vp(16), ctypes.byref(kc), vp(16), vp(16), ctypes.c_size_t(1 << 30), 0, passes, 4) == -1
    assert "null" in ours.error()
    assert lib.mlops_fbla_item_access(passes, 0, 0, 0, None, 0) == -1
    assert lib.mlops_fbla_item_call(None, None, ctypes.c_size_t(0)) == -1
