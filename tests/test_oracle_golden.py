"""Pins the CPU oracle to the reference: every array of tests/golden/fbla_golden.npz was produced by the
reference's own Python code (tests/golden/make_golden.py); the inputs are regenerated here from the same seeds."""
import os

import numpy as np
import pytest

from tests import datagen

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "fbla_golden.npz"))
MODES = [("3+3", 3, 3), ("4+2", 4, 2)]


def _groups():
    _, kb, vb = datagen.baseline_case(7, 1, 4, 1, 256)
    _, ku, _ = datagen.uneven_case(8, 1, 4, 1, 256)
    return np.stack([datagen.edge_group(3), datagen.edge_group(4), kb[0, 0, :128], kb[0, 0, 128:], vb[0, 0, :128], ku[0, 0, :128],
                     ku[0, 0, 128:]])


def test_quantizer_bit_exact(oracle):
    """base, step and codes of 7 groups (edge channels, benchmark data, the reference tests' data) equal the
    reference's _quantize (attention/python/mlops/attention/fbla.py:24-40) bit for bit."""
    for g, x in enumerate(_groups()):
        base, step, code = oracle.quantize_group(x)
        assert np.array_equal(base, GOLD["quant_base"][g]), g
        assert np.array_equal(step, GOLD["quant_step"][g]), g
        assert np.array_equal(code, GOLD["quant_code"][g]), g


@pytest.mark.parametrize("mode,cb,fb", MODES)
def test_record_layout(oracle, mode, cb, fb):
    """The packer reproduces records that the reference's independent decoder
    (attention/python/tests/test_attention.py:51-69) read the expected codes from; the unpacker inverts it."""
    kcode, vcode = GOLD["quant_code"][2], GOLD["quant_code"][4]
    for j in range(8):
        kc, vc = kcode[16 * j:16 * j + 16], vcode[16 * j:16 * j + 16]
        for bits, sel, gold in ((cb, lambda c: c >> fb, GOLD[f"records_coarse_{cb}{fb}"]),
                                (fb, lambda c: c & ((1 << fb) - 1), GOLD[f"records_fine_{cb}{fb}"])):
            rec = oracle.pack_record(bits, sel(kc), sel(vc))
            assert np.array_equal(rec, gold[j])
            uk, uv = oracle.unpack_record(bits, gold[j])
            assert np.array_equal(uk, sel(kc)) and np.array_equal(uv, sel(vc))


def test_encode_layout(oracle):
    """A cache built by the oracle from [1, 1, 512] tokens: three closed groups whose records and metadata decode to
    the quantizer's output, as the reference's test_record_layout checks (test_attention.py:72-86)."""
    _, k, v = datagen.baseline_case(21, 1, 1, 1, 512)
    for mode, cb, fb in MODES:
        c = oracle.encode(k, v, mode)
        for x, tensor in ((k, 0), (v, 1)):
            for g in range(3):
                base, step, code = oracle.quantize_group(x[0, 0, 128 * g:128 * g + 128])
                m = c["meta"][0, g].reshape(2, 32, 2, 4)[tensor]
                assert np.array_equal(m[:, 0].reshape(128), base) and np.array_equal(m[:, 1].reshape(128), step)
                for j in range(8):
                    hi = oracle.unpack_record(cb, c["coarse"][0, 8 * g + j])[tensor]
                    lo = oracle.unpack_record(fb, c["fine"][0, 8 * g + j])[tensor]
                    assert np.array_equal((hi.astype(int) << fb) | lo, code[16 * j:16 * j + 16])
        assert not c["coarse"][0, 24:].any() and not c["meta"][0, 3:].any()   # the open group is not quantized
        assert np.array_equal(c["sink_k"][0], k[0, 0, :128]) and np.array_equal(c["open_v"][0], v[0, 0, 384:])


def test_qhat_definition(oracle):
    """q-hat and sq of the decode oracle's quantize_query equal fbla_reference._quantize_q
    (attention/python/mlops/attention/fbla_reference.py:62-71), through a one-group decode whose scores expose them.
    Checked directly on the definition: qhat = rint(z * fl(127 / max|z|)), sq = max|z| * sl / 127."""
    q_bits, _, _ = datagen.baseline_case(11, 1, 64, 1, 1)
    qf = datagen.bf16_to_f32(q_bits[0])
    steps = datagen.bf16_to_f32(GOLD["quant_step"][[2, 5]])
    z = (qf[:, None, :] * steps[None, :, :]).astype(np.float32)
    amax = np.abs(z).max(-1, keepdims=True)
    r = (np.float32(127.0) / amax).astype(np.float32)
    qh = np.rint(z.astype(np.float64) * r.astype(np.float64)).astype(np.int8)
    assert np.array_equal(qh, GOLD["qhat_codes"])
    sl = np.float32(np.float32(1.0 / np.sqrt(np.float32(128.0))) * np.float32(1.4426950408889634))
    sq = (amax * np.float32(sl * np.float32(1.0 / 127.0))).astype(np.float32)
    assert np.allclose(sq, GOLD["qhat_sq"], rtol=3e-7, atol=0)


DECODE_CASES = [("uneven", "uneven_case", 0), ("baseline", "baseline_case", 1001)]


@pytest.mark.parametrize("name,gen,seed", DECODE_CASES)
@pytest.mark.parametrize("mode,cb,fb", MODES)
@pytest.mark.parametrize("tau", [1e30, 3e-3, 1e-30])
def test_decode_model(oracle, name, gen, seed, mode, cb, fb, tau):
    """The oracle's decode equals the reference's float64 decode model (test_attention.py:111-169) on 1000 tokens,
    4 q heads / 2 KV heads. Tolerance 2e-6 x max|out| (measured 2e-7): that model scales q by sl before quantizing it (a different
    rounding of the same q-hat, which the header and the kernels do not do), so a q-hat may differ by one count."""
    q, k, v = getattr(datagen, gen)(seed, 1, 4, 2, 1000)
    got = oracle.decode(q, oracle.encode(k, v, mode), tau=tau)
    want = GOLD[f"decode_{name}_{cb}{fb}_{tau:g}"]
    err = np.abs(got - want).max() / np.abs(want).max()
    assert err < 2e-6, err


@pytest.mark.parametrize("mode,cb,fb", MODES)
def test_prefill_model(oracle, mode, cb, fb):
    """Chunked prefill (chunks 300, 84, 516 as test_attention.py:205-217) against the reference's model of the DP4A
    path: the decode model of each position with every block refined."""
    q, k, v = datagen.uneven_case(11, 1, 4, 2, 900, q_rows=900)
    c = oracle.empty(1, 2, 1024, mode)
    outs = [oracle.prefill(q[:, :, a:b], k[:, :, a:b], v[:, :, a:b], c) for a, b in ((0, 300), (300, 384), (384, 900))]
    out = np.concatenate(outs, 2)
    for i, t in enumerate(GOLD["prefill_positions"]):
        want = GOLD[f"prefill_{cb}{fb}"][i][0]
        err = np.abs(out[0, :, t] - want).max() / np.abs(want).max()
        assert err < 2e-6, (t, err)
    e = oracle.encode(k, v, mode, capacity=1024)
    for key in ("coarse", "fine", "meta", "sink_k", "sink_v", "open_k", "open_v"):
        assert np.array_equal(c[key], e[key]), key


@pytest.mark.parametrize("mode,cb,fb", MODES)
def test_append_matches_encode(oracle, mode, cb, fb):
    """Token-by-token growth closes groups exactly as a one-shot encode (test_attention.py:195-207)."""
    _, k, v = datagen.uneven_case(7, 1, 4, 2, 700)
    c = oracle.encode(k[:, :, :100], v[:, :, :100], mode, capacity=1024)
    for t in range(100, 700):
        oracle.append(c, k[:, :, t:t + 1], v[:, :, t:t + 1])
        if t in (127, 128, 255, 256, 699):
            e = oracle.encode(k[:, :, :t + 1], v[:, :, :t + 1], mode, capacity=1024)
            for key in ("coarse", "fine", "meta", "sink_k", "sink_v", "open_k", "open_v"):
                assert np.array_equal(c[key], e[key]), (t, key)


def test_decode_close_to_exact_attention(oracle):
    """Distance to float64 attention in units of |v|, as test_attention.py:181-192 (threshold 4e-3)."""
    q, k, v = datagen.uneven_case(5, 1, 4, 2, 4096)
    for mode, _, _ in MODES:
        got = oracle.decode(q, oracle.encode(k, v, mode))
        exact = oracle.exact_decode(q, k, v)
        vf = datagen.bf16_to_f32(v).astype(np.float64)
        err = np.linalg.norm(got[0] - exact[0], axis=-1).mean() / np.sqrt((vf ** 2).sum(-1).mean())
        assert err < 4e-3, err
