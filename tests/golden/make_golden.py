"""Generates tests/golden/fbla_golden.npz by IMPORTING the reference's own Python code (CPU only):

  * attention/python/mlops/attention/fbla.py            _quantize  (the tests' quantizer definition)
  * attention/python/mlops/attention/fbla_reference.py  _quantize_q (the kernels' q-hat definition)
  * attention/python/tests/test_attention.py            _unpack (independent record decoder), _model (float64
                                                        decode model; with tau -> 0 it is also the model of the
                                                        DP4A prefill of one position, test_attention.py:213-225)

Run in the build container, where the reference tree is mounted:
    python tests/golden/make_golden.py <path to the reference tree>
The fixture holds only OUTPUTS of reference code; the inputs are regenerated from seeds by tests/datagen.py.
Records are packed by the oracle and accepted into the fixture only after the reference's decoder has read the
expected codes back from them.
"""
import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from tests import datagen  # noqa: E402
from oracle import fbla_oracle as orc  # noqa: E402


def load_reference(ref_root):
    att = os.path.join(ref_root, "attention", "python")
    for name in ("mlops", "mlops.attention", "mlops.attention._C"):
        sys.modules.setdefault(name, types.ModuleType(name))
    sys.modules["mlops.attention"]._C = sys.modules["mlops.attention._C"]

    def load(name, path):
        spec = importlib.util.spec_from_file_location(name, path)
        mod = importlib.util.module_from_spec(spec)
        sys.modules[name] = mod
        spec.loader.exec_module(mod)
        return mod

    fbla = load("mlops.attention.fbla", os.path.join(att, "mlops", "attention", "fbla.py"))
    ref = load("mlops.attention.fbla_reference", os.path.join(att, "mlops", "attention", "fbla_reference.py"))
    tests = load("ref_test_attention", os.path.join(att, "tests", "test_attention.py"))
    return fbla, ref, tests


def bf(bits):
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).view(torch.bfloat16)


def bits_of(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


DECODE_CASES = [  # (name, generator, seed, q_heads, kv_heads, tokens)
    ("uneven", "uneven_case", 0, 4, 2, 1000),
    ("baseline", "baseline_case", 1001, 4, 2, 1000),
]
TAUS = [1e30, 3e-3, 1e-30]
PREFILL_POS = [0, 15, 16, 127, 128, 129, 255, 256, 300, 383, 384, 511, 640, 899]


def main(ref_root):
    fbla, ref, rtests = load_reference(ref_root)
    out = {}

    # ---- A: quantizer -------------------------------------------------------------------------------------------
    _, kb, vb = datagen.baseline_case(7, 1, 4, 1, 256)
    _, ku, _ = datagen.uneven_case(8, 1, 4, 1, 256)
    groups = np.stack([datagen.edge_group(3), datagen.edge_group(4), kb[0, 0, :128], kb[0, 0, 128:], vb[0, 0, :128], ku[0, 0, :128],
                       ku[0, 0, 128:]])                       # [7, 128, 128]
    x = bf(groups).reshape(1, 1, 7 * 128, 128)
    base, step, code = fbla._quantize(x, 7)
    out["quant_base"] = bits_of(base)[0, 0]
    out["quant_step"] = bits_of(step)[0, 0]
    out["quant_code"] = code[0, 0].numpy().reshape(7, 128, 128)

    # ---- B: record layout ---------------------------------------------------------------------------------------
    kcode, vcode = out["quant_code"][2], out["quant_code"][4]     # one K group, one V group
    for mode, (cb, fb, _) in orc.FORMATS.items():
        recs_c = np.stack([orc.pack_record(cb, kcode[16 * j:16 * j + 16] >> fb, vcode[16 * j:16 * j + 16] >> fb) for j in range(8)])
        recs_f = np.stack([orc.pack_record(fb, kcode[16 * j:16 * j + 16] & ((1 << fb) - 1), vcode[16 * j:16 * j + 16] & ((1 << fb) - 1))
                           for j in range(8)])
        for recs, bits, sel in ((recs_c, cb, lambda c: c >> fb), (recs_f, fb, lambda c: c & ((1 << fb) - 1))):
            uk, uv = rtests._unpack(torch.from_numpy(recs), bits)   # the reference's decoder
            assert np.array_equal(uk.numpy().reshape(128, 128), sel(kcode.astype(np.int64))), (mode, bits, "K")
            assert np.array_equal(uv.numpy().reshape(128, 128), sel(vcode.astype(np.int64))), (mode, bits, "V")
        out[f"records_coarse_{cb}{fb}"] = recs_c
        out[f"records_fine_{cb}{fb}"] = recs_f

    # ---- C: q-hat -------------------------------------------------------------------------------------------------
    q_bits, _, _ = datagen.baseline_case(11, 1, 64, 1, 1)
    qf = datagen.bf16_to_f32(q_bits[0])                               # [64, 128]
    steps = datagen.bf16_to_f32(out["quant_step"][[2, 5]])            # two K step rows
    z = torch.from_numpy(qf[:, None, :] * steps[None, :, :])          # exact in FP32
    sl = (1.0 / np.sqrt(128.0)) * ref.LOG2E
    qh, sq = ref._quantize_q(z, 8, sl)
    out["qhat_codes"] = qh.numpy().astype(np.int8)
    out["qhat_sq"] = sq.numpy().astype(np.float32)

    # ---- D: decode model ------------------------------------------------------------------------------------------
    for name, gen, seed, hq, hk, n in DECODE_CASES:
        q, k, v = getattr(datagen, gen)(seed, 1, hq, hk, n)
        for mode, (cb, fb, _) in orc.FORMATS.items():
            for tau in TAUS:
                m = rtests._model(bf(q), bf(k), bf(v), cb, fb, tau)
                out[f"decode_{name}_{cb}{fb}_{tau:g}"] = m.numpy()

    # ---- E: prefill positions = decode model with every block refined ------------------------------------------------
    q, k, v = datagen.uneven_case(11, 1, 4, 2, 900, q_rows=900)
    for mode, (cb, fb, _) in orc.FORMATS.items():
        rows = []
        for t in PREFILL_POS:
            m = rtests._model(bf(q[:, :, t]), bf(k[:, :, :t + 1]), bf(v[:, :, :t + 1]), cb, fb, 1e-30)
            rows.append(m.numpy())
        out[f"prefill_{cb}{fb}"] = np.stack(rows)                     # [pos, 1, 4, 128]
    out["prefill_positions"] = np.array(PREFILL_POS, np.int32)

    path = os.path.join(HERE, "fbla_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes;", len(out), "arrays")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ["MLOPS_REFERENCE_ROOT"])
